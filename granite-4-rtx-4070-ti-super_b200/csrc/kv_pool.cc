// Host-side paged KV pool: which pool rows a sequence's cache positions live in.
//
// This is the controller behind the d_pt / kv_rows tables the KV-write and
// attention kernels index through. Behaviour follows the reference's PagedKV
// (engine/src/kv_pool.h:102-199, engine/src/kv_pool.cc): pages of
// tokens_per_page consecutive pool rows; a sequence holds a dense block table
// (page i covers positions [i B, (i + 1) B)); full pages can be published in a
// prefix cache keyed by the chained FNV-1a hash of the token prefix and shared,
// reference counted, by later sequences with the same prefix; pages nobody
// references but the cache still holds are retained and evicted least recently
// used first when an allocation finds the free stack empty. Row of position p:
// block_table[p / B] * B + p % B (engine/src/kv_pool.cc:285-298).
//
// The observable behaviour - page ids handed out, row tables, counts - is the
// reference's, call for call (tests drive both with the same random call
// sequences); the bookkeeping is not: page tokens live in one flat array, the
// chained prefix hash of a sequence is kept per page boundary instead of being
// re-derived from the first page on every lookup, and the retained pages sit
// in a set ordered by their last-use tick, so an eviction is a set lookup, not a
// scan over the pool.
#include "../../include/granite4_b200.h"

#include <algorithm>
#include <cstdint>
#include <new>
#include <set>
#include <unordered_map>
#include <utility>
#include <vector>

namespace {

constexpr std::uint64_t kFnvOffset = 1469598103934665603ULL;  // engine/src/kv_pool.cc:20-21
constexpr std::uint64_t kFnvPrime = 1099511628211ULL;

std::uint64_t fnv_extend(std::uint64_t h, const std::uint32_t* data, std::size_t n) {
  for (std::size_t i = 0; i < n; ++i) {
    h ^= static_cast<std::uint64_t>(data[i]);
    h *= kFnvPrime;
  }
  return h;
}

struct PageState {
  std::uint64_t key = 0;        // cache key once published
  std::uint64_t last_used = 0;  // tick of the last publication or reuse
  int refs = 0;
  int filled = 0;  // token ids stored for this page (<= B)
  bool cached = false;
};

struct SequenceState {
  std::vector<int> pages;             // block table
  std::vector<std::uint64_t> chain;   // chain[i]: hash of the tokens of pages [0, i); grown lazily
  long long filled = 0;
  bool live = false;
};

}  // namespace

struct granite4_kv_pool {
  int num_pages = 0, B = 0;
  std::vector<PageState> page;
  std::vector<std::uint32_t> tokens;  // [num_pages][B]
  std::vector<SequenceState> seq;
  std::vector<int> free_stack;        // the back is handed out first
  std::unordered_map<std::uint64_t, int> cache;
  std::set<std::pair<std::uint64_t, int>> retained;  // (last_used, page) of cached pages with no reference
  std::uint64_t tick = 0;
  long long evicted = 0;

  std::uint32_t* page_tokens(int id) { return tokens.data() + static_cast<std::size_t>(id) * B; }
  bool alive(int s) const { return s >= 0 && s < static_cast<int>(seq.size()) && seq[s].live; }

  void reset_free_stack() {
    free_stack.resize(num_pages);
    for (int i = 0; i < num_pages; ++i) free_stack[i] = i;
  }

  void wipe(PageState& p) {
    p.key = 0, p.last_used = 0, p.filled = 0;
  }

  void touch(int id) {  // a cached page was published or reused
    PageState& p = page[id];
    if (p.cached && p.refs == 0) retained.erase({p.last_used, id});
    p.last_used = ++tick;
    if (p.cached && p.refs == 0) retained.insert({p.last_used, id});
  }

  void take(int s, int id) {
    PageState& p = page[id];
    if (p.cached && p.refs == 0) retained.erase({p.last_used, id});
    p.refs += 1;
    seq[s].pages.push_back(id);
  }

  void drop(int id) {
    PageState& p = page[id];
    if (p.refs > 0) p.refs -= 1;
    if (p.refs != 0) return;
    if (p.cached) {
      retained.insert({p.last_used, id});  // still cached: retained, evictable
      return;
    }
    wipe(p);
    free_stack.push_back(id);
  }

  bool evict_one() {
    if (retained.empty()) return false;
    const int id = retained.begin()->second;
    retained.erase(retained.begin());
    PageState& p = page[id];
    const auto it = cache.find(p.key);
    if (it != cache.end() && it->second == id) cache.erase(it);
    p.cached = false;
    wipe(p);
    free_stack.push_back(id);
    ++evicted;
    return true;
  }

  // Hash of the tokens of the first `upto` pages of the sequence (all of them full but possibly
  // the last one it holds), continued from where the previous call stopped.
  std::uint64_t chain_key(int s, std::size_t upto) {
    SequenceState& q = seq[s];
    if (q.chain.empty()) q.chain.push_back(kFnvOffset);
    while (q.chain.size() <= upto) {
      const int id = q.pages[q.chain.size() - 1];
      q.chain.push_back(fnv_extend(q.chain.back(), page_tokens(id), static_cast<std::size_t>(page[id].filled)));
    }
    return q.chain[upto];
  }
  // The stored hashes stay valid only for pages whose tokens can no longer change.
  void trim_chain(int s, std::size_t full_pages) {
    SequenceState& q = seq[s];
    if (q.chain.size() > full_pages + 1) q.chain.resize(full_pages + 1);
  }

  long long count(int which) const {
    long long n = 0;
    switch (which) {
      case GRANITE4_KV_POOL_FREE_PAGES: return static_cast<long long>(free_stack.size());
      case GRANITE4_KV_POOL_USED_PAGES: return num_pages - static_cast<long long>(free_stack.size());
      case GRANITE4_KV_POOL_SHARED_PAGES:
        for (const PageState& p : page) n += p.refs > 1;
        return n;
      case GRANITE4_KV_POOL_CACHED_PAGES: return static_cast<long long>(cache.size());
      case GRANITE4_KV_POOL_EVICTED_PAGES: return evicted;
      case GRANITE4_KV_POOL_RETAINED_PAGES:
        for (const PageState& p : page) n += p.cached && p.refs == 0;
        return n;
      case GRANITE4_KV_POOL_LIVE_SEQUENCES:
        for (const SequenceState& q : seq) n += q.live;
        return n;
      default: return -1;
    }
  }
};

extern "C" {

granite4_kv_pool* granite4_kv_pool_create(int num_pages, int tokens_per_page) {
  if (num_pages < 0 || tokens_per_page <= 0) return nullptr;
  granite4_kv_pool* pool = new (std::nothrow) granite4_kv_pool;
  if (pool == nullptr) return nullptr;
  pool->num_pages = num_pages, pool->B = tokens_per_page;
  pool->page.resize(num_pages);
  pool->tokens.resize(static_cast<std::size_t>(num_pages) * tokens_per_page);
  pool->reset_free_stack();
  return pool;
}

void granite4_kv_pool_destroy(granite4_kv_pool* pool) { delete pool; }

int granite4_kv_pool_create_sequence(granite4_kv_pool* pool) {
  if (pool == nullptr) return -1;
  // engine/src/kv_pool.cc:134-137: a sequence without a page is useless
  if (pool->count(GRANITE4_KV_POOL_LIVE_SEQUENCES) >= std::max(1, pool->num_pages)) return -1;
  pool->seq.emplace_back();
  pool->seq.back().live = true;
  return static_cast<int>(pool->seq.size()) - 1;
}

long long granite4_kv_pool_match_prefix(granite4_kv_pool* pool, int seq, const uint32_t* tokens, long long n) {
  if (pool == nullptr || !pool->alive(seq) || pool->seq[seq].filled != 0 || (tokens == nullptr && n > 0)) return 0;
  const int B = pool->B;
  long long pos = 0;
  while (pos + B <= n) {
    const std::uint64_t key = fnv_extend(pool->chain_key(seq, static_cast<std::size_t>(pos / B)), tokens + pos, B);
    const auto it = pool->cache.find(key);
    if (it == pool->cache.end()) break;
    const int id = it->second;
    if (pool->page[id].filled != B) break;
    if (!std::equal(tokens + pos, tokens + pos + B, pool->page_tokens(id))) break;  // a hash collision
    pool->take(seq, id);
    pool->touch(id);
    pool->seq[seq].filled += B;
    pos += B;
  }
  return pos;
}

int granite4_kv_pool_reserve(granite4_kv_pool* pool, int seq, long long token_count, const uint32_t* tokens,
                             long long n) {
  if (pool == nullptr || !pool->alive(seq) || token_count < 0 || n < token_count ||
      (tokens == nullptr && token_count > 0))
    return 0;
  SequenceState& q = pool->seq[seq];
  if (token_count <= q.filled) return 1;
  const long long B = pool->B;
  const long long held = static_cast<long long>(q.pages.size()) * B;
  const long long overflow = token_count > held ? token_count - held : 0;
  const long long pages_needed = (overflow + B - 1) / B;
  // make room first; nothing has been changed if this fails
  while (static_cast<long long>(pool->free_stack.size()) < pages_needed)
    if (!pool->evict_one()) return 0;
  if (q.filled < held) {  // fill the partial last page before appending new ones
    const int id = q.pages.back();
    const long long take = std::min(held - q.filled, token_count - q.filled);
    std::copy(tokens + q.filled, tokens + q.filled + take, pool->page_tokens(id) + pool->page[id].filled);
    pool->page[id].filled += static_cast<int>(take);
    q.filled += take;
    if (q.filled >= token_count) return 1;
  }
  const long long start = q.filled;
  for (long long k = 0; k < pages_needed; ++k) {
    const int id = pool->free_stack.back();
    pool->free_stack.pop_back();
    const long long lo = start + k * B, hi = std::min(lo + B, token_count);
    PageState& p = pool->page[id];
    p = PageState{};
    std::copy(tokens + lo, tokens + hi, pool->page_tokens(id));
    p.filled = static_cast<int>(hi - lo);
    pool->take(seq, id);
    q.filled = hi;
    if (hi < lo + B) break;
  }
  return 1;
}

int granite4_kv_pool_mark_written(granite4_kv_pool* pool, int seq, long long page_index) {
  if (pool == nullptr || !pool->alive(seq)) return 0;
  SequenceState& q = pool->seq[seq];
  if (page_index < 0 || page_index >= static_cast<long long>(q.pages.size())) return 0;
  const int id = q.pages[static_cast<std::size_t>(page_index)];
  PageState& p = pool->page[id];
  if (p.refs != 1 || p.filled != pool->B) return 0;  // shared pages are published already; partial ones cannot be
  const std::uint64_t key =
      fnv_extend(pool->chain_key(seq, static_cast<std::size_t>(page_index)), pool->page_tokens(id), pool->B);
  p.key = key;
  const auto it = pool->cache.find(key);
  if (it != pool->cache.end() && it->second != id) {
    // a colliding older entry is no longer addressable; its page stays as it is
    PageState& old = pool->page[it->second];
    if (old.cached && old.refs == 0) pool->retained.erase({old.last_used, it->second});
    old.cached = false;
  }
  pool->cache[key] = id;
  p.cached = true;
  p.last_used = ++pool->tick;
  return 1;
}

int granite4_kv_pool_row_table(const granite4_kv_pool* pool, int seq, long long n, int* out) {
  if (pool == nullptr || !pool->alive(seq) || out == nullptr || n < 0 || n > pool->seq[seq].filled) return 0;
  const SequenceState& q = pool->seq[seq];
  const int B = pool->B;
  for (long long p = 0; p < n; ++p) out[p] = q.pages[static_cast<std::size_t>(p / B)] * B + static_cast<int>(p % B);
  return 1;
}

void granite4_kv_pool_reset_sequence(granite4_kv_pool* pool, int seq) {
  if (pool == nullptr || !pool->alive(seq)) return;
  SequenceState& q = pool->seq[seq];
  for (const int id : q.pages) pool->drop(id);
  q.pages.clear();
  q.chain.clear();
  q.filled = 0;
}

void granite4_kv_pool_truncate_sequence(granite4_kv_pool* pool, int seq, long long n_tokens) {
  if (pool == nullptr || !pool->alive(seq) || n_tokens < 0) return;
  SequenceState& q = pool->seq[seq];
  const long long B = pool->B;
  const std::size_t keep = static_cast<std::size_t>((n_tokens + B - 1) / B);
  if (q.pages.size() < keep) return;  // nothing held beyond n_tokens
  for (std::size_t i = keep; i < q.pages.size(); ++i) pool->drop(q.pages[i]);
  q.pages.resize(keep);
  q.filled = std::min(q.filled, n_tokens);
  // The last kept page is brought in line with the new length in every case. (The reference does
  // this only when a page was dropped; when none is, it leaves the page's token record long.)
  if (keep > 0) {
    PageState& last = pool->page[q.pages.back()];
    if (last.cached) {
      q.filled = static_cast<long long>(keep) * B;  // a published page is full and shared: kept whole
    } else {
      const long long in_last = q.filled > static_cast<long long>(keep - 1) * B ? q.filled - static_cast<long long>(keep - 1) * B : 0;
      if (last.filled > in_last) last.filled = static_cast<int>(in_last);
    }
  }
  pool->trim_chain(seq, keep > 0 ? keep - 1 : 0);
}

void granite4_kv_pool_release(granite4_kv_pool* pool, int seq) {
  if (pool == nullptr || !pool->alive(seq)) return;
  granite4_kv_pool_reset_sequence(pool, seq);
  pool->seq[seq].live = false;
}

void granite4_kv_pool_clear(granite4_kv_pool* pool) {
  if (pool == nullptr) return;
  pool->seq.clear();
  pool->cache.clear();
  pool->retained.clear();
  for (PageState& p : pool->page) p = PageState{};
  pool->reset_free_stack();
  pool->tick = 0;
  pool->evicted = 0;
}

long long granite4_kv_pool_count(const granite4_kv_pool* pool, int which) {
  return pool == nullptr ? -1 : pool->count(which);
}

long long granite4_kv_pool_sequence_tokens(const granite4_kv_pool* pool, int seq) {
  return (pool == nullptr || !pool->alive(seq)) ? 0 : pool->seq[seq].filled;
}

long long granite4_kv_pool_block_table(const granite4_kv_pool* pool, int seq, int* out, long long capacity) {
  if (pool == nullptr || !pool->alive(seq)) return 0;
  const std::vector<int>& pages = pool->seq[seq].pages;
  const long long n = static_cast<long long>(pages.size());
  if (out != nullptr)
    for (long long i = 0; i < std::min(n, capacity); ++i) out[i] = pages[static_cast<std::size_t>(i)];
  return n;
}

int granite4_kv_pool_ref_count(const granite4_kv_pool* pool, int page) {
  return (pool == nullptr || page < 0 || page >= pool->num_pages) ? 0 : pool->page[page].refs;
}

int granite4_kv_pool_page_in_cache(const granite4_kv_pool* pool, int page) {
  return (pool == nullptr || page < 0 || page >= pool->num_pages) ? 0 : pool->page[page].cached;
}

int granite4_kv_pool_move_rows(const granite4_kv_pool* pool, int seq, const int* src_pos, const int* dst_pos,
                               int n, int* src_rows, int* dst_rows) {
  // engine/src/forward_gpu.cu:3508-3522: logical positions of an accepted draft path -> pool rows
  if (pool == nullptr || !pool->alive(seq) || n < 0 || n > GRANITE4_MAX_TREE_DEPTH || src_pos == nullptr ||
      dst_pos == nullptr || src_rows == nullptr || dst_rows == nullptr)
    return -1;
  const SequenceState& q = pool->seq[seq];
  const long long mapped = static_cast<long long>(q.pages.size()) * pool->B;
  for (int i = 0; i < n; ++i) {
    if (src_pos[i] < 0 || dst_pos[i] < 0 || src_pos[i] >= mapped || dst_pos[i] >= mapped || dst_pos[i] > src_pos[i])
      return -1;
    for (int j = i + 1; j < n; ++j)
      if (src_pos[j] == dst_pos[i]) return -1;
    src_rows[i] = q.pages[static_cast<std::size_t>(src_pos[i] / pool->B)] * pool->B + src_pos[i] % pool->B;
    dst_rows[i] = q.pages[static_cast<std::size_t>(dst_pos[i] / pool->B)] * pool->B + dst_pos[i] % pool->B;
  }
  return 0;
}

}  // extern "C"
