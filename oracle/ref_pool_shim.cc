// The reference engine's paged KV pool (engine/src/kv_pool.{h,cc}, compiled from where they lie)
// behind a C interface shaped like the library's granite4_kv_pool_*, so that a test can drive
// both with the same calls. Test infrastructure only; nothing of the reference is copied here.
#include "kv_pool.h"  // from the reference tree, via -I
#include "kv_pool_controller.h"

#include <algorithm>
#include <cstdint>
#include <vector>

using granite4::KvPoolConfig;
using granite4::KvPoolController;
using granite4::PagedKV;

extern "C" {

void* g4ref_pool_create(int num_pages, int tokens_per_page) {
  KvPoolConfig c;
  c.tokens_per_page = static_cast<std::size_t>(tokens_per_page);
  c.num_pages = static_cast<std::size_t>(num_pages);
  return new PagedKV(c);
}
void g4ref_pool_destroy(void* p) { delete static_cast<PagedKV*>(p); }
int g4ref_pool_create_sequence(void* p) { return static_cast<PagedKV*>(p)->create_sequence(); }
long long g4ref_pool_match_prefix(void* p, int seq, const std::uint32_t* tokens, long long n) {
  return static_cast<long long>(static_cast<PagedKV*>(p)->match_prefix(seq, PagedKV::Tokens(tokens, tokens + n)));
}
int g4ref_pool_reserve(void* p, int seq, long long count, const std::uint32_t* tokens, long long n) {
  return static_cast<PagedKV*>(p)->reserve(seq, static_cast<std::size_t>(count), PagedKV::Tokens(tokens, tokens + n));
}
int g4ref_pool_mark_written(void* p, int seq, long long page_index) {
  return static_cast<PagedKV*>(p)->mark_written(seq, static_cast<std::size_t>(page_index));
}
int g4ref_pool_row_table(void* p, int seq, long long n, int* out) {
  return static_cast<PagedKV*>(p)->row_table(seq, static_cast<std::size_t>(n), out);
}
void g4ref_pool_reset_sequence(void* p, int seq) { static_cast<PagedKV*>(p)->reset_sequence(seq); }
void g4ref_pool_truncate_sequence(void* p, int seq, long long n) {
  static_cast<PagedKV*>(p)->truncate_sequence(seq, static_cast<std::size_t>(n));
}
void g4ref_pool_release(void* p, int seq) { static_cast<PagedKV*>(p)->release(seq); }
void g4ref_pool_clear(void* p) { static_cast<PagedKV*>(p)->clear(); }
long long g4ref_pool_count(void* p, int which) {
  PagedKV* k = static_cast<PagedKV*>(p);
  switch (which) {
    case 0: return static_cast<long long>(k->free_pages());
    case 1: return static_cast<long long>(k->used_pages());
    case 2: return static_cast<long long>(k->shared_pages());
    case 3: return static_cast<long long>(k->cached_pages());
    case 4: return static_cast<long long>(k->evicted_pages());
    case 5: return static_cast<long long>(k->retained_pages());
    case 6: return static_cast<long long>(k->live_sequences());
    default: return -1;
  }
}
long long g4ref_pool_sequence_tokens(void* p, int seq) {
  return static_cast<long long>(static_cast<PagedKV*>(p)->sequence_tokens(seq));
}
long long g4ref_pool_block_table(void* p, int seq, int* out, long long capacity) {
  const std::vector<std::size_t>& bt = static_cast<PagedKV*>(p)->block_table(seq);
  if (out != nullptr)
    for (long long i = 0; i < std::min<long long>(capacity, static_cast<long long>(bt.size())); ++i)
      out[i] = static_cast<int>(bt[static_cast<std::size_t>(i)]);
  return static_cast<long long>(bt.size());
}
int g4ref_pool_ref_count(void* p, int page) {
  return static_cast<int>(static_cast<PagedKV*>(p)->ref_count(static_cast<std::size_t>(page)));
}
int g4ref_pool_page_in_cache(void* p, int page) {
  return static_cast<PagedKV*>(p)->page_in_cache(static_cast<std::size_t>(page)) ? 1 : 0;
}


// ---- the reference's serve-loop controller (engine/src/kv_pool_controller.{h,cc}) ----------------
void* g4ref_ctl_create(int num_pages, int tokens_per_page) {
  KvPoolConfig c;
  c.tokens_per_page = static_cast<std::size_t>(tokens_per_page);
  c.num_pages = static_cast<std::size_t>(num_pages);
  return new KvPoolController(c);
}
void g4ref_ctl_destroy(void* p) { delete static_cast<KvPoolController*>(p); }
void g4ref_ctl_shutdown(void* p) { static_cast<KvPoolController*>(p)->shutdown(); }
int g4ref_ctl_new_slot(void* p) { return static_cast<KvPoolController*>(p)->new_slot(); }
void g4ref_ctl_release_slot(void* p, int slot) { static_cast<KvPoolController*>(p)->release_slot(slot); }
int g4ref_ctl_prefill(void* p, int slot, const std::uint32_t* prompt, long long n, int* seq_out, long long* reused_out) {
  const KvPoolController::Prefill r = static_cast<KvPoolController*>(p)->prefill(slot, PagedKV::Tokens(prompt, prompt + n));
  if (seq_out != nullptr) *seq_out = r.seq;
  if (reused_out != nullptr) *reused_out = static_cast<long long>(r.reused);
  return r.ok ? 1 : 0;
}
void g4ref_ctl_commit(void* p, int slot, const std::uint32_t* tokens, long long n) {
  static_cast<KvPoolController*>(p)->commit(slot, PagedKV::Tokens(tokens, tokens + n));
}
int g4ref_ctl_open_slot(void* p) { return static_cast<KvPoolController*>(p)->open_slot(); }
int g4ref_ctl_ensure(void* p, int slot, long long n) {
  return static_cast<KvPoolController*>(p)->ensure(slot, static_cast<std::size_t>(n)) ? 1 : 0;
}
void g4ref_ctl_trim(void* p, int slot, long long n) { static_cast<KvPoolController*>(p)->trim(slot, static_cast<std::size_t>(n)); }
void g4ref_ctl_drop(void* p, int slot) { static_cast<KvPoolController*>(p)->drop(slot); }
long long g4ref_ctl_slot_pages(void* p, int slot) {
  return static_cast<long long>(static_cast<KvPoolController*>(p)->slot_pages(slot));
}
long long g4ref_ctl_pages_missing(void* p, int slot, long long n) {
  return static_cast<long long>(static_cast<KvPoolController*>(p)->pages_missing(slot, static_cast<std::size_t>(n)));
}
int g4ref_ctl_row_table(void* p, int slot, long long n, int* out) {
  return static_cast<KvPoolController*>(p)->row_table(slot, static_cast<std::size_t>(n), out) ? 1 : 0;
}
long long g4ref_ctl_committed(void* p, int slot) {
  return static_cast<long long>(static_cast<KvPoolController*>(p)->committed(slot));
}
long long g4ref_ctl_last_reused(void* p, int slot) {
  return static_cast<long long>(static_cast<KvPoolController*>(p)->last_reused(slot));
}
long long g4ref_ctl_max_slots(void* p) { return static_cast<long long>(static_cast<KvPoolController*>(p)->max_slots()); }
long long g4ref_ctl_count(void* p, int which) {
  KvPoolController* k = static_cast<KvPoolController*>(p);
  switch (which) {
    case 0: return static_cast<long long>(k->free_pages());
    case 1: return static_cast<long long>(k->used_pages());
    case 2: return static_cast<long long>(k->shared_pages());
    case 3: return static_cast<long long>(k->cached_pages());
    case 4: return static_cast<long long>(k->evicted_pages());
    case 5: return static_cast<long long>(k->retained_pages());
    default: return -1;
  }
}

}  // extern "C"
