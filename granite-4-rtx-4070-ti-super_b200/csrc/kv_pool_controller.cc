// Serve-loop controller over the paged KV pool: session slots.
//
// The pool (kv_pool.cc) hands out pages to sequences and keeps the prefix cache; it knows nothing
// about sessions. A serve loop owns a fixed set of session slots, one per concurrent request, and
// wants three things of each: start a request (adopt whatever page-aligned prefix of the prompt is
// already cached, reserve the rest), account for every generated token (grow by a page at page
// boundaries, publish pages as they fill), and a position -> pool row table for the KV-write and
// attention kernels. A second family of calls serves resident conversations that never share pages:
// open a slot, grow it, give pages back, drop it.
//
// Behaviour follows the reference's KvPoolController (engine/src/kv_pool_controller.h:32-112,
// engine/src/kv_pool_controller.cc) call for call - slot ids, return values, row tables and the
// pool's counts are the same for the same traffic (tests drive both). Pure host code: it reasons in
// pages and token ids, never in bytes or device pointers.
//
// The implementation is a slot table over the C interface of the pool. Differences in form: slots
// are searched through a free list threaded through the idle ones, lowest id first (the reference
// scans all slots for the first idle one - same id, found without the scan), and the
// placeholder ids that ensure() hands to the pool come from one zero buffer that only ever grows.
#include "../../include/granite4_b200.h"

#include <algorithm>
#include <cstdint>
#include <new>
#include <set>
#include <vector>

namespace {

struct SlotState {
  int seq = -1;
  long long marked_pages = 0;  // leading pages already published (shared ones included)
  long long reused = 0;        // page-aligned tokens the last prefill found cached
  bool in_use = false;
};

}  // namespace

struct granite4_kv_ctl {
  granite4_kv_pool* pool = nullptr;
  int num_pages = 0, B = 0;
  std::vector<SlotState> slots;
  std::set<int> idle;  // ids of slots not in use, ordered: the lowest is recycled first
  std::vector<std::uint32_t> zeros;

  SlotState* at(int slot) {
    return (slot < 0 || slot >= static_cast<int>(slots.size())) ? nullptr : &slots[static_cast<std::size_t>(slot)];
  }
  const SlotState* at(int slot) const {
    return (slot < 0 || slot >= static_cast<int>(slots.size())) ? nullptr : &slots[static_cast<std::size_t>(slot)];
  }
  void set_in_use(int slot, bool on) {
    SlotState& s = slots[static_cast<std::size_t>(slot)];
    if (s.in_use == on) return;
    s.in_use = on;
    if (on) idle.erase(slot); else idle.insert(slot);
  }
  // engine/src/kv_pool_controller.cc:153-160: publish every page that became full since the last call
  void mark_new_full(SlotState& s, long long n_tokens) {
    const long long full = n_tokens / B;
    for (long long i = s.marked_pages; i < full; ++i) granite4_kv_pool_mark_written(pool, s.seq, i);
    s.marked_pages = full;
  }
};

extern "C" {

granite4_kv_ctl* granite4_kv_ctl_create(int num_pages, int tokens_per_page) {
  granite4_kv_pool* pool = granite4_kv_pool_create(num_pages, tokens_per_page);
  if (pool == nullptr) return nullptr;
  granite4_kv_ctl* c = new (std::nothrow) granite4_kv_ctl;
  if (c == nullptr) {
    granite4_kv_pool_destroy(pool);
    return nullptr;
  }
  c->pool = pool, c->num_pages = num_pages, c->B = tokens_per_page;
  return c;
}

void granite4_kv_ctl_shutdown(granite4_kv_ctl* c) {
  if (c == nullptr) return;
  for (const SlotState& s : c->slots)
    if (s.in_use) granite4_kv_pool_release(c->pool, s.seq);
  granite4_kv_pool_clear(c->pool);
  c->slots.clear();
  c->idle.clear();
}

void granite4_kv_ctl_destroy(granite4_kv_ctl* c) {
  if (c == nullptr) return;
  granite4_kv_ctl_shutdown(c);
  granite4_kv_pool_destroy(c->pool);
  delete c;
}

granite4_kv_pool* granite4_kv_ctl_pool(granite4_kv_ctl* c) { return c == nullptr ? nullptr : c->pool; }

int granite4_kv_ctl_new_slot(granite4_kv_ctl* c) {
  if (c == nullptr) return -1;
  // An idle slot keeps its pool sequence (reset, not released), so its id is stable across requests.
  // As in the reference, recycling leaves it idle: prefill() or open_slot() puts it in use.
  if (!c->idle.empty()) {
    const int slot = *c->idle.begin();
    SlotState& s = c->slots[static_cast<std::size_t>(slot)];
    s.marked_pages = 0, s.reused = 0;
    return slot;
  }
  const int seq = granite4_kv_pool_create_sequence(c->pool);
  if (seq < 0) return -1;  // live sequences are capped at the number of pages
  SlotState s;
  s.seq = seq, s.in_use = true;
  c->slots.push_back(s);
  return static_cast<int>(c->slots.size()) - 1;
}

void granite4_kv_ctl_release_slot(granite4_kv_ctl* c, int slot) {
  SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr) return;
  granite4_kv_pool_reset_sequence(c->pool, s->seq);  // private pages freed, published ones retained
  c->set_in_use(slot, false);
  s->marked_pages = 0, s->reused = 0;
}

int granite4_kv_ctl_prefill(granite4_kv_ctl* c, int slot, const uint32_t* prompt, long long n, int* seq_out,
                            long long* reused_out) {
  if (seq_out != nullptr) *seq_out = -1;
  if (reused_out != nullptr) *reused_out = 0;
  SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr || n < 0 || (n > 0 && prompt == nullptr)) return 0;
  granite4_kv_pool_reset_sequence(c->pool, s->seq);  // whatever an earlier request left on the slot
  s->marked_pages = 0;
  s->reused = granite4_kv_pool_match_prefix(c->pool, s->seq, prompt, n);
  if (!granite4_kv_pool_reserve(c->pool, s->seq, n, prompt, n)) {
    granite4_kv_pool_reset_sequence(c->pool, s->seq);  // give back what match_prefix adopted
    c->set_in_use(slot, false);
    s->reused = 0;
    return 0;
  }
  c->set_in_use(slot, true);
  c->mark_new_full(*s, n);
  if (seq_out != nullptr) *seq_out = s->seq;
  if (reused_out != nullptr) *reused_out = s->reused;
  return 1;
}

void granite4_kv_ctl_commit(granite4_kv_ctl* c, int slot, const uint32_t* all_tokens, long long n) {
  SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr || !s->in_use || n < 0 || (n > 0 && all_tokens == nullptr)) return;
  if (n <= granite4_kv_pool_sequence_tokens(c->pool, s->seq)) return;  // nothing new
  if (!granite4_kv_pool_reserve(c->pool, s->seq, n, all_tokens, n)) return;
  c->mark_new_full(*s, n);
}

int granite4_kv_ctl_open_slot(granite4_kv_ctl* c) {
  const int slot = granite4_kv_ctl_new_slot(c);
  if (slot < 0) return -1;
  c->set_in_use(slot, true);
  return slot;
}

int granite4_kv_ctl_ensure(granite4_kv_ctl* c, int slot, long long n_tokens) {
  SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr || !s->in_use || n_tokens < 0) return 0;
  if (n_tokens <= granite4_kv_pool_sequence_tokens(c->pool, s->seq)) return 1;
  // the pool wants the full id list; these pages are never published, so the ids are placeholders
  if (static_cast<long long>(c->zeros.size()) < n_tokens) c->zeros.resize(static_cast<std::size_t>(n_tokens), 0u);
  return granite4_kv_pool_reserve(c->pool, s->seq, n_tokens, c->zeros.data(), n_tokens);
}

void granite4_kv_ctl_trim(granite4_kv_ctl* c, int slot, long long n_tokens) {
  SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr || !s->in_use) return;
  granite4_kv_pool_truncate_sequence(c->pool, s->seq, n_tokens);
}

void granite4_kv_ctl_drop(granite4_kv_ctl* c, int slot) {
  SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr || !s->in_use) return;
  granite4_kv_pool_reset_sequence(c->pool, s->seq);
  s->marked_pages = 0, s->reused = 0;
}

long long granite4_kv_ctl_slot_pages(const granite4_kv_ctl* c, int slot) {
  const SlotState* s = c == nullptr ? nullptr : c->at(slot);
  return (s == nullptr || !s->in_use) ? 0 : granite4_kv_pool_block_table(c->pool, s->seq, nullptr, 0);
}

long long granite4_kv_ctl_pages_missing(const granite4_kv_ctl* c, int slot, long long n_tokens) {
  if (c == nullptr || n_tokens < 0) return 0;
  const long long want = (n_tokens + c->B - 1) / c->B, have = granite4_kv_ctl_slot_pages(c, slot);
  return want > have ? want - have : 0;
}

int granite4_kv_ctl_row_table(const granite4_kv_ctl* c, int slot, long long n, int* out) {
  const SlotState* s = c == nullptr ? nullptr : c->at(slot);
  if (s == nullptr || !s->in_use) return 0;
  return granite4_kv_pool_row_table(c->pool, s->seq, n, out);
}

long long granite4_kv_ctl_committed(const granite4_kv_ctl* c, int slot) {
  const SlotState* s = c == nullptr ? nullptr : c->at(slot);
  return (s == nullptr || !s->in_use) ? 0 : granite4_kv_pool_sequence_tokens(c->pool, s->seq);
}

long long granite4_kv_ctl_last_reused(const granite4_kv_ctl* c, int slot) {
  const SlotState* s = c == nullptr ? nullptr : c->at(slot);
  return s == nullptr ? 0 : s->reused;
}

long long granite4_kv_ctl_max_slots(const granite4_kv_ctl* c) { return c == nullptr ? 0 : c->num_pages; }

long long granite4_kv_ctl_count(const granite4_kv_ctl* c, int which) {
  return c == nullptr ? -1 : granite4_kv_pool_count(c->pool, which);
}

}  // extern "C"
