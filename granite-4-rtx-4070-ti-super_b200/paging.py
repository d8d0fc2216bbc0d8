"""Host side of the paged KV write: position -> pool-row tables for 16-token pages.

The device kernels only ever see integer pool rows; how pages are allocated is the
serving loop's business. These helpers restate the one rule the reference's pool uses
(``engine/src/kv_pool.cc:285-298``, ``engine/src/kv_pool.h:137-151``): logical position p of
a sequence lives in physical row ``block_table[p // B] * B + p % B`` with B tokens per page
(``engine/src/kv_pool.h:83``: 16). Pure numpy, no device work.
"""
from __future__ import annotations

import numpy as np

TOKENS_PER_PAGE = 16


def row_table(block_table, n_positions: int, tokens_per_page: int = TOKENS_PER_PAGE) -> np.ndarray:
    """Physical row of each logical position [0, n_positions) of one sequence."""
    block_table = np.asarray(block_table, dtype=np.int64)
    need = (n_positions + tokens_per_page - 1) // tokens_per_page
    if need > block_table.size:
        raise ValueError(f"{n_positions} positions need {need} pages, the sequence has "
                         f"{block_table.size}")
    p = np.arange(n_positions, dtype=np.int64)
    return (block_table[p // tokens_per_page] * tokens_per_page + p % tokens_per_page).astype(np.int32)


def validate_rows(kv_rows, pool_rows: int) -> None:
    """The reference checks a table for range and distinctness before handing it to the device
    (``engine/src/forward_gpu.cu:3570-3586``); two tokens must never share a pool row."""
    kv_rows = np.asarray(kv_rows)
    if kv_rows.size and (kv_rows.min() < 0 or kv_rows.max() >= pool_rows):
        raise ValueError("pool row out of range")
    if np.unique(kv_rows).size != kv_rows.size:
        raise ValueError("pool rows are not distinct")


def permuted_block_tables(n_sequences: int, pages_per_sequence: int, pool_pages: int, seed: int):
    """Disjoint block tables drawn from one random permutation of the pool's pages."""
    if n_sequences * pages_per_sequence > pool_pages:
        raise ValueError("pool too small")
    perm = np.random.default_rng(seed).permutation(pool_pages)
    return [perm[s * pages_per_sequence:(s + 1) * pages_per_sequence] for s in range(n_sequences)]


def batch_rows(block_tables, first_positions, tokens_per_sequence: int,
               tokens_per_page: int = TOKENS_PER_PAGE):
    """Per-row (RoPE position, pool row) arrays for a batch of sequences, sequence-major.

    Sequence s contributes tokens at RoPE positions first_positions[s] + [0, tokens_per_sequence)
    and stores token i in the page block_tables[s][i // B] at slot (first_positions[s] + i) % B
    when that stays inside the page run, i.e. its pages hold this chunk from slot 0 of the
    first page on: logical index within the chunk decides the page, as in row_table().
    """
    pos, rows = [], []
    for bt, p0 in zip(block_tables, first_positions):
        pos.append(np.arange(p0, p0 + tokens_per_sequence, dtype=np.int32))
        rows.append(row_table(bt, tokens_per_sequence, tokens_per_page))
    return np.concatenate(pos), np.concatenate(rows)


class KvPool:
    """The library's host-side paged KV pool (``granite4_kv_pool_*``): the reference's
    ``PagedKV`` (``engine/src/kv_pool.h:102-199``) behind the C ABI. Method names and meanings
    are the reference's; token id lists are sequences of non-negative ints."""

    COUNTS = {"free_pages": 0, "used_pages": 1, "shared_pages": 2, "cached_pages": 3,
              "evicted_pages": 4, "retained_pages": 5, "live_sequences": 6}

    def __init__(self, num_pages: int, tokens_per_page: int = TOKENS_PER_PAGE):
        from . import capi
        self._lib = capi.lib()
        self._p = self._lib.granite4_kv_pool_create(num_pages, tokens_per_page)
        if not self._p:
            raise ValueError("granite4_kv_pool_create failed")
        self.num_pages, self.tokens_per_page = num_pages, tokens_per_page

    def close(self):
        if getattr(self, "_p", None):
            self._lib.granite4_kv_pool_destroy(self._p)
            self._p = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _tok(tokens):
        a = np.ascontiguousarray(tokens, dtype=np.uint32)
        return a, a.ctypes.data, a.size

    def create_sequence(self) -> int:
        return self._lib.granite4_kv_pool_create_sequence(self._p)

    def match_prefix(self, seq: int, tokens) -> int:
        a, ptr, n = self._tok(tokens)
        return self._lib.granite4_kv_pool_match_prefix(self._p, seq, ptr, n)

    def reserve(self, seq: int, token_count: int, tokens) -> bool:
        a, ptr, n = self._tok(tokens)
        return bool(self._lib.granite4_kv_pool_reserve(self._p, seq, token_count, ptr, n))

    def mark_written(self, seq: int, page_index: int) -> bool:
        return bool(self._lib.granite4_kv_pool_mark_written(self._p, seq, page_index))

    def row_table(self, seq: int, n: int):
        """int32 [n] pool rows of positions [0, n), or None when n exceeds the sequence."""
        out = np.empty(max(n, 1), np.int32)
        ok = self._lib.granite4_kv_pool_row_table(self._p, seq, n, out.ctypes.data)
        return out[:n] if ok else None

    def reset_sequence(self, seq: int):
        self._lib.granite4_kv_pool_reset_sequence(self._p, seq)

    def truncate_sequence(self, seq: int, n_tokens: int):
        self._lib.granite4_kv_pool_truncate_sequence(self._p, seq, n_tokens)

    def release(self, seq: int):
        self._lib.granite4_kv_pool_release(self._p, seq)

    def clear(self):
        self._lib.granite4_kv_pool_clear(self._p)

    def count(self, name: str) -> int:
        return self._lib.granite4_kv_pool_count(self._p, self.COUNTS[name])

    def sequence_tokens(self, seq: int) -> int:
        return self._lib.granite4_kv_pool_sequence_tokens(self._p, seq)

    def block_table(self, seq: int):
        n = self._lib.granite4_kv_pool_block_table(self._p, seq, None, 0)
        out = np.empty(max(n, 1), np.int32)
        self._lib.granite4_kv_pool_block_table(self._p, seq, out.ctypes.data, n)
        return out[:n]

    def ref_count(self, page: int) -> int:
        return self._lib.granite4_kv_pool_ref_count(self._p, page)

    def page_in_cache(self, page: int) -> bool:
        return bool(self._lib.granite4_kv_pool_page_in_cache(self._p, page))

    def move_rows(self, seq: int, src_pos, dst_pos):
        """Pool rows (src, dst) of logical positions for granite4_kernel_kv_move, or None when
        the reference's checks refuse the move list."""
        n = len(src_pos)
        s = np.ascontiguousarray(src_pos, np.int32)
        d = np.ascontiguousarray(dst_pos, np.int32)
        so, do = np.empty(max(n, 1), np.int32), np.empty(max(n, 1), np.int32)
        rc = self._lib.granite4_kv_pool_move_rows(self._p, seq, s.ctypes.data, d.ctypes.data, n, so.ctypes.data,
                                                  do.ctypes.data)
        return (so[:n], do[:n]) if rc == 0 else None


class KvPoolController:
    """The library's serve-loop controller over the pool (``granite4_kv_ctl_*``): the reference's
    ``KvPoolController`` (``engine/src/kv_pool_controller.h:32-112``) behind the C ABI. Method
    names and meanings are the reference's."""

    def __init__(self, num_pages: int, tokens_per_page: int = TOKENS_PER_PAGE):
        from . import capi
        self._lib = capi.lib()
        self._p = self._lib.granite4_kv_ctl_create(num_pages, tokens_per_page)
        if not self._p:
            raise ValueError("granite4_kv_ctl_create failed")
        self.num_pages, self.tokens_per_page = num_pages, tokens_per_page

    def close(self):
        if getattr(self, "_p", None):
            self._lib.granite4_kv_ctl_destroy(self._p)
            self._p = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def new_slot(self) -> int:
        return self._lib.granite4_kv_ctl_new_slot(self._p)

    def release_slot(self, slot: int):
        self._lib.granite4_kv_ctl_release_slot(self._p, slot)

    def shutdown(self):
        self._lib.granite4_kv_ctl_shutdown(self._p)

    def prefill(self, slot: int, prompt):
        """(ok, pool sequence id, page-aligned tokens already cached)."""
        import ctypes as C
        a, ptr, n = KvPool._tok(prompt)
        seq, reused = C.c_int(-1), C.c_longlong(0)
        ok = self._lib.granite4_kv_ctl_prefill(self._p, slot, ptr, n, C.byref(seq), C.byref(reused))
        return bool(ok), seq.value, reused.value

    def commit(self, slot: int, all_tokens):
        a, ptr, n = KvPool._tok(all_tokens)
        self._lib.granite4_kv_ctl_commit(self._p, slot, ptr, n)

    def open_slot(self) -> int:
        return self._lib.granite4_kv_ctl_open_slot(self._p)

    def ensure(self, slot: int, n_tokens: int) -> bool:
        return bool(self._lib.granite4_kv_ctl_ensure(self._p, slot, n_tokens))

    def trim(self, slot: int, n_tokens: int):
        self._lib.granite4_kv_ctl_trim(self._p, slot, n_tokens)

    def drop(self, slot: int):
        self._lib.granite4_kv_ctl_drop(self._p, slot)

    def slot_pages(self, slot: int) -> int:
        return self._lib.granite4_kv_ctl_slot_pages(self._p, slot)

    def pages_missing(self, slot: int, n_tokens: int) -> int:
        return self._lib.granite4_kv_ctl_pages_missing(self._p, slot, n_tokens)

    def row_table(self, slot: int, n: int):
        out = np.empty(max(n, 1), np.int32)
        ok = self._lib.granite4_kv_ctl_row_table(self._p, slot, n, out.ctypes.data)
        return out[:n] if ok else None

    def committed(self, slot: int) -> int:
        return self._lib.granite4_kv_ctl_committed(self._p, slot)

    def last_reused(self, slot: int) -> int:
        return self._lib.granite4_kv_ctl_last_reused(self._p, slot)

    def max_slots(self) -> int:
        return self._lib.granite4_kv_ctl_max_slots(self._p)

    def count(self, name: str) -> int:
        return self._lib.granite4_kv_ctl_count(self._p, KvPool.COUNTS[name])
