"""The host-side paged KV pool (granite4_kv_pool_*): the reference's known answers
(engine/tests/test_kv_pool.cc, read as text) and, where oracle/_ref is built, a call-for-call
comparison with the reference's own PagedKV on random call sequences. CPU only."""
import ctypes as C
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libg4ref.so")


@pytest.fixture(scope="module")
def paging():
    import granite4_b200  # noqa: F401
    from granite4_b200 import _build, paging
    if _build.is_stale():
        _build.build()
    return paging


def toks(start, n):
    return list(range(start, start + n))


def test_alloc_locate_and_row_table_known_answers(paging):
    # engine/tests/test_kv_pool.cc:247-300 (4 pages of 4 tokens)
    pool = paging.KvPool(4, 4)
    a = pool.create_sequence()
    assert pool.reserve(a, 4, toks(0, 4))
    pool.release(a)
    b = pool.create_sequence()
    assert pool.reserve(b, 8, toks(10, 8))
    bt = pool.block_table(b)
    tbl = pool.row_table(b, 8)
    assert (tbl == [bt[p // 4] * 4 + p % 4 for p in range(8)]).all()
    assert tbl[0] + 1 == tbl[1] and tbl[4] == bt[1] * 4
    assert pool.row_table(b, 9) is None and pool.row_table(-1, 1) is None
    # a shared cached prefix page followed by private pages
    pool.clear()
    p0 = pool.create_sequence()
    pool.reserve(p0, 4, toks(50, 4))
    assert pool.mark_written(p0, 0)
    pool.release(p0)
    assert pool.count("retained_pages") == 1
    r = pool.create_sequence()
    assert pool.match_prefix(r, toks(50, 12)) == 4
    assert pool.reserve(r, 12, toks(50, 12))
    rt = pool.block_table(r)
    assert len(rt) == 3
    rtbl = pool.row_table(r, 12)
    assert rtbl[0] == rt[0] * 4 and rtbl[0] != rtbl[4]
    assert (rtbl[4:] == [rt[p // 4] * 4 + p % 4 for p in range(4, 12)]).all()
    pool.close()


def test_prefix_sharing_lru_eviction_and_bounds(paging):
    pool = paging.KvPool(4, 4)
    s1 = pool.create_sequence()
    assert pool.reserve(s1, 8, toks(0, 8))
    assert pool.mark_written(s1, 0) and pool.mark_written(s1, 1)
    s2 = pool.create_sequence()
    assert pool.match_prefix(s2, toks(0, 8) + [99]) == 8          # both pages shared
    assert pool.count("shared_pages") == 2 and pool.ref_count(int(pool.block_table(s1)[0])) == 2
    assert not pool.mark_written(s2, 0)                           # shared pages are published already
    pool.release(s1)
    pool.release(s2)
    assert pool.count("retained_pages") == 2 and pool.count("free_pages") == 2
    # a request for 3 pages must evict one retained page, the least recently used
    s3 = pool.create_sequence()
    assert pool.reserve(s3, 12, toks(100, 12))
    assert pool.count("evicted_pages") == 1 and pool.count("retained_pages") == 1
    # pages still referenced are never evicted: asking for more than is left fails
    s4 = pool.create_sequence()
    assert not pool.reserve(s4, 12, toks(200, 12))
    assert pool.reserve(s4, 4, toks(200, 4))
    # no more sequences than pages
    pool.clear()
    ids = [pool.create_sequence() for _ in range(5)]
    assert ids[:4] == [0, 1, 2, 3] and ids[4] == -1
    pool.close()


def test_move_rows_follow_the_block_table(paging):
    pool = paging.KvPool(8, 4)
    s = pool.create_sequence()
    assert pool.reserve(s, 10, toks(0, 10))
    rows = pool.row_table(s, 10)
    src, dst = pool.move_rows(s, [5, 7, 9], [4, 5, 6])
    assert (src == rows[[5, 7, 9]]).all() and (dst == rows[[4, 5, 6]]).all()
    assert pool.move_rows(s, [3], [4]) is None        # never moved to a later position
    assert pool.move_rows(s, [5, 4], [4, 3]) is None  # a later move would read an overwritten row
    assert pool.move_rows(s, [12], [2]) is None       # beyond the sequence's pages
    pool.close()


class RefPool:
    """The reference's PagedKV through oracle/_ref (same method names as paging.KvPool)."""

    def __init__(self, num_pages, tokens_per_page):
        self.lib = C.CDLL(REF_LIB)
        L = self.lib
        L.g4ref_pool_create.restype = C.c_void_p
        L.g4ref_pool_create.argtypes = [C.c_int, C.c_int]
        for name, res, args in (
                ("destroy", None, [C.c_void_p]), ("create_sequence", C.c_int, [C.c_void_p]),
                ("match_prefix", C.c_longlong, [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong]),
                ("reserve", C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_void_p, C.c_longlong]),
                ("mark_written", C.c_int, [C.c_void_p, C.c_int, C.c_longlong]),
                ("row_table", C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_void_p]),
                ("reset_sequence", None, [C.c_void_p, C.c_int]),
                ("truncate_sequence", None, [C.c_void_p, C.c_int, C.c_longlong]),
                ("release", None, [C.c_void_p, C.c_int]), ("clear", None, [C.c_void_p]),
                ("count", C.c_longlong, [C.c_void_p, C.c_int]),
                ("sequence_tokens", C.c_longlong, [C.c_void_p, C.c_int]),
                ("block_table", C.c_longlong, [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong]),
                ("ref_count", C.c_int, [C.c_void_p, C.c_int]), ("page_in_cache", C.c_int, [C.c_void_p, C.c_int])):
            fn = getattr(L, "g4ref_pool_" + name)
            fn.restype, fn.argtypes = res, args
        self.p = L.g4ref_pool_create(num_pages, tokens_per_page)

    def _tok(self, tokens):
        a = np.ascontiguousarray(tokens, dtype=np.uint32)
        return a, a.ctypes.data, a.size

    def create_sequence(self): return self.lib.g4ref_pool_create_sequence(self.p)
    def match_prefix(self, s, t):
        a, ptr, n = self._tok(t)
        return self.lib.g4ref_pool_match_prefix(self.p, s, ptr, n)
    def reserve(self, s, c, t):
        a, ptr, n = self._tok(t)
        return bool(self.lib.g4ref_pool_reserve(self.p, s, c, ptr, n))
    def mark_written(self, s, i): return bool(self.lib.g4ref_pool_mark_written(self.p, s, i))
    def row_table(self, s, n):
        out = np.empty(max(n, 1), np.int32)
        return out[:n] if self.lib.g4ref_pool_row_table(self.p, s, n, out.ctypes.data) else None
    def reset_sequence(self, s): self.lib.g4ref_pool_reset_sequence(self.p, s)
    def truncate_sequence(self, s, n): self.lib.g4ref_pool_truncate_sequence(self.p, s, n)
    def release(self, s): self.lib.g4ref_pool_release(self.p, s)
    def clear(self): self.lib.g4ref_pool_clear(self.p)
    def count(self, name): return self.lib.g4ref_pool_count(self.p, {"free_pages": 0, "used_pages": 1, "shared_pages": 2, "cached_pages": 3, "evicted_pages": 4, "retained_pages": 5, "live_sequences": 6}[name])
    def sequence_tokens(self, s): return self.lib.g4ref_pool_sequence_tokens(self.p, s)
    def block_table(self, s):
        n = self.lib.g4ref_pool_block_table(self.p, s, None, 0)
        out = np.empty(max(n, 1), np.int32)
        self.lib.g4ref_pool_block_table(self.p, s, out.ctypes.data, n)
        return out[:n]
    def ref_count(self, pg): return self.lib.g4ref_pool_ref_count(self.p, pg)
    def page_in_cache(self, pg): return bool(self.lib.g4ref_pool_page_in_cache(self.p, pg))
    def close(self): self.lib.g4ref_pool_destroy(self.p)


@pytest.mark.skipif(not os.path.isfile(REF_LIB), reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("seed", range(8))
def test_random_call_sequences_match_the_reference_pool(paging, seed):
    """Random serve-loop traffic against both pools: every return value, block table, row table
    and count agrees after every call. Requests share a few prompt stems, so prefix sharing,
    retention and least-recently-used eviction all happen (asserted at the end). Left out on
    purpose: a truncate that drops no page but shortens the sequence, where this pool corrects
    the reference's token record."""
    rng = np.random.default_rng(seed)
    P, B = int(rng.integers(8, 20)), int(rng.choice([2, 4, 16]))
    mine, ref = paging.KvPool(P, B), RefPool(P, B)
    stems = [rng.integers(0, 50, 5 * B).tolist() for _ in range(3)]
    seqs, prompt = [], {}
    seen = {"matched": 0, "evicted": 0, "shared": 0, "retained": 0, "reserve_failed": 0}

    def both(name, *args):
        a, b = getattr(mine, name)(*args), getattr(ref, name)(*args)
        if isinstance(a, np.ndarray) or isinstance(b, np.ndarray):
            assert (a is None) == (b is None) and (a is None or (a == b).all()), (name, args)
        else:
            assert a == b, (name, args, a, b)
        return a

    def check(step):
        for name in paging.KvPool.COUNTS:
            both("count", name)
        for q in seqs:
            n = both("sequence_tokens", q)
            both("block_table", q)
            both("row_table", q, n)
        for pg in range(P):
            both("ref_count", pg)
            both("page_in_cache", pg)
        seen["evicted"] = max(seen["evicted"], mine.count("evicted_pages"))
        seen["shared"] = max(seen["shared"], mine.count("shared_pages"))
        seen["retained"] = max(seen["retained"], mine.count("retained_pages"))

    for step in range(1500):
        op = int(rng.integers(0, 12))
        if op == 0 or not seqs:
            if len(seqs) < 5:
                a = both("create_sequence")
                if a >= 0:
                    seqs.append(a)
        elif op <= 4:  # a new request on a slot: drop what it held, adopt a cached prefix, reserve the rest
            s = int(rng.choice(seqs))
            both("reset_sequence", s)
            stem = stems[int(rng.integers(0, 3))]
            cut = int(rng.integers(0, len(stem) // B + 1)) * B if rng.random() < 0.8 else int(rng.integers(0, len(stem)))
            prompt[s] = stem[:cut] + rng.integers(0, 50, int(rng.integers(1, 2 * B))).tolist()
            seen["matched"] += both("match_prefix", s, prompt[s]) > 0
            if not both("reserve", s, len(prompt[s]), prompt[s]):
                seen["reserve_failed"] += 1
            for i in range(len(prompt[s]) // B):
                if rng.random() < 0.8:
                    both("mark_written", s, i)
        elif op <= 7:  # decode: the sequence grows by a few tokens
            s = int(rng.choice(seqs))
            prompt[s] = prompt.get(s, [])[:mine.sequence_tokens(s)] + rng.integers(0, 50, int(rng.integers(1, 4))).tolist()
            if not both("reserve", s, len(prompt[s]), prompt[s]):
                seen["reserve_failed"] += 1
            if rng.random() < 0.5:
                both("mark_written", s, int(rng.integers(0, 8)))
        elif op == 8:  # hand pages back
            s = int(rng.choice(seqs))
            filled, pages = mine.sequence_tokens(s), len(mine.block_table(s))
            n = int(rng.integers(0, filled + 2))
            if (n + B - 1) // B >= pages and n < filled:
                n = filled  # the one documented difference: not exercised
            mine.truncate_sequence(s, n)
            ref.truncate_sequence(s, n)
        elif op == 9:  # calls on ids that do not exist or are dead
            s = int(rng.integers(-2, len(seqs) + 3))
            both("match_prefix", s, stems[0])
            both("mark_written", s, 0)
            both("row_table", s, 1)
        elif op == 10 and rng.random() < 0.3:
            s = int(rng.choice(seqs))
            mine.release(s)
            ref.release(s)
            seqs.remove(s)
        elif op == 11 and rng.random() < 0.02:
            mine.clear()
            ref.clear()
            seqs, prompt = [], {}
        check(step)
    assert seen["matched"] > 20 and seen["evicted"] > 5 and seen["shared"] > 0 and seen["retained"] > 0, seen
    mine.close()
    ref.close()
