"""The serve-loop controller over the paged KV pool (granite4_kv_ctl_*): the reference's known
answers (engine/tests/test_kv_pool_controller.cc, read as text: a pool of 4 pages of 4 tokens) and,
where oracle/_ref is built, a call-for-call comparison with the reference's own KvPoolController
under random serve-loop traffic. CPU only."""
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


def prompt(base, n):
    return list(range(base, base + n))


def rows_valid(rows, pages, B):
    """engine/tests/test_kv_pool_controller.cc:49-67: in range, distinct, slot within the page kept."""
    rows = np.asarray(rows)
    return (rows >= 0).all() and (rows < pages * B).all() and len(set(rows.tolist())) == len(rows) and \
        (rows % B == np.arange(len(rows)) % B).all()


def test_slot_capacity_and_recycling(paging):
    c = paging.KvPoolController(4, 4)
    assert c.max_slots() == 4
    assert [c.new_slot() for _ in range(5)] == [0, 1, 2, 3, -1]
    c.release_slot(0)
    assert c.new_slot() == 0
    c.close()


def test_prefill_rows_and_prefix_reuse(paging):
    c = paging.KvPoolController(4, 4)
    a = c.new_slot()
    ok, seq, reused = c.prefill(a, prompt(100, 10))
    assert ok and seq >= 0 and reused == 0 and c.committed(a) == 10 and c.count("free_pages") == 1
    assert rows_valid(c.row_table(a, 10), 4, 4)
    c.close()
    # concurrent: the second session holds the same pages
    c = paging.KvPoolController(4, 4)
    a, b = c.new_slot(), c.new_slot()
    assert c.prefill(a, prompt(100, 16))[::2] == (True, 0)
    assert c.prefill(b, prompt(100, 16))[::2] == (True, 16)
    assert c.committed(b) == 16 and c.count("shared_pages") == 4 and c.count("used_pages") == 4
    assert c.count("free_pages") == 0
    c.close()
    # sequential: pages of a finished session are retained and come back
    c = paging.KvPoolController(4, 4)
    a = c.new_slot()
    assert c.prefill(a, prompt(100, 16))[0]
    c.release_slot(a)
    assert c.count("retained_pages") == 4
    b = c.new_slot()
    assert c.prefill(b, prompt(100, 16))[::2] == (True, 16) and c.count("retained_pages") == 0
    c.close()
    # partial: three shared pages, a private tail
    c = paging.KvPoolController(4, 4)
    a, b = c.new_slot(), c.new_slot()
    c.prefill(a, prompt(100, 12))
    assert c.prefill(b, prompt(100, 12) + [999, 998])[::2] == (True, 12)
    assert c.committed(b) == 14 and c.count("free_pages") == 0
    ra, rb = c.row_table(a, 12), c.row_table(b, 14)
    assert (ra == rb[:12]).all() and len(set(rb.tolist())) == 14  # shared prefix -> the same pool rows
    c.close()


def test_commit_growth_failure_eviction_release_shutdown(paging):
    c = paging.KvPoolController(4, 4)
    a = c.new_slot()
    c.prefill(a, prompt(100, 6))
    assert c.committed(a) == 6 and c.count("cached_pages") == 1
    before = c.row_table(a, 6)
    c.commit(a, prompt(100, 6) + [900, 901])
    assert c.committed(a) == 8 and c.count("cached_pages") == 2
    after = c.row_table(a, 8)
    assert rows_valid(after, 4, 4) and (after[:6] == before).all()  # rows never move under growth
    c.commit(a, prompt(100, 6) + [900, 901])  # nothing new: no effect
    assert c.committed(a) == 8 and c.count("free_pages") == 2
    c.close()
    c = paging.KvPoolController(4, 4)
    a = c.new_slot()
    assert c.prefill(a, prompt(100, 20)) == (False, -1, 0)  # 20 > 16: refused, nothing held
    assert c.committed(a) == 0 and c.count("free_pages") == 4
    c.close()
    c = paging.KvPoolController(4, 4)
    a = c.new_slot()
    c.prefill(a, prompt(100, 16))
    c.release_slot(a)
    b = c.new_slot()
    assert c.prefill(b, prompt(500, 16))[::2] == (True, 0)
    assert c.count("evicted_pages") == 4 and c.count("used_pages") == 4
    c.close()
    c = paging.KvPoolController(4, 4)
    a = c.new_slot()
    c.prefill(a, prompt(100, 8))
    c.release_slot(a)
    assert c.committed(a) == 0 and c.count("retained_pages") == 2
    assert c.prefill(a, prompt(100, 8))[::2] == (True, 8) and c.committed(a) == 8
    c.shutdown()
    assert c.count("free_pages") == 4 and c.committed(a) == 0 and c.count("cached_pages") == 0
    c.close()


def test_resident_sessions(paging):
    c = paging.KvPoolController(4, 4)
    a, b = c.open_slot(), c.open_slot()
    assert a >= 0 and b >= 0 and a != b
    assert c.ensure(a, 8) and c.ensure(b, 8) and c.count("free_pages") == 0
    ra, rb = c.row_table(a, 8), c.row_table(b, 8)
    assert len(set(ra.tolist()) | set(rb.tolist())) == 16
    assert not c.ensure(a, 12) and c.committed(a) == 8 and (c.row_table(a, 8) == ra).all()
    c.trim(b, 4)
    assert c.count("free_pages") == 1 and c.ensure(a, 12)
    ra3 = c.row_table(a, 12)
    assert (ra3[:8] == ra).all() and rows_valid(ra3, 4, 4) and (c.row_table(b, 4) == rb[:4]).all()
    c.close()
    c = paging.KvPoolController(4, 4)
    a = c.open_slot()
    assert c.pages_missing(a, 10) == 3 and c.ensure(a, 10) and c.slot_pages(a) == 3
    assert c.pages_missing(a, 12) == 0 and c.pages_missing(a, 13) == 1
    c.trim(a, 5)
    assert c.slot_pages(a) == 2 and c.committed(a) == 5 and c.ensure(a, 9)
    c.drop(a)
    assert c.slot_pages(a) == 0 and c.count("free_pages") == 4 and c.count("cached_pages") == 0
    c.close()


class RefController:
    """The reference's KvPoolController through oracle/_ref, with paging.KvPoolController's methods."""

    def __init__(self, pages, B):
        self.lib = lib = C.CDLL(REF_LIB)
        vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
        for name, res, args in (
                ("create", vp, [i, i]), ("destroy", None, [vp]), ("shutdown", None, [vp]), ("new_slot", i, [vp]),
                ("release_slot", None, [vp, i]), ("prefill", i, [vp, i, vp, ll, C.POINTER(i), C.POINTER(ll)]),
                ("commit", None, [vp, i, vp, ll]), ("open_slot", i, [vp]), ("ensure", i, [vp, i, ll]),
                ("trim", None, [vp, i, ll]), ("drop", None, [vp, i]), ("slot_pages", ll, [vp, i]),
                ("pages_missing", ll, [vp, i, ll]), ("row_table", i, [vp, i, ll, vp]), ("committed", ll, [vp, i]),
                ("last_reused", ll, [vp, i]), ("max_slots", ll, [vp]), ("count", ll, [vp, i])):
            fn = getattr(lib, "g4ref_ctl_" + name)
            fn.restype, fn.argtypes = res, args
        self.p = lib.g4ref_ctl_create(pages, B)

    @staticmethod
    def _tok(tokens):
        a = np.ascontiguousarray(tokens, dtype=np.uint32)
        return a, a.ctypes.data, a.size

    def new_slot(self): return self.lib.g4ref_ctl_new_slot(self.p)
    def release_slot(self, s): self.lib.g4ref_ctl_release_slot(self.p, s)
    def shutdown(self): self.lib.g4ref_ctl_shutdown(self.p)

    def prefill(self, s, tokens):
        a, ptr, n = self._tok(tokens)
        seq, reused = C.c_int(-1), C.c_longlong(0)
        ok = self.lib.g4ref_ctl_prefill(self.p, s, ptr, n, C.byref(seq), C.byref(reused))
        return bool(ok), seq.value, reused.value

    def commit(self, s, tokens):
        a, ptr, n = self._tok(tokens)
        self.lib.g4ref_ctl_commit(self.p, s, ptr, n)

    def open_slot(self): return self.lib.g4ref_ctl_open_slot(self.p)
    def ensure(self, s, n): return bool(self.lib.g4ref_ctl_ensure(self.p, s, n))
    def trim(self, s, n): self.lib.g4ref_ctl_trim(self.p, s, n)
    def drop(self, s): self.lib.g4ref_ctl_drop(self.p, s)
    def slot_pages(self, s): return self.lib.g4ref_ctl_slot_pages(self.p, s)
    def pages_missing(self, s, n): return self.lib.g4ref_ctl_pages_missing(self.p, s, n)

    def row_table(self, s, n):
        out = np.empty(max(n, 1), np.int32)
        return out[:n] if self.lib.g4ref_ctl_row_table(self.p, s, n, out.ctypes.data) else None

    def committed(self, s): return self.lib.g4ref_ctl_committed(self.p, s)
    def last_reused(self, s): return self.lib.g4ref_ctl_last_reused(self.p, s)
    def max_slots(self): return self.lib.g4ref_ctl_max_slots(self.p)

    def count(self, name):
        return self.lib.g4ref_ctl_count(self.p, {"free_pages": 0, "used_pages": 1, "shared_pages": 2,
                                                  "cached_pages": 3, "evicted_pages": 4, "retained_pages": 5}[name])

    def close(self): self.lib.g4ref_ctl_destroy(self.p)


@pytest.mark.skipif(not os.path.isfile(REF_LIB), reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("seed", range(8))
def test_random_serve_loop_traffic_matches_the_reference_controller(paging, seed):
    """Requests that share a few prompt stems arrive on a handful of slots, generate tokens, finish;
    resident sessions grow, shrink and drop beside them; calls on dead and out-of-range slots are
    mixed in. After every call both controllers agree on every return value, every slot's row table,
    page count and token count, and every pool count. Left out on purpose: a trim that drops no page
    but shortens the token count (the pool beneath records the kept page's ids differently there)."""
    rng = np.random.default_rng(100 + seed)
    P, B = int(rng.integers(8, 24)), int(rng.choice([2, 4, 16]))
    mine, ref = paging.KvPoolController(P, B), RefController(P, B)
    stems = [rng.integers(0, 50, 6 * B).tolist() for _ in range(3)]
    slots, tokens, resident = [], {}, set()
    seen = {"reused": 0, "evicted": 0, "shared": 0, "refused": 0, "recycled": 0, "grow_refused": 0}
    counts = ("free_pages", "used_pages", "shared_pages", "cached_pages", "evicted_pages", "retained_pages")

    def both(name, *args):
        a, b = getattr(mine, name)(*args), getattr(ref, name)(*args)
        if isinstance(a, np.ndarray) or isinstance(b, np.ndarray):
            assert (a is None) == (b is None) and (a is None or (a == b).all()), (name, args)
        else:
            assert a == b, (name, args, a, b)
        return a

    def check():
        for name in counts:
            both("count", name)
        for s in range(-1, len(slots) + 2):
            n = both("committed", s)
            both("slot_pages", s)
            both("last_reused", s)
            both("row_table", s, n)
            both("pages_missing", s, n + B + 1)
        seen["evicted"] = max(seen["evicted"], mine.count("evicted_pages"))
        seen["shared"] = max(seen["shared"], mine.count("shared_pages"))

    for step in range(1200):
        op = int(rng.integers(0, 14))
        if op == 0 or not slots:
            s = both("open_slot") if rng.random() < 0.3 else both("new_slot")
            if s >= 0 and s not in slots:
                slots.append(s)
            elif s >= 0:
                seen["recycled"] += 1
        elif op <= 4:  # a new request on a slot
            s = int(rng.choice(slots))
            stem = stems[int(rng.integers(0, 3))]
            cut = int(rng.integers(0, len(stem) // B + 1)) * B if rng.random() < 0.8 else int(rng.integers(0, len(stem)))
            tokens[s] = stem[:cut] + rng.integers(0, 50, int(rng.integers(1, 3 * B))).tolist()
            ok, _, reused = both("prefill", s, tokens[s])
            seen["reused"] += reused > 0
            seen["refused"] += not ok
            resident.discard(s)
        elif op <= 7:  # generated tokens
            s = int(rng.choice(slots))
            tokens[s] = tokens.get(s, [])[:mine.committed(s)] + rng.integers(0, 50, int(rng.integers(1, 4))).tolist()
            both("commit", s, tokens[s])
        elif op == 8:  # a resident session grows
            s = int(rng.choice(slots))
            if not both("ensure", s, int(rng.integers(0, 5 * B))):
                seen["grow_refused"] += 1
        elif op == 9:  # ... and hands pages back
            s = int(rng.choice(slots))
            filled, pages = mine.committed(s), mine.slot_pages(s)
            n = int(rng.integers(0, filled + 2))
            if (n + B - 1) // B >= pages and n < filled:
                n = filled
            both("trim", s, n)
        elif op == 10:
            both("drop", int(rng.choice(slots)))
        elif op == 11:
            both("release_slot", int(rng.choice(slots)))
        elif op == 12:  # slots that do not exist
            s = int(rng.integers(-2, len(slots) + 3))
            if s < 0 or s >= len(slots):
                both("prefill", s, stems[0])
                both("commit", s, stems[0])
                both("ensure", s, 3)
                both("trim", s, 0)
                both("drop", s)
                both("release_slot", s)
        elif op == 13 and rng.random() < 0.02:
            both("shutdown")
            slots, tokens = [], {}
        check()
    assert seen["reused"] > 20 and seen["evicted"] > 5 and seen["shared"] > 0 and seen["refused"] > 0, seen
    assert seen["recycled"] > 0 and seen["grow_refused"] > 0, seen
    mine.close()
    ref.close()
