"""The reference's split-KV attention contract (granite4::attn_split, engine/src/attention_gpu.h:15-68)
over the int8 paged pool, through granite4_attn_split_int8: consecutive rows of one sequence (host
or device base position), rows that are sequences of their own, caller-described row groups,
draft-tree rows that see their ancestors' slots, and the sliding window.

The oracle evaluates each row on its own: which pool rows a row may see is written out on the host
as an explicit per-row table (tree tails and window offsets folded in), and the golden bf16 pipeline
(engine/src/kernel_math.h:265-331, pinned bit for bit to the reference through oracle/_ref) runs over
it - the reference's own statement of the contract: "each row's arithmetic is that of a single-row
call at its position". Tolerance: 0.03 absolute against that pipeline, the reference's bar for this
kernel (engine/tests/test_kernels.cu:2055, :2282), and 0.01 against an unrounded float64 evaluation.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
Hq, Hk, D = 32, 8, 128
ATT_TOL = 0.03
SCALE = 1.0 / 128


@pytest.fixture(scope="module")
def K():
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi, kernels
    capi.lib()
    yield kernels
    assert capi.lib().device_status() == 0


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def f32_of(bits):
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def pool(seed, stride):
    rng = np.random.default_rng(seed)
    ck = rng.integers(-127, 128, (Hk, stride, D), dtype=np.int8)
    cv = rng.integers(-127, 128, (Hk, stride, D), dtype=np.int8)
    ks = (rng.random((Hk, stride), dtype=np.float32) * 0.02 + 0.005).astype(np.float32)
    vs = (rng.random((Hk, stride), dtype=np.float32) * 0.02 + 0.005).astype(np.float32)
    return ck, cv, ks, vs


def f64_rows(q, ck, cv, ks, vs, seen):
    """Unrounded evaluation: row r attends to the pool rows seen[r], in that order."""
    rows = q.shape[0]
    qf = f32_of(q).astype(np.float64).reshape(rows, Hq, D)
    out = np.zeros((rows, Hq, D))
    for r in range(rows):
        sel = np.asarray(seen[r])
        for h in range(Hq):
            k = ck[h // 4, sel].astype(np.float64) * ks[h // 4, sel, None]
            v = cv[h // 4, sel].astype(np.float64) * vs[h // 4, sel, None]
            lg = SCALE * (k @ qf[r, h])
            p = np.exp(lg - lg.max())
            out[r, h] = (p / p.sum()) @ v
    return out


def check(port, got_bits, q, pl, seen):
    """seen[r]: the pool rows row r attends to, oldest first."""
    ck, cv, ks, vs = pl
    rows = q.shape[0]
    tables = [np.asarray(s, np.int32) for s in seen]
    pos = np.array([len(s) - 1 for s in seen], np.int32)
    want = f32_of(port.attn_decode_int8(q, ck, cv, ks, vs, pos, tables, Hq, Hk, D, SCALE)).reshape(rows, Hq, D)
    got = f32_of(got_bits).reshape(rows, Hq, D)
    exact = f64_rows(q, ck, cv, ks, vs, seen)
    assert np.abs(got - want).max() < ATT_TOL
    assert np.abs(got - exact).max() < 0.01


def out_bits(t):
    return t.cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("rows,base,max_len", [(1, 0, 64), (1, 777, 1024), (4, 1000, 1024), (3, 61, 4096),
                                               (16, 4000, 4096), (7, 0, 4096)])
@pytest.mark.parametrize("paged", [False, True])
def test_consecutive_rows_of_one_sequence(K, port, rows, base, max_len, paged):
    """d_row_pos NULL: rows at base, base + 1, ...; base by value and read from the device; with and
    without a page table; a pool far larger than the sequence (max_len < stride)."""
    stride = 8192
    pl = pool(1, stride)
    rng = np.random.default_rng(rows * 100 + base)
    table = rng.permutation(stride).astype(np.int32) if paged else None
    q = bf16_bits(2.0 * rng.standard_normal((rows, Hq * D)))
    seen = [(table if paged else np.arange(stride))[: base + r + 1] for r in range(rows)]
    for by_device in (False, True):
        out = torch.empty(rows, Hq * D, dtype=torch.int16, device=DEV)
        d_pos = dev(np.array([base], np.int32)) if by_device else None
        assert K.attn_split_int8(dev(q), *[dev(x) for x in pl], SCALE, Hq, Hk, D, stride, out,
                                 kv_base=-5 if by_device else base, d_pos=d_pos,
                                 pt=None if table is None else dev(table), max_len=max_len) == 0
        check(port, out_bits(out), q, pl, seen)


def test_rows_as_sequences_and_caller_described_groups(K, port):
    """Nine rows: a verify group of three rows of session A, one decode row of session B, a group of
    four of session C, one row of session D - once ungrouped (every row its own block), once with
    group words r0 | nr << 8. Same results either way."""
    stride, max_len = 4096, 4096
    pl = pool(2, stride)
    rng = np.random.default_rng(9)
    sess = [rng.permutation(stride).astype(np.int32) for _ in range(4)]
    layout = [(0, 3, 500), (1, 1, 4095), (2, 4, 63), (3, 1, 0)]  # (session, rows, first position)
    row_sess, pos = [], []
    for s, n, p0 in layout:
        row_sess += [s] * n
        pos += list(range(p0, p0 + n))
    rows = len(pos)
    q = bf16_bits(2.0 * rng.standard_normal((rows, Hq * D)))
    d_tables = [dev(t) for t in sess]
    row_pt = torch.tensor([d_tables[s].data_ptr() for s in row_sess], dtype=torch.int64, device=DEV)
    seen = [sess[s][: p + 1] for s, p in zip(row_sess, pos)]
    words, r0 = [], 0
    for _, n, _ in layout:
        words.append(r0 | (n << 8))
        r0 += n
    outs = []
    for grp in (None, np.array(words, np.int32)):
        out = torch.empty(rows, Hq * D, dtype=torch.int16, device=DEV)
        assert K.attn_split_int8(dev(q), *[dev(x) for x in pl], SCALE, Hq, Hk, D, stride, out, max_len=max_len,
                                 row_pos=dev(np.array(pos, np.int32)), row_pt=row_pt,
                                 row_grp=None if grp is None else dev(grp)) == 0
        check(port, out_bits(out), q, pl, seen)
        outs.append(out_bits(out))
    # grouping changes which block reads a tile, not the arithmetic of a row's own tiles
    assert np.abs(f32_of(outs[0]) - f32_of(outs[1])).max() < 0.01


@pytest.mark.parametrize("tbase", [0, 15, 16, 1000, 2047])
@pytest.mark.parametrize("grouped", [False, True])
def test_draft_tree_rows_see_their_ancestors(K, port, tbase, grouped):
    """One session with tbase + 1 committed positions and a draft tree of 11 nodes stored at slots
    tbase + 1 + node. A node at depth k sits at position tbase + k and attends to the committed
    positions plus the slots of its ancestors and itself (row_tail), not to its siblings. Grouped:
    group words of up to four rows sharing tbase; otherwise one row per block."""
    stride, max_len = 4096, 2048 + 16
    pl = pool(3, stride)
    rng = np.random.default_rng(tbase + 7)
    table = rng.permutation(stride).astype(np.int32)
    parent = [-1, 0, 0, 1, 1, 2, 3, 3, 6, 8, 9]  # node 10 is at depth 7
    rows = len(parent)
    tails, pos = np.zeros((rows, 8), np.int32), []
    for n in range(rows):
        chain, a = [], n
        while a >= 0:
            chain.append(tbase + 1 + a)
            a = parent[a]
        chain.reverse()  # root first, the node itself last
        tails[n, : len(chain)] = chain
        pos.append(tbase + len(chain))
    q = bf16_bits(2.0 * rng.standard_normal((rows, Hq * D)))
    seen = [np.concatenate([table[: tbase + 1], table[tails[n, : pos[n] - tbase]]]) for n in range(rows)]
    d_table = dev(table)
    row_pt = torch.full((rows,), d_table.data_ptr(), dtype=torch.int64, device=DEV)
    grp = dev(np.array([0 | (4 << 8), 4 | (4 << 8), 8 | (3 << 8)], np.int32)) if grouped else None
    out = torch.empty(rows, Hq * D, dtype=torch.int16, device=DEV)
    assert K.attn_split_int8(dev(q), *[dev(x) for x in pl], SCALE, Hq, Hk, D, stride, out, max_len=max_len,
                             row_pos=dev(np.array(pos, np.int32)), row_pt=row_pt, row_grp=grp,
                             row_tbase=dev(np.full(rows, tbase, np.int32)), row_tail=dev(tails)) == 0
    check(port, out_bits(out), q, pl, seen)


@pytest.mark.parametrize("window", [1, 17, 64, 300, 5000])
def test_sliding_window(K, port, window):
    """window > 0: a row attends to (pos - window, pos]. Decode rows at several positions through
    their own tables, and a verify group of four consecutive rows; contexts long enough that whole
    splits lie below the window."""
    stride, max_len = 8192, 8192
    pl = pool(4, stride)
    rng = np.random.default_rng(window)
    pos = np.array([0, 5, 16, 299, 300, 4000, 8191], np.int32)
    rows = len(pos)
    tables = [rng.permutation(stride).astype(np.int32) for _ in range(rows)]
    d_tables = [dev(t) for t in tables]
    row_pt = torch.tensor([t.data_ptr() for t in d_tables], dtype=torch.int64, device=DEV)
    q = bf16_bits(2.0 * rng.standard_normal((rows, Hq * D)))
    seen = [tables[r][max(0, pos[r] + 1 - window): pos[r] + 1] for r in range(rows)]
    out = torch.empty(rows, Hq * D, dtype=torch.int16, device=DEV)
    assert K.attn_split_int8(dev(q), *[dev(x) for x in pl], SCALE, Hq, Hk, D, stride, out, max_len=max_len,
                             row_pos=dev(pos), row_pt=row_pt, window=window) == 0
    check(port, out_bits(out), q, pl, seen)
    # four consecutive rows of one sequence (device base position)
    base = 5000
    q4 = bf16_bits(2.0 * rng.standard_normal((4, Hq * D)))
    seen4 = [tables[0][max(0, base + r + 1 - window): base + r + 1] for r in range(4)]
    out4 = torch.empty(4, Hq * D, dtype=torch.int16, device=DEV)
    assert K.attn_split_int8(dev(q4), *[dev(x) for x in pl], SCALE, Hq, Hk, D, stride, out4, d_pos=dev(np.array([base], np.int32)),
                             pt=d_tables[0], max_len=max_len, window=window) == 0
    check(port, out_bits(out4), q4, pl, seen4)


def test_window_on_tree_rows(K, port):
    """Both at once: the window counts logical positions, ancestors' slots included."""
    stride, max_len, tbase, window = 2048, 1024, 500, 40
    pl = pool(5, stride)
    rng = np.random.default_rng(11)
    table = rng.permutation(stride).astype(np.int32)
    tails = np.zeros((3, 8), np.int32)
    tails[0, :1] = [tbase + 1]
    tails[1, :2] = [tbase + 1, tbase + 2]
    tails[2, :3] = [tbase + 1, tbase + 2, tbase + 3]
    pos = np.array([tbase + 1, tbase + 2, tbase + 3], np.int32)
    q = bf16_bits(2.0 * rng.standard_normal((3, Hq * D)))
    seen = []
    for n in range(3):
        logical = np.concatenate([table[: tbase + 1], table[tails[n, : pos[n] - tbase]]])
        seen.append(logical[max(0, pos[n] + 1 - window):])
    d_table = dev(table)
    row_pt = torch.full((3,), d_table.data_ptr(), dtype=torch.int64, device=DEV)
    out = torch.empty(3, Hq * D, dtype=torch.int16, device=DEV)
    assert K.attn_split_int8(dev(q), *[dev(x) for x in pl], SCALE, Hq, Hk, D, stride, out, max_len=max_len,
                             row_pos=dev(pos), row_pt=row_pt, row_grp=dev(np.array([0 | (3 << 8)], np.int32)),
                             row_tbase=dev(np.full(3, tbase, np.int32)), row_tail=dev(tails), window=window) == 0
    check(port, out_bits(out), q, pl, seen)


def test_argument_rules(K):
    """engine/src/attention_split.cu:1096-1105: what the reference refuses, this refuses."""
    stride = 256
    pl = [dev(x) for x in pool(6, stride)]
    q = torch.zeros(2, Hq * D, dtype=torch.int16, device=DEV)
    out = torch.empty_like(q)
    pos = dev(np.array([3, 4], np.int32))
    tbl = dev(np.arange(stride, dtype=np.int32))
    row_pt = torch.full((2,), tbl.data_ptr(), dtype=torch.int64, device=DEV)
    ok = dict(max_len=stride)
    assert K.attn_split_int8(q, *pl, SCALE, Hq, Hk, D, stride, out, kv_base=3, **ok) == 0
    assert K.attn_split_int8(q, *pl, SCALE, Hq, Hk, D, stride, out, kv_base=255, **ok) == -1  # base + rows > max_len
    assert K.attn_split_int8(q, *pl, SCALE, Hq, Hk, D, stride, out, row_pos=pos, **ok) == -1  # row_pos without row_pt
    assert K.attn_split_int8(q, *pl, SCALE, Hq, Hk, D, stride, out, row_pos=pos, row_pt=row_pt,
                             row_tbase=pos, **ok) == -1  # tbase without tail
    assert K.attn_split_int8(q, *pl, SCALE, Hq, Hk, D, stride, out, kv_base=3, window=-1, **ok) == -1
    assert K.attn_split_int8(q, *pl, SCALE, Hq, Hk, D, stride, out, kv_base=3, max_len=stride + 1) == -1
    assert K.attn_split_int8(q, *pl, SCALE, 16, Hk, D, stride, out, kv_base=3, **ok) == -1  # Hq != 4 Hk
    torch.cuda.synchronize()
