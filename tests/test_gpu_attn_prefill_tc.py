"""The tcgen05 form of the prefill attention (chunks of 64 rows or more through
granite4_prefill_attention_int8) against the oracle and against the mma.sync form.

Oracle: the reference's golden bf16 pipeline (engine/src/kernel_math.h:265-331) over the int8
pool, one row at a time. Tolerances as for every attention kernel here: 0.03 absolute against that
pipeline (engine/tests/test_kernels.cu:2055), 0.01 against an unrounded float64 evaluation.
Random pools with random per-row scales, permuted page tables, chunks that start at position 0 and
chunks that continue a prefix, row counts that are and are not multiples of the 64-row CTA tile.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
Hq, Hk, D = 32, 8, 128
SCALE = 1.0 / 128
ATT_TOL = 0.03


@pytest.fixture(scope="module")
def K():
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi, kernels
    capi.lib()
    yield kernels
    assert capi.lib().device_status() == 0, "a bounded wait ran out in a kernel"


def bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def f32_of(bits):
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def dev(a):
    a = np.ascontiguousarray(a)
    return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(DEV)


def pool(seed, stride):
    rng = np.random.default_rng(seed)
    ck = rng.integers(-127, 128, (Hk, stride, D), dtype=np.int8)
    cv = rng.integers(-127, 128, (Hk, stride, D), dtype=np.int8)
    ks = (rng.random((Hk, stride), dtype=np.float32) * 0.02 + 0.005).astype(np.float32)
    vs = (rng.random((Hk, stride), dtype=np.float32) * 0.02 + 0.005).astype(np.float32)
    return ck, cv, ks, vs


def f64_rows(q, pl, tables, pos):
    ck, cv, ks, vs = pl
    rows = q.shape[0]
    qf = f32_of(q).astype(np.float64).reshape(rows, Hq, D)
    out = np.zeros((rows, Hq, D))
    for r in range(rows):
        sel = tables[r][: pos[r] + 1]
        for h in range(Hq):
            k = ck[h // 4, sel].astype(np.float64) * ks[h // 4, sel, None]
            v = cv[h // 4, sel].astype(np.float64) * vs[h // 4, sel, None]
            lg = SCALE * (k @ qf[r, h])
            p = np.exp(lg - lg.max())
            out[r, h] = (p / p.sum()) @ v
    return out


def close(a, b, tol):
    """Within tol absolute plus one bf16 step of the value (the output is bf16)."""
    return bool((np.abs(a - b) <= tol + 2.0 ** -7 * np.abs(b)).all())


def run(K, q, pl, base, stride, table):
    out = torch.empty(q.shape[0], Hq * D, dtype=torch.int16, device=DEV)
    assert K.prefill_attention_int8(dev(q), SCALE, Hq, Hk, D, base, stride, out, *[dev(x) for x in pl],
                                    pt=None if table is None else dev(table)) == 0
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("rows,base,paged,sigma", [(64, 0, False, 1.0), (64, 0, True, 2.0), (100, 37, True, 2.0),
                                                   (257, 0, True, 1.0), (320, 1000, True, 3.0), (1000, 24, False, 2.0)])
def test_tensor_core_form_against_the_oracle_and_the_mma_sync_form(K, port, monkeypatch, rows, base, paged, sigma):
    stride = 2048
    pl = pool(rows + base, stride)
    rng = np.random.default_rng(rows * 7 + base)
    table = rng.permutation(stride).astype(np.int32) if paged else None
    q = bf16_bits(sigma * rng.standard_normal((rows, Hq * D)))
    monkeypatch.setenv("G4_PREFILL_TC", "1")
    got = run(K, q, pl, base, stride, table)
    monkeypatch.setenv("G4_PREFILL_TC", "0")
    other = run(K, q, pl, base, stride, table)
    # every row: the two forms agree to a bf16 step of the output (both round p to f16; they differ in
    # summation order)
    assert close(f32_of(got), f32_of(other), 0.01)
    # sampled rows against the oracle and the float64 evaluation (first and last rows of CTA tiles included)
    sel = np.unique(np.r_[0:4, 30:34, 62:66, rows // 2, rows - 3:rows]).astype(int)
    sel = sel[sel < rows]
    pos = (base + sel).astype(np.int32)
    tbl = table if table is not None else np.arange(stride, dtype=np.int32)
    want = f32_of(port.attn_decode_int8(q[sel], *pl, pos, [tbl] * len(sel), Hq, Hk, D, SCALE))
    assert np.abs(f32_of(got[sel]) - want).max() < ATT_TOL
    exact = f64_rows(q[sel], pl, [tbl] * len(sel), pos)
    assert close(f32_of(got[sel]).reshape(len(sel), Hq, D), exact, 0.01)


def test_peaked_softmax_rescales_the_accumulator(K, monkeypatch):
    """Queries of magnitude ~60: logits spread over some +-25 binary orders, so that along a prefix
    the running maximum jumps by more than 2^12 several times: the accumulator is then rescaled in
    tensor memory; a few keys are made dominant late in the prefix. At these magnitudes the golden
    pipeline's own bf16 rounding of the logits is the larger error, so the yardsticks are the
    unrounded float64 evaluation and the mma.sync form."""
    rows, stride = 192, 512
    ck, cv, ks, vs = pool(5, stride)
    ks[:, 100] *= 3.0
    ks[:, 180] *= 4.0
    rng = np.random.default_rng(6)
    qb = bf16_bits(60.0 * rng.standard_normal((rows, Hq * D)))
    monkeypatch.setenv("G4_PREFILL_TC", "1")
    got = run(K, qb, (ck, cv, ks, vs), 0, stride, None)
    monkeypatch.setenv("G4_PREFILL_TC", "0")
    other = run(K, qb, (ck, cv, ks, vs), 0, stride, None)
    assert close(f32_of(got), f32_of(other), 0.02)
    sel = np.r_[0:3, 63:66, 99:103, 179:183, 189:192]
    tbl = np.arange(stride, dtype=np.int32)
    exact = f64_rows(qb[sel], (ck, cv, ks, vs), [tbl] * len(sel), sel.astype(np.int32))
    assert close(f32_of(got[sel]).reshape(len(sel), Hq, D), exact, 0.02)


def test_a_query_head_that_is_not_a_number_stays_in_its_rows(K):
    """One head of one query row is NaN: that row and head come out NaN, every other output is what it
    is without the NaN to a bf16 step (rows do not share softmax state), and no wait runs out."""
    rows, stride = 200, 512
    pl = pool(11, stride)
    rng = np.random.default_rng(12)
    q = bf16_bits(rng.standard_normal((rows, Hq * D)))
    clean = run(K, q, pl, 0, stride, None)
    q2 = q.copy()
    q2[70, 5 * D:6 * D] = 0x7FC0
    got = run(K, q2, pl, 0, stride, None).reshape(rows, Hq, D)
    clean = clean.reshape(rows, Hq, D)
    assert (got[70, 5] & 0x7FFF > 0x7F80).all()
    keep = np.ones((rows, Hq), bool)
    keep[70, 5] = False
    assert close(f32_of(got[keep]), f32_of(clean[keep]), 0.0)  # (when a maximum moves may differ within the warp)
