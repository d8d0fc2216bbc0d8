"""Pins the CPU oracle (oracle/g4_oracle.c) before anything is compared with it.

Three layers of evidence, all CPU-only:
  1. the reference's own known-answer tests for this path, re-asserted on the port
     (engine/tests/test_kernel_math.cc, engine/tests/test_fp8_convert.cc);
  2. golden vectors recorded from the reference's host code (tests/golden/*.npz, written
     by tests/golden/make_golden.py) - available everywhere;
  3. where oracle/_ref/libg4ref.so exists, the port against the reference's compiled code
     on fresh random inputs, bit for bit.
"""
import math
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


# --------------------------------------------------------------------------- 1. known answers
def test_bf16_known_answers(port):
    # engine/tests/test_kernel_math.cc:29-51
    for v in (0.5, 1.0, 2.0, -1.0, 128.0, -128.0, math.ldexp(1.0, -133)):
        assert port.bf16_to_f32(port.f32_to_bf16(v)) == v
    assert port.f32_to_bf16(1.0 + 2.0 ** -8) == port.f32_to_bf16(1.0)  # tie -> even
    assert port.bf16_to_f32(port.f32_to_bf16(1.0 + 2.0 ** -7)) == 1.0 + 2.0 ** -7
    assert port.f32_to_bf16(-0.0) & 0x8000
    a = 1.0 + 3.5 * 2.0 ** -7
    assert port.bf16_to_f32(port.f32_to_bf16(a)) == 1.0 + 4.0 * 2.0 ** -7


def _norm_f32(port, x, w, eps):
    """rmsnorm on float values that are exactly bf16-representable, output as floats."""
    xb = np.array([[port.f32_to_bf16(v) for v in x]], np.uint16)
    wb = np.array([port.f32_to_bf16(v) for v in w], np.uint16)
    _, n = port.add_rmsnorm(xb, None, wb, eps, 1.0, want_h=False)
    return [port.bf16_to_f32(b) for b in n[0]]


def test_rmsnorm_known_answers(port):
    # engine/tests/test_kernel_math.cc:53-75 (eps must be > 0 in the device launchers; the
    # eps = 0 cases there are host-only, so a denormal-small eps stands in for them)
    n = 8
    assert _norm_f32(port, [2.0] * n, [1.0] * n, 1e-30) == [1.0] * n
    assert _norm_f32(port, [2.0] * n, [2.0] * n, 1e-30) == [2.0] * n
    got = _norm_f32(port, [2.0] * n, [1.0] * n, 1e-5)
    want = port.bf16_to_f32(port.f32_to_bf16(np.float32(2.0) / np.sqrt(np.float32(4.0) + np.float32(1e-5))))
    assert got == [want] * n
    assert _norm_f32(port, [0.0] * n, [1.0] * n, 1e-5) == [0.0] * n  # zero row: 0, not NaN


def test_rope_known_answers(port):
    # engine/tests/test_kernel_math.cc:77-110
    c, s = port.rope_tables(1e7, 8, 1)
    assert (c == 1.0).all() and (s == 0.0).all()
    c, s = port.rope_tables(1e7, 8, 2)
    assert abs(c[1, 0] - math.cos(1.0)) < 1e-5 and abs(s[1, 0] - math.sin(1.0)) < 1e-5
    # rotation by 0.5 rad on x = [2, 4, 1, 3] (a = {2, 4}, b = {1, 3}), then the inverse
    cc, ss = np.float32(math.cos(np.float32(0.5))), np.float32(math.sin(np.float32(0.5)))
    x = np.array([[port.f32_to_bf16(v) for v in (2.0, 4.0, 1.0, 3.0)]], np.uint16)
    ct, st = np.full((1, 2), cc, np.float32), np.full((1, 2), ss, np.float32)
    y = [port.bf16_to_f32(b) for b in port.rope_rows(x, ct, st)[0]]
    cd, sd = math.cos(0.5), math.sin(0.5)
    want = [2 * cd - 1 * sd, 4 * cd - 3 * sd, 1 * cd + 2 * sd, 3 * cd + 4 * sd]
    for g, wv in zip(y, want):
        assert abs(g - wv) <= abs(wv) * 2.0 ** -8 + 1e-6  # one bf16 rounding of the f32 result


def test_silu_known_answers(port):
    # engine/tests/test_kernel_math.cc:141-150
    assert port.silu(0.0) == 0.0
    assert abs(port.silu(1.0) - 1.0 / (1.0 + math.exp(-1.0))) < 1e-7
    assert port.silu(-0.5) < 0.0


def test_kv8_known_answers(port):
    # engine/tests/test_kernel_math.cc:724-764
    assert port.kv8_scale(127.0) == 1.0
    for x, q in ((0.0, 0), (1.0, 1), (-1.0, -1), (127.0, 127), (-127.0, -127), (127.4, 127),
                 (-127.4, -127), (0.5, 1), (-0.5, -1)):
        assert port.kv8_quant(x, 1.0) == q
    assert port.kv8_quant(1.0, 0.0) == 0 and port.kv8_dequant(0, 0.0) == 0.0
    rng = np.random.default_rng(0x8AB4)
    worst = 0.0
    for r in range(64):
        amax = np.float32(abs(rng.uniform(-1, 1)) * (1 + r % 7))
        s = port.kv8_scale(amax)
        for x in rng.uniform(-amax, amax, 32).astype(np.float32):
            q = port.kv8_quant(x, s)
            dq = port.kv8_dequant(q, s)
            assert dq == np.float32(s) * np.float32(q)
            assert abs(x - dq) <= s * 0.5 + 1e-7
            worst = max(worst, abs(x - dq) / max(amax, 1e-30))
    assert worst <= 1.0 / 254.0 + 1e-6


def test_rng_stream(port, ref):
    # engine/tests/test_kernel_math.cc:766-790: determinism + range; here also port == reference
    a = port.fill_bf16(123, 2.0, 5000)
    assert (a == port.fill_bf16(123, 2.0, 5000)).all()
    assert (a != port.fill_bf16(456, 2.0, 5000)).any()
    assert (a == ref.fill_bf16(123, 2.0, 5000)).all()
    vals = np.array([port.bf16_to_f32(b) for b in a[:2000]])
    assert vals.min() >= -2.0 and vals.max() <= 2.0


def test_fp8_special_values(port):
    # engine/tests/test_fp8_convert.cc:197-236
    inf, nan = float("inf"), float("nan")
    cases = [(0.0, 0x00), (-0.0, 0x80), (448.0, 0x7E), (-448.0, 0xFE), (464.0, 0x7E), (-464.0, 0xFE),
             (463.9999999999999, 0x7E), (inf, 0x7E), (-inf, 0xFE), (nan, 0x7F), (-nan, 0x7F),
             (2.0 ** -9, 0x01), (2.0 * 2.0 ** -9, 0x02), (2.0 ** -6, 0x08), (1.5 * 2.0 ** -7, 0x06),
             (450.0, 0x7E)]
    for v, want in cases:
        assert port.fp8_encode(v) == want, (v, want)


def _grid():
    """All non-negative finite e4m3 values in code order (test_fp8_convert.cc build_grid)."""
    vals = []
    for code in range(0x7F):
        e, m = code >> 3, code & 7
        vals.append(m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))
    return vals


def test_fp8_ties_to_even_and_round_trip(port):
    # engine/tests/test_fp8_convert.cc:173-195, :283-298
    g = _grid()
    for i in range(len(g) - 1):
        mid = g[i] + (g[i + 1] - g[i]) / 2.0
        even = i if i % 2 == 0 else i + 1
        assert port.fp8_encode(mid) == even
        assert port.fp8_encode(-mid) == (even | 0x80)
    for code in range(256):
        if code & 0x7F == 0x7F:
            continue
        assert port.fp8_encode(port.fp8_decode(code)) == code
        assert abs(port.fp8_decode(code)) == g[code & 0x7F]


def test_fp8_nearest_on_random_doubles(port):
    # engine/tests/test_fp8_convert.cc:138-171: the code must be the nearest grid point
    g = np.array(_grid())
    rng = np.random.default_rng(0xC0FFEE)
    v = np.abs(rng.standard_normal(20000)) * np.exp2(rng.integers(-12, 9, 20000))
    v = v[v < 448.0]
    for x in v[:6000]:
        c = port.fp8_encode(x)
        best = np.abs(g - x).min()
        assert abs(g[c] - x) <= best * (1 + 1e-15)


# --------------------------------------------------------------------------- 2. golden vectors
def test_golden_fp8_codec(port):
    z = golden("fp8_codec")
    enc = np.array([port.fp8_encode(port.bf16_to_f32(b)) for b in range(0x10000)], np.uint8)
    assert (enc == z["encode_all_bf16"]).all()
    dec = np.array([port.fp8_decode(c) for c in range(256)], np.float32)
    assert np.array_equal(dec, z["decode_all"], equal_nan=True)


@pytest.mark.parametrize("name", ["rmsnorm_64x256", "rmsnorm_4x4096"])
def test_golden_rmsnorm(port, name):
    z = golden(name)
    _, n = port.add_rmsnorm(z["x"], None, z["w"], 1e-5, 1.0, want_h=False)
    assert (n == z["n"]).all()
    # the seeded inputs themselves are reproduced by the port's RNG
    rows, cols = z["x"].shape
    seed = 0x4242 if name == "rmsnorm_64x256" else 0x6262
    stream = port.fill_bf16(seed, 4.0, rows * cols + cols)
    assert (stream[:rows * cols].reshape(rows, cols) == z["x"]).all() and (stream[rows * cols:] == z["w"]).all()


def test_golden_rope(port):
    z = golden("rope_128x128")
    c, s = port.rope_tables(1e7, 128, 128)
    assert (c[:4] == z["cos_head"]).all() and (s[-2:] == z["sin_tail"]).all()
    assert (port.rope_rows(z["x"], c, s) == z["y"]).all()


def test_golden_kv8(port):
    z = golden("kv8_256x128")
    x = z["x"]
    ck, cv, ks, vs = port.kv_append_int8(x.reshape(256, 1, 128), x.reshape(256, 1, 128),
                                         np.arange(256, dtype=np.int32), 1, 128, 256)
    assert (ck[0] == z["codes"]).all() and (ks[0] == z["scales"]).all()
    assert (cv[0] == z["codes"]).all() and (vs[0] == z["scales"]).all()
    assert (z["codes"][0] == 0).all() and z["scales"][0] == 0.0  # the all-zero row


def test_golden_config1_add_rmsnorm(port):
    z = golden("c1_add_rmsnorm_f32")
    h, n = port.add_rmsnorm(z["y"], z["res"], z["w"], 1e-5, 0.22)
    assert (h == z["h"]).all() and (n == z["n"]).all()
    codes, scale, amax = port.quant_fp8(n)
    assert (codes == z["codes"]).all() and scale == z["scale"] and amax == z["amax"]


def test_golden_add_rmsnorm_bf16(port):
    z = golden("add_rmsnorm_bf16_6x4096")
    for tag, rm in (("rm1", 1.0), ("rm022", 0.22)):
        h, n = port.add_rmsnorm(z["y"], z["res"], z["w"], 1e-5, rm)
        assert (h == z[f"h_{tag}"]).all() and (n == z[f"n_{tag}"]).all()
        codes, scale, _ = port.quant_fp8(n)
        assert (codes == z[f"codes_{tag}"]).all() and scale == z[f"scale_{tag}"]


def test_golden_embed(port):
    z = golden("embed_9x4096")
    assert (port.embed_rows(z["ids"], 0, 9, z["emb"], 12.0) == z["out12"]).all()
    assert (port.embed_rows(z["ids"], 0, 9, z["emb"], 1.0) == z["out1"]).all()
    assert (z["out1"] == z["emb"][z["ids"]]).all()  # multiplier 1 is a bit copy


def test_golden_rope_kv(port):
    z = golden("rope_kv_20")
    c, s = port.rope_tables(1e7, 128, 1024)
    for mode in (0, 1):
        q_rot, ck, cv, ks, vs = port.rope_kv_int8(z["qkv"], c, s, z["pos"], z["kv_rows"], 32, 8, 128,
                                                  64, mode)
        assert (q_rot == z[f"q_rot_{mode}"]).all()
        assert (ck == z[f"ck_{mode}"]).all() and (cv == z[f"cv_{mode}"]).all()
        assert (ks == z[f"ks_{mode}"]).all() and (vs == z[f"vs_{mode}"]).all()
    assert (z["ck_0"] != z["ck_1"]).any()  # the two K rounding modes really differ


def test_golden_swiglu(port):
    z = golden("swiglu_3x12800")
    act = port.swiglu(z["gate"], z["up"])
    assert (act == z["act"]).all()
    codes, scale, _ = port.quant_fp8(act)
    assert (codes == z["codes"]).all() and scale == z["scale"]
    z = golden("silu_mul_f32_2x12800")
    gu = z["gu"]
    assert (port.swiglu(gu[:, :12800], gu[:, 12800:]) == z["act"]).all()


# --------------------------------------------------------------------------- 3. port vs reference
def test_port_matches_reference_random(port, ref):
    rng = np.random.default_rng(7)
    rows, cols = 11, 4096
    y = port.fill_bf16(11, 4.0, rows * cols).reshape(rows, cols)
    res = port.fill_bf16(12, 4.0, rows * cols).reshape(rows, cols)
    w = port.fill_bf16(13, 1.5, cols)
    for rm in (1.0, 0.22):
        a, b = port.add_rmsnorm(y, res, w, 1e-5, rm), ref.add_rmsnorm(y, res, w, 1e-5, rm)
        assert (a[0] == b[0]).all() and (a[1] == b[1]).all()
        qa, qb = port.quant_fp8(a[1]), ref.quant_fp8(b[1])
        assert (qa[0] == qb[0]).all() and qa[1] == qb[1]
    yf = rng.standard_normal((rows, cols)).astype(np.float32)
    rf = rng.standard_normal((rows, cols)).astype(np.float32)
    a, b = port.add_rmsnorm(yf, rf, w, 1e-5, 0.22), ref.add_rmsnorm(yf, rf, w, 1e-5, 0.22)
    assert (a[0] == b[0]).all() and (a[1] == b[1]).all()
    c1, s1 = port.rope_tables(1e7, 128, 700)
    c2, s2 = ref.rope_tables(1e7, 128, 700)
    assert (c1 == c2).all() and (s1 == s2).all()
    qkv = port.fill_bf16(15, 4.0, rows * 48 * 128).reshape(rows, -1)
    pos = rng.integers(0, 700, rows).astype(np.int32)
    kvr = rng.permutation(32)[:rows].astype(np.int32)
    for mode in (0, 1):
        A = port.rope_kv_int8(qkv, c1, s1, pos, kvr, 32, 8, 128, 32, mode)
        B = ref.rope_kv_int8(qkv, c1, s1, pos, kvr, 32, 8, 128, 32, mode)
        assert all((x == z).all() for x, z in zip(A, B))
    g = port.fill_bf16(17, 6.0, rows * 12800).reshape(rows, 12800)
    u = port.fill_bf16(18, 6.0, rows * 12800).reshape(rows, 12800)
    assert (port.swiglu(g, u) == ref.swiglu(g, u)).all()
    ids = rng.integers(0, rows, 5).astype(np.int32)
    assert (port.embed_rows(ids, 0, 5, y, 12.0) == ref.embed_rows(ids, 0, 5, y, 12.0)).all()


def test_port_matches_reference_fp8_doubles(port, ref):
    rng = np.random.default_rng(3)
    v = rng.standard_normal(40000) * np.exp2(rng.integers(-14, 10, 40000))
    for x in v:
        assert port.fp8_encode(x) == ref.fp8_encode(x)


def test_greedy_pick_known_answers_and_reference(port, ref):
    # engine/tests/test_kernel_math.cc:683-688 (values rounded to bf16 keep their order)
    def bits(vals):
        return np.array([[port.f32_to_bf16(v) for v in vals]], np.uint16)
    assert port.argmax_rows(bits([0.1, 0.6, 0.2, 0.1]))[0] == 1
    assert port.argmax_rows(bits([0.5, 0.5]))[0] == 0          # tie -> smallest id
    assert port.argmax_rows(bits([-0.0, 0.0, -1.0]))[0] == 0   # +0 is not above -0
    rng = np.random.default_rng(77)
    logits = (rng.standard_normal((64, 1000)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    logits[:, 500:] = logits[:, :500]  # every maximum appears twice: the first must win
    got = port.argmax_rows(logits)
    assert (got < 500).all()
    if ref is not None:
        assert (got == ref.argmax_rows(logits)).all()


def _random_pool(seed, Hk, stride, d):
    rng = np.random.default_rng(seed)
    ck = rng.integers(-127, 128, (Hk, stride, d), dtype=np.int8)
    cv = rng.integers(-127, 128, (Hk, stride, d), dtype=np.int8)
    ks = (rng.random((Hk, stride), dtype=np.float32) * 0.02 + 0.005).astype(np.float32)
    vs = (rng.random((Hk, stride), dtype=np.float32) * 0.02 + 0.005).astype(np.float32)
    return ck, cv, ks, vs


def test_attention_oracle_matches_reference_golden_pipeline(port, ref):
    """Decode attention over an int8 pool: the port restates gqa_attention_bf16
    (engine/src/kernel_math.h:265-331) over rows dequantised to bf16; bit for bit against the
    reference's own function, and close to an unrounded float64 evaluation."""
    Hq, Hk, d, stride = 8, 2, 128, 96
    ck, cv, ks, vs = _random_pool(21, Hk, stride, d)
    rng = np.random.default_rng(22)
    q = (rng.standard_normal((3, Hq * d)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    pos = np.array([0, 40, 95], np.int32)
    tables = [rng.permutation(stride).astype(np.int32) for _ in range(3)]
    scale = 1.0 / 128
    got = port.attn_decode_int8(q, ck, cv, ks, vs, pos, tables, Hq, Hk, d, scale)
    if ref is not None:
        assert (got == ref.attn_decode_int8(q, ck, cv, ks, vs, pos, tables, Hq, Hk, d, scale)).all()
    qf = (q.astype(np.uint32) << 16).view(np.float32).astype(np.float64).reshape(3, Hq, d)
    gotf = (got.astype(np.uint32) << 16).view(np.float32).reshape(3, Hq, d)
    for r in range(3):
        rows_ = tables[r][:pos[r] + 1]
        for h in range(Hq):
            k = ck[h // 4, rows_].astype(np.float64) * ks[h // 4, rows_, None]
            v = cv[h // 4, rows_].astype(np.float64) * vs[h // 4, rows_, None]
            lg = scale * (k @ qf[r, h])
            p = np.exp(lg - lg.max())
            want = (p / p.sum()) @ v
            assert np.abs(gotf[r, h] - want).max() < 0.03  # the reference's own device tolerance
    # no cache positions (negative position): zeros
    z = port.attn_decode_int8(q[:1], ck, cv, ks, vs, np.array([-1], np.int32), None, Hq, Hk, d, scale)
    assert (z == 0).all()


def _gemm_kw(g):
    return dict(a_scale=float(g["a_scale"]), w_scales=tuple(float(x) for x in g["w_scales"]),
                segs=tuple(int(x) for x in g["segs"]))


def test_gemm_known_answers_golden_and_reference(port, ref):
    # engine/tests/test_kernel_math.cc:700-720: A [[1, 2], [3, 4]], B [[1, -1], [2, 0.5]], scale 2
    a = np.array([[port.fp8_encode(v) for v in r] for r in ((1, 2), (3, 4))], np.uint8)
    b = np.array([[port.fp8_encode(v) for v in r] for r in ((1, -1), (2, 0.5))], np.uint8)
    # K must not matter for the restatement: pad K to 16 with zero codes
    a16, b16 = np.zeros((2, 16), np.uint8), np.zeros((2, 16), np.uint8)
    a16[:, :2], b16[:, :2] = a, b
    c = port.gemm_fp8(a16, b16, a_scale=1.0, w_scales=(2.0,), kind="f32")
    assert np.abs(c - np.array([[-2, 6], [-2, 16]], np.float32)).max() < 1e-4
    g = golden("gemm_fp8_40x72x256")
    kw = _gemm_kw(g)
    assert (port.gemm_fp8(g["a"], g["w"], **kw) == g["out_bf16"]).all()
    assert (port.gemm_fp8(g["a"], g["w"], kind="f32", **kw) == g["out_f32"]).all()
    assert (port.gemm_fp8(g["a"], g["w"], residual=g["residual"], resid_scale=float(g["resid_scale"]), **kw)
            == g["out_residual"]).all()
    if ref is not None:
        rng = np.random.default_rng(5)
        a = rng.integers(0, 256, (9, 96), dtype=np.uint8)
        w = rng.integers(0, 256, (11, 96), dtype=np.uint8)
        a[(a & 0x7f) == 0x7f] = 0x30
        w[(w & 0x7f) == 0x7f] = 0x30
        assert (port.gemm_fp8(a, w, a_scale=0.01, w_scales=(0.5, 0.25), segs=(4,), kind="f32")
                == ref.gemm_fp8(a, w, a_scale=0.01, w_scales=(0.5, 0.25), segs=(4,), kind="f32")).all()
