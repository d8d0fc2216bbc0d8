"""Generates tests/golden/*.npz from the REFERENCE's own host code.

Run where a reference checkout is mounted (its root is the REF default of oracle/Makefile):

    python tests/golden/make_golden.py

It builds oracle/_ref/libg4ref.so (the reference's kernel_math.h + fp8_convert.cc behind
oracle/ref_shim.cc) and records, for seeded inputs that mirror the reference's device-test
fixtures (engine/tests/test_kernels.cu), the outputs the reference formulation gives. The
.npz files are small and committed; the tests compare both the C port and the CUDA kernels
with them, on machines where the reference tree does not exist.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import g4_oracle  # noqa: E402


def f32_to_bf16_bits(ref, a):
    flat = np.ascontiguousarray(a, np.float32).ravel()
    return np.array([ref.f32_to_bf16(x) for x in flat], np.uint16).reshape(a.shape)


def main():
    g4_oracle.build()
    ref = g4_oracle.load("reference")
    out = {}

    # -- rmsnorm 64 x 256, seed 0x4242 (engine/tests/test_kernels.cu:1019-1055): x then w from
    #    one stream
    stream = ref.fill_bf16(0x4242, 4.0, 64 * 256 + 256)
    x, w = stream[:64 * 256].reshape(64, 256), stream[64 * 256:]
    _, n = ref.add_rmsnorm(x, None, w, 1e-5, 1.0, want_h=False)
    out["rmsnorm_64x256"] = dict(x=x, w=w, n=n)

    # -- rmsnorm 4 x 4096, seed 0x6262 (test_kernels.cu:2618-2647)
    stream = ref.fill_bf16(0x6262, 4.0, 4 * 4096 + 4096)
    x, w = stream[:4 * 4096].reshape(4, 4096), stream[4 * 4096:]
    _, n = ref.add_rmsnorm(x, None, w, 1e-5, 1.0, want_h=False)
    out["rmsnorm_4x4096"] = dict(x=x, w=w, n=n)

    # -- rope 128 positions, d = 128, theta 1e7, seed 0x1337 (test_kernels.cu:1057-1090)
    x = ref.fill_bf16(0x1337, 4.0, 128 * 128).reshape(128, 128)
    c, s = ref.rope_tables(1e7, 128, 128)
    out["rope_128x128"] = dict(x=x, y=ref.rope_rows(x, c, s), cos_head=c[:4].copy(), sin_head=s[:4].copy(),
                               cos_tail=c[-2:].copy(), sin_tail=s[-2:].copy())

    # -- kv8 rows: 256 x 128, seed 0x8abc, zero row / 1e-5 row / 0.25, 3, 32, 256
    #    (test_kernels.cu:355-449); rows are generated one after the other from one stream
    import ctypes as C
    lib = C.CDLL(ref.path)
    lib.g4ref_rng_u64.argtypes = [C.c_uint64, C.c_long, C.c_void_p]
    u = np.empty(256 * 128, np.uint64)
    lib.g4ref_rng_u64(0x8abc, u.size, u.ctypes.data_as(C.c_void_p))
    unit = ((u >> np.uint64(41)).astype(np.float32) * np.float32(2.0 ** -23))
    scale = np.empty(256, np.float32)
    for r in range(256):
        scale[r] = 0.0 if r == 0 else 1e-5 if r == 1 else (0.25, 3.0, 32.0, 256.0)[r % 4]
    vals = (unit.reshape(256, 128) * np.float32(2.0) - np.float32(1.0)) * scale[:, None]
    kx = f32_to_bf16_bits(ref, vals.astype(np.float32))
    ck, cv, ks, vs = ref.kv_append_int8(kx.reshape(256, 1, 128), kx.reshape(256, 1, 128),
                                        np.arange(256, dtype=np.int32), 1, 128, 256)
    out["kv8_256x128"] = dict(x=kx, codes=ck[0], scales=ks[0])

    # -- config 1: decode add + norm, 1 row x 4096, f32 x and residual ~ N(0,1), rm 0.22,
    #    w ~ N(1, 0.02), eps 1e-5, bf16 + FP8 outputs; seed 0
    rng = np.random.default_rng(0)
    y = rng.standard_normal((1, 4096)).astype(np.float32)
    res = rng.standard_normal((1, 4096)).astype(np.float32)
    w = f32_to_bf16_bits(ref, (1.0 + 0.02 * rng.standard_normal(4096)).astype(np.float32))
    h, n = ref.add_rmsnorm(y, res, w, 1e-5, 0.22)
    codes, sc, amax = ref.quant_fp8(n)
    out["c1_add_rmsnorm_f32"] = dict(y=y, res=res, w=w, h=h, n=n, codes=codes,
                                     scale=np.float32(sc), amax=np.float32(amax))

    # -- the same op on bf16 inputs, 6 rows, both multipliers
    yb = f32_to_bf16_bits(ref, rng.standard_normal((6, 4096)).astype(np.float32))
    rb = f32_to_bf16_bits(ref, rng.standard_normal((6, 4096)).astype(np.float32))
    d = dict(y=yb, res=rb, w=w)
    for tag, rm in (("rm1", 1.0), ("rm022", 0.22)):
        h, n = ref.add_rmsnorm(yb, rb, w, 1e-5, rm)
        codes, sc, amax = ref.quant_fp8(n)
        d.update({f"h_{tag}": h, f"n_{tag}": n, f"codes_{tag}": codes, f"scale_{tag}": np.float32(sc)})
    out["add_rmsnorm_bf16_6x4096"] = d

    # -- embedding gather: 50-row table x 4096 ~ N(0, 0.02), 9 ids, mult 12 and 1
    emb = f32_to_bf16_bits(ref, (0.02 * rng.standard_normal((50, 4096))).astype(np.float32))
    ids = rng.integers(0, 50, 9).astype(np.int32)
    out["embed_9x4096"] = dict(emb=emb, ids=ids, out12=ref.embed_rows(ids, 0, 9, emb, 12.0),
                               out1=ref.embed_rows(ids, 0, 9, emb, 1.0))

    # -- RoPE + int8 paged KV: 20 token rows, Granite heads, permuted 16-token pages, positions
    #    with an offset; both K rounding modes
    Hq, Hk, dd, stride = 32, 8, 128, 64
    qkv = f32_to_bf16_bits(ref, rng.standard_normal((20, (Hq + 2 * Hk) * dd)).astype(np.float32))
    pos = (1000 + np.arange(20)).astype(np.int32)
    pages = rng.permutation(stride // 16)[:2]
    kvr = (pages[np.arange(20) // 16] * 16 + np.arange(20) % 16).astype(np.int32)
    c, s = ref.rope_tables(1e7, dd, 1024)
    d = dict(qkv=qkv, pos=pos, kv_rows=kvr)
    for mode in (0, 1):
        q_rot, ck, cv, ks, vs = ref.rope_kv_int8(qkv, c, s, pos, kvr, Hq, Hk, dd, stride, mode)
        d.update({f"q_rot_{mode}": q_rot, f"ck_{mode}": ck, f"cv_{mode}": cv, f"ks_{mode}": ks,
                  f"vs_{mode}": vs})
    out["rope_kv_20"] = d

    # -- SwiGLU: 3 rows x 12800 bf16 ~ N(0,1), bf16 + FP8
    g = f32_to_bf16_bits(ref, rng.standard_normal((3, 12800)).astype(np.float32))
    u = f32_to_bf16_bits(ref, rng.standard_normal((3, 12800)).astype(np.float32))
    act = ref.swiglu(g, u)
    codes, sc, amax = ref.quant_fp8(act)
    out["swiglu_3x12800"] = dict(gate=g, up=u, act=act, codes=codes, scale=np.float32(sc))
    # f32 [rows][2 I] form of the reference's prefill kernel
    gu = rng.standard_normal((2, 2 * 12800)).astype(np.float32)
    out["silu_mul_f32_2x12800"] = dict(gu=gu, act=ref.swiglu(gu[:, :12800], gu[:, 12800:]))

    # -- FP8 e4m3 codec: every bf16 pattern, and every code's value
    allbf = np.arange(0x10000, dtype=np.uint32).astype(np.uint16)
    enc = np.array([ref.fp8_encode(ref.bf16_to_f32(int(b))) for b in allbf], np.uint8)
    dec = np.array([ref.fp8_decode(c) for c in range(256)], np.float32)
    out["fp8_codec"] = dict(encode_all_bf16=enc, decode_all=dec)

    # -- FP8 x FP8 GEMM with the reference's epilogue kinds: codes of values in [-2, 2) as the
    #    reference's device fixture draws its weights (engine/tests/test_kernels.cu:1120-1129),
    #    three weight segments, K over two 128-byte blocks and a ragged M / N
    grng = np.random.default_rng(0xdead)
    ga = np.array([ref.fp8_encode(v) for v in grng.uniform(-2, 2, 40 * 256)], np.uint8).reshape(40, 256)
    gw = np.array([ref.fp8_encode(v) for v in grng.uniform(-2, 2, 72 * 256)], np.uint8).reshape(72, 256)
    gres = f32_to_bf16_bits(ref, grng.standard_normal((40, 72)).astype(np.float32))
    kw = dict(a_scale=0.125, w_scales=(0.001, 0.002, 0.0005), segs=(32, 48))
    out["gemm_fp8_40x72x256"] = dict(
        a=ga, w=gw, residual=gres, a_scale=np.float32(kw["a_scale"]), w_scales=np.array(kw["w_scales"], np.float32),
        segs=np.array(kw["segs"], np.int32), resid_scale=np.float32(0.22),
        out_bf16=ref.gemm_fp8(ga, gw, **kw), out_f32=ref.gemm_fp8(ga, gw, kind="f32", **kw),
        out_residual=ref.gemm_fp8(ga, gw, residual=gres, resid_scale=0.22, **kw))

    for name, arrays in out.items():
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
