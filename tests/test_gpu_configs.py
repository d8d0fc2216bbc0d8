"""The benchmark configurations at their real sizes, and row sharding over two real GPUs.

test_gpu_parity.py pins every kernel on shapes the CPU oracle walks through in a moment. The
tests here repeat the comparison at the sizes that are actually timed - the decode chain of 1 to 8
rows on a Granite-size table, the 32768-row long-context batch, one layer of the 65536-row sweep -
with the oracle spread over the host's cores, and run two half shards on two devices against the
whole batch on one. Tolerances are the ones stated at the top of test_gpu_parity.py: everything
bit-exact except SwiGLU's bf16 output (1 ulp), whose FP8 codes are the oracle quantiser applied to
the device's own bf16 values.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
Hq, Hk, D, H, I, VOCAB = 32, 8, 128, 4096, 12800, 100352


def _threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def par(fn, rows):
    """fn(lo, hi) over contiguous row ranges on all host cores (the oracle's C calls drop the GIL)."""
    from oracle import g4_oracle
    return g4_oracle.parallel_rows(fn, rows, _threads())


def bits(t):
    """bf16 (or int16) CUDA tensor -> host uint16 bit patterns."""
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    a = t.cpu().numpy()
    return a.view(np.uint16) if a.dtype == np.int16 else a


def ulp_distance(a, b):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return np.abs(key(a) - key(b))


@pytest.fixture(scope="module")
def K():
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi, kernels
    capi.lib()  # raises if the CUDA library is missing: no fallback
    yield kernels
    assert capi.lib().device_status() == 0, "a kernel reported a bounded wait that ran out"


@pytest.fixture(scope="module")
def table():
    """Granite-size embedding table, N(0, 0.02) in bf16: the device tensor and its host bits."""
    g = torch.Generator(device=DEV).manual_seed(2024)
    t = torch.empty(VOCAB, H, dtype=torch.bfloat16, device=DEV)
    for lo in range(0, VOCAB, 12544):  # in slabs: no 1.6 GB float32 temporary
        t[lo:lo + 12544] = (0.02 * torch.randn(12544, H, generator=g, device=DEV)).to(torch.bfloat16)
    yield t, bits(t)
    del t
    torch.cuda.empty_cache()


def rand_bits(gen, *shape, sigma=1.0):
    return (sigma * torch.randn(*shape, generator=gen, device=gen.device)).to(torch.bfloat16)


# =========================================================================== configuration 2
@pytest.mark.parametrize("B", [1, 2, 4, 8])
def test_config2_decode_chain(K, port, table, B):
    """Decode chain of B sessions: gather from the 100352 x 4096 table (ids uniform, multiplier 12),
    residual add + RMSNorm -> FP8, RoPE of Q [32 x 128] and K [8 x 128] at positions uniform in
    [0, 8192) with the int8 KV append through per-session page tables (K rounded to bf16 before it is
    quantised, as the reference's decode path does), SwiGLU of gate / up [12800] -> FP8. Every output
    of every step against the oracle."""
    from granite4_b200 import capi
    emb, emb_host = table
    g = torch.Generator(device=DEV).manual_seed(100 + B)
    rng = np.random.default_rng(200 + B)
    ids = rng.integers(0, VOCAB, B).astype(np.int32)
    pos = rng.integers(0, 8192, B).astype(np.int32)
    y = rand_bits(g, B, H)
    w = (1 + 0.02 * torch.randn(H, generator=g, device=DEV)).to(torch.bfloat16)
    q, k, v = rand_bits(g, B, Hq * D), rand_bits(g, B, Hk * D), rand_bits(g, B, Hk * D)
    gate, up = rand_bits(g, B, I), rand_bits(g, B, I)
    stride = 8 * 8192
    # every session owns 8192 pool rows, in 16-token pages in permuted order
    tables = []
    for r in range(B):
        pages = rng.permutation(512) + 512 * r
        tables.append(torch.from_numpy((np.repeat(pages, 16) * 16 + np.arange(8192) % 16).astype(np.int32)).to(DEV))
    kv_rows = np.array([int(tables[r][int(pos[r])].item()) for r in range(B)], np.int32)
    desc = capi.MultiRows()
    desc.n = B
    for r in range(B):
        desc.pos[r] = int(pos[r])
        desc.pt[r] = tables[r].data_ptr()
    d_rows = K.multi_rows_to_device(desc, DEV)
    t = K.RopeTables(1e7, D, 8192, DEV)

    h = torch.empty(B, H, dtype=torch.bfloat16, device=DEV)
    n8 = torch.empty(B, H, dtype=torch.uint8, device=DEV)
    sa = torch.zeros(2, 2, dtype=torch.float32, device=DEV)
    ck = torch.zeros(Hk, stride, D, dtype=torch.int8, device=DEV)
    cv = torch.zeros_like(ck)
    ks = torch.zeros(Hk, stride, dtype=torch.float32, device=DEV)
    vs = torch.zeros_like(ks)
    q_rot = torch.empty(B, Hq * D, dtype=torch.bfloat16, device=DEV)
    act = torch.empty(B, I, dtype=torch.bfloat16, device=DEV)
    a8 = torch.empty(B, I, dtype=torch.uint8, device=DEV)
    assert K.embed_gather(torch.from_numpy(ids).to(DEV), emb, 12.0, h) == 0
    h_emb = bits(h)
    assert K.add_rmsnorm_fp8(y, h, w, 1e-5, 0.22, h_out=h, n_fp8=n8, scale_amax=sa[0]) == 0
    assert K.gpu_multi_rope_append(q, k, v, t.cos, t.sin, d_rows, B, Hq, Hk, D, 8, ck, cv, ks, vs, stride,
                                   q_rot) == 0
    assert K.swiglu_fp8(gate, up, act, a8, sa[1]) == 0
    torch.cuda.synchronize()

    want_emb = port.embed_rows(ids, 0, B, emb_host, 12.0)
    assert (h_emb == want_emb).all()
    want_h, want_n = port.add_rmsnorm(bits(y), want_emb, bits(w), 1e-5, 0.22)
    codes, scale, amax = port.quant_fp8(want_n)
    assert (bits(h) == want_h).all() and (n8.cpu().numpy() == codes).all()
    assert sa[0, 0].item() == scale and sa[0, 1].item() == amax
    c, s = port.rope_tables(1e7, D, 8192)
    qkv = np.concatenate([bits(q), bits(k), bits(v)], axis=1)
    want = port.rope_kv_int8(qkv, c, s, pos, kv_rows, Hq, Hk, D, stride, 1)
    assert (bits(q_rot) == want[0]).all()
    for got, w_ in zip((ck, cv, ks, vs), want[1:]):
        assert (got.cpu().numpy() == w_).all()
    got_act = bits(act)
    assert ulp_distance(got_act, port.swiglu(bits(gate), bits(up))).max() <= 1
    a_codes, a_scale, a_amax = port.quant_fp8(got_act)
    assert (a8.cpu().numpy() == a_codes).all() and sa[1, 0].item() == a_scale and sa[1, 1].item() == a_amax
    t.close()


# =========================================================================== configuration 4
def test_config4_swiglu_and_embedding_at_32768_rows(K, port, table):
    """The long-context batch's other two ops at full size (RoPE + KV and add + norm are covered in
    test_gpu_parity.py): SwiGLU -> FP8 over 32768 x 12800 and the gather of 32768 rows, both against
    the oracle over EVERY row."""
    rows = 32768
    emb, emb_host = table
    ids = np.random.default_rng(41).integers(0, VOCAB, rows).astype(np.int32)
    out = torch.empty(rows, H, dtype=torch.bfloat16, device=DEV)
    assert K.embed_gather(torch.from_numpy(ids).to(DEV), emb, 12.0, out) == 0
    got = bits(out)
    del out
    parts = par(lambda lo, hi: port.embed_rows(ids, lo, hi - lo, emb_host, 12.0), rows)
    assert (got == np.concatenate(parts)).all()
    del got, parts

    g = torch.Generator(device=DEV).manual_seed(42)
    gate, up = rand_bits(g, rows, I), rand_bits(g, rows, I)
    act = torch.empty(rows, I, dtype=torch.bfloat16, device=DEV)
    c8 = torch.empty(rows, I, dtype=torch.uint8, device=DEV)
    sa = torch.zeros(2, dtype=torch.float32, device=DEV)
    assert K.swiglu_fp8(gate, up, act, c8, sa) == 0
    torch.cuda.synchronize()
    gb, ub, ab = bits(gate), bits(up), bits(act)
    want = np.concatenate(par(lambda lo, hi: port.swiglu(gb[lo:hi], ub[lo:hi]), rows))
    dist = ulp_distance(ab, want)
    assert dist.max() <= 1 and (dist != 0).mean() < 2e-3
    del want, dist, gb, ub
    amax = max(par(lambda lo, hi: port.amax_bf16(ab[lo:hi]), rows))
    scale = port.fp8_scale_from_amax(amax)
    assert sa[1].item() == amax and sa[0].item() == scale
    codes = c8.cpu().numpy()
    bad = par(lambda lo, hi: int((port.quant_fp8_with_scale(ab[lo:hi], scale) != codes[lo:hi]).sum()), rows)
    assert sum(bad) == 0
    # the scratch-free form (no bf16 copy between the sweeps) writes the same codes
    c8b = torch.empty_like(c8)
    assert K.swiglu_fp8(gate, up, None, c8b, sa) == 0
    assert torch.equal(c8, c8b)


# =========================================================================== configuration 5
def test_config5_one_layer_and_final_norm_at_65536_rows(K, port):
    """One layer of the box-scale sweep plus the final norm, at the single-GPU shard size the
    benchmark times (65536 rows), run the way the benchmark runs it (one library call per layer).
    The hidden state, both norms' FP8 outputs and scales, q_rot, the whole KV pool and the final
    norm are compared with the oracle over every row; SwiGLU on 2048 sampled rows, with its
    per-tensor maximum taken by the oracle over the device's bf16 activations of every row."""
    from granite4_b200 import glue
    rows = 65536
    seq = glue.GlueSequence(rows, device=DEV, seed=5, sets=1, layers=1)
    seq.reset()
    seq.run_fast()
    torch.cuda.synchronize()
    s = seq.shapes
    buf = seq.sets[0]
    w = bits(seq.w)
    h0, ya = bits(seq.h0), bits(buf["y_attn"])
    p1 = par(lambda lo, hi: port.add_rmsnorm(ya[lo:hi], h0[lo:hi], w[0, 0], s.eps, s.residual_multiplier), rows)
    h1 = np.concatenate([p[0] for p in p1])
    n1 = np.concatenate([p[1] for p in p1])
    del p1, ya, h0
    amax1 = max(par(lambda lo, hi: port.amax_bf16(n1[lo:hi]), rows))
    assert seq.scales[0, 0, 1].item() == amax1
    assert seq.scales[0, 0, 0].item() == port.fp8_scale_from_amax(amax1)
    del n1  # (its codes were overwritten by the second norm: n_fp8 is one buffer in the sweep)
    ym = bits(buf["y_mlp"])
    p2 = par(lambda lo, hi: port.add_rmsnorm(ym[lo:hi], h1[lo:hi], w[0, 1], s.eps, s.residual_multiplier), rows)
    h2 = np.concatenate([p[0] for p in p2])
    n2 = np.concatenate([p[1] for p in p2])
    del p2, ym, h1
    assert (bits(seq.h) == h2).all()
    amax2 = max(par(lambda lo, hi: port.amax_bf16(n2[lo:hi]), rows))
    scale2 = port.fp8_scale_from_amax(amax2)
    assert seq.scales[0, 1, 1].item() == amax2 and seq.scales[0, 1, 0].item() == scale2
    codes = seq.n_fp8.cpu().numpy()
    assert sum(par(lambda lo, hi: int((port.quant_fp8_with_scale(n2[lo:hi], scale2) != codes[lo:hi]).sum()),
                   rows)) == 0
    del n2, codes
    wf = bits(seq.w_final)
    fin = np.concatenate([p[1] for p in par(
        lambda lo, hi: port.add_rmsnorm(h2[lo:hi], None, wf, s.eps, 1.0, want_h=False), rows)])
    assert (bits(seq.out) == fin).all()
    del fin, h2
    # RoPE + KV write: every row, the whole pool
    c, sn = port.rope_tables(s.rope_theta, s.head_dim, seq.max_pos)
    qkv = bits(buf["qkv"])
    pos, kvr = seq.pos_rows.cpu().numpy(), seq.kv_rows.cpu().numpy()
    caches = (np.zeros((Hk, rows, D), np.int8), np.zeros((Hk, rows, D), np.int8),
              np.zeros((Hk, rows), np.float32), np.zeros((Hk, rows), np.float32))
    qr = par(lambda lo, hi: port.rope_kv_int8(qkv[lo:hi], c, sn, pos[lo:hi], kvr[lo:hi], Hq, Hk, D, rows, 0,
                                              caches)[0], rows)
    assert (bits(seq.q_rot) == np.concatenate(qr)).all()
    for got, want in zip((seq.cache_k[0], seq.cache_v[0], seq.k_scale[0], seq.v_scale[0]), caches):
        assert (got.cpu().numpy() == want).all()
    del qr, qkv, caches
    # SwiGLU: sampled rows against the formula, the tensor maximum over all rows
    act = bits(seq.act_ws)
    amax3 = max(par(lambda lo, hi: port.amax_bf16(act[lo:hi]), rows))
    scale3 = port.fp8_scale_from_amax(amax3)
    assert seq.scales[0, 2, 1].item() == amax3 and seq.scales[0, 2, 0].item() == scale3
    pick = np.sort(np.random.default_rng(55).choice(rows, 2048, replace=False))
    idx = torch.from_numpy(pick).to(DEV)
    gs, us = bits(buf["gate"][idx]), bits(buf["up"][idx])
    want = np.concatenate(par(lambda lo, hi: port.swiglu(gs[lo:hi], us[lo:hi]), len(pick)))
    assert ulp_distance(act[pick], want).max() <= 1
    a_codes = seq.act_fp8[idx].cpu().numpy()
    assert (a_codes == port.quant_fp8_with_scale(np.ascontiguousarray(act[pick]), scale3)).all()


# =========================================================================== two real devices
def _copy_shard(dst, src, lo, hi):
    for a, b in zip(dst.sets, src.sets):
        for name in a:
            a[name].copy_(b[name][lo:hi])
    dst.h0.copy_(src.h0[lo:hi])
    dst.w.copy_(src.w)
    dst.w_final.copy_(src.w_final)
    dst.set_rows(src.pos_rows[lo:hi].cpu(), src.kv_rows[lo:hi].cpu())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_half_shards_on_two_devices_equal_the_whole_batch(K):
    """The row partition on real devices: rows [0, n/2) on cuda:0 and [n/2, n) on cuda:1 against
    all n rows on cuda:0. Every bf16 output and the KV pool rows are bit-identical; the FP8 codes
    are identical where the shard's maximum equals the batch's, and otherwise decode to the same
    values within the two e4m3 grids. The cuda:1 shard, re-run on cuda:0, gives the same bits
    (same shard, same scale)."""
    from granite4_b200 import capi, glue
    rows, layers, pool = 4096, 2, 8192
    kvr = torch.randperm(pool, generator=torch.Generator().manual_seed(3))[:rows].to(torch.int32)
    pos = torch.randint(0, 8192, (rows,), generator=torch.Generator().manual_seed(4), dtype=torch.int32)
    whole = glue.GlueSequence(rows, device="cuda:0", seed=77, layers=layers, pool_rows=pool, max_pos=8192)
    whole.set_rows(pos, kvr)
    halves = []
    for i, device in enumerate(("cuda:0", "cuda:1", "cuda:0")):
        lo, hi = ((0, rows // 2), (rows // 2, rows), (rows // 2, rows))[i]
        part = glue.GlueSequence(rows // 2, device=device, seed=1, layers=layers, pool_rows=pool, max_pos=8192)
        _copy_shard(part, whole, lo, hi)
        halves.append((part, lo, hi))
    for seq in [whole] + [p for p, _, _ in halves]:
        seq.reset()
        seq.run_fast()
    for d in (0, 1):
        torch.cuda.synchronize(d)
        torch.cuda.set_device(d)
        assert capi.lib().device_status() == 0
    torch.cuda.set_device(0)
    for part, lo, hi in halves[:2]:
        for name in ("h", "out", "q_rot"):
            assert torch.equal(getattr(part, name).cpu(), getattr(whole, name)[lo:hi].cpu()), name
        mine = part.kv_rows.cpu().long()
        for name in ("cache_k", "cache_v", "k_scale", "v_scale"):
            assert torch.equal(getattr(part, name)[:, :, mine].cpu(), getattr(whole, name)[:, :, mine].cpu()), name
        for codes, slot in (("n_fp8", (layers - 1, 1)), ("act_fp8", (layers - 1, 2))):
            ps, ws = part.scales[slot].cpu(), whole.scales[slot].cpu()
            a, b = getattr(part, codes).cpu(), getattr(whole, codes)[lo:hi].cpu()
            if ps[1].item() == ws[1].item():
                assert torch.equal(a, b), codes
            else:
                fa = a.view(torch.float8_e4m3fn).float() * ps[0]
                fb = b.view(torch.float8_e4m3fn).float() * ws[0]
                assert ((fa - fb).abs() <= 0.126 * torch.maximum(fa.abs(), fb.abs()) + 2.0 ** -8 * ws[0]).all()
    # the same shard on the other device: the same bits, FP8 included
    other, same = halves[1][0], halves[2][0]
    for name in ("h", "out", "q_rot", "n_fp8", "act_fp8", "scales", "cache_k", "cache_v", "k_scale", "v_scale"):
        assert torch.equal(getattr(other, name).cpu(), getattr(same, name).cpu()), name
    shard_max = torch.maximum(halves[0][0].scales[..., 1].cpu(), other.scales[..., 1].cpu())
    assert torch.equal(shard_max, whole.scales[..., 1].cpu())  # batch maximum = max of the shards'
