"""Host-side mirror of the reference engine's launch interface for the layer glue kernels.

Same names, argument order and return convention (0 / -1) as the reference's launchers
(``engine/src/prefill_gemm.h``, ``engine/src/kernels_phase2.cu``, ``engine/src/forward_gpu_api.h``),
over PyTorch CUDA tensors: torch only provides device memory and the stream, every
computation happens in the library's own kernels. bf16 tensors may be passed as
``torch.bfloat16`` or as ``torch.uint16``/``int16`` bit patterns; FP8 outputs are ``uint8``.

Each call launches on torch's current stream of the tensor's device.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi

_BF16_OK = (torch.bfloat16, torch.uint16, torch.int16)


def _p(t, *dtypes):
    """Device pointer of a contiguous CUDA tensor (None passes through)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("expected a CUDA tensor: these kernels have no CPU path")
    if not t.is_contiguous():
        raise ValueError("expected a contiguous tensor")
    if dtypes and t.dtype not in dtypes:
        raise TypeError(f"unexpected dtype {t.dtype}, wanted one of {dtypes}")
    return t.data_ptr()


def _enter(t):
    """Select the tensor's device and torch's current stream on it for the launch."""
    lib = capi.lib()
    torch.cuda.set_device(t.device)
    lib.granite4_b200_set_stream(torch.cuda.current_stream(t.device).cuda_stream)
    return lib


# ---- a1 ---------------------------------------------------------------------------------
def prefill_embed_rows(d_tokens, start, rows, emb, mult, out):
    """engine/src/prefill_gemm.h:42-43. out[r] = bf16(mult * emb[d_tokens[start + r]])."""
    lib = _enter(emb)
    return lib.granite4_prefill_embed_rows(_p(d_tokens, torch.int32), start, rows, _p(emb, *_BF16_OK),
                                           mult, _p(out, *_BF16_OK), emb.shape[-1])


def embed_gather(d_tokens, emb, mult, out):
    """granite4_kernel_embed_gather: no 65535-row limit, out-of-vocabulary ids give zero rows."""
    lib = _enter(emb)
    return lib.granite4_kernel_embed_gather(_p(d_tokens, torch.int32), d_tokens.numel(),
                                            _p(emb, *_BF16_OK), emb.shape[0], mult,
                                            _p(out, *_BF16_OK), emb.shape[1])


# ---- a2 / a5 ------------------------------------------------------------------------------
def rmsnorm(d_x, d_w, eps, rows, cols, d_out, batched=False):
    """engine/src/kernels_phase2.cu:910-936 (granite4_kernel_rmsnorm[_batched])."""
    lib = _enter(d_x)
    fn = lib.granite4_kernel_rmsnorm_batched if batched else lib.granite4_kernel_rmsnorm
    return fn(_p(d_x, *_BF16_OK), _p(d_w, *_BF16_OK), eps, rows, cols, _p(d_out, *_BF16_OK))


def add_rmsnorm_fp8(y, res, w, eps, resid_mult, h_out=None, n_bf16=None, n_fp8=None,
                    scale_amax=None, rstd=None):
    """granite4_kernel_add_rmsnorm_fp8. y / res: bf16 or float32 [rows][cols]; res may be None.
    scale_amax: float32[2] receiving {scale, amax} when n_fp8 is given. rstd: optional
    float32[rows], receives 1/rms of every row and lets the FP8 sweep skip the reduction."""
    lib = _enter(y)
    rows, cols = y.shape
    return lib.granite4_kernel_add_rmsnorm_fp8(
        _p(y), int(y.dtype == torch.float32), _p(res), int(res is not None and res.dtype == torch.float32),
        _p(w, *_BF16_OK), eps, resid_mult, rows, cols, _p(h_out, *_BF16_OK), _p(n_bf16, *_BF16_OK),
        _p(n_fp8, torch.uint8), _p(scale_amax, torch.float32), _p(rstd, torch.float32))


def add_rmsnorm_fp8_noalloc(y, res, w, eps, resid_mult, h_out, n_fp8, scale_amax):
    """granite4_kernel_add_rmsnorm_fp8_noalloc: the op for callers that cannot allocate device
    memory; its per-row scratch is a fixed array inside the library (at most 65536 rows)."""
    lib = _enter(y)
    rows, cols = y.shape
    return lib.granite4_kernel_add_rmsnorm_fp8_noalloc(
        _p(y), int(y.dtype == torch.float32), _p(res), int(res is not None and res.dtype == torch.float32),
        _p(w, *_BF16_OK), eps, resid_mult, rows, cols, _p(h_out, *_BF16_OK), _p(n_fp8, torch.uint8),
        _p(scale_amax, torch.float32))


def fp8_quant(x, codes, scale_amax):
    """granite4_kernel_fp8_quant: per-tensor e4m3 of a bf16 tensor."""
    lib = _enter(x)
    return lib.granite4_kernel_fp8_quant(_p(x, *_BF16_OK), x.numel(), _p(codes, torch.uint8),
                                         _p(scale_amax, torch.float32))


# ---- a3 -----------------------------------------------------------------------------------
class _DevArray:
    """Zero-copy view of raw device memory for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False),
                                         "version": 2}


class RopeTables:
    """Device cos/sin tables built by granite4_rope_tables_build, which allocates them with
    cudaMalloc as the reference's does. `cos` / `sin` are float32 [max_pos][head_dim/2] views
    of that memory; close() (or collection) frees it through granite4_b200_free."""

    def __init__(self, theta, head_dim, max_pos, device=None):
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        torch.cuda.set_device(device)
        self._lib = capi.lib()
        c, s = C.c_void_p(), C.c_void_p()
        rc = self._lib.granite4_rope_tables_build(theta, head_dim, max_pos, C.byref(c), C.byref(s))
        if rc != 0:
            raise RuntimeError("granite4_rope_tables_build failed")
        self.device, self.max_pos, self.half = device, max_pos, head_dim // 2
        self.cos_ptr, self.sin_ptr = c.value, s.value
        shape = (max_pos, self.half)
        self.cos = torch.as_tensor(_DevArray(self.cos_ptr, shape, "<f4"), device=device)
        self.sin = torch.as_tensor(_DevArray(self.sin_ptr, shape, "<f4"), device=device)

    def close(self):
        if getattr(self, "cos_ptr", None):
            self.cos = self.sin = None
            self._lib.granite4_b200_free(self.cos_ptr)
            self._lib.granite4_b200_free(self.sin_ptr)
            self.cos_ptr = self.sin_ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _tbl(t):
    return t if isinstance(t, int) else _p(t, torch.float32)


def rope(d_x, d_cos, d_sin, rows, head_dim, d_out):
    """engine/src/kernels_phase2.cu:938-951 (granite4_kernel_rope)."""
    lib = _enter(d_x)
    return lib.granite4_kernel_rope(_p(d_x, *_BF16_OK), _tbl(d_cos), _tbl(d_sin), rows, head_dim,
                                    _p(d_out, *_BF16_OK))


def kv_append_int8_batched(d_src_k, d_src_v, d_cache_k, d_cache_v, d_cache_k_scale,
                           d_cache_v_scale, base_pos, rows, stride, Hk, d, d_pt=None):
    """engine/src/kernels_phase2.cu:1107-1131."""
    lib = _enter(d_src_k)
    return lib.granite4_kernel_kv_append_int8_batched(
        _p(d_src_k, *_BF16_OK), _p(d_src_v, *_BF16_OK), _p(d_cache_k, torch.int8),
        _p(d_cache_v, torch.int8), _p(d_cache_k_scale, torch.float32),
        _p(d_cache_v_scale, torch.float32), base_pos, rows, stride, Hk, d, _p(d_pt, torch.int32))


def prefill_rope_split_append_int8(qkv, cos_tbl, sin_tbl, base_pos, rows, Hq, Hk, d, stride, q_rot,
                                   cache_k, cache_v, cache_k_scale, cache_v_scale, d_pt=None):
    """engine/src/prefill_gemm.h:58-64."""
    lib = _enter(qkv)
    return lib.granite4_prefill_rope_split_append_int8(
        _p(qkv, *_BF16_OK), _tbl(cos_tbl), _tbl(sin_tbl), base_pos, rows, Hq, Hk, d, stride,
        _p(q_rot, *_BF16_OK), _p(cache_k, torch.int8), _p(cache_v, torch.int8),
        _p(cache_k_scale, torch.float32), _p(cache_v_scale, torch.float32), _p(d_pt, torch.int32))


def gpu_multi_rope_append(q, k, v, cos_tbl, sin_tbl, d_rows, rows, Hq, Hk, d, bits, cache_k, cache_v,
                          k_scale, v_scale, stride, q_rot):
    """engine/src/forward_gpu_api.h:224-227. d_rows: uint8 CUDA tensor holding a MultiRows."""
    lib = _enter(q)
    return lib.granite4_gpu_multi_rope_append(
        _p(q, *_BF16_OK), _p(k, *_BF16_OK), _p(v, *_BF16_OK), _tbl(cos_tbl), _tbl(sin_tbl), _p(d_rows),
        rows, Hq, Hk, d, bits, _p(cache_k), _p(cache_v), _p(k_scale, torch.float32),
        _p(v_scale, torch.float32), stride, _p(q_rot, *_BF16_OK))


def gpu_multi_rope(x, cos_tbl, sin_tbl, d_rows, rows, heads, d, out):
    """engine/src/forward_gpu_api.h:219-220: row r rotated at position d_rows.pos[r]."""
    lib = _enter(x)
    return lib.granite4_gpu_multi_rope(_p(x, *_BF16_OK), _tbl(cos_tbl), _tbl(sin_tbl), _p(d_rows), rows,
                                       heads, d, _p(out, *_BF16_OK))


def gpu_multi_kv_append(k, v, bits, cache_k, cache_v, k_scale, v_scale, d_rows, rows, stride, Hk, d):
    """engine/src/forward_gpu_api.h:227-229: bits 8 (int8 + scales) or 16 (bf16 copy)."""
    lib = _enter(k)
    return lib.granite4_gpu_multi_kv_append(
        _p(k, *_BF16_OK), _p(v, *_BF16_OK), bits, _p(cache_k), _p(cache_v),
        _p(k_scale, torch.float32), _p(v_scale, torch.float32), _p(d_rows), rows, stride, Hk, d)


def rope_at_pos(d_x, d_cos_row, d_sin_row, heads, d, d_out):
    """engine/src/forward_gpu.cu:3814-3826: one position; the table pointers are that position's
    row (pass e.g. ``tables.cos[pos]`` of a float32 tensor, or an integer device address)."""
    lib = _enter(d_x)
    return lib.granite4_kernel_rope_at_pos(_p(d_x, *_BF16_OK), _tbl(d_cos_row), _tbl(d_sin_row), heads,
                                           d, _p(d_out, *_BF16_OK))


def rope_at_pos_batched(d_x, d_cos_rows, d_sin_rows, rows, heads, d, d_out):
    """engine/src/forward_gpu.cu:3828-3842: row r uses row r of the table pointers."""
    lib = _enter(d_x)
    return lib.granite4_kernel_rope_at_pos_batched(_p(d_x, *_BF16_OK), _tbl(d_cos_rows),
                                                   _tbl(d_sin_rows), rows, heads, d,
                                                   _p(d_out, *_BF16_OK))


def kv_append_batched(d_src_k, d_src_v, d_cache_k, d_cache_v, base_pos, rows, stride, Hk, d,
                      d_pt=None):
    """engine/src/kernels_phase2.cu:1087-1105: bf16 cache append of rows <= 16."""
    lib = _enter(d_src_k)
    return lib.granite4_kernel_kv_append_batched(
        _p(d_src_k, *_BF16_OK), _p(d_src_v, *_BF16_OK), _p(d_cache_k, *_BF16_OK),
        _p(d_cache_v, *_BF16_OK), base_pos, rows, stride, Hk, d, _p(d_pt, torch.int32))


def verify_qkv_stage(d_q, d_k, d_v, d_cos_rows, d_sin_rows, base_pos, rows, Hq, Hk, d, cache_stride,
                     d_q_rot, d_k_rot, d_cache_k, d_cache_v, d_pt=None):
    """engine/src/forward_gpu.cu:3847-3874: RoPE q and k, append rotated k and raw v (bf16)."""
    lib = _enter(d_q)
    return lib.granite4_kernel_verify_qkv_stage(
        _p(d_q, *_BF16_OK), _p(d_k, *_BF16_OK), _p(d_v, *_BF16_OK), _tbl(d_cos_rows),
        _tbl(d_sin_rows), base_pos, rows, Hq, Hk, d, cache_stride, _p(d_q_rot, *_BF16_OK),
        _p(d_k_rot, *_BF16_OK), _p(d_cache_k, *_BF16_OK), _p(d_cache_v, *_BF16_OK),
        _p(d_pt, torch.int32))


def prefill_rope_split_append(qkv, cos_tbl, sin_tbl, base_pos, rows, Hq, Hk, d, stride, q_rot,
                              cache_k, cache_v, d_pt=None):
    """engine/src/prefill_gemm.h:48-52: the prefill step for a bf16 cache."""
    lib = _enter(qkv)
    return lib.granite4_prefill_rope_split_append(
        _p(qkv, *_BF16_OK), _tbl(cos_tbl), _tbl(sin_tbl), base_pos, rows, Hq, Hk, d, stride,
        _p(q_rot, *_BF16_OK), _p(cache_k, *_BF16_OK), _p(cache_v, *_BF16_OK), _p(d_pt, torch.int32))


def multi_rows_to_device(desc: capi.MultiRows, device):
    """Upload a MultiRows descriptor; returns a uint8 CUDA tensor to pass as d_rows."""
    raw = bytes(desc)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)


def rope_kv_int8_paged(qkv, cos_tbl, sin_tbl, pos_rows, kv_rows, Hq, Hk, d, stride, max_pos,
                       k_from_bf16, q_rot, cache_k, cache_v, k_scale, v_scale):
    """granite4_kernel_rope_kv_int8_paged: per-row RoPE positions and pool rows."""
    lib = _enter(qkv)
    return lib.granite4_kernel_rope_kv_int8_paged(
        _p(qkv, *_BF16_OK), _tbl(cos_tbl), _tbl(sin_tbl), _p(pos_rows, torch.int32),
        _p(kv_rows, torch.int32), qkv.shape[0], Hq, Hk, d, stride, max_pos, int(k_from_bf16),
        _p(q_rot, *_BF16_OK), _p(cache_k, torch.int8), _p(cache_v, torch.int8),
        _p(k_scale, torch.float32), _p(v_scale, torch.float32))


# ---- decode-step glue -----------------------------------------------------------------------
def argmax_rows(logits, out, d_pos=None, vocab_map=None):
    """granite4_kernel_argmax_rows: first index of each row's maximum of bf16 logits [rows][V]."""
    lib = _enter(logits)
    rows, V = logits.shape
    return lib.granite4_kernel_argmax_rows(_p(logits, *_BF16_OK), rows, V, _p(out, torch.int32),
                                           _p(d_pos, torch.int32), _p(vocab_map, torch.int32))


def argmax_advance(logits, d_rows, ids_out=None):
    """granite4_kernel_argmax_advance: greedy pick + token scatter / position advance in one launch."""
    lib = _enter(logits)
    rows, V = logits.shape
    return lib.granite4_kernel_argmax_advance(_p(logits, *_BF16_OK), rows, V, _p(d_rows), _p(ids_out, torch.int32))


def gpu_multi_embed(d_rows, rows, emb, mult, out):
    """granite4_gpu_multi_embed: out[r] = bf16(mult * emb[token of row r at its slot])."""
    lib = _enter(emb)
    return lib.granite4_gpu_multi_embed(_p(d_rows), rows, _p(emb, *_BF16_OK), emb.shape[0], mult,
                                        _p(out, *_BF16_OK), emb.shape[1])


def multi_scatter_advance(d_rows, ids):
    """granite4_kernel_multi_scatter_advance: d_rows is the uint8 tensor holding a MultiRows."""
    lib = _enter(ids)
    return lib.granite4_kernel_multi_scatter_advance(_p(d_rows), _p(ids, torch.int32))


def kv_move(src_rows, dst_rows, bits, cache_k, cache_v, k_scale, v_scale, layers, Hk, stride, d):
    """granite4_kernel_kv_move: src_rows / dst_rows are host sequences of physical pool rows."""
    lib = _enter(cache_k)
    n = len(src_rows)
    arr = C.c_int * max(n, 1)
    return lib.granite4_kernel_kv_move(arr(*src_rows), arr(*dst_rows), n, bits, _p(cache_k), _p(cache_v),
                                       _p(k_scale, torch.float32), _p(v_scale, torch.float32), layers,
                                       Hk, stride, d)


def attn_decode_scratch_bytes(rows, rows_per_group, Hk, max_len):
    return capi.lib().granite4_attn_decode_scratch_bytes(rows, rows_per_group, Hk, max_len)


def attn_decode_int8_paged(q, cache_k, cache_v, k_scale, v_scale, row_pos, Hq, Hk, d, stride, max_len,
                           scale, out, rows_per_group=1, row_pt=None, pt=None, scratch=None):
    """granite4_kernel_attn_decode_int8_paged. row_pt: int64 CUDA tensor of per-row table addresses
    (``table.data_ptr()`` values), pt: one int32 table for every row; scratch: uint8 CUDA tensor of
    at least attn_decode_scratch_bytes(...) bytes (allocated here when not given)."""
    lib = _enter(q)
    rows = q.shape[0]
    need = lib.granite4_attn_decode_scratch_bytes(rows, rows_per_group, Hk, max_len)
    if scratch is None and need > 0:
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    return lib.granite4_kernel_attn_decode_int8_paged(
        _p(q, *_BF16_OK), _p(cache_k, torch.int8), _p(cache_v, torch.int8), _p(k_scale, torch.float32),
        _p(v_scale, torch.float32), _p(row_pos, torch.int32), _p(row_pt, torch.int64),
        _p(pt, torch.int32), rows, rows_per_group, Hq, Hk, d, stride, max_len, scale,
        _p(scratch, torch.uint8), 0 if scratch is None else scratch.numel(), _p(out, *_BF16_OK))


def attn_split_int8(q, cache_k, cache_v, k_scale, v_scale, scale, Hq, Hk, d, stride, out, kv_base=0, d_pos=None,
                    pt=None, max_len=0, row_pos=None, row_pt=None, row_grp=None, row_tbase=None, row_tail=None,
                    window=0, scratch=None):
    """granite4_attn_split_int8: the reference's attn_split contract (engine/src/attention_gpu.h:39-68)
    over the int8 pool. row_pt: int64 CUDA tensor of per-row table addresses; row_grp: int32 group
    words r0 | nr << 8; row_tbase int32 [rows], row_tail int32 [rows][8]."""
    lib = _enter(q)
    rows = q.shape[0]
    need = lib.granite4_attn_split_scratch_bytes(Hq, rows, max_len if max_len > 0 else stride)
    if scratch is None:
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    return lib.granite4_attn_split_int8(
        _p(q, *_BF16_OK), _p(cache_k, torch.int8), _p(cache_v, torch.int8), _p(k_scale, torch.float32),
        _p(v_scale, torch.float32), scale, Hq, Hk, d, kv_base, _p(d_pos, torch.int32), rows, stride,
        _p(scratch, torch.uint8), scratch.numel(), _p(out, *_BF16_OK), _p(pt, torch.int32), max_len,
        _p(row_pos, torch.int32), _p(row_pt, torch.int64), _p(row_grp, torch.int32),
        0 if row_grp is None else row_grp.numel(), _p(row_tbase, torch.int32), _p(row_tail, torch.int32), window)


def prefill_attention_int8(q_rot, scale, Hq, Hk, d, base_pos, stride, out, cache_k, cache_v, k_scale, v_scale,
                           pt=None, scratch=None):
    """granite4_prefill_attention_int8 (engine/src/prefill_gemm.h:86-101 with the int8 cache): causal
    attention of q_rot's rows at positions base_pos, base_pos + 1, ... of one sequence."""
    lib = _enter(q_rot)
    return lib.granite4_prefill_attention_int8(
        _p(q_rot, *_BF16_OK), scale, Hq, Hk, d, base_pos, q_rot.shape[0], stride, _p(out, *_BF16_OK),
        _p(cache_k, torch.int8), _p(cache_v, torch.int8), _p(k_scale, torch.float32), _p(v_scale, torch.float32),
        _p(pt, torch.int32), _p(scratch, torch.uint8), 0 if scratch is None else scratch.numel())


# ---- FP8 x FP8 GEMM -----------------------------------------------------------------------
def gemm_fp8_workspace(M, N, K, device):
    """A zeroed workspace that lets gemm_fp8 split K for an M x N x K GEMM (None: no split wanted)."""
    need = capi.lib().granite4_gemm_fp8_workspace_bytes(M, N, K)
    return torch.zeros(need, dtype=torch.uint8, device=device) if need > 0 else None


def fp8_encode_with_amax(x, codes, scale_amax):
    """granite4_kernel_fp8_encode_with_amax: codes of a bf16 tensor whose max |x| is already in
    scale_amax[1] (the fused SwiGLU epilogue of gemm_fp8 leaves it there)."""
    lib = _enter(x)
    return lib.granite4_kernel_fp8_encode_with_amax(_p(x, *_BF16_OK), x.numel(), _p(codes, torch.uint8),
                                                    _p(scale_amax, torch.float32))


def gemm_fp8(a_fp8, w_fp8, out, a_scale=None, w_scales=(1.0,), segs=(), residual=None, resid_scale=1.0,
             workspace=None, swiglu_scale_amax=None):
    """granite4_kernel_gemm_fp8: out[M][N] = a_scale * w_scale(n) * a_fp8[M][K] x w_fp8[N][K]^T.
    a_fp8 / w_fp8: uint8 e4m3 codes (a_fp8 may be a row-strided view); a_scale: float32 CUDA tensor
    whose element 0 is the activation scale; w_scales: up to three per-segment weight scales with
    the segment ends in segs; out: bf16 or float32 [M][N] (row-strided allowed); residual: bf16,
    same pitch as out (GemmOut::kResidual, engine/src/prefill_gemm.h:12-16). workspace: uint8 CUDA
    tensor from gemm_fp8_workspace (zeroed once; reusable call after call). swiglu_scale_amax: float32[2];
    when given, w_fp8 is gate rows then up rows and out [M][N / 2] gets bf16(silu(gate) * up), its
    max |.| going to swiglu_scale_amax[1] (GRANITE4_GEMM_OUT_SWIGLU)."""
    lib = _enter(a_fp8)
    M, K = a_fp8.shape
    N = w_fp8.shape[0]
    ws = list(w_scales) + [w_scales[-1]] * (3 - len(w_scales))
    sg = list(segs) + [2 ** 31 - 1] * (2 - len(segs))
    ep = capi.GemmFp8Epilogue()
    ep.d_a_scale = _p(a_scale, torch.float32)
    ep.w_scale0, ep.w_scale1, ep.w_scale2 = ws
    ep.seg1, ep.seg2 = sg
    ep.resid_scale = resid_scale
    ep.ldc = out.stride(0)
    if swiglu_scale_amax is not None:
        kind, ep.d_out_bf16 = capi.GEMM_OUT_SWIGLU, out.data_ptr()
        ep.d_out_scale_amax = _p(swiglu_scale_amax, torch.float32)
    elif out.dtype == torch.float32:
        kind, ep.d_out_f32 = capi.GEMM_OUT_F32, out.data_ptr()
    else:
        kind = capi.GEMM_OUT_BF16 if residual is None else capi.GEMM_OUT_RESIDUAL
        ep.d_out_bf16 = out.data_ptr()
        if residual is not None:
            if residual.stride(0) != out.stride(0):
                raise ValueError("the residual must have the output's row pitch")
            ep.d_residual = residual.data_ptr()
    if w_fp8.dtype != torch.uint8 or a_fp8.dtype != torch.uint8 or not w_fp8.is_contiguous() or a_fp8.stride(1) != 1:
        raise ValueError("a_fp8 / w_fp8 must be uint8 code matrices with unit column stride")
    return lib.granite4_kernel_gemm_fp8(kind, a_fp8.data_ptr(), a_fp8.stride(0), w_fp8.data_ptr(), M, N, K,
                                        C.byref(ep), _p(workspace, torch.uint8),
                                        0 if workspace is None else workspace.numel())


# ---- a4 -----------------------------------------------------------------------------------
def prefill_silu_mul(gu, I, rows, act):
    """engine/src/prefill_gemm.h:105: gu float32 [rows][2 I] -> act bf16 [rows][I]."""
    lib = _enter(gu)
    return lib.granite4_prefill_silu_mul(_p(gu, torch.float32), I, rows, _p(act, *_BF16_OK))


def swiglu_fp8(gate, up, act_bf16=None, act_fp8=None, scale_amax=None, ld=None):
    """granite4_kernel_swiglu_fp8. gate / up: [rows][I] bf16 or float32; they may be column
    views of one [rows][2 I] buffer (pass ld = 2 I; contiguity is then not checked)."""
    lib = capi.lib()
    torch.cuda.set_device(gate.device)
    lib.granite4_b200_set_stream(torch.cuda.current_stream(gate.device).cuda_stream)
    rows, I = gate.shape
    if ld is None:
        ld = gate.stride(0)
    return lib.granite4_kernel_swiglu_fp8(gate.data_ptr(), up.data_ptr(),
                                          int(gate.dtype == torch.float32), ld, rows, I,
                                          _p(act_bf16, *_BF16_OK), _p(act_fp8, torch.uint8),
                                          _p(scale_amax, torch.float32))
