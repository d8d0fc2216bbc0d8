"""The per-layer glue sequence of the Granite 4.2 8B forward over a shard of token rows.

This is the order in which the reference's prefill path calls the glue kernels
(``engine/src/forward_gpu.cu:2751-2863``), with the GEMMs and the attention between them
left out: their outputs are inputs here.

    embed (once)                                               a1
    per layer:  h += rm * y_attn ; n1 = norm(h) -> FP8          a2   (y_attn: O-projection output)
                RoPE(q, k) + int8 paged KV write from qkv       a3   (qkv: QKV GEMM output)
                h += rm * y_mlp  ; n2 = norm(h) -> FP8          a2   (y_mlp: down-projection output)
                act = SwiGLU(gate, up) -> FP8                   a4   (gate/up GEMM output)
    final norm of h -> bf16                                    a5

Rows are independent (the per-tensor FP8 scale is per launch, i.e. per shard), so several
GPUs each run this on their own rows with nothing exchanged.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import capi, kernels


@dataclass(frozen=True)
class GraniteShapes:
    """engine/src/model_config.h:18-25 (sizes), :35-42 (scalars; the multipliers are runtime
    arguments there and default to 1.0 - the values here are the benchmark configuration's)."""
    hidden: int = 4096
    intermediate: int = 12800
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    layers: int = 40
    vocab: int = 100352
    eps: float = 1e-5
    residual_multiplier: float = 0.22
    embedding_multiplier: float = 12.0
    rope_theta: float = 1e7

    @property
    def qkv_width(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim


# algorithmic bytes per token row of each kernel: every input read once, every output written
# once, per-launch tables and weights not counted
def bytes_per_row(s: GraniteShapes) -> dict:
    H, I, d = s.hidden, s.intermediate, s.head_dim
    q, kv = s.q_heads * d, s.kv_heads * d
    return {
        "embed": 4 + 2 * H + 2 * H,
        "add_rmsnorm_fp8": 2 * H + 2 * H + 2 * H + H,
        "rope_kv_int8": 2 * q + 2 * kv + 2 * kv + 2 * 4 * (d // 2) + 4 + 2 * q + 2 * kv + 2 * 4 * s.kv_heads,
        "swiglu_fp8": 2 * I + 2 * I + I,
        "final_norm": 2 * H + 2 * H,
    }


def bytes_per_token(s: GraniteShapes) -> int:
    b = bytes_per_row(s)
    return s.layers * (2 * b["add_rmsnorm_fp8"] + b["rope_kv_int8"] + b["swiglu_fp8"]) + b["final_norm"]


# kernels (not memsets) the sequence launches per layer and at the end
KERNELS_PER_LAYER = 2 * 2 + 1 + 2
KERNELS_FINAL = 1


class GlueSequence:
    """Device buffers for `rows` token rows and the calls that run the sequence over them.

    Inputs that stand for GEMM / attention outputs are filled with seeded N(0, 1) bf16 values;
    `sets` independent copies are rotated layer by layer so that no kernel finds its inputs in
    L2 from the previous layer even at small row counts.
    """

    def __init__(self, rows: int, shapes: GraniteShapes = GraniteShapes(), device="cuda",
                 seed: int = 0, sets: int = 2, layers: int | None = None, pool_rows: int | None = None,
                 max_pos: int | None = None, workspace: bool = True):
        s = self.shapes = shapes
        self.rows, self.device = rows, torch.device(device)
        self.layers = s.layers if layers is None else layers
        self.pool_rows = rows if pool_rows is None else pool_rows
        self.max_pos = max(rows, 1) if max_pos is None else max_pos
        g = torch.Generator(device=self.device).manual_seed(seed)
        bf = torch.bfloat16

        def randn(*shape):
            return torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32).to(bf)

        self.sets = []
        for _ in range(sets):
            self.sets.append({
                "y_attn": randn(rows, s.hidden), "y_mlp": randn(rows, s.hidden),
                "qkv": randn(rows, s.qkv_width),
                "gate": randn(rows, s.intermediate), "up": randn(rows, s.intermediate),
            })
        self.h0 = randn(rows, s.hidden)  # stands for the embedding output
        self.h = torch.empty_like(self.h0)
        # norm weights ~ N(1, 0.02): [layers][2][hidden] + final
        self.w = (1.0 + 0.02 * torch.randn(self.layers, 2, s.hidden, generator=g, device=self.device)).to(bf)
        self.w_final = (1.0 + 0.02 * torch.randn(s.hidden, generator=g, device=self.device)).to(bf)
        self.n_fp8 = torch.empty(rows, s.hidden, dtype=torch.uint8, device=self.device)
        self.q_rot = torch.empty(rows, s.q_heads * s.head_dim, dtype=bf, device=self.device)
        self.act_fp8 = torch.empty(rows, s.intermediate, dtype=torch.uint8, device=self.device)
        self.out = torch.empty(rows, s.hidden, dtype=bf, device=self.device)
        self.scales = torch.zeros(self.layers, 3, 2, dtype=torch.float32, device=self.device)
        # scratch the FP8 ops may use between their two sweeps: 1/rms per row, and the bf16
        # activation of SwiGLU (so the exponential is evaluated once). workspace=False runs the
        # same ops without any scratch (the second sweep then recomputes).
        self.workspace = workspace
        self.rstd = torch.empty(rows, dtype=torch.float32, device=self.device) if workspace else None
        self.act_ws = torch.empty(rows, s.intermediate, dtype=bf, device=self.device) if workspace else None
        # int8 paged pool per layer: codes [L][Hk][pool_rows][d], scales [L][Hk][pool_rows]
        self.cache_k = torch.zeros(self.layers, s.kv_heads, self.pool_rows, s.head_dim, dtype=torch.int8,
                                   device=self.device)
        self.cache_v = torch.zeros_like(self.cache_k)
        self.k_scale = torch.zeros(self.layers, s.kv_heads, self.pool_rows, dtype=torch.float32,
                                   device=self.device)
        self.v_scale = torch.zeros_like(self.k_scale)
        self.tables = kernels.RopeTables(s.rope_theta, s.head_dim, self.max_pos, self.device)
        # identity placement unless set_rows() says otherwise
        self.pos_rows = torch.arange(rows, dtype=torch.int32, device=self.device) % self.max_pos
        self.kv_rows = torch.arange(rows, dtype=torch.int32, device=self.device) % self.pool_rows
        self.launches = 0
        self._args = None

    def set_rows(self, pos_rows, kv_rows):
        self.pos_rows = torch.as_tensor(pos_rows, dtype=torch.int32).to(self.device)
        self.kv_rows = torch.as_tensor(kv_rows, dtype=torch.int32).to(self.device)
        self._args = None

    def reset(self):
        self.h.copy_(self.h0)

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} returned {rc}")

    def layer_ops(self, layer: int):
        """The four launcher calls of one layer as (name, thunk) pairs, in order."""
        s, k = self.shapes, kernels
        buf = self.sets[layer % len(self.sets)]
        ws = self.workspace
        return [
            ("add_rmsnorm_fp8", lambda: k.add_rmsnorm_fp8(
                buf["y_attn"], self.h, self.w[layer, 0], s.eps, s.residual_multiplier, h_out=self.h,
                n_fp8=self.n_fp8, scale_amax=self.scales[layer, 0], rstd=self.rstd if ws else None)),
            ("rope_kv_int8", lambda: k.rope_kv_int8_paged(
                buf["qkv"], self.tables.cos, self.tables.sin, self.pos_rows, self.kv_rows, s.q_heads,
                s.kv_heads, s.head_dim, self.pool_rows, self.max_pos, 0, self.q_rot, self.cache_k[layer],
                self.cache_v[layer], self.k_scale[layer], self.v_scale[layer])),
            ("add_rmsnorm_fp8", lambda: k.add_rmsnorm_fp8(
                buf["y_mlp"], self.h, self.w[layer, 1], s.eps, s.residual_multiplier, h_out=self.h,
                n_fp8=self.n_fp8, scale_amax=self.scales[layer, 1], rstd=self.rstd if ws else None)),
            ("swiglu_fp8", lambda: k.swiglu_fp8(
                buf["gate"], buf["up"], act_bf16=self.act_ws if ws else None, act_fp8=self.act_fp8,
                scale_amax=self.scales[layer, 2])),
        ]

    def final_op(self):
        s = self.shapes
        return ("final_norm", lambda: kernels.rmsnorm(self.h, self.w_final, s.eps, self.rows, s.hidden,
                                                      self.out))

    def _layer_args(self, layer: int) -> capi.GlueLayerArgs:
        s = self.shapes
        buf = self.sets[layer % len(self.sets)]
        a = capi.GlueLayerArgs()
        a.y_attn, a.y_mlp, a.qkv = buf["y_attn"].data_ptr(), buf["y_mlp"].data_ptr(), buf["qkv"].data_ptr()
        a.gate, a.up = buf["gate"].data_ptr(), buf["up"].data_ptr()
        a.w_attn_norm, a.w_mlp_norm = self.w[layer, 0].data_ptr(), self.w[layer, 1].data_ptr()
        a.cos_tbl, a.sin_tbl = self.tables.cos_ptr, self.tables.sin_ptr
        a.pos_rows, a.kv_rows = self.pos_rows.data_ptr(), self.kv_rows.data_ptr()
        a.hidden, a.n_attn_fp8, a.n_mlp_fp8 = self.h.data_ptr(), self.n_fp8.data_ptr(), self.n_fp8.data_ptr()
        a.q_rot, a.act_fp8 = self.q_rot.data_ptr(), self.act_fp8.data_ptr()
        a.cache_k, a.cache_v = self.cache_k[layer].data_ptr(), self.cache_v[layer].data_ptr()
        a.k_scale, a.v_scale = self.k_scale[layer].data_ptr(), self.v_scale[layer].data_ptr()
        a.scales = self.scales[layer].data_ptr()
        a.rstd = self.rstd.data_ptr() if self.workspace else None
        a.act_ws = self.act_ws.data_ptr() if self.workspace else None
        a.rows, a.hidden_size, a.intermediate = self.rows, s.hidden, s.intermediate
        a.q_heads, a.kv_heads, a.head_dim = s.q_heads, s.kv_heads, s.head_dim
        a.pool_rows, a.max_pos, a.eps, a.resid_mult = self.pool_rows, self.max_pos, s.eps, s.residual_multiplier
        return a

    def run_fast(self):
        """The same step with one library call per layer (granite4_glue_layer): identical
        launches, a fraction of the host time. Argument blocks are built once and reused."""
        lib = capi.lib()
        if self._args is None:
            self._args = [self._layer_args(layer) for layer in range(self.layers)]
            self._arg_refs = [C.byref(a) for a in self._args]
        torch.cuda.set_device(self.device)
        lib.granite4_b200_set_stream(torch.cuda.current_stream(self.device).cuda_stream)
        for ref in self._arg_refs:
            self._check(lib.granite4_glue_layer(ref), "granite4_glue_layer")
        self.launches += self.layers * KERNELS_PER_LAYER
        name, thunk = self.final_op()
        self._check(thunk(), name)
        self.launches += KERNELS_FINAL

    def fingerprint(self, sample_rows: int = 64) -> torch.Tensor:
        """Everything a finished step left behind, condensed into one uint8 tensor whose length
        depends only on the shapes: the integer sums of the bit patterns of every output buffer
        over ALL rows (hidden state, final norm, FP8 codes, q_rot, the int8 pool and its scales of
        every layer, every {scale, amax} slot), followed by the raw bits of `sample_rows` evenly
        spaced rows of the row-shaped outputs and of their K/V pool rows in the first and last
        layer. Two runs of the same shard agree on it bit for bit; ranks exchange it after a timed
        region to be compared with an independent re-run."""
        def total(t):
            flat = t.reshape(-1)
            if flat.element_size() == 2:
                flat = flat.view(torch.int16)
            elif flat.element_size() == 4:
                flat = flat.view(torch.int32)
            return flat.sum(dtype=torch.int64).reshape(1)
        sums = [total(t) for t in (self.h, self.out, self.n_fp8, self.act_fp8, self.q_rot, self.cache_k,
                                   self.cache_v, self.k_scale, self.v_scale, self.scales)]
        k = max(1, min(sample_rows, self.rows))
        pick = torch.arange(k, device=self.device) * (self.rows // k)
        pool = self.kv_rows[pick].long()
        parts = [torch.cat(sums).view(torch.uint8), self.scales.reshape(-1).view(torch.uint8)]
        for t in (self.h, self.out, self.n_fp8, self.act_fp8, self.q_rot):
            parts.append(t[pick].reshape(-1).view(torch.uint8))
        for layer in sorted({0, self.layers - 1}):
            for t in (self.cache_k, self.cache_v, self.k_scale, self.v_scale):
                parts.append(t[layer][:, pool].contiguous().reshape(-1).view(torch.uint8))
        return torch.cat(parts)

    def run(self, wrap=None):
        """One step: all layers, then the final norm. Enqueues only; does not synchronise.
        `wrap(name, thunk)` may run the thunk itself (e.g. between two events) and must return
        its status code."""
        for layer in range(self.layers):
            for name, thunk in self.layer_ops(layer):
                self._check(wrap(name, thunk) if wrap else thunk(), name)
            self.launches += KERNELS_PER_LAYER
        name, thunk = self.final_op()
        self._check(wrap(name, thunk) if wrap else thunk(), name)
        self.launches += KERNELS_FINAL


class HostGlue:
    """The layer glue over HOST buffers (granite4_host_glue_*): the library stages pinned host
    tensors through device memory it owns, overlapping the copies of one layer call with the
    kernels and the read-back of the previous one. The residual stream and the int8 KV pool
    stay on the device between calls."""

    def __init__(self, max_rows: int, shapes: GraniteShapes = GraniteShapes(), device="cuda",
                 layers: int | None = None, pool_rows: int | None = None, max_pos: int | None = None):
        self.shapes, self.max_rows = shapes, max_rows
        self.device = torch.device(device)
        self.layers = shapes.layers if layers is None else layers
        self.pool_rows = max_rows if pool_rows is None else pool_rows
        self.max_pos = max_rows if max_pos is None else max_pos
        torch.cuda.set_device(self.device)
        self._lib = capi.lib()
        self._ctx = self._lib.granite4_host_glue_create(
            max_rows, shapes.hidden, shapes.intermediate, shapes.q_heads, shapes.kv_heads, shapes.head_dim,
            self.layers, self.pool_rows, self.max_pos, shapes.rope_theta)
        if not self._ctx:
            raise RuntimeError("granite4_host_glue_create failed")

    def h2d_bytes(self, rows):
        return self._lib.granite4_host_glue_h2d_bytes(self._ctx, rows)

    def d2h_bytes(self, rows):
        return self._lib.granite4_host_glue_d2h_bytes(self._ctx, rows)

    def layer(self, layer: int, io: "capi.HostLayerIO"):
        rc = self._lib.granite4_host_glue_layer(self._ctx, layer, C.byref(io))
        if rc != 0:
            raise RuntimeError(f"granite4_host_glue_layer returned {rc}")

    def final_norm(self, w_host, eps, rows, out_host):
        rc = self._lib.granite4_host_glue_final_norm(self._ctx, w_host.data_ptr(), eps, rows,
                                                     out_host.data_ptr())
        if rc != 0:
            raise RuntimeError(f"granite4_host_glue_final_norm returned {rc}")

    def sync(self):
        if self._lib.granite4_host_glue_sync(self._ctx) != 0:
            raise RuntimeError("granite4_host_glue_sync failed")

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.granite4_host_glue_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def host_layer_io(tensors: dict, rows: int, eps: float, resid_mult: float) -> "capi.HostLayerIO":
    """Fill a HostLayerIO from CPU tensors (pinned for asynchronous copies). Keys are the struct's
    pointer fields; hidden_in / hidden_out may be absent."""
    io = capi.HostLayerIO()
    for name, _ in capi.HostLayerIO._fields_:
        if name in ("rows", "eps", "resid_mult"):
            continue
        t = tensors.get(name)
        if t is not None:
            if t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name}: expected a contiguous CPU tensor")
            setattr(io, name, t.data_ptr())
    io.rows, io.eps, io.resid_mult = rows, eps, resid_mult
    return io
