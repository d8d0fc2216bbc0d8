"""ctypes binding of libgranite4_b200.so: one Python callable per C-ABI entry point.

The signatures are the ones declared in ``include/granite4_b200.h``; device pointers are
passed as integers (``tensor.data_ptr()``) or ``None``. There is no fallback of any kind:
if the shared library is missing, loading raises, and every wrapper returns the entry
point's own status code (0 / -1) exactly as a C caller would see it.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_vp = C.c_void_p

# name -> (restype, argtypes); must list every function include/granite4_b200.h declares
SIGNATURES = {
    "granite4_get_model_info": (None, [_vp]),
    "granite4_status": (None, [_vp]),
    "granite4_b200_set_stream": (C.c_int, [_vp]),
    "granite4_b200_device_status": (C.c_int, [C.POINTER(C.c_uint)]),
    "granite4_b200_free": (C.c_int, [_vp]),
    "granite4_prefill_embed_rows": (C.c_int, [_vp, C.c_int, C.c_int, _vp, C.c_float, _vp, C.c_int]),
    "granite4_kernel_embed_gather": (C.c_int, [_vp, C.c_longlong, _vp, C.c_int, C.c_float, _vp,
                                               C.c_int]),
    "granite4_kernel_rmsnorm": (C.c_int, [_vp, _vp, C.c_float, C.c_int, C.c_int, _vp]),
    "granite4_kernel_rmsnorm_batched": (C.c_int, [_vp, _vp, C.c_float, C.c_int, C.c_int, _vp]),
    "granite4_kernel_add_rmsnorm_fp8": (C.c_int, [_vp, C.c_int, _vp, C.c_int, _vp, C.c_float,
                                                  C.c_float, C.c_int, C.c_int, _vp, _vp, _vp, _vp,
                                                  _vp]),
    "granite4_kernel_add_rmsnorm_fp8_noalloc": (C.c_int, [_vp, C.c_int, _vp, C.c_int, _vp, C.c_float,
                                                          C.c_float, C.c_int, C.c_int, _vp, _vp, _vp]),
    "granite4_kernel_fp8_quant": (C.c_int, [_vp, C.c_longlong, _vp, _vp]),
    "granite4_rope_tables_build": (C.c_int, [C.c_double, C.c_int, C.c_int, C.POINTER(_vp),
                                             C.POINTER(_vp)]),
    "granite4_kernel_rope": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, _vp]),
    "granite4_kernel_kv_append_int8_batched": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_int,
                                                         C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "granite4_prefill_rope_split_append_int8": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int,
                                                          C.c_int, C.c_int, C.c_int, _vp, _vp, _vp,
                                                          _vp, _vp, _vp]),
    "granite4_gpu_multi_rope_append": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int,
                                                 C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp,
                                                 C.c_int, _vp]),
    "granite4_gpu_multi_rope": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "granite4_gpu_multi_kv_append": (C.c_int, [_vp, _vp, C.c_int, _vp, _vp, _vp, _vp, _vp, C.c_int,
                                               C.c_int, C.c_int, C.c_int]),
    "granite4_kernel_rope_at_pos": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, _vp]),
    "granite4_kernel_rope_at_pos_batched": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "granite4_kernel_kv_append_batched": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int,
                                                    C.c_int, C.c_int, _vp]),
    "granite4_kernel_verify_qkv_stage": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int,
                                                   C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp,
                                                   _vp]),
    "granite4_prefill_rope_split_append": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int,
                                                     C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp]),
    "granite4_kernel_rope_kv_int8_paged": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int,
                                                     C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                     _vp, _vp, _vp, _vp, _vp]),
    "granite4_kernel_argmax_rows": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp, _vp]),
    "granite4_kernel_multi_scatter_advance": (C.c_int, [_vp, _vp]),
    "granite4_kernel_argmax_advance": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp]),
    "granite4_gpu_multi_embed": (C.c_int, [_vp, C.c_int, _vp, C.c_int, C.c_float, _vp, C.c_int]),
    "granite4_kernel_kv_move": (C.c_int, [C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.c_int, _vp,
                                          _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "granite4_kv_pool_create": (_vp, [C.c_int, C.c_int]),
    "granite4_kv_pool_destroy": (None, [_vp]),
    "granite4_kv_pool_create_sequence": (C.c_int, [_vp]),
    "granite4_kv_pool_match_prefix": (C.c_longlong, [_vp, C.c_int, _vp, C.c_longlong]),
    "granite4_kv_pool_reserve": (C.c_int, [_vp, C.c_int, C.c_longlong, _vp, C.c_longlong]),
    "granite4_kv_pool_mark_written": (C.c_int, [_vp, C.c_int, C.c_longlong]),
    "granite4_kv_pool_row_table": (C.c_int, [_vp, C.c_int, C.c_longlong, _vp]),
    "granite4_kv_pool_reset_sequence": (None, [_vp, C.c_int]),
    "granite4_kv_pool_truncate_sequence": (None, [_vp, C.c_int, C.c_longlong]),
    "granite4_kv_pool_release": (None, [_vp, C.c_int]),
    "granite4_kv_pool_clear": (None, [_vp]),
    "granite4_kv_pool_count": (C.c_longlong, [_vp, C.c_int]),
    "granite4_kv_pool_sequence_tokens": (C.c_longlong, [_vp, C.c_int]),
    "granite4_kv_pool_block_table": (C.c_longlong, [_vp, C.c_int, _vp, C.c_longlong]),
    "granite4_kv_pool_ref_count": (C.c_int, [_vp, C.c_int]),
    "granite4_kv_pool_page_in_cache": (C.c_int, [_vp, C.c_int]),
    "granite4_kv_pool_move_rows": (C.c_int, [_vp, C.c_int, _vp, _vp, C.c_int, _vp, _vp]),
    "granite4_kv_ctl_create": (_vp, [C.c_int, C.c_int]),
    "granite4_kv_ctl_destroy": (None, [_vp]),
    "granite4_kv_ctl_shutdown": (None, [_vp]),
    "granite4_kv_ctl_pool": (_vp, [_vp]),
    "granite4_kv_ctl_new_slot": (C.c_int, [_vp]),
    "granite4_kv_ctl_release_slot": (None, [_vp, C.c_int]),
    "granite4_kv_ctl_prefill": (C.c_int, [_vp, C.c_int, _vp, C.c_longlong, C.POINTER(C.c_int),
                                          C.POINTER(C.c_longlong)]),
    "granite4_kv_ctl_commit": (None, [_vp, C.c_int, _vp, C.c_longlong]),
    "granite4_kv_ctl_open_slot": (C.c_int, [_vp]),
    "granite4_kv_ctl_ensure": (C.c_int, [_vp, C.c_int, C.c_longlong]),
    "granite4_kv_ctl_trim": (None, [_vp, C.c_int, C.c_longlong]),
    "granite4_kv_ctl_drop": (None, [_vp, C.c_int]),
    "granite4_kv_ctl_slot_pages": (C.c_longlong, [_vp, C.c_int]),
    "granite4_kv_ctl_pages_missing": (C.c_longlong, [_vp, C.c_int, C.c_longlong]),
    "granite4_kv_ctl_row_table": (C.c_int, [_vp, C.c_int, C.c_longlong, _vp]),
    "granite4_kv_ctl_committed": (C.c_longlong, [_vp, C.c_int]),
    "granite4_kv_ctl_last_reused": (C.c_longlong, [_vp, C.c_int]),
    "granite4_kv_ctl_max_slots": (C.c_longlong, [_vp]),
    "granite4_kv_ctl_count": (C.c_longlong, [_vp, C.c_int]),
    "granite4_attn_decode_scratch_bytes": (C.c_longlong, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "granite4_kernel_attn_decode_int8_paged": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int,
                                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                         C.c_int, C.c_float, _vp, C.c_longlong, _vp]),
    "granite4_attn_split_scratch_bytes": (C.c_longlong, [C.c_int, C.c_int, C.c_int]),
    "granite4_attn_split_int8": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int,
                                           _vp, C.c_int, C.c_int, _vp, C.c_longlong, _vp, _vp, C.c_int, _vp, _vp,
                                           _vp, C.c_int, _vp, _vp, C.c_int]),
    "granite4_gemm_fp8_workspace_bytes": (C.c_longlong, [C.c_int, C.c_int, C.c_int]),
    "granite4_kernel_gemm_fp8": (C.c_int, [C.c_int, _vp, C.c_longlong, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp,
                                           C.c_longlong]),
    "granite4_prefill_attention_int8": (C.c_int, [_vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                  C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_longlong]),
    "granite4_kernel_fp8_encode_with_amax": (C.c_int, [_vp, C.c_longlong, _vp, _vp]),
    "granite4_prefill_silu_mul": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "granite4_kernel_swiglu_fp8": (C.c_int, [_vp, _vp, C.c_int, C.c_longlong, C.c_int, C.c_int,
                                             _vp, _vp, _vp]),
    "granite4_glue_layer": (C.c_int, [_vp]),
    "granite4_host_glue_create": (_vp, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_int, C.c_int, C.c_double]),
    "granite4_host_glue_destroy": (None, [_vp]),
    "granite4_host_glue_layer": (C.c_int, [_vp, C.c_int, _vp]),
    "granite4_host_glue_final_norm": (C.c_int, [_vp, _vp, C.c_float, C.c_int, _vp]),
    "granite4_host_glue_sync": (C.c_int, [_vp]),
    "granite4_host_glue_h2d_bytes": (C.c_longlong, [_vp, C.c_int]),
    "granite4_host_glue_d2h_bytes": (C.c_longlong, [_vp, C.c_int]),
}


class GlueLayerArgs(C.Structure):
    """granite4_glue_layer_args: device pointers of one layer's glue."""
    _fields_ = [(n, _vp) for n in (
        "y_attn", "y_mlp", "qkv", "gate", "up", "w_attn_norm", "w_mlp_norm", "cos_tbl", "sin_tbl",
        "pos_rows", "kv_rows", "hidden", "n_attn_fp8", "n_mlp_fp8", "q_rot", "cache_k", "cache_v",
        "k_scale", "v_scale", "act_fp8", "scales", "rstd", "act_ws")] + [(n, C.c_int) for n in (
            "rows", "hidden_size", "intermediate", "q_heads", "kv_heads", "head_dim", "pool_rows",
            "max_pos")] + [("eps", C.c_float), ("resid_mult", C.c_float)]


class HostLayerIO(C.Structure):
    """granite4_host_layer_io: HOST pointers of one layer call."""
    _fields_ = [(n, _vp) for n in (
        "y_attn", "y_mlp", "qkv", "gate", "up", "w_attn_norm", "w_mlp_norm", "pos_rows", "kv_rows",
        "hidden_in", "hidden_out", "n_attn_fp8", "n_mlp_fp8", "q_rot", "act_fp8", "scales")] + [
            ("rows", C.c_int), ("eps", C.c_float), ("resid_mult", C.c_float)]


class GemmFp8Epilogue(C.Structure):
    """granite4_gemm_fp8_epilogue (the FP8 counterpart of GemmEpilogue, engine/src/prefill_gemm.h:21-30)."""
    _fields_ = [("d_a_scale", _vp), ("w_scale0", C.c_float), ("w_scale1", C.c_float), ("w_scale2", C.c_float),
                ("seg1", C.c_int), ("seg2", C.c_int), ("d_out_bf16", _vp), ("d_out_f32", _vp),
                ("d_residual", _vp), ("resid_scale", C.c_float), ("ldc", C.c_int),
                ("d_out_scale_amax", _vp)]


GEMM_OUT_BF16, GEMM_OUT_F32, GEMM_OUT_RESIDUAL, GEMM_OUT_SWIGLU = 0, 1, 2, 3
MAX_VERIFY_ROWS = 16
MAX_TREE_DEPTH = 8


class ModelInfo(C.Structure):
    """granite4_model_info (engine/src/capi.h:32-45 in the reference)."""
    _fields_ = [("model_id", C.c_char_p), ("num_layers", C.c_long), ("hidden_size", C.c_long),
                ("intermediate_size", C.c_long), ("num_attention_heads", C.c_long),
                ("num_key_value_heads", C.c_long), ("head_dim", C.c_long),
                ("vocab_size", C.c_long), ("max_context_length", C.c_long),
                ("gpu_target", C.c_char_p)]


class StatusInfo(C.Structure):
    """granite4_status_info; same layout as frontend/engine_bridge.py:45-51 binds."""
    _fields_ = [("status", C.c_int), ("cuda_device_present", C.c_int),
                ("status_text", C.c_char_p), ("message", C.c_char_p)]


class MultiRows(C.Structure):
    """granite4_multi_rows = granite4::GpuMultiRows (engine/src/forward_gpu_api.h:162-182)."""
    _fields_ = [("n", C.c_int), ("pos", C.c_int * MAX_VERIFY_ROWS),
                ("pt", _vp * MAX_VERIFY_ROWS), ("tok", _vp * MAX_VERIFY_ROWS),
                ("grp", C.c_int * MAX_VERIFY_ROWS), ("tree", C.c_int),
                ("slot", C.c_int * MAX_VERIFY_ROWS), ("tbase", C.c_int * MAX_VERIFY_ROWS),
                ("tail", (C.c_int * MAX_TREE_DEPTH) * MAX_VERIFY_ROWS)]


class Library:
    """The loaded shared library with typed entry points as attributes."""

    def __init__(self, path: str | None = None):
        path = path or os.environ.get("GRANITE4_B200_LIB") or _build.LIB_PATH
        if not os.path.isfile(path):
            raise FileNotFoundError(
                f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; "
                f"g.build()'` (there is no CPU or PyTorch fallback for these kernels)")
        self.path = path
        self._dll = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self._dll, name)  # AttributeError here = ABI drift
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)

    # convenience -------------------------------------------------------------------
    def model_info(self) -> ModelInfo:
        info = ModelInfo()
        self.granite4_get_model_info(C.byref(info))
        return info

    def status(self) -> StatusInfo:
        st = StatusInfo()
        self.granite4_status(C.byref(st))
        return st

    def device_status(self) -> int:
        out = C.c_uint(0)
        if self.granite4_b200_device_status(C.byref(out)) != 0:
            raise RuntimeError("granite4_b200_device_status failed")
        return out.value


_lib: Library | None = None


def lib() -> Library:
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
