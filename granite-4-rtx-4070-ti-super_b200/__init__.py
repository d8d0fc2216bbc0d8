"""B200 (sm_100a) implementation of the Granite 4.2 8B per-layer glue kernels.

Sub-modules:
  capi     ctypes binding of libgranite4_b200.so, one callable per C-ABI entry point
  kernels  the reference engine's launch interface over PyTorch CUDA tensors
  paging   16-token-page row tables (host side of the paged KV write)
  glue     the per-layer kernel sequence (2 x add+norm, RoPE+KV, SwiGLU, final norm)
  _build   nvcc build of the shared library

The directory name is not a Python identifier; import it through the `granite4_b200`
module at the repository root, which registers this package under that name.
"""
from . import _build  # noqa: F401

__all__ = ["capi", "kernels", "paging", "glue", "_build"]
