"""The allocation-free variant of the fused add + norm + FP8 op.

Who needs it: hosts that cannot get device memory at the moment of the call - an engine that
handed the whole card to its KV arena and weight blob when it started, or a language binding
that loads this library without the CUDA runtime and therefore has no cudaMalloc - and so
cannot supply the per-row scratch buffer the regular entry point takes. The variant keeps that
scratch in a fixed array inside the library.

The file name sorts last on purpose: if this fails, a run that stops at the first failure has
already been through every other test. It passes on its own in a fresh process as well as
after the other tests (it relies on nothing they leave behind; the shared scratch array needs
no clearing between calls).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _run_both(K, port, rows, cols, seed, rm):
    g = torch.Generator(device=DEV).manual_seed(seed)
    y = torch.randn(rows, cols, generator=g, device=DEV).to(torch.bfloat16)
    res = torch.randn(rows, cols, generator=g, device=DEV).to(torch.bfloat16)
    w = (1 + 0.02 * torch.randn(cols, generator=g, device=DEV)).to(torch.bfloat16)
    # existing entry point, caller-provided scratch
    h_ref = torch.empty_like(res)
    c_ref = torch.empty(rows, cols, dtype=torch.uint8, device=DEV)
    sa_ref = torch.zeros(2, dtype=torch.float32, device=DEV)
    rstd = torch.empty(rows, dtype=torch.float32, device=DEV)
    assert K.add_rmsnorm_fp8(y, res, w, 1e-5, rm, h_out=h_ref, n_fp8=c_ref, scale_amax=sa_ref,
                             rstd=rstd) == 0
    # the variant: no scratch argument, nothing allocated inside
    h = torch.empty_like(res)
    c = torch.empty_like(c_ref)
    sa = torch.zeros(2, dtype=torch.float32, device=DEV)
    assert K.add_rmsnorm_fp8_noalloc(y, res, w, 1e-5, rm, h, c, sa) == 0
    torch.cuda.synchronize()
    # same tolerance as the parity tests use for this op: bit-exact hidden state and codes,
    # scale within 1e-6 relative (it is in fact identical)
    assert torch.equal(h, h_ref)
    assert torch.equal(c, c_ref)
    assert abs(sa[0].item() - sa_ref[0].item()) <= 1e-6 * abs(sa_ref[0].item())
    assert sa[1].item() == sa_ref[1].item()
    # and, independently of the sibling entry point, against the CPU oracle
    want_h, want_n = port.add_rmsnorm(_bits(y), _bits(res), _bits(w), 1e-5, rm)
    codes, scale, amax = port.quant_fp8(want_n)
    assert (_bits(h) == want_h).all() and (c.cpu().numpy() == codes).all()
    assert sa[0].item() == scale and sa[1].item() == amax


def test_noalloc_matches_the_regular_entry_point_twice_in_a_row(port):
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi, kernels as K
    capi.lib()
    # two calls in a row share the library's scratch array; the second uses fewer rows, so stale
    # entries of the first remain in the array beyond its range and must not matter
    _run_both(K, port, 700, 4096, seed=11, rm=0.22)
    _run_both(K, port, 333, 4096, seed=12, rm=1.0)
    assert capi.lib().device_status() == 0


def test_noalloc_refuses_more_rows_than_its_scratch_holds(capfd):
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi
    lib = capi.lib()
    # validation happens before any launch: dummy aligned addresses are never dereferenced
    assert lib.granite4_kernel_add_rmsnorm_fp8_noalloc(16, 0, 16, 0, 16, 1e-5, 0.22, 65537, 8, 16, 16,
                                                       16) == -1
    assert "65536" in capfd.readouterr().err
    assert lib.granite4_kernel_add_rmsnorm_fp8_noalloc(16, 0, 16, 0, 16, 1e-5, 0.22, 4, 4096, None, 16,
                                                       16) == -1
