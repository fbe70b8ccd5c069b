"""cxg_spmm_csr_static: the SpMM entry point for callers that cannot hand the library a scratch
buffer (host programs whose memory pool owns the device, loops that must not hit cudaMalloc's
device-wide synchronisation, FFI bindings that carry only the operator's tensors). It runs on a
fixed scratch array inside the library, so the checks are: same output as cxg_spmm_csr, on two
calls in a row (the second call finds the first call's leftovers in the array), and a clear refusal
when the graph needs more scratch than the array holds.

This file sorts last on purpose: it is the only test of an add-on entry point, and a run that
stops at the first failure should have finished every other test by then.
"""
import ctypes

import pytest
import torch

from helpers import random_csr, randn

pytestmark = pytest.mark.gpu


def _call_static(be, ptr, idx, x, y, n, mean=False):
    """Straight through the C ABI: descriptor + stream, nothing else."""
    fn = be._lib.cxg_spmm_csr_static
    fn.argtypes = [ctypes.POINTER(be.SpmmDesc), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    desc = be._make_desc(ptr, idx, x, y, n, heads=1, feat=x.shape[-1], reduce=be.CXG_MEAN if mean else be.CXG_SUM)
    with torch.cuda.device(x.device):
        rc = fn(ctypes.byref(desc), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


def test_static_scratch_matches_workspace_entry_point(cuda):
    import cxgnncomp_backend as be
    # first call: hub row that crosses many tiles, fp32
    ptr, idx = random_csr(500, 400, 12, seed=101, hub=9000)
    x = randn((400, 128), 102)
    p, i, xg = ptr.cuda(), idx.cuda(), x.cuda()
    want = be.run_spmm_configurable(p, i, xg, 500)
    got = torch.full_like(want, float("nan"))
    assert _call_static(be, p, i, xg, got, 500) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)  # same kernels, same order: no tolerance needed
    import oracle
    assert torch.equal(got.cpu(), oracle.spmm(ptr, idx, x, tile=64))  # and the CPU oracle's bits (64-edge tiles here)
    # second call straight after, other graph, other dtype, mean: the array still holds the first call's data
    ptr2, idx2 = random_csr(300, 300, 7, seed=103, hub=4000)
    x2 = randn((300, 64), 104, dtype=torch.bfloat16)
    p2, i2, xg2 = ptr2.cuda(), idx2.cuda(), x2.cuda()
    want2 = be.sage_mean_forward(xg2, p2, i2, 300)
    got2 = torch.empty_like(want2)
    assert _call_static(be, p2, i2, xg2, got2, 300, mean=True) == 0
    torch.cuda.synchronize()
    assert torch.equal(got2.view(torch.int16), want2.view(torch.int16))
    # and the first problem again gives the first answer again
    got.fill_(float("nan"))
    assert _call_static(be, p, i, xg, got, 500) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_static_scratch_refuses_oversized_graphs(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(64, 64, 4, seed=105)
    x = randn((64, 128), 106)
    p, i, xg = ptr.cuda(), idx.cuda(), x.cuda()
    y = torch.zeros(64, 128, device="cuda")
    fn = be._lib.cxg_spmm_csr_static
    fn.argtypes = [ctypes.POINTER(be.SpmmDesc), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    desc = be._make_desc(p, i, xg, y, 64, heads=1, feat=128)
    desc.nnz = 2_000_000_000  # scratch need is computed from the declared sizes, before anything is launched
    rc = fn(ctypes.byref(desc), None)
    assert rc == -7  # CXG_ELIMIT
    msg = be._lib.cxg_last_error_string().decode()
    assert "scratch" in msg and "built-in array" in msg
    torch.cuda.synchronize()
    assert torch.all(y == 0)
