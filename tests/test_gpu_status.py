"""The library's failure reports: the status word of a call's workspace after (a) a graph whose ptr[n_dst] is larger
than the declared edge count, (b) a bounded wait that runs out. For (b) a test hook makes one barrier of the
bulk-copy SpMM / of the typed matmul pipeline impossible to complete and the wait limit is set to a fraction of a
millisecond: the kernels must give up, return, report CXG_ETIMEOUT, touch nothing outside their buffers, and the
next normal call must be correct. Nothing here faults or spins past the limit."""
import ctypes

import pytest
import torch

import oracle
from helpers import random_csr, randn, rel_err

pytestmark = pytest.mark.gpu

CXG_EINVAL, CXG_ETIMEOUT = -1, -6
GUARD = 4096


def _raw_spmm(be, desc, ws_bytes):
    """cxg_spmm_csr on a workspace followed by a guard region filled with 0xA5; returns (rc, status, guard ok)."""
    ws = torch.full((ws_bytes + GUARD,), 0xA5, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = be._spmm_fwd(ctypes.byref(desc), ctypes.c_void_p(ws.data_ptr()), ws_bytes, stream)
    status = be._spmm_status(ctypes.c_void_p(ws.data_ptr()), stream)
    return rc, status, bool(torch.all(ws[ws_bytes:] == 0xA5))


def _need(be, desc):
    need = ctypes.c_size_t(0)
    assert be._spmm_ws(desc.n_dst, desc.nnz, desc.feat, desc.heads, desc.split_edges, ctypes.byref(need)) == 0
    return need.value


def test_declared_nnz_smaller_than_ptr(cuda):
    """idx shorter than ptr[n] says: the kernels stay inside the declared edges and the workspace sized for them."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(400, 300, 10, seed=7, hub=900)
    x = randn((300, 64), 8)
    p, i, xg = ptr.cuda(), idx.cuda(), x.cuda()
    y = torch.zeros(400, 64, device="cuda")
    short = idx.shape[0] // 3
    desc = be._make_desc(p, i, xg, y, 400, heads=1, feat=64)
    desc.nnz = short
    desc.split_edges = 64
    rc, status, guard_ok = _raw_spmm(be, desc, _need(be, desc))
    assert rc == 0 and status == CXG_EINVAL and guard_ok
    assert "declared nnz" in be._lib.cxg_last_error_string().decode()
    # rows that lie inside one tile of the declared edges are still right (rows crossing tile borders are
    # finished by a second kernel, which does nothing once the error is recorded)
    done = (ptr[1:] <= short) & (ptr[1:] > ptr[:-1]) & ((ptr[:-1] // 64) == ((ptr[1:] - 1) // 64))
    assert int(done.sum()) > 20
    want = oracle.spmm(ptr, idx, x, tile=64)
    assert torch.equal(y.cpu()[done], want[done])
    # the same descriptor with the true edge count is clean
    desc.nnz = idx.shape[0]
    rc, status, guard_ok = _raw_spmm(be, desc, _need(be, desc))
    assert rc == 0 and status == 0 and guard_ok
    assert torch.equal(y.cpu(), want)


def test_spmm_bounded_wait_runs_out(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(300, 300, 8, seed=93, hub=500)
    x = randn((300, 64), 94)
    p, i, xg = ptr.cuda(), idx.cuda(), x.cuda()
    y = torch.full((300, 64), 3.0, device="cuda")
    desc = be._make_desc(p, i, xg, y, 300, heads=1, feat=64)
    desc.split_edges = 64
    desc.flags = be.CXG_SPMM_BULK_ROWS | be.CXG_SPMM_TEST_STALL
    be.set_wait_limit_cycles(200_000)  # ~0.1 ms
    try:
        rc, status, guard_ok = _raw_spmm(be, desc, _need(be, desc))
    finally:
        be.set_wait_limit_cycles(0)
    assert rc == 0 and status == CXG_ETIMEOUT and guard_ok
    assert "wait ran out" in be._lib.cxg_last_error_string().decode()
    # the context is intact: the same call without the hook gives the oracle's bits, in both row-fetch variants
    for flags in (be.CXG_SPMM_BULK_ROWS, 0):
        desc.flags = flags
        rc, status, guard_ok = _raw_spmm(be, desc, _need(be, desc))
        assert rc == 0 and status == 0 and guard_ok
        assert torch.equal(y.cpu(), oracle.spmm(ptr, idx, x, tile=64))


def test_spmm_index_ring_wait_runs_out(cuda):
    """The id ring of the lean walk (CXG_SPMM_TMA_INDEX): every warp's first chunk announces bytes that never
    arrive; the warps give up after the limit, the call reports CXG_ETIMEOUT and the next call is right."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(300, 300, 8, seed=95, hub=700)
    x = randn((300, 64), 96)
    for idx_dtype in (torch.int32, torch.int64):
        p, i, xg = ptr.cuda(), idx.cuda().to(idx_dtype), x.cuda()
        y = torch.full((300, 64), 3.0, device="cuda")
        desc = be._make_desc(p, i, xg, y, 300, heads=1, feat=64)
        desc.split_edges = 256
        desc.flags = be.CXG_SPMM_TMA_INDEX | be.CXG_SPMM_TEST_STALL
        be.set_wait_limit_cycles(200_000)  # ~0.1 ms
        try:
            rc, status, guard_ok = _raw_spmm(be, desc, _need(be, desc))
        finally:
            be.set_wait_limit_cycles(0)
        assert rc == 0 and status == CXG_ETIMEOUT and guard_ok
        desc.flags = be.CXG_SPMM_TMA_INDEX
        rc, status, guard_ok = _raw_spmm(be, desc, _need(be, desc))
        assert rc == 0 and status == 0 and guard_ok
        assert torch.equal(y.cpu(), oracle.spmm(ptr, idx, x, tile=256))


def test_typed_matmul_bounded_wait_runs_out(cuda):
    import cxgnncomp_backend as be
    R, E, K, N = 3, 2000, 64, 32
    g = torch.Generator().manual_seed(90)
    types = torch.randint(0, R, (E,), generator=g)
    for dtype in (torch.bfloat16, torch.float32):
        a, w = randn((E, K), 91).to(dtype), (randn((R, K, N), 92) * 0.2).to(dtype)
        # bucket the positions by relation, padded to blocks of 128 (TypedLinearE2EOP.preprocess)
        count = torch.bincount(types, minlength=R)
        new_types = torch.empty(E + R * 127, dtype=torch.int64, device="cuda")
        new_types[:E] = types.cuda()
        be.pad_rel(new_types, count.cuda(), 128, R, E)
        st, indices = torch.sort(new_types, stable=True)
        be.set_wait_limit_cycles(200_000)
        try:
            be.typed_matmul_raw(a.cuda(), w.cuda(), st, st.shape[0], E, src_idx=indices, extra_flags=be.CXG_TMM_TEST_STALL)
            with pytest.raises(RuntimeError, match="wait ran out"):
                be.check_device_status("typed_matmul")
        finally:
            be.set_wait_limit_cycles(0)
        c = be.typed_matmul_raw(a.cuda(), w.cuda(), st, st.shape[0], E, src_idx=indices)
        be.check_device_status("typed_matmul")
        assert rel_err(c.float().cpu(), oracle.typed_linear_f64(a, w, types)) < 1e-2


def test_status_answers_only_for_the_last_kind(cuda):
    """SpMM and typed matmul share the per-stream scratch buffer; asking about the kind that did not run last
    checks nothing instead of reading the other call's counters."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(600, 500, 6, seed=3, hub=60000)  # long chains: the streaming header counts them in word 0
    x = randn((500, 64), 4)
    be.sage_sum_forward(x.cuda(), ptr.cuda(), idx.cuda(), 600)
    be.check_device_status("typed_matmul")
    be.check_device_status("spmm")
    # row path (edge mask) on a graph without long rows: its header is cleared too
    mask = torch.ones(idx.shape[0], dtype=torch.bool)
    out = torch.zeros(600, 64, device="cuda")
    be.selective_aggr(x.cuda(), ptr.cuda(), idx.cuda(), mask.cuda(), out, 600)
    be.check_device_status("spmm")


def test_typed_wgrad_bounded_wait_runs_out(cuda):
    """The weight-gradient kernel: the producers never hand over their first tile; the roles give up after the limit,
    the status says so, and the next call is right."""
    import cxgnncomp_backend as be
    E = 4096
    st = torch.zeros(E, dtype=torch.int64, device="cuda")
    for dtype in (torch.bfloat16, torch.float32):
        x, g = randn((E, 128), 97).to(dtype).cuda(), randn((E, 64), 98).to(dtype).cuda()
        be.set_wait_limit_cycles(200_000)
        try:
            with pytest.raises(RuntimeError, match="wait ran out"):
                be.typed_wgrad(x, g, st, 1, E, extra_flags=1, check_status=True)
        finally:
            be.set_wait_limit_cycles(0)
        dw = be.typed_wgrad(x, g, st, 1, E, check_status=True)[0]
        want = x.double().t() @ g.double()
        assert rel_err(dw.cpu(), want.cpu()) < (1e-5 if dtype == torch.float32 else 1e-2)
