"""cxg_csr_transpose (device radix sort of the edges by source) against a stable CPU sort, bit for bit, and the
backward that runs on the transposed graph: deterministic and within 1e-5 of float64."""
import pytest
import torch

import oracle
from helpers import random_csr, randn, rel_err

pytestmark = pytest.mark.gpu


def _check(ptr, idx, n_dst, n_src, idx_dtype=torch.int64):
    import cxgnncomp_backend as be
    t_ptr, t_idx, t_eid, inv_deg = be.csr_transpose(ptr.cuda(), idx.to(idx_dtype).cuda(), n_dst, n_src)
    w_ptr, w_idx, w_eid = oracle.csr_transpose(ptr, idx, n_dst, n_src)
    e = int(ptr[n_dst])
    assert t_idx.dtype == idx_dtype and t_eid.dtype == idx_dtype
    assert torch.equal(t_ptr.cpu(), w_ptr)
    assert torch.equal(t_idx.cpu()[:e].long(), w_idx)
    assert torch.equal(t_eid.cpu()[:e].long(), w_eid)
    assert int(t_idx[e:].abs().sum()) == 0 and int(t_eid[e:].abs().sum()) == 0
    deg = (ptr[1:n_dst + 1] - ptr[:n_dst]).clamp(min=1).float()
    assert torch.equal(inv_deg.cpu(), 1.0 / deg)


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("n_dst,n_src,deg,hub", [(300, 257, 9, 60), (5000, 70000, 20, 30000), (17, 3, 4, 0),
                                                  (2048, 2048, 1, 0), (40, 1, 3, 0)])
def test_transpose_equals_stable_sort(cuda, n_dst, n_src, deg, hub, idx_dtype):
    ptr, idx = random_csr(n_dst, n_src, deg, seed=n_dst + n_src, hub=hub)
    _check(ptr, idx, n_dst, n_src, idx_dtype)


def test_transpose_prefix_rows_and_empty(cuda):
    """Layered batches use the first n rows of a longer graph: only ptr[n] edges take part."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(500, 400, 6, seed=5, hub=100)
    _check(ptr, idx, 123, 400)
    _check(ptr, idx, 1, 400)
    # a graph without edges
    z = torch.zeros(11, dtype=torch.int64)
    t_ptr, t_idx, t_eid, inv = be.csr_transpose(z.cuda(), torch.zeros(0, dtype=torch.int64).cuda(), 10, 7)
    assert torch.equal(t_ptr.cpu(), torch.zeros(8, dtype=torch.int64)) and t_idx.numel() == 0
    assert torch.equal(inv.cpu(), torch.ones(10))


def test_transpose_four_passes(cuda):
    """Source ids above 2^24 need four 8-bit passes."""
    n_src = (1 << 24) + 1000
    g = torch.Generator().manual_seed(3)
    ptr, _ = random_csr(3000, 10, 15, seed=4)
    idx = torch.randint(0, n_src, (int(ptr[-1]),), generator=g)
    idx[::7] = n_src - 1
    idx[1::7] = 0
    _check(ptr, idx, 3000, n_src)


def test_arxiv_transpose_full_size(cuda):
    """Configuration 1 (169,343 nodes / 2,332,487 edges, one source with 94,797 edges)."""
    from cxgnncomp import synthetic
    n, e_und = synthetic.CONFIG_SHAPES["arxiv_like"]
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0)
    _check(ptr, idx, n, n)
    # symmetric graph with sorted rows: its transpose is the graph itself
    t_ptr, t_idx, _, _ = __import__("cxgnncomp_backend").csr_transpose(ptr.cuda(), idx.cuda(), n, n)
    assert torch.equal(t_ptr.cpu(), ptr) and torch.equal(t_idx.cpu(), idx)


@pytest.mark.parametrize("mean", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_default_backward_is_deterministic(cuda, mean, dtype):
    """The default backward runs on the transposed graph from the first call on: same bits on every run,
    1e-5 (fp32) of float64, also with a hub source."""
    import cxgnncomp_backend as be
    assert be.BACKWARD_MODE == "auto"
    ptr, idx = random_csr(4000, 3000, 12, seed=77, hub=2500)
    idx[: 3000] = 5  # a hub SOURCE: 3000 terms added into one gradient row
    x = randn((3000, 64), 1).to(dtype)
    dy = randn((4000, 64), 2).to(dtype)
    grads = []
    for _ in range(2):
        be._TRANSPOSE_CACHE.clear()
        xg = x.cuda().requires_grad_(True)
        fn = be.sage_mean_forward if mean else be.sage_sum_forward
        fn(xg, ptr.cuda(), idx.cuda(), 4000).backward(dy.cuda())
        grads.append(xg.grad.clone())
    assert torch.equal(grads[0], grads[1])
    want, _ = oracle.spmm_bwd_f64(ptr, idx, dy.float(), x.shape, mean=mean)
    assert rel_err(grads[0].float().cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2)
