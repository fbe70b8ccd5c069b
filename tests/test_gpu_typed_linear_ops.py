"""Every ordering of gather / matmul / scatter that the reference offers for  Y[d] = sum_e x[src e] . W[rel e]
(cxgnncomp/typed_linear.py:10-310: TypedLinearS2EOP, S2DMMAggrOP, S2DAggrMMOP, S2DSort, S2DPushOP, NaiveS2D,
SelectMMS2EOP; cxgnncomp/graph_conv.py:205-306: RGCNOP, RGCNOP2, RGCNOP3, RGCNOP_sorted), forward and, where the
reference defines one, backward, against the float64 per-edge products of the oracle and autograd through the
reference's sorted torch formulation."""
import pytest
import torch

import oracle
from helpers import random_csr, randn, rel_err

pytestmark = pytest.mark.gpu

R, K, N = 5, 64, 32
# fp32 inputs on the tensor-core path (typed matmul): error-compensated TF32
TC_TOL = 1e-5
N_DST, N_SRC = 220, 260


def _case(seed=21, dtype=torch.float32):
    ptr, idx = random_csr(N_DST, N_SRC, 7, seed=seed, hub=400)
    g = torch.Generator().manual_seed(seed + 1)
    rel = torch.randint(0, R, (idx.shape[0],), generator=g)
    rel[rel == 3] = 1  # a relation without edges
    x = randn((N_SRC, K), seed + 2).to(dtype)
    w = (randn((R, K, N), seed + 3) * 0.2).to(dtype)
    dst = oracle.dst_of_edges(ptr)
    per_edge = oracle.typed_linear_f64(x.float(), w.float(), rel, src=idx)  # [E, N] float64
    y = torch.zeros(N_DST, N, dtype=torch.float64).index_add_(0, dst, per_edge)
    return ptr, idx, rel, x, w, dst, per_edge, y


def _ref_grads(ptr, idx, rel, x, w, go):
    """d/dx, d/dW of the reference's sorted torch formulation (typed_linear.py:262-310) by autograd on the CPU."""
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    oracle.torch_rgcn_sorted(xr, wr, ptr, idx, rel, N_DST).backward(go)
    return xr.grad, wr.grad


def test_s2e_forward(cuda):
    import cxgnncomp
    ptr, idx, rel, x, w, dst, per_edge, _ = _case()
    out = cxgnncomp.TypedLinearS2EOP.apply(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), [], 128)
    assert out.shape == per_edge.shape
    assert rel_err(out.cpu(), per_edge) < TC_TOL
    pre = cxgnncomp.TypedLinearS2EOP.preprocess(w.cuda(), rel.cuda(), idx.cuda(), 256)
    out2 = cxgnncomp.TypedLinearS2EOP.apply(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), pre, 256)
    assert rel_err(out2.cpu(), per_edge) < TC_TOL
    ob = cxgnncomp.TypedLinearS2EOP.apply(x.cuda().bfloat16(), w.cuda().bfloat16(), rel.cuda(), idx.cuda(), [], 128)
    assert rel_err(ob.float().cpu(), per_edge) < 1e-2
    with pytest.raises((NotImplementedError, RuntimeError)):
        xg = x.cuda().requires_grad_(True)
        cxgnncomp.TypedLinearS2EOP.apply(xg, w.cuda(), rel.cuda(), idx.cuda(), [], 128).sum().backward()


@pytest.mark.parametrize("op_name", ["TypedLinearS2DMMAggrOP", "TypedLinearS2DAggrMMOP", "RGCNOP", "RGCNOP2"])
def test_per_relation_loop_ops(cuda, op_name):
    """Transform-then-aggregate and aggregate-then-transform per relation (selective_aggr under the hood)."""
    import cxgnncomp
    ptr, idx, rel, x, w, dst, _, y = _case(seed=31)
    op = getattr(cxgnncomp, op_name)
    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    out = op.apply(xg, wg, ptr.cuda(), idx.cuda(), rel.cuda(), N_DST)
    assert rel_err(out.detach().cpu(), y) < 1e-5
    go = randn(y.shape, 33)
    out.backward(go.cuda())
    gx, gw = _ref_grads(ptr, idx, rel, x, w, go)
    assert rel_err(xg.grad.cpu(), gx) < 1e-5
    assert rel_err(wg.grad.cpu(), gw) < 1e-5


def test_rgcnop3_forward(cuda):
    import cxgnncomp
    ptr, idx, rel, x, w, dst, _, y = _case(seed=41)
    out = cxgnncomp.RGCNOP3.apply(x.cuda(), w.cuda(), ptr.cuda(), idx.cuda(), rel.cuda(), N_DST)
    assert rel_err(out.cpu(), y) < 1e-5
    with pytest.raises((NotImplementedError, RuntimeError)):
        xg = x.cuda().requires_grad_(True)
        cxgnncomp.RGCNOP3.apply(xg, w.cuda(), ptr.cuda(), idx.cuda(), rel.cuda(), N_DST).sum().backward()


def test_sorted_formulations(cuda):
    """TypedLinearS2DSort and RGCNOP_sorted (per-relation F.linear + index_add_), differentiable through torch."""
    import cxgnncomp
    ptr, idx, rel, x, w, dst, _, y = _case(seed=51)
    go = randn(y.shape, 53)
    gx, gw = _ref_grads(ptr, idx, rel, x, w, go)
    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    out = cxgnncomp.TypedLinearS2DSort(xg, wg, ptr.cuda(), idx.cuda(), rel.cuda(), N_DST)
    assert rel_err(out.detach().cpu(), y) < 1e-5
    out.backward(go.cuda())
    assert rel_err(xg.grad.cpu(), gx) < 1e-5 and rel_err(wg.grad.cpu(), gw) < 1e-5
    # same with the relation counts handed in, as the reference's callers do
    count = torch.bincount(rel, minlength=R)
    out_c = cxgnncomp.TypedLinearS2DSort(x.cuda(), w.cuda(), ptr.cuda(), idx.cuda(), rel.cuda(), N_DST, count.cuda())
    assert rel_err(out_c.cpu(), y) < 1e-5
    order = torch.sort(rel, stable=True).indices
    xg2, wg2 = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    out2 = cxgnncomp.RGCNOP_sorted(xg2, wg2, idx[order].cuda(), dst[order].cuda(), count, N_DST)
    assert rel_err(out2.detach().cpu(), y) < 1e-5
    out2.backward(go.cuda())
    assert rel_err(xg2.grad.cpu(), gx) < 1e-5 and rel_err(wg2.grad.cpu(), gw) < 1e-5


def test_naive_push_and_select(cuda):
    import cxgnncomp
    ptr, idx, rel, x, w, dst, per_edge, y = _case(seed=61)
    e = idx.shape[0]
    out = cxgnncomp.TypedLinearNaiveS2D(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), dst.cuda(), N_DST, e)
    assert rel_err(out.cpu(), y) < 1e-5
    # a prefix of the edges only
    half = e // 2
    y_half = torch.zeros(N_DST, N, dtype=torch.float64).index_add_(0, dst[:half], per_edge[:half])
    out_h = cxgnncomp.TypedLinearNaiveS2D(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), dst.cuda(), N_DST, half)
    assert rel_err(out_h.cpu(), y_half) < 1e-5
    push = cxgnncomp.TypedLinearS2DPushOP(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), dst.cuda(), R, N_DST, e)
    assert rel_err(push.cpu(), y) < TC_TOL
    outs = cxgnncomp.SelectMMS2EOP(x.cuda(), w.cuda(), idx.cuda(), rel.cuda())
    assert len(outs) == R
    for r in range(R):
        sel = rel == r
        assert outs[r].shape == (int(sel.sum()), N)
        if int(sel.sum()):
            assert rel_err(outs[r].cpu(), per_edge[sel]) < 1e-5


def test_against_reference_outputs(cuda, golden):
    """The fixture holds inputs and outputs of the reference's own TypedLinearS2DSort and SelectMMS2EOP run on the
    CPU (tests/golden/make_golden.py); the same inputs through every ordering of this library on the GPU."""
    import cxgnncomp
    x, w = torch.from_numpy(golden["spmm_x"]), torch.from_numpy(golden["rgcn_w"])
    ptr, idx, rel = (torch.from_numpy(golden[k]) for k in ("spmm_ptr", "spmm_idx", "rgcn_rel"))
    want = torch.from_numpy(golden["rgcn_s2dsort"])
    n = ptr.shape[0] - 1
    dst = oracle.dst_of_edges(ptr)
    for name in ("TypedLinearS2DMMAggrOP", "TypedLinearS2DAggrMMOP", "RGCNOP", "RGCNOP2", "RGCNOP3"):
        out = getattr(cxgnncomp, name).apply(x.cuda(), w.cuda(), ptr.cuda(), idx.cuda(), rel.cuda(), n)
        assert rel_err(out.cpu(), want) < 1e-5, name
    out = cxgnncomp.TypedLinearS2DSort(x.cuda(), w.cuda(), ptr.cuda(), idx.cuda(), rel.cuda(), n)
    assert rel_err(out.cpu(), want) < 1e-5
    out = cxgnncomp.TypedLinearS2DPushOP(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), dst.cuda(), w.shape[0], n,
                                         idx.shape[0])
    assert rel_err(out.cpu(), want) < TC_TOL
    per_edge = cxgnncomp.TypedLinearS2EOP.apply(x.cuda(), w.cuda(), rel.cuda(), idx.cuda(), [], 128)
    assert rel_err(torch.zeros_like(want).index_add_(0, dst, per_edge.cpu()), want) < TC_TOL
    for r, o in enumerate(cxgnncomp.SelectMMS2EOP(x.cuda(), w.cuda(), idx.cuda(), rel.cuda())):
        assert rel_err(o.cpu(), torch.from_numpy(golden[f"rgcn_select_{r}"])) < 1e-5
