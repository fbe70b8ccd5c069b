"""GAT-side kernels against the CPU oracle: edge softmax forward / backward, SDDMM, helpers."""
import pytest
import torch

import oracle
from helpers import random_csr, randn, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("heads", [1, 3, 4, 6])
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_edge_softmax_forward_backward(cuda, heads, idx_dtype):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(200, 180, 9, seed=heads, hub=9000)  # the hub row takes the CTA-per-row kernel
    a_s, a_d = randn((180, heads), 2) * 2, randn((200, heads), 3) * 2
    want, want_mask = oracle.edge_softmax_fwd(ptr, idx, a_d, a_s, 0.2)
    p, i = ptr.cuda(), idx.to(idx_dtype).cuda()
    asg, adg = a_s.cuda().requires_grad_(True), a_d.cuda().requires_grad_(True)
    got = be.edge_attention(ptr=p, idx=i, att_dst=adg, att_src=asg, num_edge=idx.shape[0], relu_l=0.2)
    assert got.shape == want.shape
    # fp32: the reference's own check against PyG is atol 1e-4 / rtol 1e-3 (test/1-kernels/valid-gat.py:110)
    assert torch.allclose(got.detach().cpu(), want, atol=1e-7, rtol=1e-5)
    # rows sum to one per head
    dst = oracle.dst_of_edges(ptr)
    sums = torch.zeros(200, heads).index_add_(0, dst, got.detach().cpu())
    deg = ptr[1:] - ptr[:-1]
    assert torch.allclose(sums[deg > 0], torch.ones_like(sums[deg > 0]), atol=1e-5)
    g = randn(want.shape, 4)
    got.backward(g.cuda())
    gd, gs = oracle.edge_softmax_bwd(ptr, idx, g, want_mask, want, 180, 0.2)
    assert torch.allclose(asg.grad.cpu().double(), gs, atol=1e-6, rtol=1e-4)
    assert torch.allclose(adg.grad.cpu().double(), gd, atol=1e-6, rtol=1e-4)


def test_edge_softmax_matches_reference_fixture(cuda, golden):
    import cxgnncomp_backend as be
    import numpy as np
    t = lambda k: torch.from_numpy(np.asarray(golden[k]))
    ptr, idx = t("spmm_ptr"), t("spmm_idx")
    got = be.edge_attention(ptr.cuda(), idx.cuda(), t("gat_att_dst").cuda(), t("gat_att_src").cuda(), idx.shape[0], 0.2)
    # fixture: MyGATConv.edge_softmax_opwise of the reference run on CPU (cxgnncomp/graph_conv.py:437-448)
    assert torch.allclose(got.cpu(), t("gat_edge_value"), atol=1e-6, rtol=1e-5)


def test_edge_softmax_empty(cuda):
    import cxgnncomp_backend as be
    ptr = torch.zeros(6, dtype=torch.int64).cuda()
    idx = torch.zeros(0, dtype=torch.int64).cuda()
    out = be.edge_attention(ptr, idx, torch.zeros(5, 2).cuda(), torch.zeros(3, 2).cuda(), 0, 0.2)
    assert out.shape == (0, 2)


def test_sddmm_and_helpers(cuda):
    import cxgnncomp_backend as be
    g = torch.Generator().manual_seed(5)
    src = torch.randint(0, 50, (700,), generator=g)
    dst = torch.randint(0, 40, (700,), generator=g)
    for heads, feat in [(4, 32), (1, 128), (3, 20)]:
        sf, df = randn((50, heads, feat), 6), randn((40, feat), 7)
        out = torch.zeros(700, heads, device="cuda")
        be.run_sddmm(src.cuda(), dst.cuda(), sf.cuda(), df.cuda(), out, 700)
        assert torch.allclose(out.cpu(), oracle.sddmm(src, dst, sf, df), atol=1e-5, rtol=1e-5)
        dfh = randn((40, heads, feat), 8)
        be.run_sddmm(src.cuda(), dst.cuda(), sf.cuda(), dfh.cuda(), out, 700)
        assert torch.allclose(out.cpu(), oracle.sddmm(src, dst, sf, dfh, per_head=True), atol=1e-5, rtol=1e-5)
    ptr, idx = random_csr(40, 50, 6, seed=9)
    sf, df = randn((50, 2, 16), 10), randn((40, 16), 11)
    vc = be.run_sddmm_vertex_centric(ptr.cuda(), idx.cuda(), sf.cuda(), df.cuda(), 40, 1, 1, 32, 8, 8, 32, 32, 0, 0)
    assert torch.allclose(vc.cpu(), oracle.sddmm(idx, oracle.dst_of_edges(ptr), sf, df), atol=1e-5, rtol=1e-5)
    # edge_value_degree == gcn_norm of the reference (graph_conv.py:587-596) on rows that have edges
    ptr, idx = random_csr(60, 60, 5, seed=12, empty_frac=0)
    ptr[1:] += torch.arange(1, 61)  # every row non-empty
    e = int(ptr[-1])
    ev = be.edge_value_degree(ptr.cuda(), 60, e).cpu()
    deg = ptr[1:] - ptr[:-1]
    assert torch.equal(ev, (1.0 / deg.float()).repeat_interleave(deg))
    ptr, idx = random_csr(60, 60, 5, seed=13)
    x = randn((60,), 14)
    y = be.spmv(ptr.cuda(), idx.cuda(), x.cuda(), 60).cpu()
    assert torch.allclose(y, oracle.spmm(ptr, idx, x.view(-1, 1)).view(-1), atol=1e-5)
    # gather: scatter-add of edge rows, and its backward
    xe = randn((idx.shape[0], 24), 15)
    dest = oracle.dst_of_edges(ptr)
    xg = xe.cuda().requires_grad_(True)
    out = be.gather(xg, dest.cuda(), 60)
    want = torch.zeros(60, 24).index_add_(0, dest, xe)
    assert torch.allclose(out.detach().cpu(), want, atol=1e-5)
    go = randn((60, 24), 16)
    out.backward(go.cuda())
    assert torch.equal(xg.grad.cpu(), go[dest])


def test_gat_aggregation_chain(cuda):
    """Scores -> edge softmax -> multi-head SpMM, forward and backward, as MyGATConv.forward_many chains them
    (cxgnncomp/graph_conv.py:458-496), against the torch op-wise formulation with autograd."""
    import cxgnncomp_backend as be
    H, C = 4, 32
    ptr, idx = random_csr(150, 150, 8, seed=17, hub=700)
    x = randn((150, H, C), 18)
    a_s, a_d = randn((150, H), 19), randn((150, H), 20)
    xr = x.clone().requires_grad_(True)
    asr, adr = a_s.clone().requires_grad_(True), a_d.clone().requires_grad_(True)
    ev = oracle.torch_edge_softmax_opwise(ptr, idx, asr, adr, idx.shape[0], 0.2)
    ref = oracle.torch_spmm_index_add(xr, ptr, idx, 150, edge_val=ev)
    go = randn(ref.shape, 21)
    ref.backward(go)
    p, i = ptr.cuda(), idx.cuda()
    xg = x.cuda().requires_grad_(True)
    asg, adg = a_s.cuda().requires_grad_(True), a_d.cuda().requires_grad_(True)
    val = be.edge_attention(p, i, adg, asg, idx.shape[0], 0.2)
    out = be.sage_sum_forward_edge_value(xg, p, i, val, 150)
    assert rel_err(out.detach().cpu(), ref.detach()) < 1e-5
    out.backward(go.cuda())
    assert rel_err(xg.grad.cpu(), xr.grad) < 1e-5
    assert rel_err(asg.grad.cpu(), asr.grad) < 1e-4
    assert rel_err(adg.grad.cpu(), adr.grad) < 1e-4


@pytest.mark.parametrize("heads,c", [(4, 32), (3, 20), (1, 7)])
def test_gat_scores_forward_backward(cuda, heads, c):
    """Both attention scores in one kernel against the reference's multiply + sum pairs
    (cxgnncomp/graph_conv.py:470-474), values and gradients."""
    import cxgnncomp_backend as be
    feat = randn((300, heads, c), 40)
    a_s, a_d = randn((1, heads, c), 41), randn((1, heads, c), 42)
    f1, s1, d1 = (t.cuda().requires_grad_(True) for t in (feat, a_s, a_d))
    got_s, got_d = be.gat_scores(f1, s1, d1, 120)
    f2, s2, d2 = (t.double().requires_grad_(True) for t in (feat, a_s, a_d))
    want_s, want_d = (f2 * s2).sum(-1), (f2[:120] * d2).sum(-1)
    assert got_s.shape == (300, heads) and got_d.shape == (120, heads)
    assert rel_err(got_s.detach().cpu(), want_s.detach()) < 1e-6 and rel_err(got_d.detach().cpu(), want_d.detach()) < 1e-6
    gs, gd = randn(want_s.shape, 43), randn(want_d.shape, 44)
    (got_s * gs.cuda()).sum().backward(retain_graph=True)
    (got_d * gd.cuda()).sum().backward()
    ((want_s * gs.double()).sum() + (want_d * gd.double()).sum()).backward()
    for a, b in ((f1, f2), (s1, s2), (d1, d2)):
        assert rel_err(a.grad.cpu(), b.grad) < 1e-5
