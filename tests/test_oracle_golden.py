"""The CPU oracle against fixtures produced by the reference's own pure-torch code
(tests/golden/make_golden.py), plus internal consistency of the oracle's two layers."""
import numpy as np
import torch

import oracle
from helpers import random_csr, randn, rel_err


def t(a):
    return torch.from_numpy(np.asarray(a))


def test_spmm_matches_reference_sparse_mm(golden):
    ptr, idx, x, val = t(golden["spmm_ptr"]), t(golden["spmm_idx"]), t(golden["spmm_x"]), t(golden["spmm_val"])
    # reference formulation: torch.sparse.mm on CSR (cxgnncomp/codegen/torch_spmm.py:4-9); the kernels are
    # validated against it at atol 1e-3 / rtol 1e-2 (test/1-kernels/valid_spmm.py:11-12). Tighter here.
    got = oracle.spmm(ptr, idx, x)
    assert torch.allclose(got, t(golden["spmm_sum"]), atol=1e-5, rtol=1e-5)
    got = oracle.spmm(ptr, idx, x, edge_val=val)
    assert torch.allclose(got, t(golden["spmm_val_sum"]), atol=1e-5, rtol=1e-5)
    # double-precision yardstick agrees too
    assert rel_err(oracle.spmm_f64(ptr, idx, x), t(golden["spmm_sum"])) < 1e-6


def test_spmm_oracle_vs_torch_formulations():
    ptr, idx = random_csr(200, 150, 7, seed=11, hub=900)
    x = randn((150, 24), 12)
    a = oracle.spmm(ptr, idx, x)
    b = oracle.torch_spmm_index_add(x, ptr, idx, 200)
    c = oracle.torch_spmm_sparse(x, ptr, idx, 200)
    assert rel_err(a, b) < 1e-5 and rel_err(a, c) < 1e-5
    m = oracle.spmm(ptr, idx, x, mean=True)
    assert rel_err(m, oracle.torch_spmm_index_add(x, ptr, idx, 200, mean=True)) < 1e-5
    # rows without edges give 0 for mean
    deg = ptr[1:] - ptr[:-1]
    assert torch.all(m[deg == 0] == 0)


def test_spmm_oracle_multihead_mask_rel_target():
    ptr, idx = random_csr(60, 50, 5, seed=13)
    x = randn((50, 4, 8), 14)
    val = torch.rand(idx.shape[0], 4, generator=torch.Generator().manual_seed(15))
    got = oracle.spmm(ptr, idx, x, edge_val=val)
    want = oracle.torch_spmm_index_add(x, ptr, idx, 60, edge_val=val)
    assert rel_err(got, want) < 1e-5
    # mask: same as removing the edges
    mask = torch.rand(idx.shape[0], generator=torch.Generator().manual_seed(16)) < 0.5
    x2 = randn((50, 16), 17)
    got = oracle.spmm(ptr, idx, x2, edge_mask=mask, out=torch.zeros(60, 16))
    dst = oracle.dst_of_edges(ptr)
    want = torch.zeros(60, 16).index_add_(0, dst[mask], x2[idx[mask]])
    assert rel_err(got, want) < 1e-5
    # relation-strided source rows (aggr_rel)
    rel = torch.randint(0, 3, (idx.shape[0],), generator=torch.Generator().manual_seed(18), dtype=torch.int32)
    xr = randn((150, 16), 19)
    got = oracle.spmm(ptr, idx, xr, edge_rel=rel, rel_stride=50)
    want = torch.zeros(60, 16).index_add_(0, dst, xr[rel.long() * 50 + idx])
    assert rel_err(got, want) < 1e-5
    # targets: output rows permuted, accumulated into an existing tensor
    perm = torch.randperm(60, generator=torch.Generator().manual_seed(20))
    base = randn((60, 16), 21)
    got = oracle.spmm(ptr, idx, x2, targets=perm, out=base.clone())
    want = base.clone()
    want[perm] += oracle.spmm(ptr, idx, x2)
    assert rel_err(got, want) < 1e-5


def test_spmm_oracle_bf16_rounding():
    ptr, idx = random_csr(40, 40, 6, seed=22)
    x = randn((40, 16), 23, dtype=torch.bfloat16)
    got = oracle.spmm(ptr, idx, x)
    want = oracle.spmm_f64(ptr, idx, x).to(torch.bfloat16)
    assert got.dtype == torch.bfloat16
    # fp32 accumulation then one rounding: at most one bf16 ulp from the exact result
    assert rel_err(got.float(), want.float()) < 2 ** -7


def test_spmm_bwd_oracle_matches_autograd():
    ptr, idx = random_csr(50, 40, 5, seed=24)
    x = randn((40, 2, 8), 25).requires_grad_(True)
    val = torch.rand(idx.shape[0], 2, generator=torch.Generator().manual_seed(26)).requires_grad_(True)
    y = oracle.torch_spmm_index_add(x, ptr, idx, 50, edge_val=val)
    dy = randn(y.shape, 27)
    y.backward(dy)
    dx, dval = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape, x=x.detach(), edge_val=val.detach(), need_dval=True)
    assert rel_err(dx, x.grad) < 1e-5 and rel_err(dval, val.grad) < 1e-5


def test_edge_softmax_matches_reference_opwise(golden):
    ptr, idx = t(golden["spmm_ptr"]), t(golden["spmm_idx"])
    a_s, a_d = t(golden["gat_att_src"]), t(golden["gat_att_dst"])
    got, mask = oracle.edge_softmax_fwd(ptr, idx, a_d, a_s, 0.2)
    # reference: MyGATConv.edge_softmax_opwise (cxgnncomp/graph_conv.py:437-448), differs by its 1e-16 epsilon
    assert torch.allclose(got, t(golden["gat_edge_value"]), atol=1e-6, rtol=1e-5)
    mine = oracle.torch_edge_softmax_opwise(ptr, idx, a_s, a_d, idx.shape[0], 0.2)
    assert torch.allclose(mine, t(golden["gat_edge_value"]), atol=1e-7, rtol=1e-6)
    # every non-empty row sums to 1 per head
    dst = oracle.dst_of_edges(ptr)
    sums = torch.zeros(ptr.shape[0] - 1, 4).index_add_(0, dst, got)
    deg = ptr[1:] - ptr[:-1]
    assert torch.allclose(sums[deg > 0], torch.ones_like(sums[deg > 0]), atol=1e-5)


def test_edge_softmax_bwd_matches_autograd():
    ptr, idx = random_csr(30, 30, 4, seed=28)
    a_s = randn((30, 3), 29).requires_grad_(True)
    a_d = randn((30, 3), 30).requires_grad_(True)
    ev = oracle.torch_edge_softmax_opwise(ptr, idx, a_s, a_d, idx.shape[0], 0.2)
    g = randn(ev.shape, 31)
    ev.backward(g)
    out, mask = oracle.edge_softmax_fwd(ptr, idx, a_d.detach(), a_s.detach(), 0.2)
    gd, gs = oracle.edge_softmax_bwd(ptr, idx, g, mask, out, 30, 0.2)
    assert torch.allclose(gs.float(), a_s.grad, atol=1e-5, rtol=1e-4)
    assert torch.allclose(gd.float(), a_d.grad, atol=1e-5, rtol=1e-4)


def test_sddmm_oracle():
    g = torch.Generator().manual_seed(32)
    src = torch.randint(0, 20, (100,), generator=g)
    dst = torch.randint(0, 15, (100,), generator=g)
    sf, df = randn((20, 4, 32), 33), randn((15, 32), 34)
    got = oracle.sddmm(src, dst, sf, df)
    want = (sf[src] * df[dst].unsqueeze(1)).sum(-1)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    dfh = randn((15, 4, 32), 35)
    got = oracle.sddmm(src, dst, sf, dfh, per_head=True)
    assert torch.allclose(got, (sf[src] * dfh[dst]).sum(-1), atol=1e-5, rtol=1e-5)


def test_gcn_norm_fixture(golden):
    ptr = t(golden["spmm_ptr"])
    deg = ptr[1:] - ptr[:-1]
    want = (1.0 / deg.float()).repeat_interleave(deg)
    assert torch.equal(want, t(golden["gcn_norm"]))


def test_rgcn_formulations_agree_with_reference(golden):
    ptr, idx, x = t(golden["spmm_ptr"]), t(golden["spmm_idx"]), t(golden["spmm_x"])
    w, rel = t(golden["rgcn_w"]), t(golden["rgcn_rel"])
    exact = oracle.typed_linear_f64(x, w, rel, src=idx)  # per-edge x[src] @ W[rel]
    dst = oracle.dst_of_edges(ptr)
    y = torch.zeros(64, w.shape[-1], dtype=torch.float64).index_add_(0, dst, exact)
    # reference: TypedLinearS2DSort (typed_linear.py:262-310) and RGCNOP_sorted (graph_conv.py:246-257)
    assert rel_err(y, t(golden["rgcn_s2dsort"])) < 1e-5
    assert rel_err(y, t(golden["rgcn_sorted"])) < 1e-5
    assert rel_err(oracle.torch_rgcn_sorted(x, w, ptr, idx, rel, 64), t(golden["rgcn_s2dsort"])) < 1e-5


def test_pad_rel_semantics():
    # TypedLinearE2EOP.preprocess (typed_linear.py:74-87): after padding, every relation's bucket is a multiple of thres
    thres, num_rel = 8, 5
    g = torch.Generator().manual_seed(36)
    types = torch.randint(0, num_rel, (203,), generator=g)
    types[types == 3] = 2  # one empty relation
    count = torch.bincount(types, minlength=num_rel)
    buf = torch.full((203 + num_rel * (thres - 1),), -7, dtype=torch.int64)
    buf[:203] = types
    padded, pidx = oracle.pad_rel(buf, count, thres, num_rel, 203, idx=torch.zeros_like(buf))
    assert torch.equal(padded[:203], types)
    tot = torch.bincount(padded, minlength=num_rel + 1)
    for r in range(num_rel):
        assert tot[r] % thres == 0 and tot[r] >= count[r] and tot[r] - count[r] < thres
    assert tot[num_rel] == num_rel * (thres - 1) - (tot[:num_rel] - count).sum()
    assert torch.all(pidx[203:] == -1)


def test_rel_schedule_oracle():
    ptr, idx = random_csr(30, 30, 4, seed=37)
    rel = torch.randint(0, 3, (idx.shape[0],), generator=torch.Generator().manual_seed(38), dtype=torch.int32)
    layers = torch.tensor([10, 20, 30], dtype=torch.int64)
    out = oracle.rel_schedule(ptr, idx, rel, layers, 3)
    assert len(out) == 10
    dst = oracle.dst_of_edges(ptr)
    total = 0
    for r in range(3):
        sp, si, st = out[3 * r:3 * r + 3]
        sel = rel == r
        assert torch.equal(si, idx[sel])
        assert torch.equal(st, torch.unique(dst[sel]))
        assert torch.equal(sp[1:] - sp[:-1], torch.bincount(dst[sel], minlength=30)[st])
        total += si.shape[0]
        for l in range(2):
            assert out[9][r, l] == int((st < layers[l]).sum())
    assert total == idx.shape[0]


def test_tiled_order_oracle():
    """The restatement of the CUDA kernel's tile-wise order: identical to the sequential sum when no row
    crosses a tile border, and within rounding of float64 otherwise."""
    ptr, idx = random_csr(100, 80, 6, seed=50, hub=3000)
    x = randn((80, 16), 51)
    seq = oracle.spmm(ptr, idx, x)
    assert torch.equal(oracle.spmm(ptr, idx, x, tile=1 << 40), seq)
    for tile in (1, 7, 64):
        t_ = oracle.spmm(ptr, idx, x, tile=tile)
        inside = (ptr[:-1] // tile) == ((ptr[1:] - 1).clamp(min=0) // tile)
        inside |= ptr[:-1] == ptr[1:]
        assert torch.equal(t_[inside], seq[inside])
        assert rel_err(t_, oracle.spmm_f64(ptr, idx, x)) < 1e-5
    m = oracle.spmm(ptr, idx, x, tile=7, mean=True)
    assert rel_err(m, oracle.spmm_f64(ptr, idx, x, mean=True)) < 1e-5


def test_gspmm_oracle_against_torch():
    """The C restatement of the dgSPARSE GSpMM against torch scatter formulations: max / min are exact, sum and
    mean agree to rounding, and the four compute ops follow the reference's operand order (x - v, x / v)."""
    from helpers import random_csr, randn
    ptr, idx = random_csr(90, 80, 5, seed=1, hub=120)
    x = randn((80, 12), 2)
    val = randn((idx.shape[0],), 3).abs() + 0.5
    dst = oracle.dst_of_edges(ptr)
    has = (ptr[1:] - ptr[:-1]) > 0
    ex = dst[:, None].expand(-1, 12)
    for cop, fn in enumerate((lambda v, t: v + t, lambda v, t: t - v, lambda v, t: v * t, lambda v, t: t / v)):
        e = fn(val[:, None], x[idx])
        mx = torch.full((90, 12), float("-inf")).scatter_reduce_(0, ex, e, "amax")
        mn = torch.full((90, 12), float("inf")).scatter_reduce_(0, ex, e, "amin")
        sm = torch.zeros(90, 12, dtype=torch.float64).index_add_(0, dst, e.double())
        assert torch.equal(oracle.gspmm(ptr, idx, x, val, 1, cop)[has], mx[has])
        assert torch.equal(oracle.gspmm(ptr, idx, x, val, 2, cop)[has], mn[has])
        assert float((oracle.gspmm(ptr, idx, x, val, 0, cop).double() - sm).abs().max()) < 1e-4
        mean = sm / (ptr[1:] - ptr[:-1]).clamp(min=1)[:, None]
        assert float((oracle.gspmm(ptr, idx, x, val, 3, cop).double() - mean).abs().max()) < 1e-5
        assert bool((oracle.gspmm(ptr, idx, x, val, 1, cop)[~has] == 0).all())  # rows without edges give 0


def test_sampler_oracle_properties():
    """The C restatement of the neighbour sampler: counts, membership, no position drawn twice, rows kept in CSR
    order, and uniform frequencies (degree 40, 5 draws, 4000 seeds: 1/8 each within 4 standard deviations)."""
    from helpers import random_csr
    ptr, idx = random_csr(200, 5000, 20, seed=4, hub=700)  # 5000 sources: duplicates within a row are rare
    frontier = torch.arange(200)
    out_ptr, out = oracle.sample_neighbors(ptr, idx, frontier, 8, 11)
    deg = ptr[1:] - ptr[:-1]
    assert torch.equal(out_ptr[1:] - out_ptr[:-1], deg.clamp(max=8))
    for r in range(200):
        row = idx[ptr[r]:ptr[r + 1]].tolist()
        got = out[out_ptr[r]:out_ptr[r + 1]].tolist()
        it = iter(row)
        assert all(any(g == v for v in it) for g in got)  # an ordered sub-sequence of the row
    ptr2, idx2 = torch.tensor([0, 40]), torch.arange(40)
    counts = torch.zeros(40)
    for s in range(4000):
        _, o = oracle.sample_neighbors(ptr2, idx2, torch.zeros(1, dtype=torch.int64), 5, s)
        assert o.unique().shape[0] == 5
        counts[o] += 1
    assert float((counts - 500).abs().max()) < 4 * (4000 * 0.125 * 0.875) ** 0.5
