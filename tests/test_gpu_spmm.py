"""CUDA SpMM through the C ABI against the CPU oracle.

Forward: bit-exact. Rows that lie inside one edge tile are summed in CSR order like the
reference's kernels (oracle.spmm); rows that cross tile borders are summed tile by tile and the
oracle repeats that order when given the tile size (oracle.spmm(..., tile=T)). Every result is
also held to 1e-5 (fp32) of the float64 sum. Backward: 1e-5 against float64 (atomic order is
not fixed, in the reference either)."""
import pytest
import torch

import oracle
from helpers import random_csr, randn, rel_err

pytestmark = pytest.mark.gpu
TILE = 64


@pytest.fixture(autouse=True)
def _fixed_tile():
    import cxgnncomp_backend as be
    old = be.SPLIT_EDGES
    be.SPLIT_EDGES = TILE
    yield
    be.SPLIT_EDGES = old


def _gpu(*ts):
    return [None if t_ is None else t_.cuda() for t_ in ts]


def _streams(x, heads=1, mask=False):
    """True when the library takes its streaming path for this feature matrix."""
    row_bytes = x[0].numel() * x.element_size()
    if mask or row_bytes % 16 or row_bytes > 1024:
        return False
    if heads > 1:
        cb = 16 if row_bytes > 256 else (8 if row_bytes > 128 else 4)
        if (x.shape[-1] * x.element_size()) % cb or heads > 16:
            return False
    return True


def _want(ptr, idx, x, heads=1, **kw):
    """Oracle output in the order the library uses for this shape (hub rows in these tests are
    shorter than the split of the row-per-group path, so that path is plainly sequential)."""
    return oracle.spmm(ptr, idx, x, tile=TILE if _streams(x, heads) else 0, **kw)


@pytest.mark.parametrize("feat", [1, 4, 31, 32, 33, 47, 64, 100, 128, 256, 300, 512])
@pytest.mark.parametrize("mean", [False, True])
def test_sum_mean_fp32_bit_exact(cuda, feat, mean):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(300, 257, 9, seed=feat, hub=60)
    x = randn((257, feat), feat + 1)
    want = _want(ptr, idx, x, mean=mean)
    p, i, xg = _gpu(ptr, idx, x)
    fn = be.sage_mean_forward if mean else be.sage_sum_forward
    got = fn(xg, p, i, 300).cpu()
    assert torch.equal(got, want)
    assert rel_err(got, oracle.spmm_f64(ptr, idx, x, mean=mean)) < 1e-5
    if not mean:
        got32 = be.run_spmm_configurable_int32(p.int(), i.int(), xg, 300, 1, 1, 32, 8, 8, 32, 32, 0, 0).cpu()
        assert torch.equal(got32, want)


@pytest.mark.parametrize("feat", [16, 64, 128, 256, 40, 512])
def test_bf16_bit_exact(cuda, feat):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(200, 200, 12, seed=40 + feat, hub=60)
    x = randn((200, feat), 41, dtype=torch.bfloat16)
    p, i, xg = _gpu(ptr, idx, x)
    got = be.sage_sum_forward(xg, p, i, 200).cpu()
    assert got.dtype == torch.bfloat16
    assert torch.equal(got.view(torch.int16), _want(ptr, idx, x).view(torch.int16))
    gm = be.sage_mean_forward(xg, p, i, 200).cpu()
    assert torch.equal(gm.view(torch.int16), _want(ptr, idx, x, mean=True).view(torch.int16))


def test_empty_and_ragged(cuda):
    import cxgnncomp_backend as be
    # all rows empty
    ptr = torch.zeros(11, dtype=torch.int64)
    idx = torch.zeros(0, dtype=torch.int64)
    x = randn((5, 8), 1)
    p, i, xg = _gpu(ptr, idx, x)
    assert torch.all(be.sage_sum_forward(xg, p, i, 10) == 0)
    assert torch.all(be.sage_mean_forward(xg, p, i, 10) == 0)
    # leading and trailing empty rows around a few edges
    ptr = torch.tensor([0, 0, 0, 3, 3, 5, 5, 5], dtype=torch.int64)
    idx = torch.tensor([1, 4, 2, 0, 3], dtype=torch.int64)
    p, i = _gpu(ptr, idx)
    got = torch.full((7, 8), 7.0, device="cuda")
    be._spmm_forward(xg, p, i, 7, out=got)
    assert torch.equal(got.cpu(), oracle.spmm(ptr, idx, x))
    # num_node == 0 means "all rows" (aggr.cu:118); a prefix of the rows otherwise
    ptr, idx = random_csr(50, 30, 3, seed=2)
    x = randn((30, 12), 3)
    p, i, xg = _gpu(ptr, idx, x)
    full = _want(ptr, idx, x)
    assert torch.equal(be.sage_sum_forward(xg, p, i, 0).cpu(), full)
    assert torch.equal(be.sage_sum_forward(xg, p, i, 17).cpu(), _want(ptr[:18], idx, x))
    # a single row holding every edge
    ptr = torch.tensor([0, 40], dtype=torch.int64)
    idx = torch.arange(40, dtype=torch.int64) % 30
    p, i = _gpu(ptr, idx)
    assert torch.equal(be.sage_sum_forward(xg, p, i, 1).cpu(), _want(ptr, idx, x))


@pytest.mark.parametrize("tile", [1, 7, 32, 100, 512])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tiles_and_long_rows(cuda, tile, dtype):
    """Hub rows spanning many tiles, including chains beyond 64 partials (blocked addition)."""
    import cxgnncomp_backend as be
    be.SPLIT_EDGES = tile
    ptr, idx = random_csr(120, 90, 20, seed=tile, hub=5000)
    x = randn((90, 128), 5, dtype=dtype)
    p, i, xg = _gpu(ptr, idx, x)
    got = be.sage_sum_forward(xg, p, i, 120)
    again = be.sage_sum_forward(xg, p, i, 120)
    assert torch.equal(got, again)
    want = oracle.spmm(ptr, idx, x, tile=tile)
    assert torch.equal(got.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    assert rel_err(got.cpu(), oracle.spmm_f64(ptr, idx, x)) < tol
    gm = be.sage_mean_forward(xg, p, i, 120).cpu()
    assert torch.equal(gm, oracle.spmm(ptr, idx, x, mean=True, tile=tile))


@pytest.mark.parametrize("tile", [32, 64, 256, 512])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
def test_index_ring_variant(cuda, tile, idx_dtype):
    """CXG_SPMM_TMA_INDEX: source ids staged by bulk copies (two 512-byte chunks per warp) give the oracle's bits
    for every row width of the lean walk, edge counts that are not multiples of 16 bytes, tiles of one and of
    several chunks, id arrays that start 16 bytes into an allocation, and id arrays whose start is not 16-byte
    aligned (those take the per-lane loads)."""
    import cxgnncomp_backend as be
    be.SPLIT_EDGES = tile
    for seed in range(4):
        ptr, idx = random_csr(500, 400, 9, seed=100 + seed, hub=3000 + seed)
        for dtype, feat in ((torch.float32, 32), (torch.float32, 64), (torch.float32, 128),
                            (torch.bfloat16, 64), (torch.bfloat16, 128), (torch.bfloat16, 256)):
            x = randn((400, feat), 7 + seed, dtype=dtype)
            p, xg = ptr.cuda(), x.cuda()
            want = oracle.spmm(ptr, idx, x, tile=tile)
            pad = torch.zeros(idx.shape[0] + 4, dtype=idx_dtype, device="cuda")
            for off in (0, 4 if idx_dtype == torch.int32 else 2, 1):
                i = pad[off:off + idx.shape[0]]
                i.copy_(idx)
                got = be._spmm_forward(xg, p, i, 500, flags=be.CXG_SPMM_TMA_INDEX)
                assert torch.equal(got.cpu(), want), (seed, dtype, feat, off)
            acc = got.clone()
            be._spmm_forward(xg, p, i, 500, out=acc, accumulate=True, flags=be.CXG_SPMM_TMA_INDEX)
            plain = got.clone()
            be._spmm_forward(xg, p, i, 500, out=plain, accumulate=True)
            assert torch.equal(acc, plain)
        gm = be._spmm_forward(xg, p, i, 500, reduce=be.CXG_MEAN, flags=be.CXG_SPMM_TMA_INDEX)
        assert torch.equal(gm.cpu(), oracle.spmm(ptr, idx, x, mean=True, tile=tile))


@pytest.mark.parametrize("split", [8, 32, 100])
def test_row_per_group_path_split_rows(cuda, split):
    """Widths outside the streaming path (here 4 KiB rows): long rows are cut into segments whose
    partials are added in a fixed order: reproducible, and within 1e-5 of float64."""
    import cxgnncomp_backend as be
    be.SPLIT_EDGES = split
    ptr, idx = random_csr(120, 90, 20, seed=split, hub=3000)
    x = randn((90, 1024), 5)
    p, i, xg = _gpu(ptr, idx, x)
    got = be.sage_sum_forward(xg, p, i, 120)
    assert torch.equal(got, be.sage_sum_forward(xg, p, i, 120))
    assert rel_err(got.cpu(), oracle.spmm_f64(ptr, idx, x)) < 1e-5
    deg = ptr[1:] - ptr[:-1]
    short = deg <= split
    assert torch.equal(got.cpu()[short], oracle.spmm(ptr, idx, x)[short])
    gm = be.sage_mean_forward(xg, p, i, 120).cpu()
    assert rel_err(gm, oracle.spmm_f64(ptr, idx, x, mean=True)) < 1e-5


def test_edge_value_single_and_multi_head(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(150, 140, 8, seed=7, hub=60)
    g = torch.Generator().manual_seed(8)
    x = randn((140, 64), 9)
    val = torch.rand(idx.shape[0], generator=g)
    p, i, xg, vg = _gpu(ptr, idx, x, val)
    assert torch.equal(be.sage_sum_forward_edge_value(xg, p, i, vg, 150).cpu(), _want(ptr, idx, x, edge_val=val))
    for heads, c in [(4, 32), (2, 64), (8, 8), (3, 5), (4, 4)]:
        xh = randn((140, heads, c), 10 + heads)
        vh = torch.rand(idx.shape[0], heads, generator=g)
        want = _want(ptr, idx, xh, heads=heads, edge_val=vh)
        xhg, vhg = _gpu(xh, vh)
        assert torch.equal(be.sage_sum_forward_edge_value(xhg, p, i, vhg, 150).cpu(), want)
        naive = be.spmm_multihead(p, i, vhg, xhg, 150, be.SPMM_MULTIHEAD_SCHEDULE.Naive).cpu()
        assert torch.equal(naive, want)
        pre = be.spmm_multihead(p, i, vhg, xhg, 150, be.SPMM_MULTIHEAD_SCHEDULE.PreReduce).cpu()
        # reference check: sum(Naive, dim=1) vs PreReduce at 1e-2 (test/1-kernels/perf-spmm-multihead.py:47-53)
        assert rel_err(pre, want.double().sum(1)) < 1e-5
    with pytest.raises(RuntimeError, match="mean with edge value"):
        be.sage_mean_forward_edge_value(xg, p, i, vg, 150)


def test_mask_target_rel_accumulate(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(80, 70, 6, seed=11, hub=60)
    g = torch.Generator().manual_seed(12)
    x = randn((70, 32), 13)
    mask = torch.rand(idx.shape[0], generator=g) < 0.5
    base = randn((80, 32), 14)
    p, i, xg, mg = _gpu(ptr, idx, x, mask)
    out = base.clone().cuda()
    be.selective_aggr(xg, p, i, mg, out, 80)
    assert torch.equal(out.cpu(), oracle.spmm(ptr, idx, x, edge_mask=mask, out=base.clone()))
    perm = torch.randperm(80, generator=g)
    out = base.clone().cuda()
    be.target_aggr(xg, p, i, perm.cuda(), out, 80)
    assert torch.equal(out.cpu(), _want(ptr, idx, x, targets=perm, out=base.clone()))
    rel = torch.randint(0, 3, (idx.shape[0],), generator=g, dtype=torch.int32)
    xr = randn((210, 32), 15)
    got = be.aggr_rel(xr.cuda(), p, i, rel.cuda(), 80, 3).cpu()
    assert torch.equal(got, _want(ptr, idx, xr, edge_rel=rel, rel_stride=70))


def test_backward_sum_mean_value(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(130, 110, 7, seed=16, hub=900)
    x = randn((110, 128), 17)
    dy = randn((130, 128), 18)
    p, i = _gpu(ptr, idx)
    for mean in (False, True):
        xg = x.cuda().requires_grad_(True)
        y = (be.sage_mean_forward if mean else be.sage_sum_forward)(xg, p, i, 130)
        y.backward(dy.cuda())
        dx, _ = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape, mean=mean)
        assert rel_err(xg.grad.cpu(), dx) < 1e-5
    raw = be.run_spmm_configurable_bwd(p, i, x.cuda(), dy.cuda(), 130, 1, 1, 1, 1, 1, 1, 32, 0, 0).cpu()
    assert rel_err(raw, oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)[0]) < 1e-5
    # edge values with gradients for both x and the values, 1 head and 4 heads
    g = torch.Generator().manual_seed(19)
    for shape, vshape in [((110, 64), (idx.shape[0],)), ((110, 4, 32), (idx.shape[0], 4))]:
        xv = randn(shape, 20)
        val = torch.rand(vshape, generator=g)
        dyv = randn((130,) + shape[1:], 21)
        xg = xv.cuda().requires_grad_(True)
        vg = val.cuda().requires_grad_(True)
        y = be.sage_sum_forward_edge_value(xg, p, i, vg, 130)
        y.backward(dyv.cuda())
        dx, dval = oracle.spmm_bwd_f64(ptr, idx, dyv, xv.shape, x=xv, edge_val=val, need_dval=True)
        assert rel_err(xg.grad.cpu(), dx) < 1e-5
        assert rel_err(vg.grad.cpu(), dval.reshape(vshape)) < 1e-5


def test_backward_inplace_variants(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(60, 50, 5, seed=22, hub=300)
    g = torch.Generator().manual_seed(23)
    dy = randn((60, 4, 16), 24)
    val = torch.rand(idx.shape[0], 4, generator=g)
    p, i = _gpu(ptr, idx)
    grad_x = torch.zeros(50, 4, 16, device="cuda")
    be.spmm_multihead_bwd(p, i, val.cuda(), dy.cuda(), grad_x, 60)
    dx, _ = oracle.spmm_bwd_f64(ptr, idx, dy, (50, 4, 16), edge_val=val)
    assert rel_err(grad_x.cpu(), dx) < 1e-5
    mask = torch.rand(idx.shape[0], generator=g) < 0.4
    dy2 = randn((60, 24), 25)
    gx = torch.zeros(50, 24, device="cuda")
    be.selective_aggr_bwd(dy2.cuda(), p, i, mask.cuda(), gx, 60)
    assert rel_err(gx.cpu(), oracle.spmm_bwd_f64(ptr, idx, dy2, (50, 24), edge_mask=mask)[0]) < 1e-5
    perm = torch.randperm(60, generator=g)
    gx = torch.zeros(50, 24, device="cuda")
    be.target_aggr_backward(dy2.cuda(), p, i, perm.cuda(), gx, 60)
    assert rel_err(gx.cpu(), oracle.spmm_bwd_f64(ptr, idx, dy2, (50, 24), targets=perm)[0]) < 1e-5


def test_arxiv_shape_config(cuda):
    """Configuration 1: 169,343 nodes / 2,332,487 edges power-law graph, F = 128 fp32, forward and backward."""
    import cxgnncomp_backend as be
    from cxgnncomp import synthetic
    be.SPLIT_EDGES = 256
    n, e_und = synthetic.CONFIG_SHAPES["arxiv_like"]
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0)
    assert idx.shape[0] == 2 * e_und + n == 2_332_487
    x = synthetic.node_features(n, 128, seed=0)
    p, i, xg = _gpu(ptr, idx, x)
    xg.requires_grad_(True)
    y = be.sage_sum_forward(xg, p, i, n)
    yc = y.detach().cpu()
    assert torch.equal(yc, oracle.spmm(ptr, idx, x, tile=256))
    # rows inside one tile carry exactly the bits of the sequential (reference-order) sum
    inside = (ptr[:-1] // 256) == ((ptr[1:] - 1) // 256)
    assert int(inside.sum()) > n // 2
    assert torch.equal(yc[inside], oracle.spmm(ptr, idx, x)[inside])
    # per-row error relative to the row's largest magnitude, against float64
    exact = oracle.spmm_f64(ptr, idx, x)
    err = (yc.double() - exact).abs().amax(1) / exact.abs().amax(1).clamp(min=1e-30)
    deg = ptr[1:] - ptr[:-1]
    assert float(err[deg <= 4096].max()) < 1e-5
    assert rel_err(yc, exact) < 1e-5
    # hub rows (up to 94,797 terms): fp32 rounding grows with the row length for any order; the tiled
    # order must not be worse than the reference's sequential order
    seq_err = (oracle.spmm(ptr, idx, x).double() - exact).abs().amax(1) / exact.abs().amax(1).clamp(min=1e-30)
    assert float(err[deg > 4096].max()) <= max(1e-5, float(seq_err[deg > 4096].max()))
    dy = synthetic.node_features(n, 128, seed=1)
    y.backward(dy.cuda())
    dx, _ = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)
    # default path: forward kernel over the transposed graph (built on the device by this first backward);
    # no atomics, so the hub row of 94,797 terms is summed in a fixed tiled order
    assert rel_err(xg.grad.cpu(), dx) < 1e-5
    light = torch.bincount(idx, minlength=n) <= 4096
    assert rel_err(xg.grad.cpu()[light], dx[light]) < 1e-5
    # size-independent property: A is symmetric here with sorted rows, so A^T == A and the transposed-graph
    # backward is bit for bit the forward kernel on dy (AggrOP.backward relies on the symmetry,
    # cxgnncomp/graph_conv.py:57-77)
    fwd_on_dy = be.run_spmm_configurable(p, i, dy.cuda(), n)
    assert torch.equal(xg.grad, fwd_on_dy)
    # the atomic scatter (BACKWARD_MODE = "scatter", the reference's formulation) adds the hub row's terms in
    # no fixed order: its rounding error grows with sqrt(terms) and varies from run to run (7e-5 .. 1e-4 here)
    be.BACKWARD_MODE = "scatter"
    try:
        xs = x.cuda().requires_grad_(True)
        be.sage_sum_forward(xs, p, i, n).backward(dy.cuda())
    finally:
        be.BACKWARD_MODE = "auto"
    assert rel_err(xs.grad.cpu(), dx) < 3e-4
    assert rel_err(xs.grad.cpu()[light], dx[light]) < 1e-5


@pytest.mark.parametrize("feat", [128, 36, 7])
@pytest.mark.parametrize("rop", [0, 1, 2, 3])
def test_gspmm_bit_exact(cuda, feat, rop):
    """GSpMM_u / GSpMM_u_e (dgSPARSE surface: int32 CSR, fp32): every reduce op, every compute op, rows without
    edges, vector and scalar column paths; bit-exact against the C restatement."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(300, 260, 7, seed=50 + feat, hub=900)
    x = randn((260, feat), 51)
    val = randn((idx.shape[0],), 52).abs() + 0.5
    p32, i32 = ptr.int().cuda(), idx.int().cuda()
    got = be.GSpMM_u(p32, i32, x.cuda(), be.REDUCEOP(rop))
    assert torch.equal(got.cpu(), oracle.gspmm(ptr, idx, x, None, rop))
    for cop in range(4):
        got = be.GSpMM_u_e(p32, i32, val.cuda(), x.cuda(), be.REDUCEOP(rop), be.COMPUTEOP(cop))
        assert torch.equal(got.cpu(), oracle.gspmm(ptr, idx, x, val, rop, cop)), (rop, cop)
    if rop == 1:  # max against torch on the rows that have edges
        dst = oracle.dst_of_edges(ptr)
        want = torch.full((300, feat), float("-inf")).scatter_reduce_(0, dst[:, None].expand(-1, feat), x[idx], "amax")
        has = (ptr[1:] - ptr[:-1]) > 0
        assert torch.equal(be.GSpMM_u(p32, i32, x.cuda(), be.MAX).cpu()[has], want[has])


def test_multihead_head_sum(cuda):
    """spmm_multihead with the PreReduce / Optimal schedules returns the heads summed (spmm_host.cu:158-196)."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(200, 180, 6, seed=60)
    x = randn((180, 4, 32), 61)
    val = randn((idx.shape[0], 4), 62)
    naive = be.spmm_multihead(ptr.cuda(), idx.cuda(), val.cuda(), x.cuda(), 200, be.Naive)
    opt = be.spmm_multihead(ptr.cuda(), idx.cuda(), val.cuda(), x.cuda(), 200, be.Optimal)
    assert opt.shape == (200, 32)
    want = naive[:, 0].clone()
    for h in range(1, 4):
        want += naive[:, h]
    assert torch.equal(opt, want)


@pytest.mark.parametrize("mean", [False, True])
@pytest.mark.parametrize("with_val", [False, True])
def test_backward_over_transposed_graph(cuda, mean, with_val, monkeypatch):
    """dX = A^T dY as a forward aggregation over the cached transposed graph: equal to the float64 oracle within
    fp32 rounding, bit-identical from run to run (no atomics), and the same numbers as the scatter kernel."""
    import cxgnncomp_backend as be
    if mean and with_val:
        pytest.skip("sage_mean_forward_edge_value raises in the reference too")
    ptr, idx = random_csr(500, 450, 9, seed=33, hub=700)
    x = randn((450, 64), 34)
    dy = randn((500, 64), 35)
    val = randn((idx.shape[0],), 36) if with_val else None

    def grad(mode):
        monkeypatch.setattr(be, "BACKWARD_MODE", mode)
        xg = x.cuda().requires_grad_(True)
        if with_val:
            out = be.sage_sum_forward_edge_value(xg, ptr.cuda(), idx.cuda(), val.cuda(), 500)
        else:
            out = (be.sage_mean_forward if mean else be.sage_sum_forward)(xg, ptr.cuda(), idx.cuda(), 500)
        out.backward(dy.cuda())
        return xg.grad.cpu()

    want = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape, edge_val=val, mean=mean)[0]
    a, b, c = grad("transpose"), grad("transpose"), grad("scatter")
    assert torch.equal(a, b)
    assert rel_err(a, want) < 1e-6
    assert rel_err(c, want) < 1e-5
    # automatic mode: the transposed graph is built by the first backward of a graph and reused afterwards
    be._TRANSPOSE_CACHE.clear()
    p, i = ptr.cuda(), idx.cuda()
    monkeypatch.setattr(be, "BACKWARD_MODE", "auto")
    for k in range(3):
        xg = x.cuda().requires_grad_(True)
        be.sage_sum_forward(xg, p, i, 500).backward(dy.cuda())
        assert len(be._TRANSPOSE_CACHE) == 1
        assert torch.equal(xg.grad.cpu(), a) or mean or with_val


@pytest.mark.parametrize("dtype,width", [(torch.bfloat16, 128), (torch.float32, 128), (torch.float32, 5),
                                         (torch.bfloat16, 7), (torch.int64, 3)])
def test_gather_rows(cuda, dtype, width):
    """The pack kernel of the needed-rows exchange: out[i] = x[rows[i]], any even row size."""
    import cxgnncomp_backend as be
    g = torch.Generator().manual_seed(width)
    x = (torch.randn(1000, width, generator=g) * 100).to(dtype)
    rows = torch.randint(0, 1000, (2500,), generator=g)
    got = be.gather_rows(x.cuda(), rows.cuda())
    assert torch.equal(got.cpu(), x[rows])
    assert be.gather_rows(x.cuda(), rows[:0].cuda()).shape == (0, width)


def test_spmm_into_overwrites_and_accumulates(cuda):
    import cxgnncomp_backend as be
    ptr, idx = random_csr(300, 280, 7, seed=95, hub=400)
    x = randn((280, 64), 96)
    p, i, xg = ptr.cuda(), idx.cuda(), x.cuda()
    want = be.run_spmm_configurable(p, i, xg, 300)
    out = torch.full((300, 64), 7.0, device="cuda")
    assert be.spmm_into(out, p, i, xg, 300) is out and torch.equal(out, want)
    be.spmm_into(out, p, i, xg, 300, accumulate=True)
    assert rel_err(out.cpu(), 2 * want.cpu()) < 1e-6
    mean = torch.empty_like(out)
    be.spmm_into(mean, p, i, xg, 300, reduce="mean")
    assert torch.equal(mean, be._spmm_forward(xg, p, i, 300, reduce=be.CXG_MEAN))
    # the lean and the general instantiation of the tiled walk give the same bits, also when accumulating, and
    # so does the grid that leaves room on the SMs
    for dtype in (torch.float32, torch.bfloat16):
        xd = xg.to(dtype)
        y0 = randn((300, 64), 97).to(dtype).cuda()
        for acc in (False, True):
            lean, shared, general = y0.clone(), y0.clone(), y0.clone()
            be.spmm_into(lean, p, i, xd, 300, accumulate=acc)
            be.spmm_into(shared, p, i, xd, 300, accumulate=acc, share_sms=True)
            be._spmm_forward(xd, p, i, 300, out=general, accumulate=acc, flags=be.CXG_SPMM_GENERIC_WALK)
            assert torch.equal(lean, general) and torch.equal(shared, general)
