"""Per-configuration measurements of the aggregation path (configurations 1, 2 and 4; `bench.py` covers 5).

    python bench_layers.py [--configs c1,c2,c4] [--steps K]

Prints one JSON line per configuration: GPU time per pass (CUDA events, 256 MiB L2 flush between passes),
algorithmic bytes / flops and the fraction of the measured HBM (or tensor) peak, the reference's CPU
formulation timed on the host cores of the same box (torch index_add_ / segment softmax / per-relation
linear), and the largest relative error against the CPU oracle. Inputs are synthetic and seeded (see
cxgnncomp/synthetic.py).
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "cxgnn-compute_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def gpu_ms(fn, steps, flush):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def cpu_ms(fn, reps=5, budget=25.0):
    fn()
    ts, t0 = [], time.time()
    while len(ts) < reps and time.time() - t0 < budget:
        t = time.perf_counter()
        fn()
        ts.append((time.perf_counter() - t) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp(min=1e-30))


def config1(steps, flush):
    """GCN aggregation, 169,343 nodes / 2,332,487 edges, F = 128 fp32, forward and backward w.r.t. features."""
    import cxgnncomp_backend as be
    import oracle
    from cxgnncomp import synthetic
    n, e_und = synthetic.CONFIG_SHAPES["arxiv_like"]
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0)
    x = synthetic.node_features(n, 128, seed=0)
    dy = synthetic.node_features(n, 128, seed=1)
    p, i, xg, dyg = ptr.cuda(), idx.cuda(), x.cuda(), dy.cuda()
    nnz = idx.shape[0]
    fwd = gpu_ms(lambda: be.run_spmm_configurable(p, i, xg, n), steps, flush)
    bwd = gpu_ms(lambda: be.run_spmm_configurable_bwd(p, i, xg, dyg, n), steps, flush)
    bwd_sym = gpu_ms(lambda: be.run_spmm_configurable(p, i, dyg, n), steps, flush)  # AggrOP.backward on a symmetric graph
    y = be.run_spmm_configurable(p, i, xg, n).cpu()
    err_f = rel(y, oracle.spmm_f64(ptr, idx, x))
    err_b = rel(be.run_spmm_configurable_bwd(p, i, xg, dyg, n).cpu(), oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)[0])
    xr = x.clone().requires_grad_(True)
    dst = oracle.dst_of_edges(ptr)

    def cpu_fb():
        xr.grad = None
        out = torch.zeros(n, 128).index_add_(0, dst, xr.index_select(0, idx))
        out.backward(dy)

    torch.set_num_threads(os.cpu_count() or 1)
    c_fwd = cpu_ms(lambda: oracle.torch_spmm_sparse(x, ptr, idx, n))
    c_fb = cpu_ms(cpu_fb)
    b_alg = 2 * n * 128 * 4 + nnz * 8 + (n + 1) * 8
    return {"config": "c1 GCN SpMM fwd/bwd", "nodes": n, "nnz": nnz, "gpu_fwd_ms": fwd, "gpu_bwd_scatter_ms": bwd,
            "gpu_bwd_symmetric_ms": bwd_sym, "b_alg_bytes": b_alg, "fwd_GBps": b_alg / fwd / 1e6,
            "fwd_gflops": 2 * nnz * 128 / fwd / 1e6, "cpu_fwd_sparse_mm_ms": c_fwd, "cpu_fwd_bwd_index_add_ms": c_fb,
            "cpu_cores": torch.get_num_threads(), "max_rel_err_fwd": err_f, "max_rel_err_bwd": err_b}


def config2(steps, flush):
    """GAT layer, 4 heads x 32, 128-dim input, LeakyReLU 0.2, on the configuration-1 graph; forward + backward."""
    import cxgnncomp
    import oracle
    from cxgnncomp import synthetic
    n, e_und = synthetic.CONFIG_SHAPES["arxiv_like"]
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0)
    x = synthetic.node_features(n, 128, seed=0)
    torch.manual_seed(0)
    conv = cxgnncomp.MyGATConv(128, 32, heads=4, concat=True).cuda()
    p, i = ptr.cuda(), idx.cuda()
    xg = x.cuda().requires_grad_(True)
    go = synthetic.node_features(n, 128, seed=2).cuda()
    nnz = idx.shape[0]

    def fb():
        xg.grad = None
        conv.zero_grad(set_to_none=True)
        conv(xg, p, i, n, n, nnz).backward(go)

    def fwd():
        with torch.no_grad():
            return conv(xg, p, i, n, n, nnz)

    t_fb, t_f = gpu_ms(fb, steps, flush), gpu_ms(fwd, steps, flush)
    W, a_s, a_d = conv.lin_src.detach().cpu(), conv.att_src.detach().cpu(), conv.att_dst.detach().cpu()
    xr = x.clone().requires_grad_(True)
    gc = go.cpu()

    def cpu_fb():
        xr.grad = None
        h = F.linear(xr, W).view(-1, 4, 32)
        ev = oracle.torch_edge_softmax_opwise(ptr, idx, (h * a_s).sum(-1), (h * a_d).sum(-1), nnz, 0.2)
        out = oracle.torch_spmm_index_add(h, ptr, idx, n, edge_val=ev).reshape(-1, 128)
        out.backward(gc)
        return out

    torch.set_num_threads(os.cpu_count() or 1)
    ref = cpu_fb().detach()
    c_fb = cpu_ms(cpu_fb, reps=3)
    fb()
    err = rel(fwd().cpu(), ref)
    err_g = rel(xg.grad.cpu(), xr.grad)
    # fused aggregate bytes: x_src rows + scores in, out rows + values out, idx, ptr
    b_alg = 2 * n * 4 * (32 * 4 + 4) + nnz * (8 + 4 * 4) + (n + 1) * 8
    return {"config": "c2 GAT layer fwd+bwd (4 heads x 32)", "nodes": n, "nnz": nnz, "gpu_fwd_ms": t_f,
            "gpu_fwd_bwd_ms": t_fb, "aggregate_b_alg_bytes": b_alg, "cpu_fwd_bwd_ms": c_fb,
            "cpu_cores": torch.get_num_threads(), "max_rel_err_fwd": err, "max_rel_err_grad_x": err_g}


def config4(steps, flush, scale=1.0):
    """RGCN layer, 8 relations, 1.94 M nodes / 21 M edges, 128 -> 64, fp32 (TF32 products) and bf16."""
    import cxgnncomp
    import cxgnncomp_backend as be
    import oracle
    from cxgnncomp import synthetic
    n, e_und = synthetic.CONFIG_SHAPES["rgcn_like"]
    n, e_und = int(n * scale), int(e_und * scale)  # scale < 1 keeps the mean degree (for profiler captures)
    dev = torch.device("cuda")
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0, device=dev)
    nnz = idx.shape[0]
    rel_t = synthetic.edge_relations(nnz, 8, seed=0, device=dev)
    hbm, tens, _ = peaks()
    out = {"config": "c4 RGCN layer (8 relations, 128 -> 64)", "nodes": n, "nnz": nnz}
    for dtype, name in ((torch.float32, "fp32_tf32"), (torch.bfloat16, "bf16")):
        torch.manual_seed(0)
        conv = cxgnncomp.MyRGCNConv(128, 64, 8).cuda().to(dtype)
        x = synthetic.node_features(n, 128, seed=0, device=dev, dtype=dtype)
        with torch.no_grad():
            t_sched = {}
            for sched in ("e2e", "fused_gather", "fused_scatter", "transform_first"):
                conv.schedule = sched
                conv(x, ptr, idx, rel_t, n)  # builds the relation buckets once, like the reference caches them
                t_sched[sched] = gpu_ms(lambda: conv(x, ptr, idx, rel_t, n), steps, flush)
            conv.schedule = "fused_gather"
            t_layer = t_sched["fused_gather"]
            st, num_item, indices = conv.preprocessed[:3]
            xe = x[idx]
            t_mm = gpu_ms(lambda: be.typed_matmul_raw(xe, conv.linear.data, st, st.shape[0], nnz, src_idx=indices),
                          steps, flush)
            y = conv(x, ptr, idx, rel_t, n)
        elem = 2 if dtype == torch.bfloat16 else 4
        flops = 2.0 * nnz * 128 * 64
        b_mm = nnz * (128 + 64) * elem + 8 * 128 * 64 * elem + nnz * 9
        # parity on a row sample against float64
        rows = torch.randint(0, n, (2000,), generator=torch.Generator().manual_seed(1)).sort().values.unique()
        pc, ic, rc = ptr.cpu(), idx.cpu(), rel_t.cpu()
        W = conv.linear.detach().float().cpu()
        xc = x.float().cpu()
        errs = []
        for r in rows.tolist():
            e0, e1 = int(pc[r]), int(pc[r + 1])
            if e1 == e0:
                continue
            ref = oracle.typed_linear_f64(xc, W, rc[e0:e1], src=ic[e0:e1]).sum(0) / (e1 - e0)
            errs.append(float((y[r].float().cpu().double() - ref).abs().max() / ref.abs().max().clamp(min=1e-30)))
        out[name] = {"layer_ms": t_layer, "layer_ms_by_schedule": t_sched, "typed_matmul_ms": t_mm, "typed_matmul_tflops": flops / t_mm / 1e9,
                     "typed_matmul_frac_tensor_peak": flops / t_mm / 1e9 / tens,
                     "typed_matmul_b_alg_GBps": b_mm / t_mm / 1e6, "typed_matmul_frac_hbm_peak": b_mm / t_mm / 1e6 / hbm,
                     "max_rel_err_sampled_rows": max(errs)}
        del conv, x, xe, y
        torch.cuda.empty_cache()
    # CPU: the reference's sorted formulation on a 1/8 row sample (typed_linear.py:262-310)
    r1 = n // 8
    pc, ic, rc = ptr[:r1 + 1].cpu(), idx[:int(ptr[r1])].cpu(), rel_t[:int(ptr[r1])].cpu()
    xc = torch.randn(n, 128)
    W = torch.randn(8, 128, 64)
    torch.set_num_threads(os.cpu_count() or 1)
    out["cpu_sorted_formulation_ms_one_eighth_of_rows"] = cpu_ms(lambda: oracle.torch_rgcn_sorted(xc, W, pc, ic, rc, r1),
                                                               reps=3)
    out["cpu_cores"] = torch.get_num_threads()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c4")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--c4-scale", type=float, default=1.0, help="shrink configuration 4 (nodes and edges) by this factor")
    args = ap.parse_args()
    assert torch.cuda.is_available(), "needs a CUDA device"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    table = {"c1": config1, "c2": config2, "c4": config4}
    for c in args.configs.split(","):
        res = table[c](args.steps, flush, args.c4_scale) if c == "c4" else table[c](args.steps, flush)
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
