"""Per-configuration measurements of the aggregation path (configurations 1, 2 and 4; `bench.py` covers 5).

    python bench_layers.py [--configs c1,c2,c3,c4] [--steps K]
    python -m torch.distributed.run --nproc-per-node P ... bench_layers.py      (configuration 3, one replica per GPU)

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


def config1(steps, flush, cpu=True):
    """GCN aggregation, 169,343 nodes / 2,332,487 edges, F = 128 fp32, forward and backward w.r.t. features.
    cpu=False skips the timing of the CPU formulation (the error checks against the oracle stay)."""
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
    want_b = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)[0]
    be.BACKWARD_MODE = "scatter"  # the reference's formulation: atomic adds, order not fixed
    bwd = gpu_ms(lambda: be.run_spmm_configurable_bwd(p, i, xg, dyg, n), steps, flush)
    err_b = rel(be.run_spmm_configurable_bwd(p, i, xg, dyg, n).cpu(), want_b)
    be.BACKWARD_MODE = "auto"  # default: forward kernel over the transposed graph, built on the device and cached
    t_build = gpu_ms(lambda: be.csr_transpose(p, i, n, n), steps, flush)

    def bwd_cold():
        be._TRANSPOSE_CACHE.clear()
        return be.run_spmm_configurable_bwd(p, i, xg, dyg, n)

    bwd_first = gpu_ms(bwd_cold, steps, flush)
    bwd_t = gpu_ms(lambda: be.run_spmm_configurable_bwd(p, i, xg, dyg, n), steps, flush)
    err_bt = rel(be.run_spmm_configurable_bwd(p, i, xg, dyg, n).cpu(), want_b)
    y = be.run_spmm_configurable(p, i, xg, n).cpu()
    err_f = rel(y, oracle.spmm_f64(ptr, idx, x))
    b_alg = 2 * n * 128 * 4 + nnz * 8 + (n + 1) * 8
    hbm = peaks()[0]
    out = {"config": "c1 GCN SpMM fwd/bwd (169,343 nodes, F=128 fp32, int64 idx)", "nodes": n, "nnz": nnz,
           "gpu_fwd_ms": fwd, "gpu_bwd_ms": bwd_t, "gpu_bwd_first_call_ms": bwd_first, "transpose_build_ms": t_build,
           "gpu_bwd_scatter_ms": bwd, "b_alg_bytes": b_alg, "fwd_GBps": b_alg / fwd / 1e6,
           "fwd_frac_hbm_peak": b_alg / fwd / 1e6 / hbm, "bwd_frac_hbm_peak": b_alg / bwd_t / 1e6 / hbm,
           "fwd_gflops": 2 * nnz * 128 / fwd / 1e6, "max_rel_err_fwd": err_f, "max_rel_err_bwd": err_bt,
           "max_rel_err_bwd_scatter": err_b,
           "note": "inputs (193 MB) fit the 126 MB L2 in large part: the kernel is latency / issue bound here, not HBM bound"}
    if cpu:
        xr = x.clone().requires_grad_(True)
        dst = oracle.dst_of_edges(ptr)

        def cpu_fb():
            xr.grad = None
            o = torch.zeros(n, 128).index_add_(0, dst, xr.index_select(0, idx))
            o.backward(dy)

        torch.set_num_threads(os.cpu_count() or 1)
        out.update({"cpu_fwd_sparse_mm_ms": cpu_ms(lambda: oracle.torch_spmm_sparse(x, ptr, idx, n)),
                    "cpu_fwd_bwd_index_add_ms": cpu_ms(cpu_fb), "cpu_cores": torch.get_num_threads()})
    return out


def config2(steps, flush, cpu=True):
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
    # the same layer with its linear transform and both of that transform's gradients on the library's tensor-core
    # kernels (an option of the layer)
    conv.tensor_core_linear = True
    fb()
    t_fb_tc, t_f_tc = gpu_ms(fb, steps, flush), gpu_ms(fwd, steps, flush)
    conv.tensor_core_linear = False
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
    c_fb = cpu_ms(cpu_fb, reps=3) if cpu else None
    # parity reference: the same formulation in float64 (in fp32 the CPU's own rounding of the 94,797-term hub
    # row is larger than the difference that is to be measured)
    x64 = x.double().requires_grad_(True)
    h64 = F.linear(x64, W.double()).view(-1, 4, 32)
    ev64 = oracle.torch_edge_softmax_opwise(ptr, idx, (h64 * a_s.double()).sum(-1), (h64 * a_d.double()).sum(-1), nnz, 0.2)
    ref = oracle.torch_spmm_index_add(h64, ptr, idx, n, edge_val=ev64).reshape(-1, 128) + conv.bias.detach().cpu().double()
    ref.backward(gc.double())
    fb()
    err = rel(fwd().cpu(), ref.detach())
    err_g = rel(xg.grad.cpu(), x64.grad)
    # fused aggregate bytes: x_src rows + scores in, out rows + values out, idx, ptr
    b_alg = 2 * n * 4 * (32 * 4 + 4) + nnz * (8 + 4 * 4) + (n + 1) * 8
    # the library's kernels of the layer, each against the HBM roofline with its own algorithmic bytes
    import cxgnncomp_backend as be
    hbm = peaks()[0]
    H = 4
    with torch.no_grad():
        h3 = F.linear(xg, conv.lin_src).view(-1, H, 32).contiguous()
        sc_s, sc_d = (h3 * conv.att_src).sum(-1).contiguous(), (h3 * conv.att_dst).sum(-1).contiguous()
        val = be.edge_attention(p, i, sc_d, sc_s, nnz, 0.2)
        dyh = go.view(-1, H, 32).contiguous()
        kern = {
            "edge_softmax_fwd": (gpu_ms(lambda: be.edge_attention(p, i, sc_d, sc_s, nnz, 0.2), steps, flush),
                                 2 * n * H * 4 + nnz * (8 + 5 * H) + (n + 1) * 8),
            "spmm_multihead_fwd": (gpu_ms(lambda: be.spmm_multihead(p, i, val, h3, n, be.Naive), steps, flush),
                                   2 * n * 128 * 4 + nnz * (8 + 4 * H) + (n + 1) * 8),
            "spmm_multihead_bwd_dx_dval": (gpu_ms(lambda: be._spmm_backward(dyh, h3, p, i, n, edge_val=val, need_dx=True,
                                                                           need_dval=True), steps, flush),
                                           3 * n * 128 * 4 + nnz * (8 + 8 * H) + (n + 1) * 8),
        }
    kernels = {k: {"ms": t, "b_alg_bytes": b, "GBps": b / t / 1e6, "frac_hbm_peak": b / t / 1e6 / hbm}
               for k, (t, b) in kern.items()}
    return {"config": "c2 GAT layer fwd+bwd (4 heads x 32)", "nodes": n, "nnz": nnz, "gpu_fwd_ms": t_f,
            "gpu_fwd_bwd_ms": t_fb, "gpu_fwd_ms_tensor_core_linear": t_f_tc, "gpu_fwd_bwd_ms_tensor_core_linear": t_fb_tc,
            "aggregate_b_alg_bytes": b_alg, "kernels": kernels, "cpu_fwd_bwd_ms": c_fb,
            "cpu_cores": torch.get_num_threads(), "max_rel_err_fwd": err, "max_rel_err_grad_x": err_g}


def config3(steps, flush, scale=1.0):
    """GraphSAGE (mean) mini-batch training, 2.449 M nodes / ~126 M edges, F 100 -> 256 -> 256 -> 47, 1024 seeds,
    fanouts 15 / 10 / 5 counted from the seeds, 8 % of the nodes as training set: epoch time with the stages of a
    step (sample, feature gather, forward + backward + Adam) timed apart, and the same step in the torch index_add
    formulation on the host cores."""
    import cxgnncomp
    import oracle
    from cxgnncomp import synthetic
    n, e_und = synthetic.CONFIG_SHAPES["products_like"]
    n, e_und = int(n * scale), int(e_und * scale)
    dev = torch.device("cuda")
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0, device=dev)
    x = synthetic.node_features(n, 100, seed=0, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    y = torch.randint(0, 47, (n,), device=dev, generator=g)
    train = torch.randperm(n, device=dev, generator=g)[:int(0.08 * n)]
    fanouts, bs = [15, 10, 5], 1024
    torch.manual_seed(0)
    model = cxgnncomp.SAGE(100, 256, 47, 3).cuda()
    opt = torch.optim.Adam(model.parameters(), lr=0.003, fused=True)
    sampler = cxgnncomp.NeighborSampler(ptr, idx, fanouts)
    nb = cxgnncomp.num_batches(train.shape[0], bs)
    cxgnncomp.train_epoch(model, opt, sampler, x, y, train, bs, epoch=0, max_batches=10)  # warm-up
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    losses = cxgnncomp.train_epoch(model, opt, sampler, x, y, train, bs, epoch=1)
    b.record()
    b.synchronize()
    epoch_ms, wall_ms = a.elapsed_time(b), (time.perf_counter() - t0) * 1e3
    # stages of a step over 20 batches, each stage once untimed first (the epoch above allocated its batches on the
    # producer's stream; the first pass on this stream pays for fresh device allocations)
    seeds_list = [train[i * bs:(i + 1) * bs] for i in range(20)]
    torch.cuda.empty_cache()

    def stage(fn):
        for i, s_ in enumerate(seeds_list):
            fn(i, s_)
        torch.cuda.synchronize()
        t = time.perf_counter()
        for i, s_ in enumerate(seeds_list):
            fn(i, s_)
        torch.cuda.synchronize()
        return (time.perf_counter() - t) * 1e3 / len(seeds_list)

    samples, batches = {}, {}

    def do_sample(i, s_):
        samples[i] = sampler.sample(s_, seed=i)

    def do_gather(i, s_):
        batches[i] = cxgnncomp.Batch(x[samples[i][0]], samples[i][1], samples[i][2], samples[i][3], samples[i][4],
                                     y=y[s_])

    t_sample = stage(do_sample)
    t_gather = stage(do_gather)

    def step(i, s_):
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.nll_loss(model(batches[i]), batches[i].y)
        loss.backward()
        opt.step()

    t_step = stage(step)
    nodes_per_batch = sum(int(s_[3][-1]) for s_ in samples.values()) / len(samples)
    edges_per_batch = sum(int(s_[4][-1]) for s_ in samples.values()) / len(samples)

    # the same step on the host cores: aggregation as index_add (the reference's CPU formulation), autograd
    torch.set_num_threads(os.cpu_count() or 1)
    params = {k: v.detach().cpu().clone().requires_grad_(True) for k, v in model.named_parameters()}
    cpu_opt = torch.optim.Adam(list(params.values()), lr=0.003)

    def cpu_step(bt):
        h, pc, ic = bt.x.cpu(), bt.ptr.cpu(), bt.idx.cpu()
        for i in range(3):
            nn_, ne_ = bt.num_node_in_layer[2 - i], bt.num_edge_in_layer[2 - i]
            wl, bl = params[f"convs.{i}.lin_l.weight"], params[f"convs.{i}.lin_l.bias"]
            if wl.shape[1] > wl.shape[0]:  # wide input: transform, then aggregate (graph_conv.py:142-152)
                agg = oracle.torch_spmm_index_add(h @ wl.t() + bl, pc[:nn_ + 1], ic[:ne_], nn_, mean=True)
            else:
                agg = oracle.torch_spmm_index_add(h, pc[:nn_ + 1], ic[:ne_], nn_, mean=True) @ wl.t() + bl
            h = agg + h[:nn_] @ params[f"convs.{i}.lin_r.weight"].t()
            if i != 2:
                h = torch.relu(torch.nn.functional.batch_norm(h, None, None, params[f"bns.{i}.weight"],
                                                              params[f"bns.{i}.bias"], training=True))
                h = torch.nn.functional.dropout(h, 0.5)
        cpu_opt.zero_grad()
        torch.nn.functional.nll_loss(h.log_softmax(-1), bt.y.cpu()).backward()
        cpu_opt.step()

    cpu_step(batches[0])
    ts = []
    for bt in (batches[1], batches[2], batches[3]):
        t = time.perf_counter()
        cpu_step(bt)
        ts.append((time.perf_counter() - t) * 1e3)
    cpu_step_ms = sorted(ts)[1]
    return {"config": "c3 GraphSAGE mini-batch training (100 -> 256 -> 256 -> 47)", "nodes": n, "nnz": int(idx.shape[0]),
            "fanouts_from_seeds": fanouts, "batch_size": bs, "train_fraction": 0.08, "batches_per_epoch": nb,
            "epoch_ms": epoch_ms, "epoch_wall_ms": wall_ms, "ms_per_batch": epoch_ms / nb,
            "stage_ms_per_batch": {"sample": t_sample, "feature_gather": t_gather, "forward_backward_adam": t_step},
            "nodes_per_batch": nodes_per_batch, "edges_per_batch": edges_per_batch,
            "loss_first_last": [float(losses[0]), float(losses[-1])],
            "cpu_step_ms_index_add_formulation": cpu_step_ms, "cpu_epoch_ms_extrapolated": cpu_step_ms * nb,
            "cpu_cores": torch.get_num_threads(),
            "note": "CPU step excludes sampling and feature gather (batches taken from the GPU sampler)"}


def config3_replicas(scale=1.0):
    """Configuration 3 as the reference's MultiModel runs it (cxgnncomp/trainer.py:14-59,307-344): one model
    replica, one sampler stream (seed 1000 + rank) and one epoch loop per GPU, no gradient exchange. Launched under
    torchrun with one rank per GPU; every rank trains one epoch of its own stream, the epoch time is the maximum over
    the ranks (device events) and the throughput is ranks x batches / that time. Rank 0 returns the record."""
    import torch.distributed as dist
    import cxgnncomp
    from cxgnncomp import synthetic
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    n, e_und = synthetic.CONFIG_SHAPES["products_like"]
    n, e_und = int(n * scale), int(e_und * scale)
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0, device=dev)  # every GPU holds the whole graph
    x = synthetic.node_features(n, 100, seed=0, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    y = torch.randint(0, 47, (n,), device=dev, generator=g)
    train = torch.randperm(n, device=dev, generator=g)[:int(0.08 * n)]
    bs = 1024
    torch.manual_seed(1000 + rank)
    model = cxgnncomp.SAGE(100, 256, 47, 3).cuda()
    opt = torch.optim.Adam(model.parameters(), lr=0.003, fused=True)
    sampler = cxgnncomp.NeighborSampler(ptr, idx, [15, 10, 5])
    nb = cxgnncomp.num_batches(train.shape[0], bs)
    cxgnncomp.train_epoch(model, opt, sampler, x, y, train, bs, epoch=1000 + rank, max_batches=10)  # warm-up
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    losses = cxgnncomp.train_epoch(model, opt, sampler, x, y, train, bs, epoch=2000 + rank)
    b.record()
    b.synchronize()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    rec = {"config": "c3 GraphSAGE mini-batch training, one replica and one batch stream per GPU, no gradient exchange",
           "n_gpus": world, "nodes": n, "nnz": int(idx.shape[0]), "fanouts_from_seeds": [15, 10, 5], "batch_size": bs,
           "train_fraction": 0.08, "batches_per_epoch_per_gpu": nb, "epoch_ms_max_over_ranks": ms,
           "batches_per_s_all_gpus": world * nb / (ms * 1e-3), "ms_per_batch_per_gpu": ms / nb,
           "loss_first_last_rank0": [float(losses[0]), float(losses[-1])]}
    if world > 1:
        dist.barrier()
    return rec if rank == 0 else None


def config4(steps, flush, scale=1.0, cpu=True, quick=False):
    """RGCN layer, 8 relations, 1.94 M nodes / 21 M edges, 128 -> 64: fp32 (error-compensated TF32, the default),
    fp32 with plain TF32 products (the reference's tl.dot precision) and bf16. quick=True times the default
    schedule only."""
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
    out = {"config": "c4 RGCN layer (8 relations, 128 -> 64, total in-degree normalisation)", "nodes": n, "nnz": nnz}
    pc, ic, rc = ptr.cpu(), idx.cpu(), rel_t.cpu()
    rows = torch.randint(0, n, (2000,), generator=torch.Generator().manual_seed(1)).sort().values.unique()
    for dtype, name, tf32 in ((torch.float32, "fp32", False), (torch.float32, "fp32_tf32", True),
                              (torch.bfloat16, "bf16", False)):
        torch.manual_seed(0)
        be.ALLOW_TF32 = tf32
        conv = cxgnncomp.MyRGCNConv(128, 64, 8).cuda().to(dtype)
        x = synthetic.node_features(n, 128, seed=0, device=dev, dtype=dtype)
        with torch.no_grad():
            t_sched = {}
            for sched in (() if quick else ("e2e", "fused_gather", "fused_scatter", "transform_first")):
                conv.schedule = sched
                conv(x, ptr, idx, rel_t, n)  # builds the relation buckets once, like the reference caches them
                t_sched[sched] = gpu_ms(lambda: conv(x, ptr, idx, rel_t, n), steps, flush)
            conv.schedule = "auto"
            conv(x, ptr, idx, rel_t, n)
            t_layer = gpu_ms(lambda: conv(x, ptr, idx, rel_t, n), steps, flush)
            if len(conv.preprocessed) == 0:
                conv.preprocessed = cxgnncomp.TypedLinearE2EOP.preprocess(conv.linear, rel_t)
            st, num_item, indices = conv.preprocessed[:3]
            xe = x[idx]
            t_mm = gpu_ms(lambda: be.typed_matmul_raw(xe, conv.linear.data, st, st.shape[0], nnz, src_idx=indices),
                          steps, flush)
            y = conv(x, ptr, idx, rel_t, n)
            # weight gradient of the per-edge typed linear (one launch; the reference loops torch.mm over the relations)
            ge = torch.randn(nnz, 64, device=dev).to(dtype)
            t_wg = gpu_ms(lambda: be.typed_wgrad(xe, ge, st, 8, nnz, idx=indices), steps, flush)
            del ge
        elem = 2 if dtype == torch.bfloat16 else 4
        flops = 2.0 * nnz * 128 * 64
        b_mm = nnz * (128 + 64) * elem + 8 * 128 * 64 * elem + nnz * 9
        b_fused = n * 128 * elem + n * 64 * elem + 8 * 128 * 64 * elem + nnz * 9  # gather -> matmul -> segment sum
        # parity on a row sample against float64
        W = conv.linear.detach().float().cpu()
        xc = x.float().cpu()
        errs = []
        for r in rows.tolist():
            e0, e1 = int(pc[r]), int(pc[r + 1])
            if e1 == e0:
                continue
            ref = oracle.typed_linear_f64(xc, W, rc[e0:e1], src=ic[e0:e1]).sum(0) / (e1 - e0)
            errs.append(float((y[r].float().cpu().double() - ref).abs().max() / ref.abs().max().clamp(min=1e-30)))
        out[name] = {"layer_ms": t_layer, "layer_ms_by_schedule": t_sched, "layer_b_alg_fused_bytes": b_fused,
                     "layer_frac_hbm_peak_fused_bytes": b_fused / t_layer / 1e6 / hbm,
                     "typed_matmul_ms": t_mm, "typed_matmul_tflops": flops / t_mm / 1e9,
                     "typed_matmul_frac_tensor_peak": flops / t_mm / 1e9 / tens,
                     "typed_matmul_b_alg_GBps": b_mm / t_mm / 1e6, "typed_matmul_frac_hbm_peak": b_mm / t_mm / 1e6 / hbm,
                     "typed_wgrad_ms": t_wg, "typed_wgrad_b_alg_GBps": nnz * (128 + 64) * elem / t_wg / 1e6,
                     "typed_wgrad_frac_hbm_peak": nnz * (128 + 64) * elem / t_wg / 1e6 / hbm,
                     "max_rel_err_sampled_rows": max(errs)}
        del conv, x, xe, y
        torch.cuda.empty_cache()
    be.ALLOW_TF32 = False
    if cpu:
        # CPU: the reference's sorted formulation on a 1/8 row sample (typed_linear.py:262-310)
        r1 = n // 8
        pc, ic, rc = ptr[:r1 + 1].cpu(), idx[:int(ptr[r1])].cpu(), rel_t[:int(ptr[r1])].cpu()
        xc = torch.randn(n, 128)
        W = torch.randn(8, 128, 64)
        torch.set_num_threads(os.cpu_count() or 1)
        out["cpu_sorted_formulation_ms_one_eighth_of_rows"] = cpu_ms(
            lambda: oracle.torch_rgcn_sorted(xc, W, pc, ic, rc, r1), reps=3)
        out["cpu_cores"] = torch.get_num_threads()
    return out


def quick(steps=5):
    """Configurations 1, 2 and 4 on the GPU only (no CPU timing): what bench.py adds to its line as "layers"."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    res = {}
    for name, fn in (("c1", lambda: config1(steps, flush, cpu=False)), ("c2", lambda: config2(steps, flush, cpu=False)),
                     ("c4", lambda: config4(steps, flush, cpu=False, quick=True))):
        t0 = time.time()
        try:
            res[name] = fn()
        except Exception as e:  # a layer record must not cost the headline line
            res[name] = {"error": f"{type(e).__name__}: {e}"}
        res[name]["wall_s"] = time.time() - t0
        torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c4")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--c4-scale", type=float, default=1.0, help="shrink configuration 4 (nodes and edges) by this factor")
    ap.add_argument("--c3-scale", type=float, default=1.0, help="shrink configuration 3 (nodes and edges) by this factor")
    ap.add_argument("--c4-default-only", action="store_true",
                    help="configuration 4: time the default schedule and the typed matmul only, no CPU timing "
                         "(a short launch list for profiler captures)")
    args = ap.parse_args()
    assert torch.cuda.is_available(), "needs a CUDA device"
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.configs == "c3r":
        # torchrun: the only multi-GPU layer record is configuration 3 as independent replicas
        rec = config3_replicas(args.c3_scale)
        if rec is not None:
            print(json.dumps(rec), flush=True)
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    table = {"c1": config1, "c2": config2, "c3": config3, "c4": config4}
    for c in args.configs.split(","):
        if c == "c4" and args.c4_default_only:
            res = config4(args.steps, flush, args.c4_scale, cpu=False, quick=True)
        elif c in ("c3", "c4"):
            res = table[c](args.steps, flush, args.c4_scale if c == "c4" else args.c3_scale)
        else:
            res = table[c](args.steps, flush)
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
