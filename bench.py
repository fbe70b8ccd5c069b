"""Benchmark of the aggregation hot path: one step = one CSR SpMM pass (sum) over the whole graph.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0). `value` is the whole-job algorithmic HBM throughput in GB/s:
compulsory bytes of one pass (every touched feature row once in, every output row once out, the
index stream, the row pointers) divided by the step time, inputs resident in HBM. `e2e` is the
same metric through the `cxgnncomp_backend` call with the step's inputs copied from pinned host
memory and its output copied back inside the timed region. `roofline` compares the SpMM call
with the measured HBM copy bandwidth of the GPU (MEASURED_PEAKS.json next to this file, when present). `cpu_baseline` times the
reference's CPU formulation (torch index_add_ / sparse.mm, all host threads) on a bounded row
sample of the same workload.

With N > 1 (torchrun, one rank per GPU) rows are split contiguously by edge count; every step each
rank's feature shard is all-gathered over NCCL into every rank's local buffer
and aggregates its own rows; total work is fixed ("strong" scaling).

`--impl reference` times the reference's own CPU formulation only (rank 0), same metric and unit.
Inputs are synthetic (seeded power-law graphs, N(0,1) features): the reference's datasets are not
available offline.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "cxgnn-compute_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOADS = {
    # name: (nodes, undirected edges, feat, dtype, idx dtype, description)
    "papers_like": (111_000_000, 744_500_000, 128, "bf16", "int32",
                    "full-graph GCN aggregation, 111M nodes / 1.6B edges, F=128 bf16 (config 5)"),
    "products_like": (2_449_029, 61_850_000, 128, "bf16", "int32",
                      "2.45M nodes / 126M edges power-law graph, F=128 bf16 (graph of config 3)"),
    "papers_tenth": (11_100_000, 74_450_000, 128, "bf16", "int32",
                     "one tenth of config 5 (11.1M nodes / 160M edges, same mean degree), F=128 bf16: profiling case"),
    "arxiv_like": (169_343, 1_081_572, 128, "f32", "int64",
                   "GCN aggregation, 169,343 nodes / 2.33M edges, F=128 fp32 (config 1)"),
}
DTYPES = {"bf16": torch.bfloat16, "f32": torch.float32}
L2_FLUSH_BYTES = 256 << 20
# Peer-copy bandwidth into one GPU over NVLink that the exchange is compared with: 770 GB/s per direction was
# measured between B200s of the kind this benchmark targets (nominal 900); override with CXG_PEER_COPY_GBPS.
PEER_COPY_GBPS = float(os.environ.get("CXG_PEER_COPY_GBPS", "770"))
# what --exchange auto picks when the needed rows are few enough: "needed" (pack + NCCL all-to-all), "put" (one gather
# kernel storing into the peers' buffers) or "putcopy" (pack + copy-engine copies into the peers' buffers)
AUTO_EXCHANGE = os.environ.get("CXG_BENCH_AUTO_EXCHANGE", "put")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the tiled kernel on one GPU, from ncu
# captures of these workloads (profiles/spmm_stream_papers.md); None where no capture exists.
NCU_DRAM_BYTES = {"papers_like": 300.59e9, "papers_tenth": 24.67e9}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (6.65 TB/s, an earlier B200 copy-bandwidth measurement)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 8 for n, v in zip(names, r[4:8]) if v == "Active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def algorithmic_bytes(n_dst, n_src_touched, nnz, feat, elem, idx_bytes):
    """Compulsory bytes of one SpMM pass: touched input rows once, output rows once, idx, ptr."""
    return n_src_touched * feat * elem + n_dst * feat * elem + nnz * idx_bytes + (n_dst + 1) * 8


def cpu_baseline_sample(ptr, idx, feat, dtype, budget_s=20.0):
    """Times the reference's CPU formulation (torch index_add_ and sparse.mm, fp32, all host threads;
    test/2-benchmark/bench-gcn.py:45-60, cxgnncomp/codegen/torch_spmm.py:4-9) on a contiguous row sample
    of the workload. Source rows are compacted so that the sample's features fit host memory.
    `ptr`/`idx` may live on the GPU; only the sample is copied to the host."""
    import oracle
    n = ptr.shape[0] - 1
    nnz = int(ptr[n])
    torch.set_num_threads(os.cpu_count() or 1)
    want_edges = min(nnz, 8_000_000)
    r0 = n // 3
    r1 = int(torch.searchsorted(ptr, ptr[r0] + want_edges).clamp(max=n))
    r1 = max(r1, min(n, r0 + 1))
    e0, e1 = int(ptr[r0]), int(ptr[r1])
    sub_idx = idx[e0:e1].long()
    uniq, inv = torch.unique(sub_idx, return_inverse=True)
    sp = (ptr[r0:r1 + 1] - e0).cpu()
    si = inv.cpu()
    rows, n_src = r1 - r0, int(uniq.shape[0])
    x = torch.randn(n_src, feat, generator=torch.Generator().manual_seed(1))
    b_alg = algorithmic_bytes(rows, n_src, e1 - e0, feat, 4, 8)
    best = {}
    t_start = time.time()
    for name, fn in (("index_add", lambda: oracle.torch_spmm_index_add(x, sp, si, rows)),
                     ("sparse_mm", lambda: oracle.torch_spmm_sparse(x, sp, si, rows))):
        fn()  # warm-up
        ts = []
        while len(ts) < 5 and (time.time() - t_start) < budget_s:
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        if ts:
            best[name] = sorted(ts)[len(ts) // 2]
    form = min(best, key=best.get)
    # The metric is the algorithmic bytes of the WHOLE workload over the time of one pass. The CPU pass is
    # extrapolated from the sample by edge count (its time is per-edge gather work); the sample's own
    # algorithmic bytes per edge are several times the full graph's (few edges per distinct source), so its
    # own GB/s is reported separately and is not comparable with the GPU figure.
    elem = 2 if dtype == torch.bfloat16 else 4
    b_alg_full = algorithmic_bytes(n, n, nnz, feat, elem, idx.element_size())
    full_s = best[form] * (nnz / max(1, e1 - e0))
    return {"value": b_alg_full / full_s / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"rows [{r0},{r1}) of the workload = {rows} rows / {e1 - e0} edges / {n_src} distinct sources, "
                      f"fp32 int64, torch {form} (median of {len(ts)}), {best[form] * 1e3:.1f} ms; whole pass "
                      f"extrapolated by edge count ({nnz} edges): {full_s:.2f} s",
            "formulation": form, "ms": best[form] * 1e3, "extrapolated_pass_s": full_s,
            "sample_own_GBps": b_alg / best[form] / 1e9}


def load_synthetic():
    """cxgnncomp/synthetic.py (seeded generators, plain torch) loaded by path: importing the package would load
    the CUDA library, which the reference arm must not touch."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("cxg_synthetic", os.path.join(PKG, "cxgnncomp", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_workload(name, device, seed=0):
    synthetic = load_synthetic()
    n, e_und, feat, dt, it, desc = WORKLOADS[name]
    idx_dtype = torch.int32 if it == "int32" else torch.int64
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=seed, device=device, idx_dtype=idx_dtype)
    return ptr, idx, n, feat, DTYPES[dt], desc


def run_reference(args, rank):
    """The reference's CPU formulation on host cores (there is no CPU kernel in the reference; its
    torch formulation is what it validates against). Rank 0 only."""
    if rank != 0:
        return
    name = args.workload
    dev = torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
    ptr, idx, n, feat, dtype, desc = build_workload(name, dev)
    ts = []
    base = None
    for _ in range(args.warmup + args.steps):
        base = cpu_baseline_sample(ptr, idx, feat, dtype, budget_s=max(5.0, 60.0 / (args.warmup + args.steps)))
        ts.append(base["ms"])
    ms = sum(ts[args.warmup:]) / max(1, args.steps)
    base["value"] = base["value"] * base["ms"] / ms  # mean over the timed steps instead of the last one
    line = {"impl": "reference", "metric": "spmm_algorithmic_hbm_throughput", "value": base["value"], "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["extrapolated_pass_s"] * 1e3 * ms / base["ms"],  # one whole pass, extrapolated
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "description": desc, "nodes": n, "nnz": int(ptr[n]), "feat": feat,
                       "sample": base["sample"]},
            "extrapolated": True, "sample_ms_per_step": ms, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=os.environ.get("CXG_BENCH_WORKLOAD", "papers_like"),
                    choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", default="auto", choices=["auto", "allgather", "needed", "put", "putcopy"],
                    help="multi-GPU feature exchange: one padded all-gather; an all-to-all of only the rows each "
                         "rank's edges name (needed); or the same rows stored into the peers' buffers over NVLink by one "
                         "gather kernel (put) or by the copy engines (putcopy)")
    ap.add_argument("--exchange-chunks", type=int, default=int(os.environ.get("CXG_BENCH_EXCHANGE_CHUNKS", "0")),
                    help="needed-rows mode: cut every peer's rows into this many parts and send a part while the next "
                         "one is packed (0 = 4 parts on 2 GPUs, where it was measured; 1 part on more)")
    ap.add_argument("--overlap", default="auto", choices=["auto", "on", "off"],
                    help="aggregate the edges that read this rank's own rows while the exchange is in flight, then "
                         "accumulate the rest (auto = off: at 2 GPUs the second pass over the output rows costs what "
                         "the overlap hides, 45.1 vs 44.4 ms per step)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--backward", action="store_true",
                    help="also time the backward of the step (dX = A^T dY over the transposed local graph, then the "
                         "return of the remote rows' partial gradients to their owners) and add it as \"backward\"")
    ap.add_argument("--no-layers", action="store_true",
                    help="skip the per-layer records of configurations 1, 2 and 4 (added at 1 GPU by default)")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    # Libraries below (NCCL prints its version banner) write to file descriptor 1; keep it clean for the
    # one JSON line by pointing it at stderr until the result is printed.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch.distributed as dist
    import cxgnncomp_backend as be
    from cxgnncomp import synthetic
    from cxgnncomp.distributed import NeededRowsExchange, RowPartition, exchange_features, reduce_gradients

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ptr, idx, n, feat, dtype, desc = build_workload(args.workload, dev)
    nnz = int(ptr[n])
    elem = 2 if dtype == torch.bfloat16 else 4
    idx_bytes = idx.element_size()
    part = RowPartition(ptr, world)
    r0, r1 = part.rows(rank)
    ex, exchange_mode, remote_rows = None, "none", 0
    if world > 1:
        lptr, lidx = part.local_graph(ptr, idx, rank, gather_ids=False)
        full_ptr = ptr
        del idx
        torch.cuda.empty_cache()
        exchange_mode = args.exchange
        remote_all = (world - 1) * part.shard_rows
        if exchange_mode in ("auto", "needed", "put", "putcopy"):
            ex = NeededRowsExchange(part, lptr, lidx, rank, n)
            frac = torch.tensor([ex.remote_rows() / max(remote_all, 1)], dtype=torch.float64, device=dev)
            dist.all_reduce(frac, op=dist.ReduceOp.MAX)
            if exchange_mode == "auto":
                exchange_mode = AUTO_EXCHANGE if float(frac[0]) < 0.8 else "allgather"
        if exchange_mode in ("needed", "put", "putcopy"):
            lidx = ex.lidx
            remote_rows = ex.remote_rows()
        else:
            ex = None
            lidx = part.to_gather_ids(lidx)
            remote_rows = remote_all
    else:
        lptr, lidx, full_ptr = ptr, idx, ptr
    torch.cuda.empty_cache()
    n_local = r1 - r0

    # features: every rank draws the same stream. All-gather mode re-lays the matrix out as the
    # [world, shard_rows, F] gather buffer; needed-rows mode keeps this rank's shard followed by the remote
    # rows its edges name.
    x_full = synthetic.node_features(n, feat, seed=0, device=dev, dtype=dtype)
    send_buf = None
    if world > 1 and ex is None:
        xg = torch.zeros((part.gather_rows(), feat), dtype=dtype, device=dev)
        for j in range(world):
            b0, b1 = part.rows(j)
            part.shard(xg, j).copy_(x_full[b0:b1])
        x_full = xg
        del xg
        x_own = part.shard(x_full, rank)
    elif world > 1:
        xb = torch.empty((ex.buffer_rows(), feat), dtype=dtype, device=dev)  # [own shard | remote rows]
        ex.own(xb).copy_(x_full[r0:r1])
        x_full = xb
        del xb
        torch.cuda.empty_cache()
        x_own = ex.own(x_full)
        send_buf = torch.empty((ex.send_rows.shape[0], feat), dtype=dtype, device=dev)
    else:
        x_own = x_full
    y = torch.empty((n_local, feat), dtype=dtype, device=dev)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    b_alg_total = algorithmic_bytes(n, n, nnz, feat, elem, idx_bytes)
    b_alg_local = algorithmic_bytes(n_local, n, int(lptr[n_local]), feat, elem, idx_bytes)

    putters = {}
    if exchange_mode in ("put", "putcopy"):
        from cxgnncomp.distributed import PeerExchange
        put_chunks = args.exchange_chunks if args.exchange_chunks > 0 else 4
        put_mode = "kernel" if exchange_mode == "put" else "copy"
        try:
            putters[x_full.data_ptr()] = PeerExchange(ex, x_full, send_buf, mode=put_mode, chunks=put_chunks)
        except RuntimeError as e:  # raised on every rank together: no IPC between these processes
            sys.stderr.write(f"peer mappings unavailable ({e}); using the NCCL all-to-all\n")
            exchange_mode = "needed"
    # Overlap: the edges whose source is one of this rank's own rows are aggregated while the remote rows travel,
    # the rest is accumulated onto them afterwards (one more pass over the output rows)
    overlap = ex is not None and args.overlap == "on"
    exchange_chunks = args.exchange_chunks if args.exchange_chunks > 0 else (4 if world == 2 else 1)
    if overlap:
        seg_graphs = ex.segment_graphs(lptr, 1)  # [own-source edges, remote-source edges]
        comm_stream = torch.cuda.Stream()
        chunk_events = [torch.cuda.Event()]

    def exchange(buf=None):
        """The feature buffer (x_full by default) receives what this rank's aggregation reads: every shard (one
        NCCL all-gather) or the rows its edges name (pack + one NCCL all-to-all)."""
        buf = x_full if buf is None else buf
        if putters:
            putters[buf.data_ptr()].exchange()
        elif ex is not None:
            ex.exchange(buf, send_buf, chunks=exchange_chunks)
        else:
            exchange_features(buf, part, rank)

    def own_rows(buf):
        """This rank's own feature rows inside a feature buffer."""
        if world == 1:
            return buf
        return ex.own(buf) if ex is not None else part.shard(buf, rank)

    def aggregate_segments(buf, out, wait=True):
        """Own-source edges first, then one accumulating pass over the edges that read remote rows as soon as the
        exchange is complete (fixed order of additions)."""
        main = torch.cuda.current_stream()
        share = exchange_mode == "needed"  # NCCL's copy kernels need room on the SMs; copy engines do not
        be.spmm_into(out, seg_graphs[0][0], seg_graphs[0][1], buf, n_local, share_sms=share)
        if wait:
            main.wait_event(chunk_events[0])
        return be.spmm_into(out, seg_graphs[1][0], seg_graphs[1][1], buf, n_local, accumulate=True)

    def step(buf=None, out=None):
        buf = x_full if buf is None else buf
        out = y if out is None else out
        if overlap:
            comm_stream.wait_stream(torch.cuda.current_stream())  # the own rows of buf are in place
            with torch.cuda.stream(comm_stream):
                exchange(buf)
                chunk_events[0].record(comm_stream)
            return aggregate_segments(buf, out)
        if world > 1:
            exchange(buf)
        return be.spmm_into(out, lptr, lidx, buf, n_local)

    def timed(fn, k):
        """k calls of fn, each between its own pair of events on the current stream, L2 flushed before."""
        total = 0.0
        for _ in range(k):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            total += a.elapsed_time(b)
        return total

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = be.kernel_launch_count()
    ms_total = timed(step, args.steps)
    launches = be.kernel_launch_count() - launches0
    barrier()
    # kernel-only time of the SpMM call (no exchange), for the roofline
    spmm_ms = timed(lambda: be.spmm_into(y, lptr, lidx, x_full, n_local), args.steps) / args.steps
    barrier()
    # the segmented aggregation alone (rows already exchanged): what the step costs beyond it is exposed exchange
    seg_ms = timed(lambda: aggregate_segments(x_full, y, wait=False), args.steps) / args.steps if overlap else spmm_ms
    barrier()
    exch_ms = timed(exchange, args.steps) / args.steps if world > 1 else 0.0
    barrier()
    clocks = sampler.stop() if sampler else None

    t = torch.tensor([ms_total, spmm_ms, exch_ms, float(remote_rows), seg_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0]) / args.steps
    spmm_ms = float(t[1])
    exch_ms, remote_rows_max, seg_ms = float(t[2]), int(t[3]), float(t[4])
    value = b_alg_total / (ms_step * 1e-3) / 1e9

    # end to end: inputs from pinned host memory, result back to the host, every step
    e2e = None
    if not args.no_e2e:
        hx = torch.empty(x_own.shape, dtype=dtype).pin_memory()
        hx.copy_(x_own)
        hy = torch.empty(y.shape, dtype=dtype).pin_memory()

        ksteps = min(args.steps, 5)
        # The graph (ptr, idx) does not change between steps and stays on the device, like a layer's weights; what
        # a step brings in is the feature matrix and what it returns is the aggregated matrix.
        # Double-buffered: the upload of step k+1 runs on its own stream while step k aggregates and step k-1's
        # result returns to the host (the link is full duplex), so a step costs max(upload, download), not their sum.
        xb, yb = [x_full, torch.empty_like(x_full)], [y, torch.empty_like(y)]
        if putters:
            putters[xb[1].data_ptr()] = PeerExchange(ex, xb[1], send_buf, mode=put_mode, chunks=put_chunks)
        s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def run_pipelined(k_steps):
            for k in range(k_steps):
                b = k & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_comp[b])  # the aggregation that last read this buffer
                    own_rows(xb[b]).copy_(hx, non_blocking=True)
                    ev_in[b].record(s_in)
                s_main.wait_event(ev_in[b])
                s_main.wait_event(ev_out[b])  # the download that last read this output buffer
                step(xb[b], yb[b])
                ev_comp[b].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[b])
                    hy.copy_(yb[b], non_blocking=True)
                    ev_out[b].record(s_out)
            s_main.wait_event(ev_out[0])
            s_main.wait_event(ev_out[1])

        run_pipelined(2)
        barrier()
        a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_ev.record()
        run_pipelined(ksteps)
        b_ev.record()
        b_ev.synchronize()
        e_ms = a_ev.elapsed_time(b_ev) / ksteps
        if putters:
            putters.pop(xb[1].data_ptr()).close()
        del xb, yb
        barrier()
        te = torch.tensor([e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        h2d = hx.numel() * elem
        d2h = hy.numel() * elem
        e2e = {"value": b_alg_total / (float(te[0]) * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": float(te[0]),
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": ksteps,
               "api": ("cxgnncomp_backend.spmm_into (cxg_spmm_csr with a caller-owned output); every step the feature "
                       "matrix comes from pinned host memory and the aggregated matrix goes back to it, the graph "
                       "(ptr, idx) stays on the device; two buffer sets: upload of step k+1, exchange + aggregation "
                       "of step k and download of step k-1 overlap")}
        del hx, hy

    # backward of the step (not part of the headline): every rank aggregates the upstream gradient of its rows over
    # its transposed local graph into a gradient in the layout of the feature buffer, then the partial gradients of
    # remote rows go back to their owners (needed-rows plans: all-to-all + an accumulating aggregation over the
    # transposed request list; all-gather layout: one reduce-scatter)
    backward = None
    if args.backward:
        n_src = x_full.shape[0]
        a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_ev.record()
        t_ptr, t_idx, _, _ = be.csr_transpose(lptr, lidx, n_local, n_src, want_eid=False)
        b_ev.record()
        b_ev.synchronize()
        transpose_ms = a_ev.elapsed_time(b_ev)
        dx = torch.empty((n_src, feat), dtype=dtype, device=dev)

        def local_backward():
            return be.spmm_into(dx, t_ptr, t_idx, y, n_src)

        def return_gradients():
            if world == 1:
                return dx
            if ex is not None:
                return ex.exchange_backward(dx, send_buf)
            return reduce_gradients(dx, part, rank)

        def backward_step():
            local_backward()
            return return_gradients()

        for _ in range(2):
            backward_step()
        barrier()
        t_b = [timed(backward_step, args.steps) / args.steps]
        barrier()
        t_b.append(timed(local_backward, args.steps) / args.steps)
        barrier()
        t_b.append(timed(return_gradients, args.steps) / args.steps)
        barrier()
        tb = torch.tensor(t_b + [transpose_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tb, op=dist.ReduceOp.MAX)
        backward = {"ms_per_step": float(tb[0]), "transposed_aggregation_ms": float(tb[1]),
                    "gradient_return_ms": float(tb[2]), "transpose_once_ms": float(tb[3]),
                    "return": "none" if world == 1 else ("all-to-all + accumulating aggregation" if ex is not None
                                                         else "reduce-scatter"),
                    "note": "max over ranks; the transposed graph is built once per graph and kept"}
        del dx, t_ptr, t_idx
        torch.cuda.empty_cache()

    peak, peak_src = load_peaks()
    achieved = b_alg_local / (spmm_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_DRAM_BYTES.get(args.workload) if world == 1 else None,
                "traffic_source": "ncu capture summarised in profiles/spmm_stream_papers.md (a constant, not measured by this run)",
                "peak_source": peak_src,
                "kernel": "cxg_spmm_csr (plan + spmm_stream + fix kernels)",
                "ms": spmm_ms, "algorithmic_bytes": b_alg_local}
    if roofline["traffic"]:
        # DRAM bytes actually moved (ncu, one launch) over the event-timed duration: how busy HBM is
        roofline["hbm_util"] = roofline["traffic"] / (spmm_ms * 1e-3) / 1e9 / peak
        roofline["traffic_over_algorithmic"] = roofline["traffic"] / b_alg_local
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline_sample(full_ptr, lidx, feat, dtype)

    layers = None
    if rank == 0 and world == 1 and not args.no_layers:
        del x_full, y, lidx, lptr, ptr, full_ptr, x_own, idx
        torch.cuda.empty_cache()
        import bench_layers
        layers = bench_layers.quick()

    exchange_info = None
    if world > 1:
        # the exchange against the peer-copy rate into one GPU (PEER_COPY_GBPS)
        bytes_in = remote_rows_max * feat * elem
        exchange_info = {"mode": exchange_mode, "ms": exch_ms, "rows_into_busiest_gpu": remote_rows_max,
                         "bytes_into_busiest_gpu": bytes_in, "achieved_GBps": bytes_in / (exch_ms * 1e-3) / 1e9,
                         "nvlink_peak_GBps": PEER_COPY_GBPS, "frac": bytes_in / (exch_ms * 1e-3) / 1e9 / PEER_COPY_GBPS,
                         "allgather_rows_per_gpu": (world - 1) * part.shard_rows,
                         "overlapped": overlap, "chunks": exchange_chunks, "aggregation_alone_ms": seg_ms,
                         "exposed_ms": max(0.0, ms_step - seg_ms)}
    if rank == 0:
        line = {"metric": "spmm_algorithmic_hbm_throughput", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "f32",
                "data": "synthetic",
                "config": {"workload": args.workload, "description": desc, "nodes": n, "nnz": nnz, "feat": feat,
                           "idx_bytes": idx_bytes, "partition": f"rows by edge count over {world} GPU(s)",
                           "exchange": exchange_mode + (f" in {exchange_chunks} chunks" if exchange_mode in ("needed", "putcopy")
                                                        and exchange_chunks > 1 else "") +
                           (", overlapped with the aggregation of the rows already there" if overlap else ""),
                           "l2": "256 MiB written between timed steps; inputs exceed L2"},
                "gflops": 2.0 * nnz * feat / (ms_step * 1e-3) / 1e9, "frac_of_hbm_peak": value / peak / world,
                "gpu_launches": int(launches), "roofline": roofline, "layers": layers, "exchange": exchange_info, "backward": backward, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks}
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
