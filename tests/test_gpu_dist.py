"""Two NCCL ranks on two GPUs: the full-graph layer forward and backward through the CUDA kernels with both
feature exchanges (padded all-gather, needed-rows all-to-all), against the single-process float64 oracle.
Skipped on a single-GPU box; the host logic of the same path runs on CPU in test_dist_gloo.py."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "cxgnn-compute_b200"), os.path.join(ROOT, "tests")):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import cxgnncomp_backend as be
    from cxgnncomp import synthetic
    from cxgnncomp.distributed import NeededRowsExchange, RowPartition, exchange_features, reduce_gradients
    n, feat = 20000, 64
    ptr, idx = synthetic.powerlaw_graph(n, 150000, seed=1)
    x = synthetic.node_features(n, feat, seed=1)
    dy = synthetic.node_features(n, feat, seed=2)
    part = RowPartition(ptr, world)
    r0, r1 = part.rows(rank)
    lptr, gidx = part.local_graph(ptr, idx, rank, gather_ids=False)
    lptr, gidx = lptr.to(dev), gidx.to(dev)
    # all-gather layout
    lidx = part.to_gather_ids(gidx)
    xg = torch.zeros(part.gather_rows(), feat, device=dev)
    part.shard(xg, rank).copy_(x[r0:r1])
    exchange_features(xg, part, rank)
    y_a = be._spmm_forward(xg, lptr, lidx, r1 - r0)
    # backward on the default path: forward kernel over the transposed local graph (no atomics)
    dxg, _ = be._spmm_backward(dy[r0:r1].to(dev), None, lptr, lidx, r1 - r0, x_shape=(part.gather_rows(), feat))
    dx_a = reduce_gradients(dxg, part, rank)
    # needed-rows layout
    ex = NeededRowsExchange(part, lptr, gidx, rank, n)
    xb = torch.zeros(ex.buffer_rows(), feat, device=dev)
    ex.own(xb).copy_(x[r0:r1])
    ex.exchange(xb)
    y_b = be._spmm_forward(xb, lptr, ex.lidx, r1 - r0)
    xc = torch.zeros_like(xb)  # the same exchange in three parts per peer (pack of a part overlaps the previous send)
    ex.own(xc).copy_(x[r0:r1])
    ex.exchange(xc, chunks=3)
    assert torch.equal(xc, xb)
    dxb, _ = be._spmm_backward(dy[r0:r1].to(dev), None, lptr, ex.lidx, r1 - r0, x_shape=(ex.buffer_rows(), feat))
    dx_b = ex.exchange_backward(dxb)
    # the exchange in chunks on its own stream, aggregation of the own-source edges meanwhile and of every chunk's
    # edges as soon as its rows are there (accumulating passes in a fixed order)
    chunks = 3
    graphs = ex.segment_graphs(lptr, chunks)
    comm, events = torch.cuda.Stream(), [torch.cuda.Event() for _ in range(chunks)]
    send_buf = torch.empty((ex.send_rows.shape[0], feat), device=dev)
    runs = []
    for _ in range(2):
        xp = torch.zeros_like(xb)
        ex.own(xp).copy_(x[r0:r1])
        y_c = torch.full((r1 - r0, feat), float("nan"), device=dev)
        comm.wait_stream(torch.cuda.current_stream())
        ex.exchange_pipelined(xp, send_buf, chunks, comm, events)
        be.spmm_into(y_c, graphs[0][0], graphs[0][1], xp, r1 - r0, share_sms=True)
        for c in range(chunks):
            torch.cuda.current_stream().wait_event(events[c])
            be.spmm_into(y_c, graphs[1 + c][0], graphs[1 + c][1], xp, r1 - r0, accumulate=True, share_sms=True)
        torch.cuda.synchronize()
        assert torch.equal(xp, xb)
        runs.append(y_c)
    assert torch.equal(runs[0], runs[1])
    # the same rows moved over peer mappings of the other rank's buffer: by the copy engines, then by one gather
    # kernel that stores across NVLink (no collective kernel, no send buffer in the second form)
    from cxgnncomp.distributed import PeerExchange
    xq = torch.zeros_like(xb)
    ex.own(xq).copy_(x[r0:r1])
    for mode in os.environ.get("CXG_TEST_PEER_MODES", "copy,kernel").split(","):
        put = PeerExchange(ex, xq, send_buf, mode=mode, chunks=3)
        for _ in range(2):
            xq[ex.n_own:].zero_()
            put.exchange()
            torch.cuda.synchronize()
            assert torch.equal(xq, xb), mode
        put.fence()
        put.close()
    torch.save({"rows": (r0, r1), "y_a": y_a.cpu(), "y_b": y_b.cpu(), "y_c": runs[0].cpu(), "dx_a": dx_a.cpu(),
                "dx_b": dx_b.cpu(), "remote": ex.remote_rows()}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_layer_forward_backward(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, os.path.join(ROOT, "cxgnn-compute_b200"))
    import oracle
    from cxgnncomp import synthetic
    from helpers import rel_err
    port = 29700 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    n, feat = 20000, 64
    ptr, idx = synthetic.powerlaw_graph(n, 150000, seed=1)
    x = synthetic.node_features(n, feat, seed=1)
    dy = synthetic.node_features(n, feat, seed=2)
    y = oracle.spmm_f64(ptr, idx, x)
    dx = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)[0]
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(2)]
    assert parts[0]["rows"][1] == parts[1]["rows"][0] and parts[1]["rows"][1] == n
    for key, want, tol in (("y_a", y, 1e-5), ("y_b", y, 1e-5), ("y_c", y, 1e-5), ("dx_a", dx, 1e-5), ("dx_b", dx, 1e-5)):
        got = torch.cat([p[key] for p in parts])
        assert rel_err(got, want) < tol, (key, rel_err(got, want))
    assert all(0 < p["remote"] < n for p in parts)
