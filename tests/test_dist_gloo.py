"""Host logic of the multi-GPU full-graph layer with two gloo ranks on CPU: the edge-balanced row partition is the
same on every rank, the feature exchange rebuilds the full matrix everywhere, and the per-rank aggregations
(computed here by the CPU oracle, since the CUDA kernels need a GPU) assemble to the single-process result."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "cxgnn-compute_b200"), os.path.join(ROOT, "tests")):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from cxgnncomp import synthetic
    from cxgnncomp.distributed import RowPartition, dist_aggregate
    ptr, idx = synthetic.powerlaw_graph(3000, 20000, seed=1)
    x = synthetic.node_features(3000, 16, seed=1)
    part = RowPartition(ptr, world)
    r0, r1 = part.rows(rank)
    lptr, lidx = part.local_graph(ptr, idx, rank)
    x_gather = torch.zeros(part.gather_rows(), x.shape[1])
    part.shard(x_gather, rank).copy_(x[r0:r1])  # this rank only knows its own shard

    def aggregate(xf, p, i, n, out):
        return oracle.spmm(p, i, xf)

    y_local = dist_aggregate(x_gather, lptr, lidx, part, rank, aggregate)
    for j in range(world):
        b0, b1 = part.rows(j)
        assert torch.equal(part.shard(x_gather, j), x[b0:b1]), "exchange did not deliver every shard"
    # column ids were renumbered into the gather layout: they address the same feature rows
    _, gidx = part.local_graph(ptr, idx, rank, gather_ids=False)
    assert torch.equal(x_gather[lidx], x[gidx])
    # needed-rows exchange: only the rows this rank's edges name arrive, in the renumbered order
    from cxgnncomp.distributed import NeededRowsExchange
    ex = NeededRowsExchange(part, lptr, gidx, rank, 3000)
    x_buf = torch.zeros(ex.buffer_rows(), x.shape[1])
    ex.own(x_buf).copy_(x[r0:r1])
    ex.exchange(x_buf, pack=lambda src, rows, out: torch.index_select(src, 0, rows, out=out))
    # the chunked exchange (parts of every peer's rows sent while the next part is packed) delivers the same buffer
    x_buf2 = torch.zeros_like(x_buf)
    ex.own(x_buf2).copy_(x[r0:r1])
    ex.exchange(x_buf2, pack=lambda src, rows, out: torch.index_select(src, 0, rows, out=out), chunks=3)
    assert torch.equal(x_buf2, x_buf)
    remote_ids = torch.unique(gidx[(gidx < r0) | (gidx >= r1)])
    assert torch.equal(ex.remote, remote_ids) and ex.recv_counts[rank] == 0 and ex.send_counts[rank] == 0
    assert torch.equal(x_buf[ex.n_own:], x[remote_ids])
    assert torch.equal(x_buf[ex.lidx.long()], x[gidx])
    assert 0 < ex.remote_rows() <= 3000 - (r1 - r0)
    y_need = oracle.spmm(lptr, ex.lidx, x_buf)
    assert torch.equal(y_need, y_local)
    # the plan survives a trip through the on-disk cache and needs no collective to come back
    ex.tofile(os.path.join(out_dir, f"needed_{rank}"))
    ex2 = NeededRowsExchange.fromfile(os.path.join(out_dir, f"needed_{rank}"), part, rank, torch.device("cpu"))
    assert torch.equal(ex2.remote, ex.remote) and torch.equal(ex2.send_rows, ex.send_rows)
    assert torch.equal(ex2.lidx, ex.lidx) and ex2.lidx.dtype == ex.lidx.dtype
    assert ex2.recv_counts == ex.recv_counts and ex2.send_counts == ex.send_counts and ex2.n_own == ex.n_own
    x_buf3 = torch.zeros_like(x_buf)
    ex2.own(x_buf3).copy_(x[r0:r1])
    ex2.exchange(x_buf3, pack=lambda src, rows, out: torch.index_select(src, 0, rows, out=out))
    assert torch.equal(x_buf3, x_buf)
    # the two-phase form: own-source edges (no exchange needed) + remote-source edges
    (p_own, i_own), (p_rem, i_rem) = ex.split_graph(lptr)
    assert int(p_own[-1]) + int(p_rem[-1]) == int(lptr[-1]) and torch.equal(p_own + p_rem, lptr)
    assert bool((i_own < ex.n_own).all()) and bool((i_rem >= ex.n_own).all())
    y_two = oracle.spmm_f64(p_own, i_own, x_buf) + oracle.spmm_f64(p_rem, i_rem, x_buf)
    assert float((y_two - oracle.spmm_f64(lptr, ex.lidx, x_buf)).abs().max()) < 1e-12
    # the local graph cut by arrival time in a 3-chunk exchange: the pieces partition the edges, each reads only its
    # own part of the buffer, and accumulating them in order reproduces the aggregation
    graphs = ex.segment_graphs(lptr, 3)
    assert len(graphs) == 4 and sum(int(g[0][-1]) for g in graphs) == int(lptr[-1])
    assert torch.equal(sum(g[0] for g in graphs), lptr) and bool((graphs[0][1] < ex.n_own).all())
    plan3 = ex._chunk_plan(3)
    for c in range(3):
        rows_c = torch.cat([torch.arange(ra, rb) for (ra, rb) in plan3["recv_parts"][c]]) + ex.n_own
        assert bool(torch.isin(graphs[1 + c][1], rows_c).all())
    y_seg = sum(oracle.spmm_f64(g[0], g[1], x_buf) for g in graphs)
    assert float((y_seg - oracle.spmm_f64(lptr, ex.lidx, x_buf)).abs().max()) < 1e-12
    # backward: partial gradients for every row this rank read go back to their owners and are summed there
    dy = synthetic.node_features(3000, 16, seed=2)[r0:r1]
    dx_buf = oracle.spmm_bwd_f64(lptr, ex.lidx, dy, (ex.buffer_rows(), 16))[0]
    dx_needed = ex.exchange_backward(dx_buf).clone()
    from cxgnncomp.distributed import reduce_gradients
    dx_gather = oracle.spmm_bwd_f64(lptr, lidx, dy, (part.gather_rows(), 16))[0]
    dx_all = reduce_gradients(dx_gather, part, rank)
    assert float((dx_needed - dx_all).abs().max()) < 1e-12
    torch.save({"bounds": part.bounds, "y": y_local, "nnz": int(lptr[-1]), "dx": dx_needed},
               os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_partition_exchange_aggregate(tmp_path):
    world = 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, os.path.join(ROOT, "cxgnn-compute_b200"))
    import oracle
    from cxgnncomp import synthetic
    ptr, idx = synthetic.powerlaw_graph(3000, 20000, seed=1)
    x = synthetic.node_features(3000, 16, seed=1)
    full = oracle.spmm(ptr, idx, x)
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    assert parts[0]["bounds"] == parts[1]["bounds"]
    assert torch.equal(torch.cat([p["y"] for p in parts]), full)
    # the distributed backward assembles to the single-process transpose product
    dy = synthetic.node_features(3000, 16, seed=2)
    dx_full = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)[0]
    assert float((torch.cat([p["dx"] for p in parts]) - dx_full).abs().max()) < 1e-12
    nnz = [p["nnz"] for p in parts]
    assert sum(nnz) == idx.shape[0]
    max_deg = int((ptr[1:] - ptr[:-1]).max())
    assert abs(nnz[0] - nnz[1]) <= 2 * max_deg  # balanced by edges up to one row


def _worker4(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "cxgnn-compute_b200"), os.path.join(ROOT, "tests")):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from cxgnncomp import synthetic
    from cxgnncomp.distributed import NeededRowsExchange, RowPartition
    ptr, idx = synthetic.powerlaw_graph(2000, 9000, seed=3)
    x = synthetic.node_features(2000, 8, seed=3)
    part = RowPartition(ptr, world)
    r0, r1 = part.rows(rank)
    lptr, gidx = part.local_graph(ptr, idx, rank, gather_ids=False)
    ex = NeededRowsExchange(part, lptr, gidx, rank, 2000)
    pack = lambda src, rows, out: torch.index_select(src, 0, rows, out=out)  # noqa: E731
    bufs = []
    for chunks in (1, 3):
        buf = torch.zeros(ex.buffer_rows(), 8)
        ex.own(buf).copy_(x[r0:r1])
        ex.exchange(buf, pack=pack, chunks=chunks)
        bufs.append(buf)
    assert torch.equal(bufs[0], bufs[1])
    assert torch.equal(bufs[0][ex.lidx.long()], x[gidx])
    y = oracle.spmm(lptr, ex.lidx, bufs[0])
    dy = synthetic.node_features(2000, 8, seed=4)[r0:r1]
    dx = ex.exchange_backward(oracle.spmm_bwd_f64(lptr, ex.lidx, dy, (ex.buffer_rows(), 8))[0]).clone()
    torch.save({"y": y, "dx": dx}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_four_rank_needed_rows_exchange(tmp_path):
    """Four ranks: every rank sends to and receives from three peers, whole and in chunks; forward and backward
    assemble to the single-process results."""
    world = 4
    port = 31500 + os.getpid() % 2000
    mp.spawn(_worker4, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, os.path.join(ROOT, "cxgnn-compute_b200"))
    import oracle
    from cxgnncomp import synthetic
    ptr, idx = synthetic.powerlaw_graph(2000, 9000, seed=3)
    x = synthetic.node_features(2000, 8, seed=3)
    dy = synthetic.node_features(2000, 8, seed=4)
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    assert torch.equal(torch.cat([p["y"] for p in parts]), oracle.spmm(ptr, idx, x))
    want = oracle.spmm_bwd_f64(ptr, idx, dy, x.shape)[0]
    assert float((torch.cat([p["dx"] for p in parts]) - want).abs().max()) < 1e-12
