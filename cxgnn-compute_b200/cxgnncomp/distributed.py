"""Full-graph aggregation over several GPUs, one process per GPU.

The reference's multi-GPU layer (DistAggrOP in test/1-kernels/test_mgpu_model.py:106-224) splits nodes into
equal blocks, and for every source rank i broadcasts that rank's features and aggregates sub-graph (rank, i)
into the local output; communication and computation strictly alternate. Here rows are split contiguously by
EDGE count (so every GPU gathers about the same number of feature rows) and each rank keeps the CSR of its
own rows. The feature shards are exchanged with ONE NCCL all-gather into a local buffer laid out as
[world, shard_rows, F] (shard_rows = the longest shard; shorter shards leave their tail unused), and the
column ids of the local CSR are renumbered once into that layout, so the exchange needs no repacking and
one aggregation over the local rows follows it. Remote features are in local HBM before any kernel reads
them: no peer-memory loads.

`NeededRowsExchange` is the volume-reducing alternative (the reference's "densify" step,
test/1-kernels/test_mgpu_model.py:227-331,447-454): every rank asks each owner only for the feature rows its
own edges name. Requests are exchanged once per graph; every step the owners pack the requested rows and one
variable-size all-to-all delivers them into a compact local buffer, into whose numbering the column ids were
renumbered. It moves (rows needed from other ranks) x F instead of (world - 1) / world x N x F per rank.
"""
import os

import numpy as np
import torch
import torch.distributed as dist

from .partition import local_rows, row_partition_by_nnz


def _dump(directory, name, t):
    t.detach().cpu().contiguous().numpy().tofile(os.path.join(directory, name + ".dat"))


def _read(directory, name, dtype=np.int64):
    return torch.from_numpy(np.fromfile(os.path.join(directory, name + ".dat"), dtype=dtype))


class RowPartition:
    """Contiguous row ranges [bounds[r], bounds[r+1]) per rank, chosen from the full ptr so that the ranges hold
    about nnz / world edges each; identical on every rank."""

    def __init__(self, ptr, world):
        self.world = world
        self.bounds = row_partition_by_nnz(ptr, world)
        self.shard_rows = max(self.bounds[r + 1] - self.bounds[r] for r in range(world))

    def rows(self, rank):
        return self.bounds[rank], self.bounds[rank + 1]

    def tofile(self, directory):
        """bounds.dat: world + 1 int64 row bounds, raw like the reference's partition cache (cxgnncomp/batch.py:38-47)."""
        os.makedirs(directory, exist_ok=True)
        _dump(directory, "bounds", torch.tensor(self.bounds, dtype=torch.int64))

    @classmethod
    def fromfile(cls, directory):
        self = cls.__new__(cls)
        self.bounds = _read(directory, "bounds").tolist()
        self.world = len(self.bounds) - 1
        self.shard_rows = max(self.bounds[r + 1] - self.bounds[r] for r in range(self.world))
        return self

    def gather_rows(self):
        """Rows of the gather buffer: world * shard_rows."""
        return self.world * self.shard_rows

    def to_gather_ids(self, ids):
        """Global node id -> row of the [world, shard_rows] gather buffer."""
        b = torch.tensor(self.bounds, dtype=torch.int64, device=ids.device)
        owner = torch.bucketize(ids.long(), b[1:-1], right=True)
        return (ids.long() - b[owner] + owner * self.shard_rows).to(ids.dtype)

    def local_graph(self, ptr, idx, rank, gather_ids=True):
        """(ptr, idx) of this rank's rows; column ids in gather-buffer numbering (default) or global."""
        r0, r1 = self.rows(rank)
        lptr, lidx = local_rows(ptr, idx, r0, r1)
        if gather_ids and self.world > 1:
            lidx = self.to_gather_ids(lidx)
        return lptr, lidx

    def shard(self, x_gather, rank):
        """View of this rank's own rows inside the gather buffer."""
        r0, r1 = self.rows(rank)
        return x_gather[rank * self.shard_rows:rank * self.shard_rows + (r1 - r0)]


def exchange_features(x_gather, part, rank, group=None):
    """Every rank has written its own shard (part.shard(x_gather, rank)); afterwards every rank holds all
    shards. One in-place all-gather of equal [shard_rows, F] blocks."""
    if part.world == 1:
        return x_gather
    block = x_gather[rank * part.shard_rows:(rank + 1) * part.shard_rows]
    dist.all_gather_into_tensor(x_gather, block, group=group)
    return x_gather


def reduce_gradients(dx_gather, part, rank, group=None):
    """Backward of `exchange_features` (DistAggrOP.backward, test_mgpu_model.py:185-224): every rank holds partial
    gradients for ALL feature rows in the gather layout; the shards are summed across ranks and each rank
    receives its own (one reduce-scatter). Returns the [rows of this rank, F] gradient."""
    r0, r1 = part.rows(rank)
    if part.world == 1:
        return dx_gather[:r1 - r0]
    out = torch.empty((part.shard_rows, dx_gather.shape[1]), dtype=dx_gather.dtype, device=dx_gather.device)
    dist.reduce_scatter_tensor(out, dx_gather, group=group)
    return out[:r1 - r0]


def dist_aggregate(x_gather, lptr, lidx, part, rank, aggregate, out=None, group=None):
    """One full-graph aggregation step for this rank: exchange, then aggregate(x_gather, lptr, lidx, n_local, out)."""
    exchange_features(x_gather, part, rank, group)
    r0, r1 = part.rows(rank)
    return aggregate(x_gather, lptr, lidx, r1 - r0, out)


class NeededRowsExchange:
    """Per-graph state of the needed-rows exchange for one rank.

    The local feature buffer is [own shard | remote rows this rank's edges name, ordered by global id]; the
    rank's own rows are used in place (no copy), only remote rows travel.

    remote        sorted global ids of the remote feature rows this rank's edges read
    recv_counts   how many of them each owner holds (0 for this rank itself)
    send_rows     local row numbers (inside this rank's shard) that the other ranks asked for, grouped by asker
    send_counts   rows per asker
    lidx          the local column ids renumbered into rows of the local feature buffer
    """

    def __init__(self, part, lptr, lidx_global, rank, num_nodes, group=None):
        self.part, self.rank, self.group = part, rank, group
        world = part.world
        dev = lidx_global.device
        nnz = int(lptr[-1])
        r0, r1 = part.rows(rank)
        self.n_own = r1 - r0
        cols = lidx_global[:nnz].long()
        used = torch.zeros(num_nodes, dtype=torch.bool, device=dev)
        used[cols] = True
        used[r0:r1] = False  # own rows are addressed in place
        self.remote = torch.nonzero(used).squeeze(1)  # ascending, hence grouped by owner
        pos = torch.cumsum(used, 0, dtype=torch.int64) - 1 + self.n_own
        pos[r0:r1] = torch.arange(self.n_own, device=dev)
        self.lidx = pos[cols].to(lidx_global.dtype)
        del pos, used, cols
        bounds = torch.tensor(part.bounds, dtype=torch.int64, device=dev)
        cut = torch.searchsorted(self.remote, bounds)
        self.recv_counts = (cut[1:] - cut[:-1]).tolist()
        # tell every owner which of its rows (shard-local numbers) this rank needs
        owner = torch.repeat_interleave(torch.arange(world, device=dev), cut[1:] - cut[:-1])
        want_local = self.remote - bounds[owner]
        counts_out = torch.tensor(self.recv_counts, dtype=torch.int64, device=dev)
        counts_in = torch.empty_like(counts_out)
        dist.all_to_all_single(counts_in, counts_out, group=group)
        self.send_counts = counts_in.tolist()
        self.send_rows = torch.empty(sum(self.send_counts), dtype=torch.int64, device=dev)
        dist.all_to_all_single(self.send_rows, want_local, self.send_counts, self.recv_counts, group=group)

    def tofile(self, directory):
        """The plan of this rank as raw int64 arrays (remote.dat, send_rows.dat, lidx.dat, counts.dat = receive
        counts then send counts, meta.dat = [world, rank, n_own, bytes per lidx entry]), so that a later run skips
        the request exchange; same raw format as the reference's partition cache (cxgnncomp/batch.py:38-47)."""
        os.makedirs(directory, exist_ok=True)
        _dump(directory, "remote", self.remote)
        _dump(directory, "send_rows", self.send_rows)
        _dump(directory, "lidx", self.lidx.long())
        _dump(directory, "counts", torch.tensor(self.recv_counts + self.send_counts, dtype=torch.int64))
        _dump(directory, "meta", torch.tensor([self.part.world, self.rank, self.n_own, self.lidx.element_size()],
                                              dtype=torch.int64))

    @classmethod
    def fromfile(cls, directory, part, rank, device, group=None):
        """Rebuilds the plan written by `tofile`; no collective is needed. Raises when the cache was written for
        another partition or rank."""
        world, rank_f, n_own, isz = _read(directory, "meta").tolist()
        r0, r1 = part.rows(rank)
        if world != part.world or rank_f != rank or n_own != r1 - r0:
            raise RuntimeError(f"{directory}: cache is for world {world} rank {rank_f} ({n_own} rows)")
        self = cls.__new__(cls)
        self.part, self.rank, self.group, self.n_own = part, rank, group, n_own
        self.remote = _read(directory, "remote").to(device)
        self.send_rows = _read(directory, "send_rows").to(device)
        self.lidx = _read(directory, "lidx").to(torch.int32 if isz == 4 else torch.int64).to(device)
        counts = _read(directory, "counts").tolist()
        self.recv_counts, self.send_counts = counts[:world], counts[world:]
        return self

    def buffer_rows(self):
        """Rows of the local feature buffer: own shard + remote rows."""
        return self.n_own + self.remote.shape[0]

    def remote_rows(self):
        """Rows that cross the interconnect into this rank per step."""
        return self.remote.shape[0]

    def own(self, x_buf):
        """View of this rank's own rows at the head of the buffer."""
        return x_buf[:self.n_own]

    def split_graph(self, lptr):
        """The local CSR cut by where the source lives: ((ptr, idx) of the edges whose source is one of this rank's
        own rows, (ptr, idx) of the edges that read remote rows). Both keep every local row, so the second can be
        accumulated onto the result of the first while nothing else changes; the first needs no exchange."""
        nnz = int(lptr[-1])
        own = self.lidx[:nnz] < self.n_own
        run = torch.zeros(nnz + 1, dtype=torch.int64, device=lptr.device)
        torch.cumsum(own, 0, out=run[1:])
        ptr_own = run[lptr.long()]
        ptr_rem = lptr.long() - ptr_own
        return (ptr_own, self.lidx[:nnz][own].contiguous()), (ptr_rem, self.lidx[:nnz][~own].contiguous())

    def segment_graphs(self, lptr, chunks):
        """The local CSR cut by WHEN the source row of an edge is available in a chunked exchange: element 0 holds the
        edges that read this rank's own rows (no exchange needed), element 1 + c those that read the rows arriving
        with chunk c (part c of every peer's rows, as `_chunk_plan` cuts them). Every element keeps all local rows,
        so element k > 0 can be accumulated onto the sum of the elements before it; the order of the additions
        into an output row is then own edges, chunk 0, chunk 1, ..., each in CSR order."""
        plan = self._chunk_plan(chunks)
        nnz = int(lptr[-1])
        dev = lptr.device
        seg_of_row = torch.zeros(self.buffer_rows(), dtype=torch.int8, device=dev)
        for c in range(chunks):
            for (ra, rb) in plan["recv_parts"][c]:
                if rb > ra:
                    seg_of_row[self.n_own + ra:self.n_own + rb] = 1 + c
        seg = seg_of_row[self.lidx[:nnz].long()]
        lptr_l = lptr.long()
        graphs = []
        for k in range(chunks + 1):
            mine = seg == k
            run = torch.zeros(nnz + 1, dtype=torch.int64, device=dev)
            torch.cumsum(mine, 0, out=run[1:])
            graphs.append((run[lptr_l], self.lidx[:nnz][mine].contiguous()))
            del run, mine
        return graphs

    def exchange_pipelined(self, x_buf, send_buf, chunks, comm_stream, events, pack=None):
        """The chunked exchange issued on `comm_stream`: chunk c is packed and sent / received there and
        `events[c]` is recorded when its rows have landed in x_buf, so that another stream can start the work that
        reads them (segment 1 + c of `segment_graphs`) while later chunks are still in flight. The caller makes
        comm_stream wait for whatever produced x_buf's own rows before calling."""
        x_own = x_buf[:self.n_own]
        if pack is None:
            import cxgnncomp_backend
            pack = cxgnncomp_backend.gather_rows
        plan = self._chunk_plan(chunks)
        with torch.cuda.stream(comm_stream):
            for c in range(chunks):
                lo, hi = plan["send_chunk"][c]
                pack(x_own, plan["send_rows"][lo:hi], send_buf[lo:hi])
                ops = []
                for q in range(self.part.world):
                    (sa, sb), (ra, rb) = plan["send_parts"][c][q], plan["recv_parts"][c][q]
                    if sb > sa:
                        ops.append(dist.P2POp(dist.isend, send_buf[sa:sb], q, group=self.group))
                    if rb > ra:
                        ops.append(dist.P2POp(dist.irecv, x_buf[self.n_own + ra:self.n_own + rb], q, group=self.group))
                if ops:
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
                events[c].record(comm_stream)

    def exchange_backward(self, dx_buf, recv_buf=None, unpack=None):
        """Backward of `exchange`: dx_buf [buffer_rows, F] holds this rank's partial gradients for its own rows and
        for the remote rows it read. The remote part travels back to the owners (the forward all-to-all with the
        counts swapped) and every owner adds what it receives into its own rows. Returns the gradient of this
        rank's shard (a view of dx_buf[:n_own], updated in place).
        `unpack(dx_own, rows, recv)` adds recv[i] into dx_own[rows[i]] (default: index_add_)."""
        dx_own = dx_buf[:self.n_own]
        if recv_buf is None:
            recv_buf = torch.empty((self.send_rows.shape[0], dx_buf.shape[1]), dtype=dx_buf.dtype, device=dx_buf.device)
        dist.all_to_all_single(recv_buf, dx_buf[self.n_own:].contiguous(), self.send_counts, self.recv_counts,
                               group=self.group)
        if unpack is not None:
            unpack(dx_own, self.send_rows, recv_buf)
        elif dx_own.is_cuda and dx_own.dtype in (torch.float32, torch.bfloat16):
            # every own row gathers the received rows that belong to it, in the order they arrived (sender by
            # sender): an accumulating aggregation over the transposed request list, no atomics, same bits every run
            t_ptr, t_idx = self._unpack_graph()
            import cxgnncomp_backend
            cxgnncomp_backend.spmm_into(dx_own, t_ptr, t_idx, recv_buf, self.n_own, accumulate=True)
        else:
            dx_own.index_add_(0, self.send_rows, recv_buf)
        return dx_own

    def _unpack_graph(self):
        """CSR over this rank's own rows listing, for every row, the positions of the receive buffer that hold a
        partial gradient for it (the transpose of send_rows, built once per plan on the device)."""
        cached = getattr(self, "_unpack", None)
        if cached is None:
            import cxgnncomp_backend
            n_recv = self.send_rows.shape[0]
            ptr = torch.arange(n_recv + 1, dtype=torch.int64, device=self.send_rows.device)
            t_ptr, t_idx, _, _ = cxgnncomp_backend.csr_transpose(ptr, self.send_rows, n_recv, self.n_own, want_eid=False)
            cached = self._unpack = (t_ptr, t_idx)
        return cached

    def exchange(self, x_buf, send_buf=None, pack=None, async_op=False, chunks=1):
        """x_buf [buffer_rows, F] with this rank's shard already in x_buf[:n_own]; fills the remote part.
        `pack(x_own, rows, out)` gathers the rows the peers asked for (default: the CUDA row-gather kernel).
        async_op=True returns the collective's work handle instead of waiting for it on the current stream.
        chunks > 1 cuts every peer's rows into that many parts and sends part c while part c + 1 is packed."""
        x_own = x_buf[:self.n_own]
        if send_buf is None:
            send_buf = torch.empty((self.send_rows.shape[0], x_buf.shape[1]), dtype=x_buf.dtype, device=x_buf.device)
        if pack is None:
            import cxgnncomp_backend
            pack = cxgnncomp_backend.gather_rows
        if chunks <= 1 or async_op:
            pack(x_own, self.send_rows, send_buf)
            work = dist.all_to_all_single(x_buf[self.n_own:], send_buf, self.recv_counts, self.send_counts,
                                          group=self.group, async_op=async_op)
            return work if async_op else x_buf
        plan = self._chunk_plan(chunks)
        works = []
        for c in range(chunks):
            lo, hi = plan["send_chunk"][c]
            pack(x_own, plan["send_rows"][lo:hi], send_buf[lo:hi])
            ops = []
            for q in range(self.part.world):
                (sa, sb), (ra, rb) = plan["send_parts"][c][q], plan["recv_parts"][c][q]
                if sb > sa:
                    ops.append(dist.P2POp(dist.isend, send_buf[sa:sb], q, group=self.group))
                if rb > ra:
                    ops.append(dist.P2POp(dist.irecv, x_buf[self.n_own + ra:self.n_own + rb], q, group=self.group))
            if ops:
                works += dist.batch_isend_irecv(ops)
        for w in works:
            w.wait()
        return x_buf

    def _chunk_plan(self, chunks):
        """send_rows reordered as [part 0 of every peer | part 1 of every peer | ...] with the row ranges of every
        (chunk, peer) block on the send side (in that reordered list) and on the receive side (in the remote part
        of the buffer). Both sides cut a peer's list of k rows at the same places, i * k // chunks."""
        cached = getattr(self, "_plans", {}).get(chunks)
        if cached is not None:
            return cached
        world = self.part.world

        def cuts(counts):
            base, out = 0, []
            for k in counts:
                out.append([(base + i * k // chunks, base + (i + 1) * k // chunks) for i in range(chunks)])
                base += k
            return out  # [peer][chunk] -> (lo, hi) in the peer-major list

        send_cut, recv_cut = cuts(self.send_counts), cuts(self.recv_counts)
        order, send_parts, send_chunk, pos = [], [], [], 0
        for c in range(chunks):
            start, parts = pos, []
            for q in range(world):
                lo, hi = send_cut[q][c]
                order.append(self.send_rows[lo:hi])
                parts.append((pos, pos + hi - lo))
                pos += hi - lo
            send_parts.append(parts)
            send_chunk.append((start, pos))
        plan = {"send_rows": torch.cat(order) if order else self.send_rows, "send_parts": send_parts,
                "send_chunk": send_chunk, "recv_parts": [[recv_cut[q][c] for q in range(world)] for c in range(chunks)]}
        if not hasattr(self, "_plans"):
            self._plans = {}
        self._plans[chunks] = plan
        return plan


class PeerExchange:
    """The needed-rows exchange without a collective kernel, over peer mappings of the other ranks' feature
    buffers (CUDA IPC, every mapping opened by the GPU that writes through it: cxg_ipc_open). Two forms:

      mode "kernel": ONE gather kernel per rank stores the rows every peer asked for straight into the peers'
                     buffers (cxg_put_rows: pack and transfer fused, plain stores over NVLink);
      mode "copy":   the rows are packed into the send buffer (cxg_gather_rows, in `chunks` parts) and each peer's
                     part is copied into that peer's buffer by the copy engines (cxg_copy_async), one side stream
                     per peer; no SM takes part in the transfer.

    Ordering: a tiny all-reduce before the transfer (no rank still reads the buffer that is overwritten) and one
    after it (every sender's stores have completed); both are stream-ordered, the host never waits. `close()`
    releases the mappings (all ranks call it)."""

    def __init__(self, ex, x_buf, send_buf=None, group=None, mode="kernel", chunks=1):
        import cxgnncomp_backend as be
        self.ex, self.group, self.x_buf, self.send_buf = ex, group, x_buf, send_buf
        self.mode, self.chunks = mode, max(1, int(chunks))
        world, rank = ex.part.world, ex.rank
        dev = x_buf.device
        self.row_bytes = x_buf.shape[1] * x_buf.element_size()
        # Every rank takes part in every collective below even when a step of its own fails; the failure is agreed
        # on afterwards, so that all ranks raise together and the caller can fall back to another exchange.
        error = None
        try:
            exported = be.ipc_export(x_buf)
        except RuntimeError as e:
            exported, error = (None, 0), e
        meta = [None] * world
        dist.all_gather_object(meta, (exported[0], exported[1], ex.n_own, list(ex.recv_counts)), group=group)
        self._bases, self.dst = [], []
        for q in range(world):
            if q == rank or ex.send_counts[q] == 0:
                self.dst.append(0)
                continue
            h_q, off_q, n_own_q, recv_q = meta[q]
            assert recv_q[rank] == ex.send_counts[q], "peer expects another number of rows"
            base = 0
            if error is None and h_q is not None:
                try:
                    base = be.ipc_open(h_q, dev)
                    self._bases.append(base)
                except RuntimeError as e:
                    error = e
            elif error is None:
                error = RuntimeError(f"rank {q} could not export its buffer")
            first = n_own_q + sum(recv_q[:rank])  # q's own rows, then the rows of the owners before me
            self.dst.append(base + off_q + first * self.row_bytes if base else 0)
        ok = torch.tensor([0.0 if error is not None else 1.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if float(ok[0]) == 0.0:
            for b in self._bases:
                be.ipc_close(b, dev)
            self._bases = []
            raise RuntimeError(f"peer mappings are not available on every rank ({error})")
        seg = [0]
        for q in range(world):
            seg.append(seg[-1] + ex.send_counts[q])
        self.seg_start = seg
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        self._streams = [torch.cuda.Stream(device=dev) if d else None for d in self.dst]
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def close(self):
        import cxgnncomp_backend as be
        torch.cuda.synchronize(self.x_buf.device)
        dist.barrier(group=self.group)
        for b in self._bases:
            be.ipc_close(b, self.x_buf.device)
        self._bases = []

    def fence(self):
        """Stream-ordered rendezvous of all ranks."""
        dist.all_reduce(self._token, group=self.group)

    def exchange(self):
        """Fills the remote part of every rank's buffer; returns when the work is queued on the current stream."""
        import cxgnncomp_backend as be
        ex = self.ex
        x_own = ex.own(self.x_buf)
        self.fence()
        if self.mode == "kernel":
            be.put_rows(x_own, ex.send_rows, self.dst, self.seg_start)
        else:
            main = torch.cuda.current_stream()
            order = [(ex.rank + 1 + i) % ex.part.world for i in range(ex.part.world - 1)]  # another peer first per rank
            for c in range(self.chunks):
                for q in order:
                    if not self.dst[q]:
                        continue
                    k = ex.send_counts[q]
                    lo, hi = self.seg_start[q] + c * k // self.chunks, self.seg_start[q] + (c + 1) * k // self.chunks
                    if hi == lo:
                        continue
                    be.gather_rows(x_own, ex.send_rows[lo:hi], self.send_buf[lo:hi])
                    done = torch.cuda.Event()
                    done.record(main)
                    st = self._streams[q]
                    st.wait_event(done)
                    with torch.cuda.stream(st):
                        be.copy_async(self.dst[q] + (lo - self.seg_start[q]) * self.row_bytes, self.send_buf[lo:hi])
            for st in self._streams:
                if st is not None:
                    main.wait_stream(st)
        self.fence()
        return self.x_buf
