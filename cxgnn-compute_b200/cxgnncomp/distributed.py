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
"""
import torch
import torch.distributed as dist

from .partition import local_rows, row_partition_by_nnz


class RowPartition:
    """Contiguous row ranges [bounds[r], bounds[r+1]) per rank, chosen from the full ptr so that the ranges hold
    about nnz / world edges each; identical on every rank."""

    def __init__(self, ptr, world):
        self.world = world
        self.bounds = row_partition_by_nnz(ptr, world)
        self.shard_rows = max(self.bounds[r + 1] - self.bounds[r] for r in range(world))

    def rows(self, rank):
        return self.bounds[rank], self.bounds[rank + 1]

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


def dist_aggregate(x_gather, lptr, lidx, part, rank, aggregate, out=None, group=None):
    """One full-graph aggregation step for this rank: exchange, then aggregate(x_gather, lptr, lidx, n_local, out)."""
    exchange_features(x_gather, part, rank, group)
    r0, r1 = part.rows(rank)
    return aggregate(x_gather, lptr, lidx, r1 - r0, out)
