"""LSTM neighbourhood aggregation over degree buckets (cxgnncomp/neighbor_lstm.py:6-92 of the reference).

The rows of the CSR are expected in ascending order of degree, `deg_count[d]` rows of degree d (what the
reference's loader prepares); `module` is a batch-first torch.nn.LSTM over the feature width. Every function
returns, per destination row, the sum of the LSTM outputs over the row's neighbour sequence. The padded variant
keeps the reference's arithmetic: a group of rows is padded with zero vectors at the END of the shorter
sequences and the outputs of the padded steps are part of the sum."""
import torch


def NeighborLstmOneByOneOP(module, ptr, idx, feat):
    """One LSTM call per row (neighbor_lstm.py:6-17). Rows without neighbours are left as allocated (zeros here)."""
    n, width = ptr.shape[0] - 1, feat.shape[-1]
    out = torch.zeros((n, width), device=feat.device, dtype=feat.dtype)
    bounds = ptr.tolist()
    for r in range(n):
        lo, hi = bounds[r], bounds[r + 1]
        if hi > lo:
            seq = feat.index_select(0, idx[lo:hi])
            out[r] = module(seq, None)[0].reshape(-1, width).sum(0)
    return out


def NeighborLstmOP(module, ptr, idx, feat, deg_count):
    """One LSTM call per degree: the rows of a degree form a [rows, degree, width] batch (neighbor_lstm.py:20-38)."""
    n, width = ptr.shape[0] - 1, feat.shape[-1]
    out = torch.zeros((n, width), device=feat.device, dtype=feat.dtype)
    row = edge = 0
    for d, num in enumerate(int(c) for c in deg_count):
        if num > 0 and d > 0:  # the reference counts destination rows only for degrees > 0
            batch = feat.index_select(0, idx[edge:edge + num * d]).view(num, d, width)
            out[row:row + num] = module(batch, None)[0].reshape(num, d, -1).sum(1)
            row += num
            edge += num * d
    return out


def padded_groups(deg_count, num_center_in_batch, num_neighbor_in_batch):
    """Groups of consecutive degrees as the reference closes them (neighbor_lstm.py:52-66): a group ends at the
    degree where it has reached `num_center_in_batch` rows or `num_neighbor_in_batch` edges, or at the last degree.
    Yields (first degree, last degree, rows, first row, first edge); rows of degree 0 are not counted."""
    counts = [int(c) for c in deg_count]
    rows = edges = 0
    first_deg = None
    row0 = edge0 = 0
    for d, num in enumerate(counts):
        if num > 0 and d > 0:
            if rows == 0:
                first_deg = d
            rows += num
            edges += num * d
        if rows > 0 and (rows >= num_center_in_batch or edges >= num_neighbor_in_batch or d == len(counts) - 1):
            yield first_deg, d, rows, row0, edge0
            row0 += rows
            edge0 += edges
            rows = edges = 0


def NeighborLstmPadOP(module, ptr, idx, feat, deg_count, num_center_in_batch, num_neighbor_in_batch):
    """One LSTM call per group of degrees, shorter sequences zero-padded at the end (neighbor_lstm.py:41-92)."""
    n, width = ptr.shape[0] - 1, feat.shape[-1]
    out = torch.zeros((n, width), device=feat.device, dtype=feat.dtype)
    counts = torch.as_tensor([int(c) for c in deg_count], device=feat.device)
    for lo_deg, hi_deg, rows, row0, edge0 in padded_groups(deg_count, num_center_in_batch, num_neighbor_in_batch):
        # degree of every row of the group, and where its neighbours start inside the group's edges
        degs = torch.repeat_interleave(torch.arange(lo_deg, hi_deg + 1, device=feat.device), counts[lo_deg:hi_deg + 1])
        starts = torch.cumsum(degs, 0) - degs + edge0
        step = torch.arange(hi_deg, device=feat.device)
        valid = step.unsqueeze(0) < degs.unsqueeze(1)                      # [rows, hi_deg]
        pos = (starts.unsqueeze(1) + step.unsqueeze(0)).clamp(max=idx.shape[0] - 1)
        batch = feat.index_select(0, idx[pos.reshape(-1)]).view(rows, hi_deg, width) * valid.unsqueeze(-1)
        out[row0:row0 + rows] = module(batch, None)[0].reshape(rows, hi_deg, -1).sum(1)
    return out
