"""Index transforms on CSR graphs, same names and results as cxgnncomp/schedule.py of the
reference, written as vectorised torch ops that stay on the device of their inputs (the
reference loops in Python over numpy arrays and moves the result to the GPU at the end).
All results are integer and equal the reference's element for element.
"""
import torch


def _deg(ptr):
    return ptr[1:] - ptr[:-1]


def _segments(ptr, thres, keep_empty):
    deg = _deg(ptr)
    nseg = (deg + thres - 1) // thres
    if keep_empty:
        nseg = nseg.clamp(min=1)
    n = deg.shape[0]
    target = torch.repeat_interleave(torch.arange(n, dtype=torch.int64, device=ptr.device), nseg)
    first = torch.cumsum(nseg, 0) - nseg  # index of each row's first segment
    k = torch.arange(target.shape[0], dtype=torch.int64, device=ptr.device) - first[target]
    ends = torch.minimum(ptr[:-1][target] + (k + 1) * thres, ptr[1:][target])
    new_ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=ptr.device), ends.to(torch.int64)])
    return new_ptr, target


def neighbor_grouping(ptr, neighbor_thres=32):
    """Cut every row into segments of at most `neighbor_thres` edges (schedule.py:20-35).
    Returns (new_ptr, new_target): segment boundaries and the row each segment belongs to.
    A row without edges keeps one empty segment."""
    if not isinstance(ptr, torch.Tensor):
        ptr = torch.as_tensor(ptr)
    return _segments(ptr.to(torch.int64), int(neighbor_thres), keep_empty=True)


def neighbor_grouping_gpu(ptr, neighbor_thres=32):
    """Segment boundaries only (schedule.py:6-17). Equal to neighbor_grouping(...)[0] when no row
    is empty, which is the only case the reference's cumsum construction handles; empty rows
    contribute no segment here."""
    return _segments(ptr.to(torch.int64), int(neighbor_thres), keep_empty=False)[0]


def _edge_rows(ptr):
    n = ptr.shape[0] - 1
    return torch.repeat_interleave(torch.arange(n, dtype=torch.int64, device=ptr.device), _deg(ptr))


def partition_2d(ptr, idx, num_src, num_dst, num_parts=8):
    """Reorder the edges into num_parts x num_parts (dst block, src block) tiles, row by row inside
    a tile, dropping rows that are empty in a tile (schedule.py:38-69). Blocks have
    num // num_parts nodes, the last one takes the remainder. Returns (new_ptr, new_idx)."""
    num_src, num_dst, P = int(num_src), int(num_dst), int(num_parts)
    rows = _edge_rows(ptr)
    spp, dpp = num_src // P, num_dst // P
    bi = (rows // dpp).clamp(max=P - 1) if dpp > 0 else torch.full_like(rows, P - 1)
    bj = (idx // spp).clamp(max=P - 1) if spp > 0 else torch.full_like(idx, P - 1)
    n = ptr.shape[0] - 1
    key = (bi * P + bj) * n + rows
    order = torch.sort(key, stable=True).indices
    new_idx = idx[order]
    _, counts = torch.unique_consecutive(key[order], return_counts=True)
    new_ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=ptr.device), torch.cumsum(counts, 0)])
    return new_ptr, new_idx


def _take_rows(ptr, idx, rows):
    """CSR made of the given rows of (ptr, idx), in the given order."""
    deg = _deg(ptr)[rows]
    new_ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=ptr.device), torch.cumsum(deg, 0)])
    owner = torch.repeat_interleave(torch.arange(rows.shape[0], dtype=torch.int64, device=ptr.device), deg)
    pos = torch.arange(int(new_ptr[-1]), dtype=torch.int64, device=ptr.device) - new_ptr[:-1][owner]
    new_idx = idx[ptr[:-1][rows][owner] + pos]
    return new_ptr, new_idx


def reorder_by(ptr, idx, metric):
    """New row i is old row metric[i]; source ids are not renumbered (schedule.py:83-103)."""
    assert metric.shape[0] == ptr.shape[0] - 1
    return _take_rows(ptr, idx, metric.to(torch.int64))


def remove_from_graph(ptr, idx, remove_flag):
    """Drop the rows whose flag is set, together with their edges (schedule.py:106-121)."""
    keep = (~remove_flag.to(torch.bool)).nonzero().flatten()
    return _take_rows(ptr, idx, keep)


def remove_from_graph_by_edge(ptr, idx, remove_flag):
    """Drop the flagged edges, then the rows left without edges (schedule.py:124-144)."""
    assert remove_flag.shape == idx.shape, f"remove_flag.shape != idx.shape {remove_flag.shape} {idx.shape}"
    keep = ~remove_flag.to(torch.bool)
    n = ptr.shape[0] - 1
    rows = _edge_rows(ptr)[keep]
    deg = torch.bincount(rows, minlength=n)
    deg = deg[deg > 0]
    new_ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=ptr.device), torch.cumsum(deg, 0)])
    return new_ptr, idx[keep]
