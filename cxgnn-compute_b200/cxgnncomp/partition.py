"""Graph partitioning for multi-GPU aggregation.

`partition_2d_gpu` / `partition_2d_gpu_layered` keep the names, arguments and return triple of
cxgnncomp/partition.py (node-count blocks, sub-CSR of one (dst block, src block) tile with
local ids and the local destination id of every kept row).

Difference from the reference, on purpose: the reference builds `ptr` from degrees in ascending
destination order but orders `idx` with an unstable DESCENDING sort of the destinations
(partition.py:34-35), so its rows and its edges run in opposite directions. Here edges are in
ascending destination order, stable, which is what `target_aggr` needs; per row the multiset of
sources equals the reference's.

`row_partition_by_nnz` and `local_rows` are the contiguous, edge-balanced row split used for
full-graph layers on several GPUs (no counterpart in the reference, which splits by node count).
"""
import torch


def _block_bounds(total, num_device, rank):
    per = total // num_device
    lo = per * rank
    hi = per * (rank + 1) if rank < num_device - 1 else total
    return lo, hi


def _sub_csr(src, dst, num_node, device):
    degree = torch.bincount(dst, minlength=num_node).to(device)
    kept = (degree > 0).nonzero().flatten()
    new_ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=device),
                         torch.cumsum(degree[kept], 0).to(torch.int64)])
    order = torch.sort(dst, stable=True).indices
    return new_ptr, src[order].to(device), kept


def partition_2d_gpu(edge_index, num_device, rank_dst, rank_src, device=None):
    """Sub-graph of the edges whose destination lies in node block `rank_dst` and whose source lies
    in block `rank_src` (partition.py:4-36). Returns (ptr, idx_local, target_ids_local): only rows
    with at least one edge are kept, `target_ids_local[k]` is row k's destination minus the start
    of the destination block, `idx_local` is the source minus the start of the source block."""
    if device is None:
        device = edge_index.device
    num_node = int(torch.max(edge_index)) + 1
    lo_d, hi_d = _block_bounds(num_node, num_device, rank_dst)
    lo_s, hi_s = _block_bounds(num_node, num_device, rank_src)
    src, dst = edge_index[0], edge_index[1]
    keep = (dst >= lo_d) & (dst < hi_d) & (src >= lo_s) & (src < hi_s)
    src, dst = src[keep], dst[keep]
    new_ptr, new_src, kept = _sub_csr(src, dst, num_node, device)
    return new_ptr, new_src - lo_s, kept - lo_d


def partition_2d_gpu_layered(edge_index, num_device, rank_dst, rank_src, visit_mask, layer_id, device=None):
    """Layered variant (partition.py:39-98): sources are the nodes with visit_mask >= layer_id,
    destinations those with visit_mask >= layer_id + 1; both lists are cut into `num_device` blocks
    by position and ids are local positions inside the block."""
    if device is None:
        device = edge_index.device
    num_node = int(torch.max(edge_index)) + 1
    visit_src = (visit_mask >= layer_id).nonzero().flatten()
    visit_dst = (visit_mask >= layer_id + 1).nonzero().flatten()
    lo_d, hi_d = _block_bounds(visit_dst.shape[0], num_device, rank_dst)
    lo_s, hi_s = _block_bounds(visit_src.shape[0], num_device, rank_src)
    dst_mask = torch.zeros(num_node, dtype=torch.bool, device=device)
    dst_mask[visit_dst[lo_d:hi_d]] = True
    src_mask = torch.zeros(num_node, dtype=torch.bool, device=device)
    src_mask[visit_src[lo_s:hi_s]] = True
    src, dst = edge_index[0], edge_index[1]
    keep = dst_mask[dst] & src_mask[src]
    src, dst = src[keep], dst[keep]
    new_ptr, new_src, kept = _sub_csr(src, dst, num_node, device)
    target_ids = torch.searchsorted(visit_dst, kept) - lo_d
    new_idx = torch.searchsorted(visit_src, new_src) - lo_s
    return new_ptr, new_idx, target_ids


def row_partition_by_nnz(ptr, num_parts):
    """Boundaries r_0 = 0 <= r_1 <= ... <= r_P = N of contiguous row ranges holding about nnz / P
    edges each (binary search of k * nnz / P in ptr). Returns a Python list of P + 1 ints."""
    n = ptr.shape[0] - 1
    nnz = int(ptr[n])
    goals = torch.tensor([nnz * k // num_parts for k in range(1, num_parts)], dtype=ptr.dtype, device=ptr.device)
    cuts = torch.searchsorted(ptr, goals, right=False).clamp(max=n).tolist() if num_parts > 1 else []
    bounds = [0] + [int(c) for c in cuts] + [n]
    for k in range(1, len(bounds)):
        bounds[k] = max(bounds[k], bounds[k - 1])
    return bounds


def local_rows(ptr, idx, r0, r1):
    """CSR of rows [r0, r1) with a zero-based ptr; column ids stay global."""
    e0, e1 = int(ptr[r0]), int(ptr[r1])
    return (ptr[r0:r1 + 1] - e0).contiguous(), idx[e0:e1].contiguous()
