"""Host-side index transforms against the outputs of the reference's own functions
(fixtures made by tests/golden/make_golden.py from cxgnncomp/schedule.py and partition.py)."""
import numpy as np
import torch

import cxgnncomp
from helpers import random_csr


def t(a):
    return torch.from_numpy(np.asarray(a))


def test_neighbor_grouping(golden):
    ptr = t(golden["sched_ptr"])
    for thres in (4, 32):
        new_ptr, target = cxgnncomp.neighbor_grouping(ptr, thres)
        assert torch.equal(new_ptr, t(golden[f"ng{thres}_ptr"]))
        assert torch.equal(target, t(golden[f"ng{thres}_target"]))
    ptr_ne = t(golden["sched_ptr_noempty"])
    for thres in (4, 32):
        assert torch.equal(cxgnncomp.neighbor_grouping_gpu(ptr_ne, thres), t(golden[f"nggpu{thres}_ptr"]))
        a, b = cxgnncomp.neighbor_grouping(ptr_ne, thres)
        assert torch.equal(a, t(golden[f"ngne{thres}_ptr"])) and torch.equal(b, t(golden[f"ngne{thres}_target"]))
        # the two variants agree when no row is empty
        assert torch.equal(a, cxgnncomp.neighbor_grouping_gpu(ptr_ne, thres))


def test_partition_2d(golden):
    ptr, idx = t(golden["sched_ptr"]), t(golden["sched_idx"])
    new_ptr, new_idx = cxgnncomp.partition_2d(ptr, idx, 40, 40, num_parts=4)
    assert torch.equal(new_ptr, t(golden["p2d_ptr"]))
    assert torch.equal(new_idx, t(golden["p2d_idx"]))


def test_reorder_and_remove(golden):
    ptr, idx = t(golden["sched_ptr"]), t(golden["sched_idx"])
    a, b = cxgnncomp.reorder_by(ptr, idx, t(golden["reorder_metric"]))
    assert torch.equal(a, t(golden["reorder_ptr"])) and torch.equal(b, t(golden["reorder_idx"]))
    a, b = cxgnncomp.remove_from_graph(ptr, idx, t(golden["remove_flag"]))
    assert torch.equal(a, t(golden["remove_ptr"])) and torch.equal(b, t(golden["remove_idx"]))
    a, b = cxgnncomp.remove_from_graph_by_edge(ptr, idx, t(golden["remove_eflag"]))
    assert torch.equal(a, t(golden["remove_e_ptr"])) and torch.equal(b, t(golden["remove_e_idx"]))


def _rows(ptr, idx):
    return [sorted(idx[int(ptr[k]):int(ptr[k + 1])].tolist()) for k in range(ptr.shape[0] - 1)]


def _check_partition(mine, ref_ptr, ref_idx, ref_target):
    ptr, idx, target = mine
    assert torch.equal(ptr, ref_ptr)
    assert torch.equal(target, ref_target)
    # The reference lists the edges in DESCENDING destination order (partition.py:34-35) next to an
    # ascending ptr; read its idx from the back, row by row, to get each row's sources.
    deg = (ref_ptr[1:] - ref_ptr[:-1]).tolist()
    ref_rows, pos = [], ref_idx.shape[0]
    for d in deg:
        ref_rows.append(sorted(ref_idx[pos - d:pos].tolist()))
        pos -= d
    assert _rows(ptr, idx) == ref_rows


def test_partition_2d_gpu(golden):
    edge_index = t(golden["part_edge_index"])
    for P in (2, 4):
        total = 0
        for i in range(P):
            for j in range(P):
                k = f"part{P}_{i}_{j}"
                mine = cxgnncomp.partition_2d_gpu(edge_index, P, i, j)
                _check_partition(mine, t(golden[k + "_ptr"]), t(golden[k + "_idx"]), t(golden[k + "_target"]))
                total += mine[1].shape[0]
        # invariant asserted by the reference's test (test/1-kernels/test_partition.py:28)
        assert total == edge_index.shape[1]


def test_partition_2d_gpu_layered(golden):
    edge_index, visit = t(golden["part_edge_index"]), t(golden["part_visit_mask"])
    P = 2
    for layer in range(3):
        total = 0
        for i in range(P):
            for j in range(P):
                k = f"partl{layer}_{i}_{j}"
                mine = cxgnncomp.partition_2d_gpu_layered(edge_index, P, i, j, visit, layer)
                _check_partition(mine, t(golden[k + "_ptr"]), t(golden[k + "_idx"]), t(golden[k + "_target"]))
                total += mine[1].shape[0]
        # test/1-kernels/test_partition.py:44-51
        want = int(((visit[edge_index[0]] >= layer) & (visit[edge_index[1]] >= layer + 1)).sum())
        assert total == want


def test_row_partition_by_nnz():
    ptr, idx = random_csr(1000, 1000, 9, seed=5, hub=4000)
    for P in (1, 2, 4, 8):
        b = cxgnncomp.row_partition_by_nnz(ptr, P)
        assert b[0] == 0 and b[-1] == 1000 and len(b) == P + 1 and b == sorted(b)
        nnz = int(ptr[-1])
        parts = [int(ptr[b[k + 1]] - ptr[b[k]]) for k in range(P)]
        assert sum(parts) == nnz
        # no part exceeds its share by more than the longest row
        assert max(parts) <= nnz / P + 4000
        lp, li = cxgnncomp.local_rows(ptr, idx, b[0], b[1])
        assert lp[0] == 0 and lp[-1] == li.shape[0]
