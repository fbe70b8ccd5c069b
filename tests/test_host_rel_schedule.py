"""rel_schedule is host code in the reference (src/cpp/src/schedule.cu:5-63); the C-ABI version runs without a GPU
and must equal the oracle's restatement element for element."""
import torch

import oracle
from helpers import random_csr


def test_rel_schedule_matches_oracle():
    import cxgnncomp_backend as be
    ptr, idx = random_csr(120, 100, 6, seed=3, hub=200)
    rel = torch.randint(0, 4, (idx.shape[0],), generator=torch.Generator().manual_seed(4), dtype=torch.int32)
    rel[rel == 2] = 0  # relation 2 has no edges
    layers = torch.tensor([30, 70, 120], dtype=torch.int64)
    got = be.rel_schedule(ptr, idx, rel, layers, 4)
    want = oracle.rel_schedule(ptr, idx, rel, layers, 4)
    assert len(got) == len(want) == 13
    for a, b in zip(got, want):
        assert a.dtype == torch.int64 and torch.equal(a, b)
    assert got[6].shape[0] == 1 and got[7].shape[0] == 0 and got[8].shape[0] == 0  # the empty relation


def _dag(n, avg, seed):
    """Out-edge CSR of a random DAG (edges point from lower to higher rank of a random permutation)."""
    g = torch.Generator().manual_seed(seed)
    rank = torch.randperm(n, generator=g)
    u = torch.randint(0, n, (n * avg,), generator=g)
    v = torch.randint(0, n, (n * avg,), generator=g)
    keep = rank[u] != rank[v]
    u, v = u[keep], v[keep]
    lo = torch.where(rank[u] < rank[v], u, v)
    hi = torch.where(rank[u] < rank[v], v, u)
    order = torch.argsort(lo, stable=True)
    lo, hi = lo[order], hi[order]
    ptr = torch.zeros(n + 1, dtype=torch.int64)
    ptr[1:] = torch.cumsum(torch.bincount(lo, minlength=n), 0)
    degree = torch.bincount(hi, minlength=n)
    return ptr, hi.contiguous(), degree


def test_topo_sort_dag_and_cycle():
    """topo_sort is host code (src/cpp/src/schedule.cu:72-124): the library and the oracle agree element for
    element, a DAG comes out in a valid topological order, and a graph with a cycle is still walked to the end."""
    import cxgnncomp_backend as be
    ptr, idx, degree = _dag(300, 4, seed=9)
    got = be.topo_sort(ptr, idx, degree)
    want, done = oracle.topo_sort(ptr, idx, degree)
    assert done == 300 and torch.equal(got, want)
    pos = torch.empty(300, dtype=torch.int64)
    pos[got] = torch.arange(300)
    src = torch.repeat_interleave(torch.arange(300), ptr[1:] - ptr[:-1])
    assert bool((pos[src] < pos[idx]).all())
    assert torch.equal(torch.sort(got).values, torch.arange(300))
    # 0 -> 1 -> 2 -> 0 cycle with a tail 2 -> 3, and an isolated node 4
    ptr = torch.tensor([0, 1, 2, 4, 4, 4])
    idx = torch.tensor([1, 2, 0, 3])
    degree = torch.tensor([1, 1, 1, 1, 0])
    got = be.topo_sort(ptr, idx, degree)
    want, done = oracle.topo_sort(ptr, idx, degree)
    assert done == 5 and torch.equal(got, want)
    assert got.tolist() == [4, 0, 1, 2, 3]  # node 4 first; then every degree-1 node is released in id order
