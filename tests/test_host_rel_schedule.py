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
