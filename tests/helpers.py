"""Small seeded inputs shared by the tests."""
import torch


def random_csr(n_dst, n_src, avg_deg, seed, hub=0, empty_frac=0.1, idx_dtype=torch.int64):
    """Random multigraph in CSR form with some empty rows and, optionally, one row of `hub` edges."""
    g = torch.Generator().manual_seed(seed)
    deg = torch.poisson(torch.full((n_dst,), float(avg_deg)), generator=g).long()
    if empty_frac > 0 and n_dst > 1:
        k = max(1, int(n_dst * empty_frac))
        deg[torch.randint(0, n_dst, (k,), generator=g)] = 0
    if hub:
        deg[int(torch.randint(0, n_dst, (1,), generator=g))] = hub
    ptr = torch.zeros(n_dst + 1, dtype=torch.int64)
    ptr[1:] = torch.cumsum(deg, 0)
    idx = torch.randint(0, n_src, (int(ptr[-1]),), generator=g, dtype=torch.int64).to(idx_dtype)
    return ptr, idx


def randn(shape, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


def rel_err(a, b):
    """max |a-b| / max(|b|, 1e-30) over the whole tensor (norm-wise relative error)."""
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp(min=1e-30))
