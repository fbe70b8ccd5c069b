"""Seeded synthetic graphs in the CSR_Layer format.

The reference loads OGB-derived graphs (arxiv, products, papers100M, mag240m ...) through the
CxGNN-DL loader (cxgnncomp/data_preparation.py:59-107) and fabricates random features for
them (data_preparation.py:95-101). Those datasets are not available offline, so graphs of the
same node / edge counts and a power-law degree law are generated instead; features are
N(0,1) like the reference's `torch.randn`.
"""
import torch


def powerlaw_graph(num_nodes, num_undirected, seed=0, alpha=2.1, device="cpu", idx_dtype=torch.int64,
                   chunk=1 << 26):
    """Symmetrised power-law multigraph with one self-loop per node.

    Node weights follow a Zipf rank-size law w_i = (i+1)^(-1/(alpha-1)) over a random permutation
    of the ids (degree exponent ~alpha). Both endpoints of `num_undirected` edges are drawn
    independently in proportion to the weights (u == v draws are redrawn), every edge is stored in
    both directions, and one self-loop per node is added, so every row has at least one edge and
    nnz = 2 * num_undirected + num_nodes exactly. Rows are sorted by (dst, src); that order is the
    edge traversal order of all kernels.

    Returns (ptr int64 [N+1], idx idx_dtype [nnz]) on `device`.
    """
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    n = int(num_nodes)
    w = torch.arange(1, n + 1, dtype=torch.float64, device=dev).pow_(-1.0 / (alpha - 1.0))
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()
    del w
    perm = torch.randperm(n, generator=gen, device=dev)

    def draw(k):
        r = torch.rand(k, dtype=torch.float64, device=dev, generator=gen)
        return torch.searchsorted(cdf, r).clamp_(max=n - 1)

    keys = torch.empty(2 * num_undirected + n, dtype=torch.int64, device=dev)
    done = 0
    while done < num_undirected:
        k = min(chunk, num_undirected - done)
        u, v = draw(k), draw(k)
        while True:
            same = (u == v).nonzero().flatten()
            if same.numel() == 0:
                break
            v[same] = draw(same.numel())
        u, v = perm[u], perm[v]
        keys[2 * done:2 * done + k] = v * n + u
        keys[2 * done + k:2 * (done + k)] = u * n + v
        done += k
        del u, v
    loops = torch.arange(n, dtype=torch.int64, device=dev)
    keys[2 * num_undirected:] = loops * n + loops
    del loops, cdf, perm
    keys = torch.sort(keys).values
    bounds = torch.arange(n + 1, dtype=torch.int64, device=dev) * n
    ptr = torch.searchsorted(keys, bounds)
    del bounds
    idx = (keys % n).to(idx_dtype)
    return ptr, idx


def node_features(num_nodes, feat, seed=0, device="cpu", dtype=torch.float32, chunk_rows=1 << 22):
    """N(0,1) features [num_nodes, feat], generated in row chunks to bound temporaries."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + 7919)
    x = torch.empty((num_nodes, feat), dtype=dtype, device=dev)
    for r0 in range(0, num_nodes, chunk_rows):
        r1 = min(num_nodes, r0 + chunk_rows)
        x[r0:r1] = torch.randn((r1 - r0, feat), dtype=torch.float32, device=dev, generator=gen).to(dtype)
    return x


def edge_relations(num_edges, num_rel, seed=0, device="cpu", dtype=torch.int64):
    """Relation id per directed edge, uniform over [0, num_rel) (cxgnncomp/model.py:169-171 draws
    them with torch.randint)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + 104729)
    return torch.randint(0, num_rel, (num_edges,), generator=gen, device=dev, dtype=dtype)


def xavier_uniform(shape, fan_in, fan_out, seed=0, device="cpu", dtype=torch.float32):
    """U(-a, a), a = sqrt(6 / (fan_in + fan_out)): PyG's `glorot` (cxgnncomp/graph_conv.py:420-425)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed + 15485863)
    a = (6.0 / (fan_in + fan_out)) ** 0.5
    return ((torch.rand(shape, generator=gen, dtype=torch.float32) * 2 - 1) * a).to(device=device, dtype=dtype)


# Shapes of the benchmark configurations (nodes, undirected edges).
CONFIG_SHAPES = {
    "arxiv_like": (169_343, 1_081_572),            # nnz 2,332,487
    "products_like": (2_449_029, 61_850_000),      # nnz ~126.1 M
    "rgcn_like": (1_940_000, 9_530_000),           # nnz 21.0 M
    "papers_like": (111_000_000, 744_500_000),     # nnz 1.6 G
}
