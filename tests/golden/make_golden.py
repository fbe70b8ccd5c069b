"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN PYTHON on CPU.

Usage (only where the reference checkout is present):
    python tests/golden/make_golden.py /path/to/CxGNN-Compute

What can be executed of the reference without a GPU is its pure-torch / numpy code:
  cxgnncomp/schedule.py      neighbor_grouping{,_gpu}, partition_2d, reorder_by, remove_from_graph{,_by_edge}
  cxgnncomp/partition.py     partition_2d_gpu, partition_2d_gpu_layered
  cxgnncomp/codegen/torch_spmm.py   spmm_torch                      (the SpMM the kernels are validated against)
  cxgnncomp/codegen/rgcn_kernel.py  rgcn_scatter                    (gather -> mm -> index_add_)
  cxgnncomp/typed_linear.py  TypedLinearS2DSort, TypedLinearNaiveS2D
  cxgnncomp/graph_conv.py    MyGATConv.edge_softmax_opwise, MyGCNConv.gcn_norm, RGCNOP_sorted
  cxgnncomp/typed_linear.py  SelectMMS2EOP
  cxgnncomp/batch.py         Batch.tofile / fromfile (the raw .dat files of the partition cache)
The modules are imported from the reference tree as they are. Packages they import but that
are not installed here (the CUDA extension `cxgnncomp_backend`, torch_geometric, torch_scatter,
dgl, cxgnndl) are replaced by stubs; of those only torch_scatter's `segment_csr` / `gather_csr`
are ever called, and they are written out below from their documented semantics. `.cuda()` and
`torch.cuda.synchronize()` are made no-ops for the duration of the run.

Inputs are seeded and stored with the outputs, so the tests need neither the reference
nor this script at run time.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python make_golden.py <path to a checkout of xxcclong/CxGNN-Compute>")
REF = sys.argv[1]


class _AnyStub(types.ModuleType):
    """Module whose every attribute is a harmless placeholder."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)

        def _missing(*a, **k):
            raise RuntimeError(f"stubbed {self.__name__}.{name} was called")

        return _missing


def _segment_csr(src, indptr, reduce="sum"):
    # torch_scatter.segment_csr: reduce src[indptr[i]:indptr[i+1]] along dim 0.
    lengths = indptr[1:] - indptr[:-1]
    red = {"sum": "sum", "max": "max", "min": "min", "mean": "mean"}[reduce]
    return torch.segment_reduce(src, red, lengths=lengths, unsafe=True)


def _gather_csr(src, indptr):
    # torch_scatter.gather_csr: repeat src[i] (indptr[i+1]-indptr[i]) times.
    return torch.repeat_interleave(src, indptr[1:] - indptr[:-1], dim=0)


def install_stubs():
    for name in ["cxgnncomp_backend", "dgl", "cxgnndl", "cxgnndl_backend", "torch_geometric",
                 "torch_geometric.nn", "torch_geometric.nn.dense", "torch_geometric.nn.dense.linear",
                 "torch_geometric.nn.inits", "torch_geometric.nn.conv", "torch_geometric.loader",
                 "torch_geometric.data", "dgl.nn", "dgl.nn.pytorch", "dgl.function", "hydra", "omegaconf",
                 "torch_scatter"]:
        if name not in sys.modules:
            sys.modules[name] = _AnyStub(name)
    sys.modules["torch_geometric.nn.dense.linear"].Linear = torch.nn.Linear
    sys.modules["torch_geometric.nn.inits"].glorot = lambda t: torch.nn.init.xavier_uniform_(t) if t.dim() > 1 else t
    sys.modules["torch_scatter"].segment_csr = _segment_csr
    sys.modules["torch_scatter"].gather_csr = _gather_csr
    pkg = types.ModuleType("cxgnncomp")
    pkg.__path__ = [os.path.join(REF, "cxgnncomp")]
    sys.modules["cxgnncomp"] = pkg
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.cuda.synchronize = lambda *a, **k: None


def small_graph(n, avg_deg, seed, hub=True):
    """Random multigraph CSR with empty rows, one hub row and unsorted neighbours."""
    g = torch.Generator().manual_seed(seed)
    deg = torch.poisson(torch.full((n,), float(avg_deg)), generator=g).long()
    deg[torch.randint(0, n, (max(1, n // 8),), generator=g)] = 0
    if hub:
        deg[int(torch.randint(0, n, (1,), generator=g))] = 3 * n
    ptr = torch.zeros(n + 1, dtype=torch.int64)
    ptr[1:] = torch.cumsum(deg, 0)
    idx = torch.randint(0, n, (int(ptr[-1]),), generator=g, dtype=torch.int64)
    return ptr, idx


def main():
    install_stubs()
    schedule = importlib.import_module("cxgnncomp.schedule")
    partition = importlib.import_module("cxgnncomp.partition")
    out = {}

    # ---- schedule.py -------------------------------------------------------------------
    ptr, idx = small_graph(40, 5, seed=1)
    out["sched_ptr"], out["sched_idx"] = ptr, idx
    for thres in (4, 32):
        np_, nt_ = schedule.neighbor_grouping(ptr, thres)
        out[f"ng{thres}_ptr"], out[f"ng{thres}_target"] = np_, nt_
        # neighbor_grouping_gpu mis-sizes rows of degree 0 (up_deg = 0); it is only called on
        # graphs without empty rows, so the fixture uses one.
    ptr_ne = ptr.clone()
    deg = ptr[1:] - ptr[:-1]
    deg_ne = torch.where(deg == 0, torch.ones_like(deg), deg)
    ptr_ne[1:] = torch.cumsum(deg_ne, 0)
    out["sched_ptr_noempty"] = ptr_ne
    for thres in (4, 32):
        out[f"nggpu{thres}_ptr"] = schedule.neighbor_grouping_gpu(ptr_ne, thres)
        a, b = schedule.neighbor_grouping(ptr_ne, thres)
        out[f"ngne{thres}_ptr"], out[f"ngne{thres}_target"] = a, b
    p2_ptr, p2_idx = schedule.partition_2d(ptr, idx, 40, 40, num_parts=4)
    out["p2d_ptr"], out["p2d_idx"] = p2_ptr, p2_idx
    g = torch.Generator().manual_seed(2)
    metric = torch.randperm(40, generator=g)
    out["reorder_metric"] = metric
    out["reorder_ptr"], out["reorder_idx"] = schedule.reorder_by(ptr, idx, metric)
    flag = torch.rand(40, generator=g) < 0.3
    out["remove_flag"] = flag
    out["remove_ptr"], out["remove_idx"] = schedule.remove_from_graph(ptr, idx, flag)
    eflag = torch.rand(idx.shape[0], generator=g) < 0.4
    out["remove_eflag"] = eflag
    out["remove_e_ptr"], out["remove_e_idx"] = schedule.remove_from_graph_by_edge(ptr, idx, eflag)

    # ---- partition.py ------------------------------------------------------------------
    g = torch.Generator().manual_seed(3)
    n_node, n_edge = 53, 600
    edge_index = torch.randint(0, n_node, (2, n_edge), generator=g, dtype=torch.int64)
    edge_index[0, 0] = n_node - 1  # so that max(edge_index)+1 == n_node
    out["part_edge_index"] = edge_index
    visit_mask = torch.randint(0, 4, (n_node,), generator=g, dtype=torch.int64)
    out["part_visit_mask"] = visit_mask
    for P in (2, 4):
        for i in range(P):
            for j in range(P):
                a, b, c = partition.partition_2d_gpu(edge_index, P, i, j)
                out[f"part{P}_{i}_{j}_ptr"], out[f"part{P}_{i}_{j}_idx"], out[f"part{P}_{i}_{j}_target"] = a, b, c
    P = 2
    for layer in range(3):
        for i in range(P):
            for j in range(P):
                a, b, c = partition.partition_2d_gpu_layered(edge_index, P, i, j, visit_mask, layer)
                k = f"partl{layer}_{i}_{j}"
                out[k + "_ptr"], out[k + "_idx"], out[k + "_target"] = a, b, c

    # ---- torch formulations of the float path --------------------------------------------
    spec = importlib.util.spec_from_file_location("ref_torch_spmm", os.path.join(REF, "cxgnncomp/codegen/torch_spmm.py"))
    torch_spmm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(torch_spmm)
    ptr, idx = small_graph(64, 6, seed=4)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 32, generator=g)
    val = torch.rand(idx.shape[0], generator=g)
    out["spmm_ptr"], out["spmm_idx"], out["spmm_x"], out["spmm_val"] = ptr, idx, x, val
    out["spmm_sum"] = torch_spmm.spmm_torch(x, ptr, idx, 64)
    out["spmm_val_sum"] = torch_spmm.spmm_torch(x, ptr, idx, 64, val)

    notes = []
    try:
        graph_conv = importlib.import_module("cxgnncomp.graph_conv")
        typed_linear = importlib.import_module("cxgnncomp.typed_linear")
        rgcn_kernel = importlib.import_module("cxgnncomp.codegen.rgcn_kernel")
    except Exception as e:  # pragma: no cover - depends on the installed triton
        notes.append(f"graph_conv/typed_linear import failed: {type(e).__name__}: {e}")
        graph_conv = typed_linear = rgcn_kernel = None

    if graph_conv is not None:
        # edge softmax, op-wise formulation (graph_conv.py:437-448), 4 heads
        heads = 4
        att_src = torch.randn(64, heads, generator=g)
        att_dst = torch.randn(64, heads, generator=g)
        conv = graph_conv.MyGATConv.__new__(graph_conv.MyGATConv)
        ev = graph_conv.MyGATConv.edge_softmax_opwise(conv, ptr, idx, att_src, att_dst, idx.shape[0], 0.2)
        out["gat_att_src"], out["gat_att_dst"], out["gat_edge_value"] = att_src, att_dst, ev
        # gcn_norm (graph_conv.py:587-596)
        gcn = graph_conv.MyGCNConv.__new__(graph_conv.MyGCNConv)
        out["gcn_norm"] = graph_conv.MyGCNConv.gcn_norm(gcn, ptr, idx)
        # RGCN formulations
        R, K, N = 3, 32, 16
        w = torch.randn(R, K, N, generator=g) * 0.2
        rel = torch.randint(0, R, (idx.shape[0],), generator=g, dtype=torch.int64)
        out["rgcn_w"], out["rgcn_rel"] = w, rel
        try:
            out["rgcn_scatter"] = rgcn_kernel.rgcn_scatter(x, ptr, idx, rel, w, 64)
        except RuntimeError as e:
            # torch.mm of [E,K] with [E,K,N]: the function is ill-formed in the reference.
            notes.append(f"rgcn_scatter raises in the reference itself: {e}")
        out["rgcn_s2dsort"] = typed_linear.TypedLinearS2DSort(x, w, ptr, idx, rel, 64)
        dst = torch.repeat_interleave(torch.arange(64), ptr[1:] - ptr[:-1])
        srel, order = torch.sort(rel, stable=True)
        cnt = torch.bincount(rel, minlength=R)
        out["rgcn_sorted"] = graph_conv.RGCNOP_sorted(x, w, idx[order], dst[order], cnt.tolist(), 64)

        for i, o in enumerate(typed_linear.SelectMMS2EOP(x, w, idx, rel)):
            out[f"rgcn_select_{i}"] = o

    # ---- batch.py: the .dat wire format, bytes written by the reference's own Batch.tofile -----------------
    import tempfile
    batch_mod = importlib.import_module("cxgnncomp.batch")
    ptr_b, idx_b = small_graph(30, 4, seed=6, hub=False)
    gb = torch.Generator().manual_seed(7)
    x_b = torch.randn(30, 12, generator=gb)
    target_b = torch.randperm(50, generator=gb)[:30]
    out["batch_x"], out["batch_ptr"], out["batch_idx"], out["batch_target"] = x_b, ptr_b, idx_b, target_b
    with tempfile.TemporaryDirectory() as tmp:
        batch_mod.Batch(x_b, ptr_b, idx_b, target=target_b).tofile(tmp)
        for name in ("x", "ptr", "idx", "target"):
            out[f"batch_{name}_dat"] = np.fromfile(os.path.join(tmp, name + ".dat"), dtype=np.uint8)
        back = batch_mod.Batch(None, None, None)
        back.fromfile(tmp)
        assert torch.equal(back.x, x_b.reshape(-1)) and torch.equal(back.ptr, ptr_b) and torch.equal(back.target, target_b)
        # a sub-graph without features, as the partition cache stores them (test_mgpu_model.py:546-554)
        batch_mod.Batch(x=None, ptr=ptr_b, idx=idx_b, target=target_b).tofile(tmp + "/")

    arrays = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in out.items()}
    np.savez_compressed(os.path.join(HERE, "reference_cpu.npz"), **arrays)
    with open(os.path.join(HERE, "reference_cpu.txt"), "w") as f:
        f.write("generated by tests/golden/make_golden.py from the reference's own Python on CPU\n")
        f.write(f"torch {torch.__version__}\n")
        for n_ in notes:
            f.write(n_ + "\n")
        for k in sorted(arrays):
            f.write(f"{k} {arrays[k].dtype} {arrays[k].shape}\n")
    print("wrote", len(arrays), "arrays;", "; ".join(notes) if notes else "all reference modules imported")


if __name__ == "__main__":
    main()
