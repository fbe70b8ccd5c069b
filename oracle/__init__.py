"""CPU oracle for the aggregation path — TEST INFRASTRUCTURE ONLY.

Two layers:
  * `cxg_oracle.c` (compiled here with gcc into `_build/liborc.so`): restates the
    arithmetic of the reference's CUDA kernels in their own summation order;
  * the torch formulations below: the pure-torch expressions the reference validates
    its kernels against and that serve as its CPU path (index_add_ / sparse.mm /
    per-relation linear + index_add_).

Only tests, the smoke check and the CPU-baseline / reference legs of the benchmark may
import this package. The product (`cxgnncomp_backend`, `cxgnncomp`) never does.

Parity status: the reference ships no golden vectors and cannot be run here (every entry
point is a CUDA kernel). The restatement is pinned against the outputs of the
reference's own pure-torch formulations executed on CPU (tests/golden/make_golden.py);
the typed-matmul arithmetic (Triton `tl.dot`, a dependency absent from the reference
tree) is "parity unpinned" and checked against exact fp64 math instead.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "cxg_oracle.c")
_LIB = os.path.join(_HERE, "_build", "liborc.so")


def build(force=False):
    """gcc -O2 build of the C restatement; returns the library path."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        os.makedirs(os.path.dirname(_LIB), exist_ok=True)
        subprocess.run(["gcc", "-O2", "-std=c99", "-shared", "-fPIC", "-ffp-contract=off",
                        "-fvisibility=hidden", _SRC, "-o", _LIB, "-lm"], check=True)
    return _LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_rel_schedule_one.restype = ctypes.c_int64
    return _lib


def _np(t, dtype):
    if isinstance(t, torch.Tensor):
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        t = t.detach().cpu().numpy()
    return np.ascontiguousarray(t, dtype=dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _bf16_bits(x):
    """uint16 bit pattern array of a bf16 torch tensor."""
    return x.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def spmm(ptr, idx, x, edge_val=None, mean=False, edge_mask=None, edge_rel=None, rel_stride=0,
         targets=None, out=None, n_dst=None, tile=0):
    """Sequential-order fp32 SpMM (orc_spmm_csr). x: torch [N,F] or [N,H,F], fp32 or bf16.
    Returns a torch tensor of x's dtype; `out` (same dtype) is accumulated into.
    tile > 0 switches to the summation order of the CUDA streaming kernel at that tile size."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    n = int(n_dst) if n_dst else len(ptr_n) - 1
    bf16 = x.dtype == torch.bfloat16
    heads = x.shape[1] if x.dim() == 3 else 1
    feat = x.shape[-1]
    xa = _bf16_bits(x) if bf16 else _np(x, np.float32)
    ev = None if edge_val is None else _np(edge_val, np.float32)
    em = None if edge_mask is None else _np(edge_mask, np.uint8)
    er = None if edge_rel is None else _np(edge_rel, np.int32)
    tg = None if targets is None else _np(targets, np.int64)
    shape = (n, heads, feat) if x.dim() == 3 else (n, feat)
    accumulate = out is not None
    if accumulate:
        ya = (_bf16_bits(out) if bf16 else _np(out, np.float32)).copy()
    else:
        ya = np.zeros(shape, dtype=np.uint16 if bf16 else np.float32)
    if tile:
        # summation order of the CUDA streaming kernel with `tile` edges per tile (orc_spmm_csr_tiled)
        assert em is None, "the tiled order has no edge mask"
        lib().orc_spmm_csr_tiled(_ptr(ptr_n), _ptr(idx_n), _ptr(xa), _ptr(ya), _ptr(ev), _ptr(er),
                                 ctypes.c_int64(rel_stride), _ptr(tg), ctypes.c_int64(n), feat, heads, int(mean),
                                 int(accumulate), int(bf16), ctypes.c_int64(tile))
    else:
        lib().orc_spmm_csr(_ptr(ptr_n), _ptr(idx_n), _ptr(xa), _ptr(ya), _ptr(ev), _ptr(em), _ptr(er),
                           ctypes.c_int64(rel_stride), _ptr(tg), ctypes.c_int64(n), feat, heads, int(mean),
                           int(accumulate), int(bf16))
    if bf16:
        return torch.from_numpy(ya.view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(ya)


def spmm_f64(ptr, idx, x, edge_val=None, mean=False, n_dst=None):
    """Double-precision SpMM (orc_spmm_csr_f64); returns float64 torch tensor."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    n = int(n_dst) if n_dst else len(ptr_n) - 1
    bf16 = x.dtype == torch.bfloat16
    heads = x.shape[1] if x.dim() == 3 else 1
    feat = x.shape[-1]
    xa = _bf16_bits(x) if bf16 else _np(x, np.float32)
    ev = None if edge_val is None else _np(edge_val, np.float32)
    shape = (n, heads, feat) if x.dim() == 3 else (n, feat)
    ya = np.zeros(shape, dtype=np.float64)
    lib().orc_spmm_csr_f64(_ptr(ptr_n), _ptr(idx_n), _ptr(xa), _ptr(ya), _ptr(ev), ctypes.c_int64(n), feat,
                           heads, int(mean), int(bf16))
    return torch.from_numpy(ya)


def spmm_bwd_f64(ptr, idx, dy, x_shape, x=None, edge_val=None, edge_mask=None, targets=None, mean=False,
                 need_dval=False, n_dst=None):
    """(dx, dval) in float64 for the SpMM backward (orc_spmm_csr_bwd_f64)."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    n = int(n_dst) if n_dst else len(ptr_n) - 1
    dya = _np(dy.float(), np.float32)
    heads = dy.shape[1] if dy.dim() == 3 else 1
    feat = dy.shape[-1]
    dx = np.zeros(tuple(x_shape), dtype=np.float64)
    xa = None if x is None else _np(x.float(), np.float32)
    ev = None if edge_val is None else _np(edge_val, np.float32)
    em = None if edge_mask is None else _np(edge_mask, np.uint8)
    tg = None if targets is None else _np(targets, np.int64)
    dval = np.zeros((len(idx_n), heads), dtype=np.float64) if need_dval else None
    lib().orc_spmm_csr_bwd_f64(_ptr(ptr_n), _ptr(idx_n), _ptr(dya), _ptr(xa), _ptr(ev), _ptr(em), _ptr(tg),
                               _ptr(dx), _ptr(dval), ctypes.c_int64(n), feat, heads, int(mean))
    return torch.from_numpy(dx), (None if dval is None else torch.from_numpy(dval))


def edge_softmax_fwd(ptr, idx, att_dst, att_src, slope):
    """(values [E,H] fp32, mask [E,H] bool) per orc_edge_softmax_fwd."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    ad, as_ = _np(att_dst, np.float32), _np(att_src, np.float32)
    n, heads = ad.shape
    e = int(ptr_n[n])
    out = np.zeros((e, heads), dtype=np.float32)
    mask = np.zeros((e, heads), dtype=np.uint8)
    lib().orc_edge_softmax_fwd(_ptr(ptr_n), _ptr(idx_n), _ptr(ad), _ptr(as_), _ptr(out), _ptr(mask),
                               ctypes.c_int64(n), heads, ctypes.c_float(slope))
    return torch.from_numpy(out), torch.from_numpy(mask.astype(np.bool_))


def edge_softmax_bwd(ptr, idx, grad, mask, out, n_src, slope):
    """(grad_att_dst [N,H], grad_att_src [N_s,H]) float64 per orc_edge_softmax_bwd."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    g, o = _np(grad, np.float32), _np(out, np.float32)
    m = _np(mask, np.uint8)
    heads = g.shape[1]
    n = len(ptr_n) - 1
    gd = np.zeros((n, heads), dtype=np.float64)
    gs = np.zeros((n_src, heads), dtype=np.float64)
    lib().orc_edge_softmax_bwd(_ptr(ptr_n), _ptr(idx_n), _ptr(g), _ptr(m), _ptr(o), _ptr(gd), _ptr(gs),
                               ctypes.c_int64(n), heads, ctypes.c_float(slope))
    return torch.from_numpy(gd), torch.from_numpy(gs)


def sddmm(src, dst, src_feat, dst_feat, per_head=False):
    """out[E,H] fp32 per orc_sddmm. src_feat [N,H,F]; dst_feat [N,F] (per_head False) or [N,H,F]."""
    s, d = _np(src, np.int64), _np(dst, np.int64)
    sf, df = _np(src_feat, np.float32), _np(dst_feat, np.float32)
    heads, feat = sf.shape[1], sf.shape[2]
    out = np.zeros((len(s), heads), dtype=np.float32)
    lib().orc_sddmm(_ptr(s), _ptr(d), _ptr(sf), _ptr(df), _ptr(out), ctypes.c_int64(len(s)), feat, heads,
                    int(per_head))
    return torch.from_numpy(out)


def gspmm(ptr, idx, x, val=None, rop=0, cop=2):
    """Generalised SpMM per orc_gspmm, fp32. rop: 0 sum 1 max 2 min 3 mean; cop: 0 add 1 sub 2 mul 3 div."""
    p, i = _np(ptr, np.int64), _np(idx, np.int64)
    xv = _np(x, np.float32)
    v = None if val is None else _np(val, np.float32)
    n, feat = len(p) - 1, xv.shape[1]
    y = np.zeros((n, feat), dtype=np.float32)
    lib().orc_gspmm(_ptr(p), _ptr(i), _ptr(v), _ptr(xv), _ptr(y), ctypes.c_int64(n), feat, int(rop), int(cop))
    return torch.from_numpy(y)


def sample_neighbors(gptr, gidx, frontier, fanout, seed):
    """(out_ptr, out) per orc_sample_neighbors."""
    p, i, f = _np(gptr, np.int64), _np(gidx, np.int64), _np(frontier, np.int64)
    cnt = np.minimum(p[f + 1] - p[f], fanout)
    out_ptr = np.zeros(len(f) + 1, dtype=np.int64)
    out_ptr[1:] = np.cumsum(cnt)
    out = np.full(int(out_ptr[-1]), -1, dtype=np.int64)
    lib().orc_sample_neighbors(_ptr(p), _ptr(i), _ptr(f), ctypes.c_int64(len(f)), int(fanout), _ptr(out_ptr), _ptr(out),
                               ctypes.c_uint64(seed))
    return torch.from_numpy(out_ptr), torch.from_numpy(out)


def topo_sort(ptr, idx, degree):
    """Release order per orc_topo_sort; returns (order, number of nodes released)."""
    p, i, d = _np(ptr, np.int64), _np(idx, np.int64), _np(degree, np.int64)
    out = np.full(len(d), -1, dtype=np.int64)
    fn = lib().orc_topo_sort
    fn.restype = ctypes.c_int64
    done = fn(_ptr(p), _ptr(i), _ptr(d), ctypes.c_int64(len(d)), _ptr(out))
    return torch.from_numpy(out), int(done)


def pad_rel(rel, count, thres, num_rel, base, idx=None):
    """In-place relation padding on int64 numpy/torch arrays (orc_pad_rel); returns (rel, idx)."""
    rel_n = _np(rel, np.int64).copy()
    cnt = _np(count, np.int64)
    idx_n = None if idx is None else _np(idx, np.int64).copy()
    lib().orc_pad_rel(_ptr(rel_n), _ptr(idx_n), _ptr(cnt), int(thres), int(num_rel), ctypes.c_int64(base))
    return torch.from_numpy(rel_n), (None if idx_n is None else torch.from_numpy(idx_n))


def rel_schedule(ptr, idx, rel, num_node_in_layer, num_rel):
    """List of 3*num_rel + 1 int64 tensors as the reference returns (schedule.cu:5-63)."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    rel_n = _np(rel, np.int32)
    nl = _np(num_node_in_layer, np.int64)
    num_layer = len(nl) - 1
    n = len(ptr_n) - 1
    out = []
    counts = np.zeros((num_rel, num_layer), dtype=np.int64)
    for r in range(num_rel):
        sp = np.zeros(n + 1, dtype=np.int64)
        si = np.zeros(max(len(idx_n), 1), dtype=np.int64)
        st = np.zeros(max(n, 1), dtype=np.int64)
        ninl = np.zeros(max(num_layer, 1), dtype=np.int64)
        nt = lib().orc_rel_schedule_one(_ptr(ptr_n), _ptr(idx_n), _ptr(rel_n), ctypes.c_int64(n), r, _ptr(nl),
                                        num_layer, _ptr(sp), _ptr(si), _ptr(st), _ptr(ninl))
        out += [torch.from_numpy(sp[:nt + 1].copy()), torch.from_numpy(si[:sp[nt]].copy()),
                torch.from_numpy(st[:nt].copy())]
        counts[r, :] = ninl[:num_layer]
    out.append(torch.from_numpy(counts))
    return out


def typed_linear_f64(a, w, rel, src=None):
    """out[m] = a[src[m]] @ w[rel[m]] in float64; rows with rel outside [0,R) stay 0."""
    an, wn = _np(a.float(), np.float32), _np(w.float(), np.float32)
    rn = _np(rel, np.int64)
    sn = None if src is None else _np(src, np.int64)
    m = len(rn)
    num_rel, k, n = wn.shape
    out = np.zeros((m, n), dtype=np.float64)
    lib().orc_typed_linear_f64(_ptr(an), _ptr(wn), _ptr(sn), _ptr(rn), _ptr(out), ctypes.c_int64(m), k, n,
                               num_rel)
    return torch.from_numpy(out)


# ----------------------------------------------------------------------------------------
# The reference's pure-torch formulations ("its CPU path"), restated.
# ----------------------------------------------------------------------------------------
def csr_transpose(ptr, idx, n_dst, n_src):
    """(t_ptr, t_idx, t_eid) of the first n_dst rows: edges ordered by (source, forward edge id), i.e. a stable
    sort of idx, which is what the reference's users build with torch.sort when they need the reverse graph
    (the symmetric-graph shortcut of AggrOP.backward, cxgnncomp/graph_conv.py:57-77, avoids it)."""
    ptr_n, idx_n = _np(ptr, np.int64), _np(idx, np.int64)
    e = int(ptr_n[n_dst])
    src = idx_n[:e]
    order = np.argsort(src, kind="stable")
    dst = np.repeat(np.arange(n_dst, dtype=np.int64), np.diff(ptr_n[:n_dst + 1]))
    t_ptr = np.zeros(n_src + 1, dtype=np.int64)
    np.cumsum(np.bincount(src, minlength=n_src), out=t_ptr[1:])
    return torch.from_numpy(t_ptr), torch.from_numpy(dst[order]), torch.from_numpy(order.astype(np.int64))


def dst_of_edges(ptr, n=None):
    n = ptr.shape[0] - 1 if n is None else n
    return torch.repeat_interleave(torch.arange(n, device=ptr.device), ptr[1:n + 1] - ptr[:n])


def torch_spmm_index_add(x, ptr, idx, n_dst, mean=False, edge_val=None):
    """out.index_add_(0, dst, x[idx]) — the gather/scatter form of test/2-benchmark/bench-gcn.py:45-60
    and cxgnncomp/codegen/rgcn_kernel.py:355-366."""
    dst = dst_of_edges(ptr, n_dst)
    e = int(ptr[n_dst])
    msg = x.index_select(0, idx[:e])
    if edge_val is not None:
        msg = msg * (edge_val.unsqueeze(-1) if msg.dim() == edge_val.dim() + 1 else edge_val)
    out = torch.zeros((n_dst,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    out.index_add_(0, dst, msg)
    if mean:
        deg = (ptr[1:n_dst + 1] - ptr[:n_dst]).clamp(min=1).to(x.dtype)
        out = out / deg.view(-1, *([1] * (x.dim() - 1)))
    return out


def torch_spmm_sparse(x, ptr, idx, n_dst, val=None):
    """torch.sparse.mm on a CSR tensor — cxgnncomp/codegen/torch_spmm.py:4-9."""
    e = int(ptr[n_dst])
    if val is None:
        val = torch.ones(e, dtype=torch.float32)
    mat = torch.sparse_csr_tensor(ptr[:n_dst + 1], idx[:e], val[:e], size=(n_dst, x.shape[0]))
    return torch.sparse.mm(mat, x)


def torch_edge_softmax_opwise(ptr, idx, att_src, att_dst, num_edge, slope):
    """MyGATConv.edge_softmax_opwise (cxgnncomp/graph_conv.py:437-448) with torch_scatter's
    gather_csr / segment_csr written as repeat_interleave / segment_reduce."""
    n = ptr.shape[0] - 1
    deg = ptr[1:] - ptr[:-1]
    alpha_src = torch.index_select(att_src, 0, idx[:num_edge])
    alpha_dst = torch.repeat_interleave(att_dst[:n], deg, dim=0)
    alpha = torch.nn.functional.leaky_relu(alpha_src + alpha_dst, slope)
    with torch.no_grad():
        amax = torch.segment_reduce(alpha, "max", lengths=deg, unsafe=True)
        amax = torch.repeat_interleave(amax, deg, dim=0)
    alpha = torch.exp(alpha - amax)
    osum = torch.segment_reduce(alpha, "sum", lengths=deg, unsafe=True) + 1e-16
    osum = torch.repeat_interleave(osum, deg, dim=0)
    return alpha / osum


def torch_rgcn_sorted(x, weights, ptr, idx, rel, n_dst):
    """TypedLinearS2DSort (cxgnncomp/typed_linear.py:262-310): sort edges by relation, per relation
    F.linear(x[src], W[r].T) and index_add_ into the destinations."""
    dst = dst_of_edges(ptr, n_dst)
    num_rel = weights.shape[0]
    out = torch.zeros((n_dst, weights.shape[-1]), dtype=x.dtype, device=x.device)
    _, order = torch.sort(rel, stable=True)
    count = torch.bincount(rel, minlength=num_rel)
    src, dst = idx[order], dst[order]
    c = 0
    for r in range(num_rel):
        k = int(count[r])
        s, d = src[c:c + k], dst[c:c + k]
        c += k
        out.index_add_(0, d, torch.nn.functional.linear(x[s], weights[r].T))
    return out
