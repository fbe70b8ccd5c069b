"""Relational (RGCN) part of the `cxgnncomp_backend` surface: pad_rel, typed_linear*, aggr_rgcn_direct_func,
rel_schedule and the typed matmul entry used by `cxgnncomp.codegen.typed_matmul`
(reference: init_rel_spmm / init_compute in src/cpp/python_bindings/binding.cpp:28,44-55)."""
import ctypes
import sys

import torch

from . import (_check, _cuda, _p, _stream, _sig, _workspace, _vp, _i64, _sz, _num_rows, _INDEX_DTYPES, CXG_F32,
               CXG_BF16)

_int = ctypes.c_int
_pad = _sig("cxg_pad_rel", [_vp, _vp, _vp, _int, _int, _i64, _vp])
_tl = _sig("cxg_typed_linear", [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _vp])
_direct = _sig("cxg_rgcn_direct", [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _i64, _int, _int, _vp])
_relsched = _sig("cxg_rel_schedule_host", [_vp, _vp, _vp, _i64, _vp, _int, _int, _vp, _vp, _vp, _vp, _vp])
_tmm_ws = _sig("cxg_typed_matmul_workspace_size", [_int, _int, _int, _int, ctypes.POINTER(_sz)])
_tmm = _sig("cxg_typed_matmul", [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _int, _int, _int, _vp, _sz,
                                 _vp])


def pad_rel(rel, count, thres, num_rel, base):
    """In place: fill the num_rel*(thres-1) pad slots of `rel` behind position `base` (binding.cpp:51)."""
    _cuda(rel, "rel", (torch.int64,))
    _cuda(count, "count", (torch.int64,))
    if rel.shape[0] < base + num_rel * (thres - 1):
        raise RuntimeError("pad_rel: rel is shorter than base + num_rel * (thres - 1)")
    with torch.cuda.device(rel.device):
        _check(_pad(_p(rel), None, _p(count), int(thres), int(num_rel), int(base), _stream()), "cxg_pad_rel")


def pad_rel_idx(rel, idx, count, thres, num_rel, base):
    """pad_rel that also writes -1 into the pad slots of `idx` (binding.cpp:52)."""
    _cuda(rel, "rel", (torch.int64,))
    _cuda(idx, "idx", (torch.int64,))
    _cuda(count, "count", (torch.int64,))
    if min(rel.shape[0], idx.shape[0]) < base + num_rel * (thres - 1):
        raise RuntimeError("pad_rel_idx: rel / idx shorter than base + num_rel * (thres - 1)")
    with torch.cuda.device(rel.device):
        _check(_pad(_p(rel), _p(idx), _p(count), int(thres), int(num_rel), int(base), _stream()), "cxg_pad_rel")


def _typed_linear(x, w, out, types, src, dst, num):
    _cuda(x, "x", (torch.float32,))
    _cuda(w, "weights", (torch.float32,))
    _cuda(out, "output", (torch.float32,))
    _cuda(types, "types", (torch.int32,))
    if src is not None:
        _cuda(src, "src", (torch.int64,))
    if dst is not None:
        _cuda(dst, "dst", (torch.int64,))
    if w.dim() != 3 or w.shape[1] != x.shape[1] or w.shape[2] != out.shape[1]:
        raise RuntimeError("typed_linear: weights must be [R, in_feat, out_feat]")
    with torch.cuda.device(x.device):
        _check(_tl(_p(x), _p(w), _p(out), _p(types), _p(src), _p(dst), int(num), x.shape[0], x.shape[1], out.shape[1],
                   w.shape[0], _stream()), "cxg_typed_linear")


def typed_linear(x, weights, output, types, in_feat_tile):
    """output[i] += x[i] @ weights[types[i]] (binding.cpp:48); in_feat_tile is a tiling hint and is ignored."""
    _typed_linear(x, weights, output, types, None, None, x.shape[0])


def typed_linear_s2e(x, weights, output, src_id, types, in_feat_tile):
    """output[e] += x[src_id[e]] @ weights[types[e]] (binding.cpp:49)."""
    _typed_linear(x, weights, output, types, src_id, None, src_id.shape[0])


def typed_linear_s2d(x, weights, output, src_id, dst_id, types, in_feat_tile):
    """output[dst_id[e]] += x[src_id[e]] @ weights[types[e]], atomic (binding.cpp:50)."""
    _typed_linear(x, weights, output, types, src_id, dst_id, src_id.shape[0])


def aggr_rgcn_direct_func(x, ptr, idx, weights, rel, num_node):
    """out[d] = sum over row d of x[idx[e]] @ weights[rel[e]]; rel int32 (binding.cpp:47)."""
    _cuda(x, "x", (torch.float32,))
    _cuda(weights, "weights", (torch.float32,))
    _cuda(rel, "rel", (torch.int32,))
    _cuda(ptr, "ptr", _INDEX_DTYPES)
    _cuda(idx, "idx", _INDEX_DTYPES)
    if weights.dim() != 3 or weights.shape[1] != x.shape[1]:
        raise RuntimeError(f"feat_len weight size {x.shape[1]} {weights.shape[1]}")
    n = _num_rows(ptr, num_node)
    out = torch.empty((n, weights.shape[2]), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(_direct(_p(ptr), _p(idx), ptr.element_size(), idx.element_size(), _p(rel), _p(x), _p(weights), _p(out), n,
                       x.shape[1], weights.shape[2], _stream()), "cxg_rgcn_direct")
    return out


def rel_schedule(csr_ptr, csr_idx, rel, num_node_in_layer, num_rel):
    """Per-relation sub-graphs from CPU tensors (binding.cpp:28, schedule.cu:5-63): returns
    [ptr_0, idx_0, target_0, ..., ptr_{R-1}, idx_{R-1}, target_{R-1}, rows_in_layer[R, L]], all int64 on the CPU."""
    for t_, name, dt in ((csr_ptr, "csr_ptr", torch.int64), (csr_idx, "csr_idx", torch.int64), (rel, "rel", torch.int32),
                         (num_node_in_layer, "num_node_in_layer", torch.int64)):
        if t_.is_cuda or t_.dtype != dt or not t_.is_contiguous():
            raise RuntimeError(f"rel_schedule: {name} must be a contiguous CPU tensor of {dt}")
    n = csr_ptr.shape[0] - 1
    nnz = int(csr_ptr[n])
    layers = num_node_in_layer.shape[0] - 1
    sp = torch.zeros((num_rel, n + 1), dtype=torch.int64)
    si = torch.zeros((num_rel, max(nnz, 1)), dtype=torch.int64)
    st = torch.zeros((num_rel, max(n, 1)), dtype=torch.int64)
    counts = torch.zeros((num_rel, 2), dtype=torch.int64)
    in_layer = torch.zeros((num_rel, max(layers, 1)), dtype=torch.int64)
    _check(_relsched(csr_ptr.data_ptr(), csr_idx.data_ptr(), rel.data_ptr(), n, num_node_in_layer.data_ptr(), layers,
                     num_rel, sp.data_ptr(), si.data_ptr(), st.data_ptr(), counts.data_ptr(), in_layer.data_ptr()),
           "cxg_rel_schedule_host")
    out = []
    for r in range(num_rel):
        rows, edges = int(counts[r, 0]), int(counts[r, 1])
        # the host routine writes rows of stride nnz / n / n+1; slice each relation's part
        out += [sp[r, :rows + 1].clone(), si.view(num_rel, -1)[r, :edges].clone(), st[r, :rows].clone()]
    out.append(in_layer[:, :layers].clone())
    return out


_topo = _sig("cxg_topo_sort_host", [_vp, _vp, _vp, _i64, _vp, ctypes.POINTER(_i64)])


def topo_sort(csr_ptr, csr_idx, degree):
    """Release order of the nodes by remaining in-degree (binding.cpp:33, schedule.cu:72-124); CPU int64 tensors."""
    for t_, name in ((csr_ptr, "csr_ptr"), (csr_idx, "csr_idx"), (degree, "degree")):
        if t_.is_cuda or t_.dtype != torch.int64 or not t_.is_contiguous():
            raise RuntimeError(f"topo_sort: {name} must be a contiguous CPU int64 tensor")
    n = degree.shape[0]
    out = torch.empty(n, dtype=torch.int64)
    done = _i64(0)
    _check(_topo(csr_ptr.data_ptr(), csr_idx.data_ptr(), degree.data_ptr(), n, out.data_ptr(), ctypes.byref(done)),
           "cxg_topo_sort_host")
    if done.value != n:
        print(f"Error: graph is not a DAG, {done.value} {n}")  # the reference prints and returns the buffer
    return out


class _AggrRelDirectFunction(torch.autograd.Function):
    """AggrRelDirectFunction (rel_spmm.cu:370-432). The reference's backward returns zero gradients; here
    grad_x[idx[e]] += grad_out[d] @ W[rel[e]]^T and grad_W[r] = sum of x[idx[e]]^T grad_out[d] are computed."""

    @staticmethod
    def forward(ctx, x, ptr, idx, weights, etype, num_node, num_rel):
        ctx.save_for_backward(x, ptr, idx, weights, etype)
        ctx.num_node = num_node
        return aggr_rgcn_direct_func(x, ptr, idx, weights, etype, num_node)

    @staticmethod
    def backward(ctx, grad_out):
        x, ptr, idx, weights, etype = ctx.saved_tensors
        n = ctx.num_node
        nnz = int(ptr[n])
        grad_out = grad_out.contiguous()
        dst = torch.repeat_interleave(torch.arange(n, device=x.device), (ptr[1:n + 1] - ptr[:n]).long())
        src = idx[:nnz].long()
        grad_x = grad_w = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.zeros_like(x)
            typed_linear_s2d(grad_out, weights.transpose(1, 2).contiguous(), grad_x, dst, src, etype[:nnz], 0)
        if ctx.needs_input_grad[3]:
            grad_w = torch.zeros_like(weights)
            order = torch.sort(etype[:nnz].long(), stable=True).indices
            cnt = torch.bincount(etype[:nnz].long(), minlength=weights.shape[0]).tolist()
            c = 0
            for r, n_r in enumerate(cnt):
                sel = order[c:c + n_r]
                c += n_r
                if n_r:
                    grad_w[r] = torch.mm(x[src[sel]].t(), grad_out[dst[sel]])
        return grad_x, None, None, grad_w, None, None, None


def aggr_rel_direct(x, ptr, idx, weights, etype, num_node, num_rel):
    """out[d] = sum over row d of x[idx[e]] @ weights[etype[e]] with autograd (binding.cpp:46)."""
    return _AggrRelDirectFunction.apply(x, ptr, idx, weights, etype, num_node, num_rel)


def typed_matmul_raw(a, b, rel, m_positions, m_valid, src_idx=None, dst_idx=None, seq_output=False, exact=False,
                     out_rows=None, atomic_out=None, extra_flags=0, allow_tf32=None):
    """C = typed matmul through the C ABI. a [*, K], b [R, K, N], rel int64 per position; see cxg_typed_matmul.
    C has `out_rows` rows (default: m_positions for sequential output, else m_valid). With `atomic_out` (a
    float32 [*, N] tensor) the rows are ADDED into it with vector atomics instead (rows may repeat).
    exact: fp32 fma without tensor cores. allow_tf32 (default: cxgnncomp_backend.ALLOW_TF32): plain TF32 products
    for fp32 inputs instead of the error-compensated ones."""
    _cuda(a, "a", (torch.float32, torch.bfloat16))
    _cuda(b, "b", (a.dtype,))
    _cuda(rel, "rel", (torch.int64,))
    if src_idx is not None:
        _cuda(src_idx, "src_idx", (torch.int64,))
    if dst_idx is not None:
        _cuda(dst_idx, "dst_idx", (torch.int64,))
    num_rel, k, n = b.shape
    if a.shape[1] != k:
        raise RuntimeError("incompatible dimensions")
    flags = (1 if seq_output else 0) | int(extra_flags)
    if atomic_out is not None:
        _cuda(atomic_out, "atomic_out", (torch.float32,))
        if atomic_out.shape[1] != n:
            raise RuntimeError("atomic_out must be [*, N]")
        c = atomic_out
        flags |= 2
    else:
        if out_rows is None:
            out_rows = m_positions if (seq_output or src_idx is None) else m_valid
        # rows that no position writes are left unset, like the reference's torch.empty output
        c = torch.empty((int(out_rows), n), dtype=a.dtype, device=a.device)
    dtype = CXG_F32 if a.dtype == torch.float32 else CXG_BF16
    if allow_tf32 is None:
        allow_tf32 = sys.modules[__package__].ALLOW_TF32
    precision = 0 if exact else (1 if (allow_tf32 or dtype == CXG_BF16) else 2)
    need = _sz(0)
    _check(_tmm_ws(num_rel, k, n, dtype, ctypes.byref(need)), "cxg_typed_matmul_workspace_size")
    ws = _workspace(a.device, need.value, "typed_matmul")
    with torch.cuda.device(a.device):
        _check(_tmm(_p(a), _p(b), _p(c), _p(rel), _p(src_idx), _p(dst_idx), int(m_positions), int(m_valid), k, n, num_rel,
                    dtype, precision, flags, _p(ws), ws.numel(), _stream()), "cxg_typed_matmul")
    return c


_wg_ws = _sig("cxg_typed_wgrad_workspace_size", [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_sz)])
_wg = _sig("cxg_typed_wgrad", [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                               ctypes.c_int, ctypes.c_int, ctypes.c_uint32, _vp, _vp, _sz, _vp])
_wg_status = _sig("cxg_typed_wgrad_status", [_vp, _vp])


def typed_wgrad_supported(x, g, allow_tf32=None):
    """Shapes cxg_typed_wgrad covers: same fp32 / bf16 dtype, 128 input columns, output rows a multiple of 128 bytes,
    one stage (both tiles, twice for the error-compensated fp32 mode) within shared memory."""
    if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and g.dtype == x.dtype and x.dim() == 2
            and g.dim() == 2 and x.shape[1] == 128 and (g.shape[1] * g.element_size()) % 128 == 0
            and g.shape[1] % 16 == 0 and g.shape[1] <= 256):
        return False
    if allow_tf32 is None:
        allow_tf32 = sys.modules[__package__].ALLOW_TF32
    split = 2 if (x.dtype == torch.float32 and not allow_tf32) else 1
    positions = 64 if split == 2 else 128  # per tile, as the kernel chooses them
    return (128 + g.shape[1]) * x.element_size() * positions * split <= 224 * 1024


def typed_wgrad(x, g, sorted_rel, num_rel, num_valid=None, idx=None, idx_g=None, allow_tf32=None, extra_flags=0,
                check_status=False):
    """dW [num_rel, K, N] (float32) = per relation, the sum over its positions of x[row]^T g[row_g]; positions are the
    sorted, padded ones of TypedLinearE2EOP.preprocess (`sorted_rel` int64 per position, `idx` the row of x per
    position, `idx_g` the row of g (default: the same row); a position whose row is negative or not below num_valid
    (default: the tensors' row counts) is padding). One tensor-core launch (cxg_typed_wgrad) instead of a torch.mm
    per relation (cxgnncomp/typed_linear.py:115-137)."""
    _cuda(x, "x", (torch.float32, torch.bfloat16))
    _cuda(g, "g", (x.dtype,))
    _cuda(sorted_rel, "sorted_rel", (torch.int64,))
    if idx is not None:
        _cuda(idx, "idx", (torch.int64,))
    if idx_g is not None:
        _cuda(idx_g, "idx_g", (torch.int64,))
    m = sorted_rel.shape[0]
    k, n = x.shape[1], g.shape[1]
    x_rows = min(x.shape[0], int(num_valid)) if num_valid is not None else x.shape[0]
    g_rows = min(g.shape[0], int(num_valid)) if (num_valid is not None and idx_g is None) else g.shape[0]
    dw = torch.empty((num_rel, k, n), dtype=torch.float32, device=x.device)
    dtype = CXG_F32 if x.dtype == torch.float32 else CXG_BF16
    if allow_tf32 is None:
        allow_tf32 = sys.modules[__package__].ALLOW_TF32
    precision = 1 if (allow_tf32 or dtype == CXG_BF16) else 2
    need = _sz(0)
    _check(_wg_ws(num_rel, k, n, ctypes.byref(need)), "cxg_typed_wgrad_workspace_size")
    ws = _workspace(x.device, need.value, "typed_wgrad")
    with torch.cuda.device(x.device):
        _check(_wg(_p(x), _p(g), _p(sorted_rel), _p(idx), _p(idx_g), m, x_rows, g_rows, k, n, num_rel, dtype, precision,
                   int(extra_flags), _p(dw), _p(ws), ws.numel(), _stream()), "cxg_typed_wgrad")
        if check_status:  # synchronises; raises when a bounded device-side wait ran out
            _check(_wg_status(_p(ws), _stream()), "cxg_typed_wgrad_status")
    return dw


def typed_matmul_all_relations(x, w, allow_tf32=None, extra_flags=0):
    """[R, N, out] = x [N, K] multiplied by every relation's weight w [R, K, out] in one launch of the tensor-core
    kernel (cxg_typed_matmul with CXG_TMM_ALL_RELATIONS): the first half of TypedLinearS2DMMAggrOP
    (cxgnncomp/typed_linear.py:191-221), which the reference runs as num_rel torch.mm calls. No autograd."""
    _cuda(x, "x", (torch.float32, torch.bfloat16))
    _cuda(w, "w", (x.dtype,))
    num_rel, k, n = w.shape
    if x.dim() != 2 or x.shape[1] != k:
        raise RuntimeError("incompatible dimensions")
    m = x.shape[0]
    c = torch.empty((num_rel, m, n), dtype=x.dtype, device=x.device)
    dtype = CXG_F32 if x.dtype == torch.float32 else CXG_BF16
    if allow_tf32 is None:
        allow_tf32 = sys.modules[__package__].ALLOW_TF32
    precision = 1 if (allow_tf32 or dtype == CXG_BF16) else 2
    need = _sz(0)
    _check(_tmm_ws(num_rel, k, n, dtype, ctypes.byref(need)), "cxg_typed_matmul_workspace_size")
    ws = _workspace(x.device, need.value, "typed_matmul")
    with torch.cuda.device(x.device):
        _check(_tmm(_p(x), _p(w), _p(c), None, None, None, m, m, k, n, num_rel, dtype, precision, 8 | int(extra_flags), _p(ws), ws.numel(),
                    _stream()), "cxg_typed_matmul")
    return c


def typed_matmul_all_relations_supported(x, w):
    """Shapes the dense tensor-core mode covers (K a multiple of 16 / 8, N a multiple of 16 up to 256, both TF32
    terms of a weight matrix within shared memory for fp32)."""
    if x.dtype not in (torch.float32, torch.bfloat16) or w.dtype != x.dtype or not x.is_cuda:
        return False
    num_rel, k, n = w.shape
    elem = x.element_size()
    if k % (32 // elem) != 0 or n % 16 != 0 or n > 256 or num_rel > 148:
        return False
    split = 2 if elem == 4 else 1  # fp32: both TF32 terms of every operand
    return n * k * elem * split + 3 * 128 * min(k, 32) * elem * split <= 226 * 1024


class _TransformAllFunction(torch.autograd.Function):
    """xw[r] = x @ w[r] for every relation (forward: one tensor-core launch); backward through the dense formulas
    dx = sum_r g[r] @ w[r]^T and dw[r] = x^T @ g[r] as batched matrix products."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return typed_matmul_all_relations(x.contiguous(), w.contiguous())

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        dx = dw = None
        tf32 = sys.modules[__package__].ALLOW_TF32
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = bool(tf32)
        try:
            if ctx.needs_input_grad[0]:
                dx = torch.matmul(g, w.transpose(1, 2)).sum(0)
            if ctx.needs_input_grad[1]:
                dw = torch.matmul(x.t().unsqueeze(0), g)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old
        return dx, dw


def transform_all_relations(x, w):
    """Differentiable typed_matmul_all_relations."""
    return _TransformAllFunction.apply(x, w)


_one_rel_cache = {}


def _one_relation(n, device):
    """int64 zeros [n]: the position array of a weight gradient whose rows all belong to one relation (kept and
    re-sliced, it never changes)."""
    key = str(device)
    t = _one_rel_cache.get(key)
    if t is None or t.shape[0] < n:
        t = _one_rel_cache[key] = torch.zeros(max(n, 1 << 16), dtype=torch.int64, device=device)
    return t[:n]


class _DenseLinearFunction(torch.autograd.Function):
    """y = x @ weight^T (weight [out, in], torch.nn.functional.linear without bias) on the tensor-core kernel in its
    dense mode with one relation: fp32 inputs keep fp32 accuracy (error-compensated TF32), where the library GEMM
    torch would call runs on the fp32 SIMT pipe. dx = g @ weight goes the same way; dW = g^T @ x, a reduction over
    the rows, is the weight-gradient kernel with a single relation when the layer has 128 outputs, else torch."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return typed_matmul_all_relations(x, weight.t().contiguous().unsqueeze(0))[0]

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors
        dx = dw = None
        g = g.contiguous()
        if ctx.needs_input_grad[0]:
            w3 = weight.contiguous().unsqueeze(0)  # [1, out, in]: K = out, N = in
            if typed_matmul_all_relations_supported(g, w3):
                dx = typed_matmul_all_relations(g, w3)[0]
            else:
                dx = g @ weight
        if ctx.needs_input_grad[1]:
            if typed_wgrad_supported(g, x):  # out == 128: one relation holding every row
                dw = typed_wgrad(g, x, _one_relation(x.shape[0], x.device), 1)[0].to(weight.dtype)
            else:
                dw = g.t() @ x
        return dx, dw


def dense_linear(x, weight):
    """torch.nn.functional.linear(x, weight) for a 2-D x on the library's tensor-core kernel where its dense mode
    covers the shape (same dtype fp32 / bf16, in a multiple of 8 / 16, out a multiple of 16 up to 256), else torch."""
    if (x.dim() == 2 and x.is_cuda and x.shape[0] > 0 and weight.dtype == x.dtype and x.is_contiguous()
            and typed_matmul_all_relations_supported(x, weight.t().unsqueeze(0))):
        return _DenseLinearFunction.apply(x, weight)
    return torch.nn.functional.linear(x, weight)
