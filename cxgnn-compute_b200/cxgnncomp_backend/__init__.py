"""Drop-in for the `cxgnncomp_backend` extension module of CxGNN-Compute.

The reference builds this module with pybind11 (src/cpp/python_bindings/binding.cpp:122-130)
around CUDA kernels that take `torch::Tensor`s. Here every function is a thin host-side
wrapper: it checks the tensors, allocates the outputs with torch, and calls the matching
entry point of `libcxgnn_b200.so` through its C ABI (include/cxgnn_b200.h) with raw device
pointers on torch's current stream. Names, positional signatures and argument meaning are
those of the reference, so code written against the reference imports this module unchanged.

There is no CPU path: every function needs CUDA tensors and the compiled library, and
raises when either is missing. A negative status from the library becomes a RuntimeError
(the reference calls exit(1) or abort(), src/cpp/include/common.h:16-37).
"""
import ctypes
import enum
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "..", "csrc", "libcxgnn_b200.so")

CXG_F32, CXG_BF16 = 0, 1
CXG_SUM, CXG_MEAN = 0, 1
CXG_SPMM_ACCUMULATE = 1


def _load():
    path = os.path.abspath(os.environ.get("CXGNN_B200_LIB", _LIB_PATH))
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python {os.path.join(os.path.dirname(path), 'build.py')}` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these operators.")
    return ctypes.CDLL(path)


_lib = _load()
_vp, _i64, _i32, _u32, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_uint32, ctypes.c_size_t


class SpmmDesc(ctypes.Structure):
    """Mirror of `cxg_spmm_desc`."""
    _fields_ = [
        ("ptr", _vp), ("idx", _vp), ("x", _vp), ("y", _vp), ("edge_val", _vp), ("edge_mask", _vp),
        ("edge_rel", _vp), ("targets", _vp), ("n_dst", _i64), ("nnz", _i64), ("rel_stride", _i64),
        ("feat", _i32), ("heads", _i32), ("dtype", _i32), ("ptr_bytes", _i32), ("idx_bytes", _i32),
        ("reduce", _i32), ("flags", _u32), ("split_edges", _i32),
    ]


_lib.cxg_last_error_string.restype = ctypes.c_char_p
_lib.cxg_abi_version.restype = ctypes.c_int
_lib.cxg_kernel_launch_count.restype = ctypes.c_longlong


def kernel_launch_count():
    """Kernels launched by the library in this process so far."""
    return int(_lib.cxg_kernel_launch_count())


def _sig(name, argtypes):
    fn = getattr(_lib, name)
    fn.argtypes = argtypes
    fn.restype = ctypes.c_int
    return fn


_spmm_ws = _sig("cxg_spmm_csr_workspace_size", [_i64, _i64, _i32, _i32, _i32, ctypes.POINTER(_sz)])
_spmm_fwd = _sig("cxg_spmm_csr", [ctypes.POINTER(SpmmDesc), _vp, _sz, _vp])
_spmm_bwd = _sig("cxg_spmm_csr_backward", [ctypes.POINTER(SpmmDesc), _vp, _vp, _vp, _vp])


def _check(rc, what):
    if rc != 0:
        msg = _lib.cxg_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed with status {rc}: {msg}")


def _cuda(t, name, dtypes=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this backend has no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise RuntimeError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    return t


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_raw_stream = torch._C._cuda_getCurrentRawStream  # (device index) -> the stream's handle as an int, no Python objects


def _stream():
    """Handle of the current stream of the current device."""
    return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))


def _dev_index(device):
    return device.index if device.index is not None else torch.cuda.current_device()


class _OnDevice:
    """`with _on(device):` makes `device` current like torch.cuda.device, but costs one comparison when it already is
    (the case of every call in a one-GPU process)."""
    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = _dev_index(device)
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


_on = _OnDevice


_FEAT_DTYPES = (torch.float32, torch.bfloat16)
_INDEX_DTYPES = (torch.int64, torch.int32)
_workspaces = {}

# Rows with more edges than this are split into segments; 0 keeps the library default.
# Tests lower it to exercise the split path on small graphs.
SPLIT_EDGES = 0
# OR-ed into cxg_spmm_desc.flags; CXG_SPMM_BULK_ROWS (4) selects the bulk-copy (TMA) row fetch.
CXG_SPMM_BULK_ROWS = 4
CXG_SPMM_TEST_STALL = 8  # test hook, see include/cxgnn_b200.h
CXG_SPMM_GENERIC_WALK = 16
CXG_SPMM_TMA_INDEX = 64  # source ids staged by bulk copies into a ring in shared memory (lean walk)
CXG_SPMM_SHARE_SMS = 32
CXG_TMM_TEST_STALL = 4
CXG_TMM_NO_TMA = 16  # dense mode: 16-byte copies instead of tiled bulk tensor copies for A
CXG_TMM_GATHER4 = 32  # gathered rows through the bulk tensor copy unit (tile::gather4); slower, for measurement
EXTRA_SPMM_FLAGS = int(os.environ.get("CXG_SPMM_FLAGS", "0"))


_last_kind = {}


def _workspace(device, nbytes, kind=None):
    """Scratch buffer per (device, stream); grows on demand, contents never carry over. `kind` names the entry
    point family that uses it now (its status word is the one check_device_status can answer for)."""
    idx = _dev_index(device)
    key = (idx, _raw_stream(idx))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    _last_kind[key] = kind
    return buf


def _dtype_code(t):
    return CXG_F32 if t.dtype == torch.float32 else CXG_BF16


def _make_desc(ptr, idx, x, y, num_node, *, heads=1, feat=None, edge_val=None, edge_mask=None,
               edge_rel=None, rel_stride=0, targets=None, reduce=CXG_SUM, accumulate=False, flags=0):
    _cuda(ptr, "ptr", _INDEX_DTYPES)
    _cuda(idx, "idx", _INDEX_DTYPES)
    d = SpmmDesc()
    d.ptr, d.idx = ptr.data_ptr(), idx.data_ptr()
    d.x = x.data_ptr() if x is not None else None
    d.y = y.data_ptr() if y is not None else None
    d.edge_val = edge_val.data_ptr() if edge_val is not None else None
    d.edge_mask = edge_mask.data_ptr() if edge_mask is not None else None
    d.edge_rel = edge_rel.data_ptr() if edge_rel is not None else None
    d.targets = targets.data_ptr() if targets is not None else None
    d.n_dst = int(num_node)
    d.nnz = int(idx.shape[0])
    d.rel_stride = int(rel_stride)
    d.feat = int(feat)
    d.heads = int(heads)
    ref = x if x is not None else y
    d.dtype = _dtype_code(ref) if ref is not None else CXG_F32
    d.ptr_bytes = ptr.element_size()
    d.idx_bytes = idx.element_size()
    d.reduce = reduce
    d.flags = (CXG_SPMM_ACCUMULATE if accumulate else 0) | EXTRA_SPMM_FLAGS | int(flags)
    d.split_edges = SPLIT_EDGES
    return d


def _num_rows(ptr, num_node):
    n = int(num_node)
    if n <= 0:
        n = ptr.shape[0] - 1  # "0 means all rows", src/cpp/src/aggr.cu:118
    if n > ptr.shape[0] - 1:
        raise RuntimeError(f"num_node {n} exceeds the {ptr.shape[0] - 1} rows of ptr")
    return n


_spmm_status = _sig("cxg_spmm_csr_status", [_vp, _vp])
_tmm_status = _sig("cxg_typed_matmul_status", [_vp, _vp])


def check_device_status(kind="spmm", device=None):
    """Synchronises the current stream and raises if the LAST call on this stream was of that kind ("spmm" or
    "typed_matmul") and a bounded device-side wait of it ran out (the kernels give up after a cycle limit instead
    of spinning forever) or, for "spmm", ptr[num_node] exceeded the length of idx. The calls of one stream share
    a scratch buffer, so only the last call can be asked about; for any other kind nothing is checked."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = _dev_index(device)
    key = (idx, _raw_stream(idx))
    ws = _workspaces.get(key)
    if ws is None or _last_kind.get(key) != kind:
        return
    fn, name = (_spmm_status, "cxg_spmm_csr_status") if kind == "spmm" else (_tmm_status, "cxg_typed_matmul_status")
    with _on(device):
        _check(fn(_p(ws), _stream()), name)


_set_wait = _lib.cxg_set_wait_limit_cycles
_set_wait.argtypes = [ctypes.c_longlong]
_set_wait.restype = ctypes.c_int


def set_wait_limit_cycles(cycles):
    """Cycle limit of one bounded device-side wait for the launches that follow (0 = default, about a second)."""
    _check(_set_wait(int(cycles)), "cxg_set_wait_limit_cycles")


def _run_spmm(desc, device):
    need = _sz(0)
    _check(_spmm_ws(desc.n_dst, desc.nnz, desc.feat, desc.heads, desc.split_edges, ctypes.byref(need)),
           "cxg_spmm_csr_workspace_size")
    ws = _workspace(device, need.value, "spmm")
    with _on(device):
        _check(_spmm_fwd(ctypes.byref(desc), _p(ws), ws.numel(), _stream()), "cxg_spmm_csr")


def _spmm_forward(x, ptr, idx, num_node, *, edge_val=None, reduce=CXG_SUM, out=None, accumulate=False,
                  edge_mask=None, edge_rel=None, rel_stride=0, targets=None, flags=0):
    """y = A x for the first `num_node` rows; x is [N_s, F] or [N_s, H, F]."""
    _cuda(x, "x", _FEAT_DTYPES)
    n = _num_rows(ptr, num_node)
    heads = 1
    if x.dim() == 3:
        heads = x.shape[1]
    elif x.dim() != 2:
        raise RuntimeError("x must be [N, F] or [N, H, F]")
    feat = x.shape[-1]
    if edge_val is not None:
        _cuda(edge_val, "edge_value", (torch.float32,))
        ev_heads = edge_val.shape[1] if edge_val.dim() == 2 else 1
        if ev_heads != heads and not (heads == 1 and ev_heads == 1):
            raise RuntimeError(f"edge_value has {ev_heads} heads, x has {heads}")
    if out is None:
        shape = (n, heads, feat) if x.dim() == 3 else (n, feat)
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    desc = _make_desc(ptr, idx, x, out, n, heads=heads, feat=feat, edge_val=edge_val, edge_mask=edge_mask,
                      edge_rel=edge_rel, rel_stride=rel_stride, targets=targets, reduce=reduce,
                      accumulate=accumulate, flags=flags)
    _run_spmm(desc, x.device)
    return out


# dX = A^T dY is a forward aggregation over the transposed graph: deterministic and on the fast forward
# kernel, where the scatter kernel adds with atomics in no fixed order (like the reference's backward,
# aggr_kernel.cu:188-273). The transposed graph is built on the device (cxg_csr_transpose: a stable radix sort
# of the edges by source) the first time a backward is asked for a graph and kept in a small cache keyed by the
# ptr / idx tensors. BACKWARD_MODE: "auto" (= "transpose" wherever it applies) | "scatter" | "transpose".
BACKWARD_MODE = os.environ.get("CXG_BACKWARD_MODE", "auto")
_TRANSPOSE_CACHE = {}
_TRANSPOSE_CACHE_MAX = 8
_transpose_ws = _sig("cxg_csr_transpose_workspace_size", [_i64, ctypes.POINTER(_sz)])
_transpose = _sig("cxg_csr_transpose", [_vp, _vp, ctypes.c_int, ctypes.c_int, _i64, _i64, _i64, _vp, _vp, _vp, _vp,
                                        _vp, _sz, _vp])


def csr_transpose(ptr, idx, num_node, num_src, want_eid=True):
    """(t_ptr int64 [num_src + 1], t_idx, t_eid, inv_deg float [num_node]) of the first `num_node` rows of the CSR
    graph (ptr, idx): row s of the transposed graph lists the destinations of source s in ascending order, t_eid
    the forward edge of every transposed edge (what a stable sort of idx returns), inv_deg 1 / in-degree per
    destination. t_idx / t_eid have the dtype and length of idx; entries past ptr[num_node] are not written."""
    _cuda(ptr, "ptr", _INDEX_DTYPES)
    _cuda(idx, "idx", _INDEX_DTYPES)
    n = _num_rows(ptr, num_node)
    nnz = idx.shape[0]
    dev = ptr.device
    t_ptr = torch.empty(num_src + 1, dtype=torch.int64, device=dev)
    t_idx = torch.empty(nnz, dtype=idx.dtype, device=dev)
    t_eid = torch.empty(nnz, dtype=idx.dtype, device=dev) if want_eid else None
    inv_deg = torch.empty(n, dtype=torch.float32, device=dev)
    need = _sz(0)
    _check(_transpose_ws(nnz, ctypes.byref(need)), "cxg_csr_transpose_workspace_size")
    ws = _workspace(dev, need.value)
    with _on(dev):
        _check(_transpose(_p(ptr), _p(idx), ptr.element_size(), idx.element_size(), n, int(num_src), nnz, _p(t_ptr),
                          _p(t_idx), _p(t_eid), _p(inv_deg), _p(ws), ws.numel(), _stream()), "cxg_csr_transpose")
    return t_ptr, t_idx, t_eid, inv_deg


def _transposed_graph(ptr, idx, n, n_src):
    """Cached csr_transpose of the first n rows."""
    key = (ptr.data_ptr(), idx.data_ptr(), n, n_src, ptr._version, idx._version, str(ptr.device))
    hit = _TRANSPOSE_CACHE.get(key)
    if hit is not None:
        return hit[:4]
    entry = csr_transpose(ptr, idx, n, n_src)
    while len(_TRANSPOSE_CACHE) >= _TRANSPOSE_CACHE_MAX:
        _TRANSPOSE_CACHE.pop(next(iter(_TRANSPOSE_CACHE)))
    # ptr and idx are kept alive with the entry, so their addresses cannot be handed to another graph
    _TRANSPOSE_CACHE[key] = entry + (ptr, idx)
    return entry


def _spmm_backward(grad_out, x, ptr, idx, num_node, *, edge_val=None, reduce=CXG_SUM, need_dx=True,
                   need_dval=False, grad_x=None, edge_mask=None, edge_rel=None, rel_stride=0, targets=None,
                   x_shape=None):
    """Returns (dx fp32 or None, dval fp32 or None). `grad_x` is added into when given."""
    grad_out = _cuda(grad_out.contiguous(), "grad_out", _FEAT_DTYPES)
    n = _num_rows(ptr, num_node)
    heads = grad_out.shape[1] if grad_out.dim() == 3 else 1
    feat = grad_out.shape[-1]
    if x_shape is None:
        x_shape = x.shape
    dx_t = None
    # dx on the transposed graph (deterministic); the edge-value gradient, when asked for, is a second pass
    # over the forward edges with a fixed order of its own
    if (need_dx and BACKWARD_MODE != "scatter" and grad_x is None and edge_mask is None and edge_rel is None
            and targets is None and n > 0 and idx.shape[0] > 0):
        t_ptr, t_idx, t_eid, inv_deg = _transposed_graph(ptr, idx, n, x_shape[0])
        dy = grad_out[:n]
        if reduce == CXG_MEAN:
            dy = (dy.float() * inv_deg.view(-1, *([1] * (grad_out.dim() - 1)))).to(grad_out.dtype)
        t_val = None
        if edge_val is not None:  # the edge values in transposed order
            ev = edge_val.contiguous()
            t_val = torch.empty_like(ev)
            with _on(ev.device):
                _check(_gather(_p(ev), _p(t_eid), t_eid.element_size(), _p(t_val), min(t_eid.shape[0], ev.shape[0]),
                               ev.shape[1] if ev.dim() == 2 else 1, 1, _stream()), "cxg_gather_edges")
        dx_t = _spmm_forward(dy.contiguous(), t_ptr, t_idx, x_shape[0], edge_val=t_val)
        if dx_t.dtype != torch.float32:
            dx_t = dx_t.float()
        need_dx = False
        if not need_dval:
            return dx_t, None
    dx = None
    if need_dx:
        dx = grad_x if grad_x is not None else torch.zeros(x_shape, dtype=torch.float32, device=grad_out.device)
        _cuda(dx, "grad_x", (torch.float32,))
    dval = None
    if need_dval:
        dval = torch.zeros(edge_val.shape, dtype=torch.float32, device=grad_out.device)
        if x.dtype != grad_out.dtype:
            x = x.to(grad_out.dtype)
    desc = _make_desc(ptr, idx, x if need_dval else None, None, n, heads=heads, feat=feat, edge_val=edge_val,
                      edge_mask=edge_mask, edge_rel=edge_rel, rel_stride=rel_stride, targets=targets,
                      reduce=reduce)
    desc.dtype = _dtype_code(grad_out)
    with _on(grad_out.device):
        _check(_spmm_bwd(ctypes.byref(desc), _p(grad_out), _p(dx), _p(dval), _stream()),
               "cxg_spmm_csr_backward")
    return (dx_t if dx_t is not None else dx), dval


# --------------------------------------------------------------------------------------
# autograd-aware aggregation (reference: C++ torch::autograd::Function, src/cpp/include/aggr.h:13-33)
# --------------------------------------------------------------------------------------
class _SageFunction(torch.autograd.Function):
    """SAGEFunction / SAGEEdgeValueFunction (src/cpp/src/aggr.cu:275-303).

    The reference stashes raw device pointers of ptr/idx between forward and backward
    (aggr.cu:116-117); the tensors themselves are saved here, so they cannot dangle.
    """

    @staticmethod
    def forward(ctx, x, ptr, idx, edge_val, num_node, reduce):
        ctx.num_node = num_node
        ctx.reduce = reduce
        ctx.save_for_backward(x, ptr, idx, edge_val if edge_val is not None else torch.empty(0))
        ctx.has_val = edge_val is not None
        return _spmm_forward(x, ptr, idx, num_node, edge_val=edge_val, reduce=reduce)

    @staticmethod
    def backward(ctx, grad_out):
        x, ptr, idx, edge_val = ctx.saved_tensors
        edge_val = edge_val if ctx.has_val else None
        need_dx = ctx.needs_input_grad[0]
        need_dval = ctx.has_val and ctx.needs_input_grad[3]
        dx, dval = _spmm_backward(grad_out, x, ptr, idx, ctx.num_node, edge_val=edge_val, reduce=ctx.reduce,
                                  need_dx=need_dx, need_dval=need_dval)
        if dx is not None and dx.dtype != x.dtype:
            dx = dx.to(x.dtype)
        return dx, None, None, dval, None, None


def sage_sum_forward(x, ptr, idx, num_node):
    """out[r] = sum of x[idx[e]] over row r (binding.cpp:20, aggr.cu:390-393)."""
    return _SageFunction.apply(x, ptr, idx, None, num_node, CXG_SUM)


def sage_mean_forward(x, ptr, idx, num_node):
    """out[r] = mean of x[idx[e]] over row r, 0 for empty rows (binding.cpp:19, aggr.cu:385-388)."""
    return _SageFunction.apply(x, ptr, idx, None, num_node, CXG_MEAN)


def sage_sum_forward_edge_value(x, ptr, idx, edge_value, num_node):
    """out[r] = sum of edge_value[e] * x[idx[e]]; x [N,F] with value [E], or x [N,H,F] with value [E,H]
    (binding.cpp:17, aggr.cu:377-383)."""
    if edge_value.dim() == 2 and x.dim() == 2 and edge_value.shape[1] == 1:
        edge_value = edge_value.reshape(-1)
    return _SageFunction.apply(x, ptr, idx, edge_value, num_node, CXG_SUM)


def sage_mean_forward_edge_value(x, ptr, idx, edge_value, num_node):
    """The reference's kernel starts with assert(false) and its host code refuses the call
    ("DO NOT use mean with edge value", aggr.cu:158,163); same refusal here."""
    raise RuntimeError("sage_mean_forward_edge_value: DO NOT use mean with edge value")


# --------------------------------------------------------------------------------------
# raw SpMM family (no autograd), src/cpp/src/spmm_host.cu
# --------------------------------------------------------------------------------------
def run_spmm_configurable(ptr, idx, vin, num_node, grid_x=0, grid_y=0, block_x=0, block_y=0, rpb=0, cpb=0,
                          cpw=0, grid_map=0, block_map=0):
    """SpMM sum into a fresh [num_node, F] tensor (spmm_host.cu:6-55). The nine launch
    parameters chosen by the reference's tuner are accepted and ignored: the kernel
    picks its schedule from the row width and the degree of each row."""
    if vin.dim() != 2:
        raise RuntimeError("vin must be 2D")
    return _spmm_forward(vin, ptr, idx, num_node)


def spmm_into(out, ptr, idx, vin, num_node, reduce="sum", accumulate=False, share_sms=False):
    """SpMM into a caller-owned [num_node, F] (or [num_node, H, F]) tensor: out = A vin, or out += A vin with
    accumulate=True. Not in the reference (its outputs are always fresh tensors); for loops that keep their
    buffers, e.g. double-buffered pipelines, and for accumulating several source blocks into one output.
    share_sms=True leaves room on every SM for a kernel of another stream (an overlapping collective)."""
    _cuda(out, "out", (vin.dtype,))
    return _spmm_forward(vin, ptr, idx, num_node, out=out, accumulate=accumulate,
                         reduce=CXG_MEAN if reduce == "mean" else CXG_SUM,
                         flags=CXG_SPMM_SHARE_SMS if share_sms else 0)


def run_spmm_configurable_int32(ptr, idx, vin, num_node, *tuner_args):
    """int32 ptr/idx variant (spmm_host.cu:99-156)."""
    _cuda(ptr, "ptr", (torch.int32,))
    _cuda(idx, "idx", (torch.int32,))
    return run_spmm_configurable(ptr, idx, vin, num_node)


def run_spmm_configurable_bwd(ptr, idx, vin, grad_vout, num_node, *tuner_args):
    """grad_vin = A^T grad_vout, shaped like vin (spmm_host.cu:57-97)."""
    if grad_vout.dim() != 2:
        raise RuntimeError("vin must be 2D")
    dx, _ = _spmm_backward(grad_vout, vin, ptr, idx, num_node)
    return dx if dx.dtype == vin.dtype else dx.to(vin.dtype)


class SPMM_MULTIHEAD_SCHEDULE(enum.IntEnum):
    """binding.cpp:58-62."""
    Naive = 0
    PreReduce = 1
    Optimal = 2


Naive = SPMM_MULTIHEAD_SCHEDULE.Naive
PreReduce = SPMM_MULTIHEAD_SCHEDULE.PreReduce
Optimal = SPMM_MULTIHEAD_SCHEDULE.Optimal


_gather_rows = _sig("cxg_gather_rows", [_vp, _vp, _vp, _i64, _i64, _vp])


def gather_rows(x, rows, out=None):
    """out[i] = x[rows[i]] for a contiguous 2-D x and int64 rows (any element type of even size)."""
    _cuda(x, "x")
    _cuda(rows, "rows", (torch.int64,))
    if x.dim() != 2:
        raise RuntimeError("x must be 2-D")
    if out is None:
        out = torch.empty((rows.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    _cuda(out, "out", (x.dtype,))
    if out.shape[0] < rows.shape[0] or out.shape[1] != x.shape[1]:
        raise RuntimeError("out must be [len(rows), x.shape[1]]")
    with _on(x.device):
        _check(_gather_rows(_p(x), _p(rows), _p(out), rows.shape[0], x.shape[1] * x.element_size(), _stream()),
               "cxg_gather_rows")
    return out


_ipc_export = _sig("cxg_ipc_export", [_vp, _vp, ctypes.POINTER(_i64)])
_ipc_open = _sig("cxg_ipc_open", [_vp, ctypes.POINTER(_vp)])
_ipc_close = _sig("cxg_ipc_close", [_vp])
_copy_async = _sig("cxg_copy_async", [_vp, _vp, _i64, _vp])
_put_rows = _sig("cxg_put_rows", [_vp, _vp, _vp, _vp, ctypes.c_int, _i64, _vp])


def ipc_export(t):
    """(64-byte CUDA IPC handle of the allocation behind the CUDA tensor t, offset of t's first byte in it)."""
    _cuda(t, "tensor")
    buf = (ctypes.c_ubyte * 64)()
    off = _i64(0)
    with _on(t.device):
        _check(_ipc_export(_p(t), buf, ctypes.byref(off)), "cxg_ipc_export")
    return bytes(buf), int(off.value)


def ipc_open(handle, device):
    """Maps the allocation named by `handle` (from another process) into `device`'s context; returns its base address."""
    base = _vp(0)
    with _on(device):
        _check(_ipc_open((ctypes.c_ubyte * 64).from_buffer_copy(handle), ctypes.byref(base)), "cxg_ipc_open")
    return int(base.value)


def ipc_close(base, device):
    with _on(device):
        _check(_ipc_close(_vp(base)), "cxg_ipc_close")


def copy_async(dst_ptr, src, nbytes=None):
    """Device-to-device copy (copy engines) of the contiguous CUDA tensor `src` to the device address dst_ptr, queued
    on the current stream of src's device."""
    _cuda(src, "src")
    nbytes = src.numel() * src.element_size() if nbytes is None else int(nbytes)
    with _on(src.device):
        _check(_copy_async(_vp(dst_ptr), _p(src), nbytes, _stream()), "cxg_copy_async")


def put_rows(x, rows, peer_ptrs, seg_start):
    """Row i of `rows` (int64 positions into the 2-D x) is stored at peer_ptrs[q] + (i - seg_start[q]) * row bytes for
    the q with seg_start[q] <= i < seg_start[q + 1]; peer_ptrs[q] is an address inside a mapping from ipc_open (None
    or 0 where nothing is sent). One kernel, plain stores over NVLink. See cxg_put_rows."""
    _cuda(x, "x")
    _cuda(rows, "rows", (torch.int64,))
    n_peer = len(peer_ptrs)
    bases = (ctypes.c_void_p * n_peer)(*[None if not v else int(v) for v in peer_ptrs])
    segs = (ctypes.c_int64 * (n_peer + 1))(*[int(v) for v in seg_start])
    with _on(x.device):
        _check(_put_rows(_p(x), _p(rows), bases, segs, n_peer, x.shape[1] * x.element_size(), _stream()), "cxg_put_rows")


_sample = _sig("cxg_sample_neighbors", [_vp, _vp, ctypes.c_int, ctypes.c_int, _vp, _i64, ctypes.c_int, _vp, _vp,
                                        ctypes.c_uint64, _vp])


_sample_counts = _sig("cxg_sample_counts", [_vp, ctypes.c_int, _vp, _i64, ctypes.c_int, _vp, _vp])


def sample_neighbors(graph_ptr, graph_idx, frontier, fanout, seed):
    """min(degree, fanout) distinct in-neighbours of every frontier node, uniformly without replacement, as a CSR
    (out_ptr int64 [n + 1], out int64 global ids). Deterministic in (seed, node id). This is the step the reference
    takes from its external loader (neighbor_sample, cxgnncomp/data_preparation.py:214-215)."""
    _cuda(graph_ptr, "graph_ptr", _INDEX_DTYPES)
    _cuda(graph_idx, "graph_idx", _INDEX_DTYPES)
    _cuda(frontier, "frontier", (torch.int64,))
    n = frontier.shape[0]
    out_ptr = torch.zeros(n + 1, dtype=torch.int64, device=frontier.device)
    with _on(frontier.device):
        _check(_sample_counts(_p(graph_ptr), graph_ptr.element_size(), _p(frontier), n, int(fanout),
                              out_ptr[1:].data_ptr(), _stream()), "cxg_sample_counts")
    out_ptr[1:].cumsum_(0)
    out = torch.empty(int(out_ptr[-1]), dtype=torch.int64, device=frontier.device)
    with _on(frontier.device):
        _check(_sample(_p(graph_ptr), _p(graph_idx), graph_ptr.element_size(), graph_idx.element_size(), _p(frontier), n,
                       int(fanout), _p(out_ptr), _p(out), int(seed) & 0xFFFFFFFFFFFFFFFF, _stream()),
               "cxg_sample_neighbors")
    return out_ptr, out


_claim = _sig("cxg_renumber_claim", [_vp, _i64, _vp, _vp, _vp, _vp])
_assign = _sig("cxg_renumber_assign", [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp])


def renumber_claim(picked, local_of, fresh, n_fresh):
    """Appends the ids of `picked` that have no batch position yet (local_of == -1) to `fresh`, each once, and
    marks them claimed; n_fresh (int64 [1], device) receives the count. See cxg_renumber_claim."""
    for t_, name in ((picked, "picked"), (local_of, "local_of"), (fresh, "fresh"), (n_fresh, "n_fresh")):
        _cuda(t_, name, (torch.int64,))
    with _on(picked.device):
        _check(_claim(_p(picked), picked.shape[0], _p(local_of), _p(fresh), _p(n_fresh), _stream()),
               "cxg_renumber_claim")


def renumber_assign(fresh_sorted, base, picked, local_of):
    """local_of[fresh_sorted[i]] = base + i, then returns local_of[picked]. See cxg_renumber_assign."""
    for t_, name in ((picked, "picked"), (local_of, "local_of"), (fresh_sorted, "fresh_sorted")):
        _cuda(t_, name, (torch.int64,))
    out = torch.empty_like(picked)
    with _on(picked.device):
        _check(_assign(_p(fresh_sorted), fresh_sorted.shape[0], int(base), _p(picked), picked.shape[0], _p(local_of),
                       _p(out), _stream()), "cxg_renumber_assign")
    return out


class REDUCEOP(enum.IntEnum):
    """binding.cpp:108-113."""
    SUM = 0
    MAX = 1
    MIN = 2
    MEAN = 3


class COMPUTEOP(enum.IntEnum):
    """binding.cpp:114-119 (values of the C++ enum, dgsparse.h:15)."""
    ADD = 0
    SUB = 1
    MUL = 2
    DIV = 3


_gspmm = _sig("cxg_gspmm_csr", [_vp, _vp, ctypes.c_int, ctypes.c_int, _vp, _vp, _vp, _i64, ctypes.c_int, ctypes.c_int,
                                ctypes.c_int, _vp])


def _gspmm_call(rowptr, colind, val, b, re_op, comp_op):
    _cuda(rowptr, "A_rowptr", (torch.int32,))
    _cuda(colind, "A_colind", (torch.int32,))
    _cuda(b, "B", (torch.float32,))
    if val is not None:
        _cuda(val, "A_csrVal", (torch.float32,))
    if b.dim() != 2:
        raise RuntimeError("B must be [n_src, feat]")
    m = rowptr.shape[0] - 1
    out = torch.empty((m, b.shape[1]), dtype=torch.float32, device=b.device)
    with _on(b.device):
        _check(_gspmm(_p(rowptr), _p(colind), 4, 4, _p(val), _p(b), _p(out), m, b.shape[1], int(re_op), int(comp_op),
                      _stream()), "cxg_gspmm_csr")
    return out


def GSpMM_u(A_rowptr, A_colind, B, op):
    """out[r] = REDUCE over row r of B[colind[e]]; int32 CSR, fp32 (binding.cpp:98-104,107)."""
    return _gspmm_call(A_rowptr, A_colind, None, B, op, COMPUTEOP.MUL)


def GSpMM_u_e(A_rowptr, A_colind, A_csrVal, B, re_op, comp_op):
    """out[r] = REDUCE over row r of COMPUTE(val[e], B[colind[e]]) (binding.cpp:87-96,106)."""
    return _gspmm_call(A_rowptr, A_colind, A_csrVal, B, re_op, comp_op)


_gat_scores = _sig("cxg_gat_scores", [_vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_int, ctypes.c_int, _vp])
_gat_scores_bwd = _sig("cxg_gat_scores_backward", [_vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_int, ctypes.c_int, _vp])


_gat_att_grad_ws = _sig("cxg_gat_att_grad_workspace_size", [ctypes.c_int, ctypes.c_int, ctypes.POINTER(_sz)])
_gat_att_grad = _sig("cxg_gat_att_grad", [_vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_int, ctypes.c_int, _vp, _sz, _vp])


class _GatScoresFunction(torch.autograd.Function):
    """Both attention scores of a GAT layer from the transformed features in one kernel (the reference writes
    them as two multiply + sum pairs, cxgnncomp/graph_conv.py:470-474)."""

    @staticmethod
    def forward(ctx, feat, att_src, att_dst, num_dst):
        n, h, c = feat.shape
        a_s = torch.empty((n, h), dtype=torch.float32, device=feat.device)
        a_d = torch.empty((num_dst, h), dtype=torch.float32, device=feat.device)
        with _on(feat.device):
            _check(_gat_scores(_p(feat), _p(att_src), _p(att_dst), _p(a_s), _p(a_d), n, num_dst, h, c, _stream()),
                   "cxg_gat_scores")
        ctx.save_for_backward(feat, att_src, att_dst)
        ctx.num_dst = num_dst
        return a_s, a_d

    @staticmethod
    def backward(ctx, g_src, g_dst):
        feat, att_src, att_dst = ctx.saved_tensors
        n, h, c = feat.shape
        g_src, g_dst = g_src.contiguous(), g_dst.contiguous()
        grad_feat = grad_as = grad_ad = None
        if ctx.needs_input_grad[0]:
            grad_feat = torch.empty_like(feat)
            with _on(feat.device):
                _check(_gat_scores_bwd(_p(g_src), _p(g_dst), _p(att_src), _p(att_dst), _p(grad_feat), n, ctx.num_dst,
                                       h, c, _stream()), "cxg_gat_scores_backward")
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            grad_as, grad_ad = torch.empty_like(att_src), torch.empty_like(att_dst)
            need = _sz(0)
            _check(_gat_att_grad_ws(h, c, ctypes.byref(need)), "cxg_gat_att_grad_workspace_size")
            ws = _workspace(feat.device, need.value)
            with _on(feat.device):
                _check(_gat_att_grad(_p(feat), _p(g_src), _p(g_dst), _p(grad_as), _p(grad_ad), n, ctx.num_dst, h, c,
                                     _p(ws), ws.numel(), _stream()), "cxg_gat_att_grad")
        return grad_feat, grad_as, grad_ad, None


def gat_scores(feat, att_src, att_dst, num_dst):
    """(alpha_src [n_src, H], alpha_dst [num_dst, H]) from feat [n_src, H, C] and the attention vectors [.., H, C]."""
    _cuda(feat, "feat", (torch.float32,))
    _cuda(att_src, "att_src", (torch.float32,))
    _cuda(att_dst, "att_dst", (torch.float32,))
    if feat.dim() != 3 or att_src.numel() != feat.shape[1] * feat.shape[2] or att_dst.numel() != att_src.numel():
        raise RuntimeError("feat must be [n, H, C] and the attention vectors [H, C]")
    return _GatScoresFunction.apply(feat, att_src, att_dst, int(num_dst))


_colsum_ws = _sig("cxg_column_sum_workspace_size", [ctypes.c_int, ctypes.POINTER(_sz)])
_colsum = _sig("cxg_column_sum", [_vp, ctypes.c_int, _i64, ctypes.c_int, _vp, _vp, _sz, _vp])


def column_sum(x):
    """float32 [W]: the sum of the rows of x [N, W] (or [N, ...] flattened to W columns), added in a fixed order."""
    _cuda(x, "x", _FEAT_DTYPES)
    n = x.shape[0]
    width = x.numel() // n if n > 0 else int(torch.tensor(x.shape[1:]).prod())
    out = torch.empty(width, dtype=torch.float32, device=x.device)
    need = _sz(0)
    _check(_colsum_ws(width, ctypes.byref(need)), "cxg_column_sum_workspace_size")
    ws = _workspace(x.device, need.value)
    with _on(x.device):
        _check(_colsum(_p(x), _dtype_code(x), n, width, _p(out), _p(ws), ws.numel(), _stream()), "cxg_column_sum")
    return out


class _BiasAddFunction(torch.autograd.Function):
    """y + bias over the last dimension(s); the bias gradient is cxg_column_sum of the upstream gradient."""

    @staticmethod
    def forward(ctx, y, bias):
        ctx.bias_shape, ctx.bias_dtype = bias.shape, bias.dtype
        return y + bias

    @staticmethod
    def backward(ctx, grad):
        g_bias = None
        if ctx.needs_input_grad[1]:
            g_bias = column_sum(grad.contiguous()).view(ctx.bias_shape).to(ctx.bias_dtype)
        return grad, g_bias


def bias_add(y, bias):
    """y [N, ...] + bias [...] (bias covers all trailing dimensions of y); differentiable in both."""
    if (not y.is_cuda or y.dtype not in _FEAT_DTYPES or y.dim() < 2 or y.shape[0] == 0
            or bias.numel() * y.shape[0] != y.numel()):
        return y + bias
    return _BiasAddFunction.apply(y, bias)


_head_sum_c = _sig("cxg_head_sum", [_vp, _vp, _i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp])


def spmm_multihead(ptr, idx, val, vin, num_node, schedule=SPMM_MULTIHEAD_SCHEDULE.Optimal, block_size=256):
    """Multi-head SpMM with per-(edge, head) values (spmm_host.cu:158-196).
    Naive -> [num_node, H, F]; PreReduce / Optimal -> heads summed, [num_node, F]."""
    if vin.dim() != 3:
        raise RuntimeError("vin must be 3D, [num_node, num_head, feat_len]")
    if val.dim() != 2:
        raise RuntimeError("val must be 2D, [num_edge, num_head]")
    if vin.shape[1] != val.shape[1]:
        raise RuntimeError(f"num_head mismatch {vin.shape[1]} {val.shape[1]}")
    out = _spmm_forward(vin, ptr, idx, num_node, edge_val=val)
    if int(schedule) == int(SPMM_MULTIHEAD_SCHEDULE.Naive):
        return out
    return _head_sum(out)


def _head_sum(out):
    """[n, H, F] -> [n, F]: heads added in head order with one fp32 accumulator per column."""
    res = torch.empty((out.shape[0], out.shape[2]), dtype=out.dtype, device=out.device)
    with _on(out.device):
        _check(_head_sum_c(_p(out), _p(res), out.shape[0], out.shape[1], out.shape[2], _dtype_code(out), _stream()),
               "cxg_head_sum")
    return res


def spmm_multihead_bwd(ptr, idx, val, grad_output, grad_x, num_node, schedule=SPMM_MULTIHEAD_SCHEDULE.Optimal,
                       block_size=256):
    """grad_x[idx[e], h, :] += val[e, h] * grad_output[r, h, :]  in place (spmm_host.cu:198-214)."""
    _cuda(grad_x, "grad_x", (torch.float32,))
    _spmm_backward(grad_output, None, ptr, idx, num_node, edge_val=val, grad_x=grad_x, x_shape=grad_x.shape)
    return None


def run_spmm_multihead_configurable(ptr, idx, val, vin, num_node, *tuner_args):
    """Heads-summed multi-head SpMM, [num_node, F] (spmm_host.cu:216-256); tuner arguments ignored."""
    return spmm_multihead(ptr, idx, val, vin, num_node, SPMM_MULTIHEAD_SCHEDULE.PreReduce)


# --------------------------------------------------------------------------------------
# masked / target-indexed / relational aggregation, accumulated INTO the caller's output
# --------------------------------------------------------------------------------------
def selective_aggr(x, ptr, idx, mask, out, num_node):
    """out[r] += sum over the edges of row r whose mask is set (aggr.cu:478-492)."""
    _cuda(mask, "mask", (torch.bool, torch.uint8))
    _cuda(out, "out", (x.dtype,))
    _spmm_forward(x, ptr, idx, num_node, out=out, accumulate=True, edge_mask=mask)


def selective_aggr_bwd(grad_out, ptr, idx, mask, grad_x, num_center):
    """grad_x[idx[e]] += grad_out[r] for the masked edges (aggr.cu:494-509)."""
    _cuda(mask, "mask", (torch.bool, torch.uint8))
    _spmm_backward(grad_out, None, ptr, idx, num_center, grad_x=grad_x, edge_mask=mask, x_shape=grad_x.shape)


def target_aggr(x, ptr, idx, targets, out, num_node):
    """out[targets[r]] += sum of x[idx[e]] over row r (aggr.cu:450-463). `targets` must not
    repeat inside one call: each output row is owned by one group of lanes."""
    _cuda(targets, "targets", (torch.int64,))
    _cuda(out, "out", (x.dtype,))
    _spmm_forward(x, ptr, idx, num_node, out=out, accumulate=True, targets=targets)


def target_aggr_backward(grad_in, ptr, idx, targets, grad_out, num_node):
    """grad_out[idx[e]] += grad_in[targets[r]] (aggr.cu:465-476)."""
    _cuda(targets, "targets", (torch.int64,))
    _spmm_backward(grad_in, None, ptr, idx, num_node, grad_x=grad_out, targets=targets, x_shape=grad_out.shape)


_cidx_cache = []  # (idx, etype, versions, stride, combined), most recent last


def _combined_index(idx, etype, stride, num_rel):
    """etype[e] * stride + idx[e]: the row of the [num_rel * stride, F] table that edge e reads. Built once per
    (idx, etype) pair and kept (cache of 8), so that the relational aggregation is a plain aggregation over the
    table and takes the lean walk and the transposed-graph backward; int32 when the table has fewer than 2^31 rows."""
    ver = (idx._version, etype._version)
    for it in _cidx_cache:
        if it[0] is idx and it[1] is etype and it[2] == ver and it[3] == stride:
            return it[4]
    n = min(idx.shape[0], etype.shape[0])
    c = etype[:n].to(torch.int64) * stride + idx[:n].to(torch.int64)
    if stride * num_rel < 2 ** 31:
        c = c.to(torch.int32)
    _cidx_cache.append((idx, etype, ver, stride, c))
    if len(_cidx_cache) > 8:
        _cidx_cache.pop(0)
    return c


class _AggrRelFunction(torch.autograd.Function):
    """AggrRelFunction (src/cpp/src/rel_spmm.cu:37-135); `reduce` = CXG_MEAN divides every row by its edge count in
    the same kernel (the degree normalisation of MyRGCNConv, cxgnncomp/graph_conv.py:370-375). Edges are walked in
    CSR order with the row of the table computed per edge, which is the aggregation of the table over the combined
    index etype * N + idx: same additions in the same order as the reference's kernel."""

    @staticmethod
    def forward(ctx, x, ptr, idx, etype, num_node, num_rel, reduce):
        stride = x.shape[0] // num_rel
        cidx = _combined_index(idx, etype, stride, num_rel)
        ctx.save_for_backward(x, ptr, cidx)
        ctx.num_node, ctx.reduce = num_node, reduce
        return _spmm_forward(x, ptr, cidx, num_node, reduce=reduce)

    @staticmethod
    def backward(ctx, grad_out):
        x, ptr, cidx = ctx.saved_tensors
        dx, _ = _spmm_backward(grad_out, x, ptr, cidx, ctx.num_node, reduce=ctx.reduce)
        return dx.to(x.dtype), None, None, None, None, None, None


def aggr_rel(x, ptr, idx, etype, num_node, num_rel):
    """out[r] = sum_e x[etype[e] * N + idx[e]] with x = [num_rel * N, F] already transformed per
    relation; etype is int32 (binding.cpp:45, rel_spmm.cu:8-70)."""
    _cuda(etype, "etype", (torch.int32,))
    return _AggrRelFunction.apply(x, ptr, idx, etype, num_node, num_rel, CXG_SUM)


def aggr_rel_mean(x, ptr, idx, etype, num_node, num_rel):
    """aggr_rel divided by the number of edges of every destination (0 for destinations without edges), in one
    kernel: the aggregation + total-degree normalisation of the RGCN layer (cxgnncomp/graph_conv.py:370-375)."""
    _cuda(etype, "etype", (torch.int32,))
    return _AggrRelFunction.apply(x, ptr, idx, etype, num_node, num_rel, CXG_MEAN)


# --------------------------------------------------------------------------------------
# GAT: edge softmax, SDDMM, per-edge helpers
# --------------------------------------------------------------------------------------
_f, _int = ctypes.c_float, ctypes.c_int
_es_ws = _sig("cxg_edge_softmax_workspace_size", [_i64, _i64, ctypes.POINTER(_sz)])
_es_fwd = _sig("cxg_edge_softmax_forward", [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _i64, _i64, _int, _f, _vp, _sz, _vp])
_es_bwd = _sig("cxg_edge_softmax_backward",
               [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _f, _vp, _sz, _vp])
_sddmm = _sig("cxg_sddmm_coo", [_vp, _vp, _int, _vp, _vp, _vp, _i64, _int, _int, _int, _vp])
_evd = _sig("cxg_edge_value_degree", [_vp, _int, _vp, _i64, _vp])
_spmv = _sig("cxg_spmv_csr", [_vp, _vp, _int, _int, _vp, _vp, _i64, _vp])
_gather = _sig("cxg_gather_edges", [_vp, _vp, _int, _vp, _i64, _int, _int, _vp])


def _softmax_ws(device, n_dst, nnz):
    need = _sz(0)
    _check(_es_ws(n_dst, nnz, ctypes.byref(need)), "cxg_edge_softmax_workspace_size")
    return _workspace(device, need.value)


class _EdgeSoftmaxFunction(torch.autograd.Function):
    """EdgeSoftMaxFunction (src/cpp/src/edge_softmax.cu:97-177)."""

    @staticmethod
    def forward(ctx, ptr, idx, att_dst, att_src, num_edge, relu_l):
        _cuda(att_dst, "att_dst", (torch.float32,))
        _cuda(att_src, "att_src", (torch.float32,))
        _cuda(ptr, "ptr", _INDEX_DTYPES)
        _cuda(idx, "idx", _INDEX_DTYPES)
        n_dst, heads = att_dst.shape
        if ptr.shape[0] < n_dst + 1:
            raise RuntimeError("ptr has fewer rows than att_dst")
        out = torch.empty((num_edge, heads), dtype=torch.float32, device=att_dst.device)
        mask = torch.empty((num_edge, heads), dtype=torch.bool, device=att_dst.device)
        ws = _softmax_ws(att_dst.device, n_dst, num_edge)
        with _on(att_dst.device):
            _check(_es_fwd(_p(ptr), _p(idx), ptr.element_size(), idx.element_size(), _p(att_dst), _p(att_src), _p(out),
                           _p(mask), n_dst, num_edge, heads, float(relu_l), _p(ws), ws.numel(), _stream()),
                   "cxg_edge_softmax_forward")
        ctx.save_for_backward(ptr, idx, out, mask)
        ctx.shape = (n_dst, att_src.shape[0], heads, num_edge, float(relu_l))
        return out

    @staticmethod
    def backward(ctx, grad_out):
        ptr, idx, out, mask = ctx.saved_tensors
        n_dst, n_src, heads, num_edge, relu_l = ctx.shape
        grad_out = _cuda(grad_out.contiguous(), "grad", (torch.float32,))
        gd = torch.zeros((n_dst, heads), dtype=torch.float32, device=out.device)
        gs = torch.zeros((n_src, heads), dtype=torch.float32, device=out.device)
        ws = _softmax_ws(out.device, n_dst, num_edge)
        with _on(out.device):
            _check(_es_bwd(_p(ptr), _p(idx), ptr.element_size(), idx.element_size(), _p(grad_out), _p(mask), _p(out),
                           _p(gd), _p(gs), n_dst, num_edge, heads, relu_l, _p(ws), ws.numel(), _stream()),
                   "cxg_edge_softmax_backward")
        return None, None, gd, gs, None, None


def edge_attention(ptr, idx, att_dst, att_src, num_edge, relu_l):
    """softmax over each destination's edges of LeakyReLU(att_dst[d] + att_src[src]) -> [E, H]
    (binding.cpp:22-23, keyword arguments ptr, idx, att_dst, att_src, num_edge, relu_l)."""
    return _EdgeSoftmaxFunction.apply(ptr, idx, att_dst, att_src, int(num_edge), float(relu_l))


_gatf_ws = _sig("cxg_gat_fused_workspace_size", [_i64, _i64, _int, _int, ctypes.POINTER(_sz)])
_gatf_fwd = _sig("cxg_gat_fused_forward", [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _f,
                                           _vp, _sz, _vp])
_gatf_bwd = _sig("cxg_gat_fused_backward", [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                            _i64, _i64, _int, _int, _f, _vp, _vp, _int, _vp, _sz, _vp])
# False (default): the gradient of the destination scores is added with one atomic per edge and head, like the
# reference's backward (the only sum of the fused GAT backward whose order is not fixed); True: it is summed in a
# fixed order, bit-identical from run to run, at about 14 % more time for the layer's forward + backward.
GAT_ORDERED_ATT_GRAD = os.environ.get("CXG_GAT_ORDERED_ATT_GRAD", "0") == "1"


def gat_fused_supported(x_src):
    """True when cxg_gat_fused_forward covers this [N, H, C] feature tensor (fp32, H a power of two <= 16, rows of
    128 / 256 / 512 bytes, a lane's share of a row inside one head)."""
    if x_src.dim() != 3 or x_src.dtype != torch.float32 or not x_src.is_cuda:
        return False
    h, c = x_src.shape[1], x_src.shape[2]
    row = h * c * 4
    return h <= 16 and (h & (h - 1)) == 0 and row in (128, 256, 512) and (c * 4) % (row // 32) == 0


class _GatFusedFunction(torch.autograd.Function):
    """y = softmax-weighted neighbour sum of a GAT layer in one pass (cxg_gat_fused_forward); the backward
    recomputes the edge probabilities from the saved row maxima and sums over the transposed graph."""

    @staticmethod
    def forward(ctx, x_src, a_src, a_dst, ptr, idx, num_dst, slope):
        _cuda(x_src, "x_src", (torch.float32,))
        _cuda(a_src, "a_src", (torch.float32,))
        _cuda(a_dst, "a_dst", (torch.float32,))
        _cuda(ptr, "ptr", _INDEX_DTYPES)
        _cuda(idx, "idx", _INDEX_DTYPES)
        n = _num_rows(ptr, num_dst)
        n_src, h, c = x_src.shape
        if a_src.shape != (n_src, h) or a_dst.shape[0] < n or a_dst.shape[1] != h:
            raise RuntimeError("gat_fused: a_src must be [n_src, H] and a_dst [num_dst, H]")
        dev = x_src.device
        y = torch.empty((n, h, c), dtype=torch.float32, device=dev)
        row_max = torch.empty((n, h), dtype=torch.float32, device=dev)
        row_sum = torch.empty((n, h), dtype=torch.float32, device=dev)
        need = _sz(0)
        _check(_gatf_ws(n, idx.shape[0], h, c, ctypes.byref(need)), "cxg_gat_fused_workspace_size")
        ws = _workspace(dev, need.value)
        with _on(dev):
            _check(_gatf_fwd(_p(ptr), _p(idx), ptr.element_size(), idx.element_size(), _p(x_src), _p(a_src), _p(a_dst),
                             _p(y), _p(row_max), _p(row_sum), n, idx.shape[0], h, c, float(slope), _p(ws), ws.numel(),
                             _stream()), "cxg_gat_fused_forward")
        ctx.save_for_backward(x_src, a_src, a_dst, ptr, idx, y, row_max, row_sum)
        ctx.n, ctx.slope = n, float(slope)
        ctx.mark_non_differentiable(row_max, row_sum)
        return y, row_max, row_sum

    @staticmethod
    def backward(ctx, dy, _gmax, _gsum):
        x_src, a_src, a_dst, ptr, idx, y, row_max, row_sum = ctx.saved_tensors
        n, (n_src, h, c) = ctx.n, x_src.shape
        dev = x_src.device
        dy = _cuda(dy.contiguous(), "grad_out", (torch.float32,))
        t_ptr, t_idx, t_eid, _ = _transposed_graph(ptr, idx, n, n_src)
        ordered = GAT_ORDERED_ATT_GRAD and t_eid is not None
        dx = torch.empty_like(x_src)
        d_as = torch.empty((n_src, h), dtype=torch.float32, device=dev)
        d_ad = torch.empty((a_dst.shape[0], h), dtype=torch.float32, device=dev)
        if a_dst.shape[0] > n:
            d_ad[n:].zero_()
        need = _sz(0)
        _check(_gatf_ws(n, idx.shape[0], h, c, ctypes.byref(need)), "cxg_gat_fused_workspace_size")
        ws = _workspace(dev, need.value)
        with _on(dev):
            _check(_gatf_bwd(_p(t_ptr), _p(t_idx), t_ptr.element_size(), t_idx.element_size(), _p(dy), _p(y), _p(x_src),
                             _p(a_src), _p(a_dst), _p(row_max), _p(row_sum), _p(dx), _p(d_as), _p(d_ad), n_src, n,
                             t_idx.shape[0], h, c, ctx.slope, _p(t_eid) if ordered else None,
                             _p(ptr) if ordered else None, ptr.element_size(), _p(ws), ws.numel(), _stream()),
                   "cxg_gat_fused_backward")
        return dx, d_as, d_ad, None, None, None, None


def gat_fused(x_src, a_src, a_dst, ptr, idx, num_dst, negative_slope):
    """(y [num_dst, H, C], row_max [num_dst, H], row_sum [num_dst, H]): GAT aggregation of x_src [n_src, H, C] with
    attention scores a_src [n_src, H], a_dst [num_dst, H]; differentiable in x_src, a_src, a_dst."""
    return _GatFusedFunction.apply(x_src, a_src, a_dst, ptr, idx, int(num_dst), float(negative_slope))


def edge_value_degree(ptr, num_dst, num_edge):
    """val[e] = 1 / in-degree of e's destination (binding.cpp:24-25)."""
    _cuda(ptr, "ptr", _INDEX_DTYPES)
    out = torch.empty((int(num_edge),), dtype=torch.float32, device=ptr.device)
    with _on(ptr.device):
        _check(_evd(_p(ptr), ptr.element_size(), _p(out), int(num_dst), _stream()), "cxg_edge_value_degree")
    return out


def spmv(ptr, idx, x, num_dst):
    """y[d] = sum of x[idx[e]] over row d (binding.cpp:32)."""
    _cuda(x, "x", (torch.float32,))
    y = torch.empty((int(num_dst),), dtype=torch.float32, device=x.device)
    with _on(x.device):
        _check(_spmv(_p(ptr), _p(idx), ptr.element_size(), idx.element_size(), _p(x), _p(y), int(num_dst), _stream()),
               "cxg_spmv_csr")
    return y


def run_sddmm(src, dst, src_feat, dst_feat, output, num_edge):
    """output[e, h] = <src_feat[src[e], h, :], dst_feat[dst[e], :]> in place (binding.cpp:77,
    sddmm_host.cu:4-14). A 3-D dst_feat [N, H, F] selects the head-wise product."""
    _cuda(src_feat, "src_feat", (torch.float32,))
    _cuda(dst_feat, "dst_feat", (torch.float32,))
    _cuda(output, "output", (torch.float32,))
    _cuda(src, "src", _INDEX_DTYPES)
    _cuda(dst, "dst", (src.dtype,))
    heads, feat = src_feat.shape[1], src_feat.shape[-1]
    with _on(src_feat.device):
        _check(_sddmm(_p(src), _p(dst), src.element_size(), _p(src_feat), _p(dst_feat), _p(output), int(num_edge), feat,
                      heads, 1 if dst_feat.dim() == 3 else 0, _stream()), "cxg_sddmm_coo")
    return None


_DST_CACHE = {}


def _dst_of_edges(ptr, idx, n):
    """Destination (row) of every edge of the first n rows, in idx's dtype; kept per graph (the reference's tuned
    vertex-centric kernel avoids the expansion, sddmm_kernel.cu:27-279; here it is done once per ptr tensor)."""
    key = (ptr.data_ptr(), ptr._version, n, idx.dtype, str(ptr.device))
    hit = _DST_CACHE.get(key)
    if hit is None:
        deg = (ptr[1:n + 1] - ptr[:n]).long()
        hit = (torch.repeat_interleave(torch.arange(n, device=ptr.device, dtype=idx.dtype), deg), ptr)
        if len(_DST_CACHE) >= 8:
            _DST_CACHE.pop(next(iter(_DST_CACHE)))
        _DST_CACHE[key] = hit
    return hit[0]


def run_sddmm_vertex_centric(ptr, idx, src_feat, dst_feat, num_node, *tuner_args):
    """CSR form of run_sddmm: the destination of edge e is its row (sddmm_host.cu:16-60); returns [E, H].
    The tuner's launch integers are ignored."""
    n = _num_rows(ptr, num_node)
    dst = _dst_of_edges(ptr, idx, n)
    out = torch.zeros((idx.shape[0], src_feat.shape[1]), dtype=torch.float32, device=src_feat.device)
    run_sddmm(idx, dst, src_feat, dst_feat, out, dst.shape[0])
    return out


class _GatherFunction(torch.autograd.Function):
    """GatherFunction (src/cpp/src/aggr.cu:395-443)."""

    @staticmethod
    def forward(ctx, x_edge, dest, num_node):
        _cuda(x_edge, "input", (torch.float32,))
        _cuda(dest, "dest", _INDEX_DTYPES)
        if num_node <= 0:
            raise RuntimeError("gather: num_node must be positive")
        ctx.save_for_backward(dest)
        out = torch.zeros((num_node, x_edge.shape[1]), dtype=torch.float32, device=x_edge.device)
        with _on(x_edge.device):
            _check(_gather(_p(x_edge), _p(dest), dest.element_size(), _p(out), dest.shape[0], x_edge.shape[1], 0,
                           _stream()), "cxg_gather_edges")
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (dest,) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        g = torch.empty((dest.shape[0], grad_out.shape[1]), dtype=torch.float32, device=grad_out.device)
        with _on(grad_out.device):
            _check(_gather(_p(grad_out), _p(dest), dest.element_size(), _p(g), dest.shape[0], grad_out.shape[1], 1,
                           _stream()), "cxg_gather_edges")
        return g, None, None


def gather(x_edge, dest, num_node):
    """Scatter-add edge rows to their destination node: out[dest[e]] += x_edge[e] (binding.cpp:21)."""
    return _GatherFunction.apply(x_edge, dest, int(num_node))


# fp32 inputs of the typed matmul on the tensor cores: False (default) = error-compensated TF32 (three products per
# term, fp32 accuracy); True = plain TF32 like the reference's tl.dot (test/2-benchmark/bench-memory-rgcn.py:121
# sets allow_tf32).
ALLOW_TF32 = os.environ.get("CXG_ALLOW_TF32", "0") == "1"

from ._rgcn import (pad_rel, pad_rel_idx, typed_linear, typed_linear_s2e, typed_linear_s2d,  # noqa: E402,F401
                    aggr_rgcn_direct_func, rel_schedule, typed_matmul_raw, topo_sort, aggr_rel_direct,
                    typed_matmul_all_relations, typed_matmul_all_relations_supported, transform_all_relations,
                    dense_linear, typed_wgrad, typed_wgrad_supported)

# pybind's export_values(): the enum members are module attributes too
SUM, MAX, MIN, MEAN = REDUCEOP.SUM, REDUCEOP.MAX, REDUCEOP.MIN, REDUCEOP.MEAN
ADD, SUB, MUL, DIV = COMPUTEOP.ADD, COMPUTEOP.SUB, COMPUTEOP.MUL, COMPUTEOP.DIV
