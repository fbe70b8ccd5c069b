"""Typed-linear strategies of the reference (cxgnncomp/typed_linear.py:10-310), same names and arguments,
on the kernels of this library."""
import torch
import torch.nn.functional as F
import cxgnncomp_backend

from .codegen.typed_matmul import typed_matmul


def TypedLinearNaiveS2D(x, weights, types, src, dst, num_center, num_edge):
    """Gather features and weights per edge, multiply, scatter-add (typed_linear.py:10-21; the reference's
    torch.mm on a 3-D weight gather is ill-formed, the batched product is what it means)."""
    assert num_edge != 0
    feat = torch.index_select(x, 0, src[:num_edge])
    w = torch.index_select(weights, 0, types[:num_edge])
    out_e = torch.bmm(feat.unsqueeze(1), w).squeeze(1)
    output = torch.zeros([num_center, out_e.shape[1]], device=x.device, dtype=x.dtype)
    output.index_add_(0, dst[:num_edge], out_e)
    return output


def SelectMMS2EOP(x, weights, idx, types):
    """Per relation: torch.mm(x[idx[types == i]], weights[i]) (typed_linear.py:24-28)."""
    return [torch.mm(x[idx[types == i]], weights[i]) for i in range(weights.shape[0])]


def _dst_of_edges(ptr, num_center):
    return torch.repeat_interleave(torch.arange(num_center, device=ptr.device), ptr[1:num_center + 1] - ptr[:num_center])


class TypedLinearE2EOP(torch.autograd.Function):
    """x [E, K] (one row per edge) -> [E, N] with the weight of each edge's relation (typed_linear.py:71-137)."""

    @staticmethod
    def preprocess(weights, types, thres=256):
        """Bucket the edges by relation, every bucket padded to a multiple of `thres` (typed_linear.py:74-87).
        Returns [sorted_types, num_item, indices, count_cpu]. The sort is stable, so `indices` is reproducible
        (the reference's torch.sort is not)."""
        num_rel = weights.shape[0]
        num_item = types.shape[0]
        count = torch.bincount(types, minlength=num_rel)
        new_types = torch.empty([num_item + num_rel * (thres - 1)], device=weights.device, dtype=types.dtype)
        new_types[:num_item] = types
        cxgnncomp_backend.pad_rel(new_types, count, thres, num_rel, num_item)
        sorted_types, indices = torch.sort(new_types, stable=True)
        return [sorted_types, num_item, indices, count.cpu()]

    @staticmethod
    def forward(ctx, x, weights, types, preprocessed=[], thres=256, count=None):
        if len(preprocessed) == 4:
            sorted_types, num_item, indices, count = preprocessed
        else:
            sorted_types, num_item, indices, count = TypedLinearE2EOP.preprocess(weights, types, thres)
        output = typed_matmul(x, weights, sorted_types, num_item, indices)
        ctx.save_for_backward(x, weights, types, indices, sorted_types)
        ctx.num_item = num_item
        return output[:num_item]

    @staticmethod
    def backward(ctx, grad_out):
        x, weights, types, indices, sorted_types = ctx.saved_tensors
        num_rel = weights.shape[0]
        grad_x = None
        if ctx.needs_input_grad[0]:
            trans = torch.transpose(weights, 1, 2).contiguous()
            grad_x = typed_matmul(grad_out.contiguous(), trans, sorted_types, ctx.num_item, indices)[:ctx.num_item]
        grad_w = None
        if ctx.needs_input_grad[1]:
            # dW[r] = sum over the edges of relation r of x_e^T g_e. (The reference multiplies the unsorted
            # prefixes x[:count[i]] and grad[:count[i]] for every i, typed_linear.py:130-133, which is not
            # the gradient.)
            if cxgnncomp_backend.typed_wgrad_supported(x, grad_out):
                # one tensor-core launch over the sorted, padded positions (rows of padding positions do not exist)
                gw = cxgnncomp_backend.typed_wgrad(x.contiguous(), grad_out.contiguous(), sorted_types, num_rel,
                                                   ctx.num_item, idx=indices)
                return grad_x, gw.to(weights.dtype), None, None, None, None
            grad_w = torch.zeros_like(weights)
            order = torch.sort(types, stable=True).indices
            cnt = torch.bincount(types, minlength=num_rel).tolist()
            c = 0
            for i in range(num_rel):
                sel = order[c:c + cnt[i]]
                c += cnt[i]
                if cnt[i]:
                    grad_w[i] = torch.mm(x[sel].t().float(), grad_out[sel].float()).to(weights.dtype)
        return grad_x, grad_w, None, None, None, None


class TypedLinearS2EOP(torch.autograd.Function):
    """x [N_src, K] gathered by src_idx per edge -> [E, N] (typed_linear.py:140-188)."""

    @staticmethod
    def preprocess(weights, types, src_idx, thres):
        num_rel = weights.shape[0]
        num_item = src_idx.shape[0]
        count = torch.bincount(types, minlength=num_rel)
        pad = num_rel * (thres - 1)
        new_types = torch.empty([num_item + pad], device=weights.device, dtype=types.dtype)
        new_types[:num_item] = types
        new_src = torch.empty([num_item + pad], device=weights.device, dtype=src_idx.dtype)
        new_src[:num_item] = src_idx
        cxgnncomp_backend.pad_rel_idx(new_types, new_src, count, thres, num_rel, num_item)
        sorted_types, indices = torch.sort(new_types, stable=True)
        return [sorted_types, num_item, new_src, indices]

    @staticmethod
    def forward(ctx, x, weights, types, src_idx, preprocessed=[], thres=256, count=None):
        if len(preprocessed) == 4:
            sorted_types, num_item, new_src, indices = preprocessed
        else:
            sorted_types, num_item, new_src, indices = TypedLinearS2EOP.preprocess(weights, types, src_idx, thres)
        # position m reads row new_src[indices[m]] of x (-1 for padding) and writes row indices[m] of the output
        out = cxgnncomp_backend.typed_matmul_raw(x, weights, sorted_types, sorted_types.shape[0], x.shape[0],
                                                 src_idx=new_src[indices].contiguous(), dst_idx=indices,
                                                 out_rows=sorted_types.shape[0])
        return out[:num_item]

    @staticmethod
    def backward(ctx, grad_out):
        raise NotImplementedError("TypedLinearS2EOP has no backward in the reference either (typed_linear.py:187-188)")


class TypedLinearS2DMMAggrOP(torch.autograd.Function):
    """Transform all nodes with every relation's weight, aggregate the edges of that relation
    (typed_linear.py:191-221)."""

    @staticmethod
    def forward(ctx, x, weights, ptr, idx, rel, num_center):
        ctx.save_for_backward(x, weights, ptr, idx, rel)
        output = torch.zeros([num_center, weights.shape[-1]], device=x.device, dtype=x.dtype)
        for i in range(weights.shape[0]):
            cxgnncomp_backend.selective_aggr(torch.mm(x, weights[i]), ptr, idx, (rel == i), output, num_center)
        return output

    @staticmethod
    def backward(ctx, grad_out):
        x, weights, ptr, idx, rel = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        grad_x = torch.zeros_like(x)
        grad_weights = []
        for i in range(weights.shape[0]):
            g = torch.zeros([x.shape[0], grad_out.shape[-1]], device=x.device)
            cxgnncomp_backend.selective_aggr_bwd(grad_out, ptr, idx, (rel == i), g, grad_out.shape[0])
            grad_x += torch.mm(g, weights[i].t())
            grad_weights.append(torch.mm(x.t(), g))
        return grad_x, torch.stack(grad_weights), None, None, None, None


class TypedLinearS2DAggrMMOP(torch.autograd.Function):
    """Aggregate the edges of each relation first, transform the aggregate (typed_linear.py:224-258)."""

    @staticmethod
    def forward(ctx, x, weights, ptr, idx, rel, num_center):
        output = torch.zeros([num_center, weights.shape[-1]], device=x.device, dtype=x.dtype)
        aggr_outputs = []
        for i in range(weights.shape[0]):
            aggr = torch.zeros([num_center, weights.shape[-2]], device=x.device, dtype=x.dtype)
            cxgnncomp_backend.selective_aggr(x, ptr, idx, (rel == i), aggr, num_center)
            output += torch.mm(aggr, weights[i])
            aggr_outputs.append(aggr)
        ctx.save_for_backward(x, weights, ptr, idx, rel, torch.stack(aggr_outputs))
        return output

    @staticmethod
    def backward(ctx, grad_out):
        x, weights, ptr, idx, rel, aggr_outputs = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        grad_x = torch.zeros_like(x)
        grad_weights = []
        for i in range(weights.shape[0]):
            grad_mm = torch.mm(grad_out, weights[i].t())
            grad_weights.append(torch.mm(aggr_outputs[i].t(), grad_out))
            cxgnncomp_backend.selective_aggr_bwd(grad_mm, ptr, idx, (rel == i), grad_x, grad_out.shape[0])
        return grad_x, torch.stack(grad_weights), None, None, None, None


def TypedLinearS2DSort(x, weights, ptr, idx, rel, num_center, count=None):
    """Sort the edges by relation; per relation F.linear on the gathered sources and index_add_ into the
    destinations (typed_linear.py:262-310). Differentiable through torch."""
    dst = _dst_of_edges(ptr, num_center)
    num_rel = weights.shape[0]
    output = torch.zeros([num_center, weights.shape[-1]], device=x.device, dtype=x.dtype)
    _, indices = torch.sort(rel, stable=True)
    count = torch.bincount(rel, minlength=num_rel).cpu() if count is None else count.cpu()
    src, dst = idx[indices], dst[indices]
    cnt = 0
    for i in range(num_rel):
        k = int(count[i])
        s, d = src[cnt:cnt + k], dst[cnt:cnt + k]
        cnt += k
        output.index_add_(0, d, F.linear(x[s], weights[i].T))
    return output


def TypedLinearS2DPushOP(x, weights, types, src, dst, num_type, num_center, num_edge):
    """Transform each distinct (relation, source) pair once, then push the rows to the destinations
    (typed_linear.py:31-68)."""
    max_src = int(torch.max(src)) + 1
    key = types * max_src + src
    _, order = torch.sort(key, stable=True)
    uniq, inverse = torch.unique(key, return_inverse=True)
    type_u = torch.div(uniq, max_src, rounding_mode="floor")
    src_u = uniq % max_src
    # bucket the distinct pairs by relation (already sorted by key) and pad to the tile size
    pre = TypedLinearS2EOP.preprocess(weights, type_u, src_u, 128)
    rows = TypedLinearS2EOP.apply(x, weights, type_u, src_u, pre, 128)
    out = torch.zeros([num_center, weights.shape[-1]], dtype=x.dtype, device=x.device)
    out.index_add_(0, dst, rows[inverse])
    return out
