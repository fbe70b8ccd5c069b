import torch
import cxgnncomp_backend


class SpMMValOP(torch.autograd.Function):
    """Multi-head SpMM with per-(edge, head) values, x [N, H, F], val [E, H] -> [num_center, H, F]
    (cxgnncomp/graph_kernel.py:5-36). The reference's backward runs a scatter kernel for grad_x and an
    SDDMM for grad_val whose destination operand has no head axis (sddmm_kernel.cu:16-17), which is wrong
    for H > 1; here one fused kernel gives grad_x and the head-wise grad_val[e,h] = <grad_out[dst,h], x[src,h]>."""

    @staticmethod
    def forward(ctx, x, ptr, idx, val, num_center):
        ctx.save_for_backward(x, ptr, idx, val)
        ctx.num_center = num_center
        return cxgnncomp_backend.spmm_multihead(ptr, idx, val, x, num_center,
                                                cxgnncomp_backend.SPMM_MULTIHEAD_SCHEDULE.Naive)

    @staticmethod
    def backward(ctx, grad_out):
        x, ptr, idx, val = ctx.saved_tensors
        dx, dval = cxgnncomp_backend._spmm_backward(grad_out, x, ptr, idx, ctx.num_center, edge_val=val,
                                                    need_dx=ctx.needs_input_grad[0],
                                                    need_dval=ctx.needs_input_grad[3])
        if dx is not None and dx.dtype != x.dtype:
            dx = dx.to(x.dtype)
        return dx, None, None, dval, None
