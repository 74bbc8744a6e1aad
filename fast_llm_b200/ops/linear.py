"""Linear layers with hand-written backward passes and tensor / sequence parallel collectives.

    linear(x, W, b)                        y = x W^T + b
    mode "output" (column parallel)        W split along its output rows; with sequence parallelism the input holds
                                           T/tp tokens and is all-gathered first, and the input gradient is
                                           reduce-scattered (all-reduced without SP)
    mode "input"  (row parallel)           W split along its input columns; the partial outputs are reduce-scattered
                                           (SP) or all-reduced, the bias is added after the reduction
`transposed_weight` stores W as [in, out] (the MLP's second layer).  Weight gradients are accumulated by the GEMM
epilogue straight into the parameter's gradient buffer.  Parity: `fast_llm/functional/linear.py:27-273`.
"""

import torch

from fast_llm_b200.ops.gemm import matmul_nn, matmul_nt, matmul_tn
from fast_llm_b200.ops.param_grad import accumulate_param_grad, wgrad_target
from fast_llm_b200.parallel import fused_tp
from fast_llm_b200.parallel.ops import gather_op, reduce_op, reduce_scatter_op


def _forward_matmul(x2, weight, transposed_weight):
    return matmul_nn(x2, weight) if transposed_weight else matmul_nt(x2, weight)


def _dgrad(dy2, weight, transposed_weight):
    return matmul_nt(dy2, weight) if transposed_weight else matmul_nn(dy2, weight)


def weight_grad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor, transposed_weight: bool):
    """Accumulate dW into the gradient buffer (returns None) or return it for autograd."""
    buf, accumulate = wgrad_target(weight)
    a, b = (x2, dy2) if transposed_weight else (dy2, x2)
    if buf is not None:
        matmul_tn(a, b, out=buf.view(weight.shape), accumulate=accumulate)
        return None
    return matmul_tn(a, b, out_dtype=weight.dtype)


def bias_grad(dy2: torch.Tensor, bias: torch.Tensor):
    return accumulate_param_grad(bias, dy2.sum(0, dtype=torch.float32).to(bias.dtype) if dy2.dtype != torch.float32 else dy2.sum(0))


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, transposed_weight, mode, group, sequence_parallel):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        x_in = x2
        fused = fused_tp.usable(group, sequence_parallel, x2, weight)
        world = group.size() if group is not None else 1
        if fused is not None and mode == "output" and fused.fits(x2.shape[0] * world, x2.shape[1]):
            y = fused.all_gather_matmul(x2, weight, transposed_weight)  # the gather is the GEMM's operand fetch
        elif fused is not None and mode == "input" and fused.fits(x2.shape[0], weight.shape[1] if transposed_weight else weight.shape[0]):
            y = fused.matmul_reduce_scatter(x2, weight, transposed_weight)  # partial tiles leave from the epilogue
        else:
            if mode == "output" and sequence_parallel and group is not None:
                x2 = gather_op(x2, group, 0)
            y = _forward_matmul(x2, weight, transposed_weight)
            if mode == "input" and group is not None:
                y = reduce_scatter_op(y, group, dim=0) if sequence_parallel else reduce_op(y, group)
        if bias is not None:
            y = y + bias
        # Parameters are views of buffers that ZeRO-3 re-fills between forward and backward (with the same values):
        # keep them as plain attributes so autograd's version check does not fire.
        ctx.save_for_backward(x_in)
        ctx.weight, ctx.bias = weight, bias
        ctx.args = (transposed_weight, mode, group, sequence_parallel, shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x_in,) = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        transposed_weight, mode, group, sequence_parallel, shape = ctx.args
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        db = bias_grad(dy2, bias) if bias is not None else None
        fused = fused_tp.usable(group, sequence_parallel, dy2, x_in, weight) if mode in ("input", "output") else None
        if fused is not None:
            world = group.size()
            tokens = max(dy2.shape[0], x_in.shape[0])
            if not (fused.fits(tokens, dy2.shape[1] if mode == "input" else x_in.shape[1]) and tokens == min(dy2.shape[0], x_in.shape[0]) * world):
                fused = None
        if fused is not None:
            return _Linear._backward_fused(ctx, fused, dy2, x_in, weight, transposed_weight, mode, db)
        x2 = x_in
        if mode == "input" and sequence_parallel and group is not None:
            dy2 = gather_op(dy2, group, 0)
        gather_handle = None
        if mode == "output" and sequence_parallel and group is not None:
            x2, gather_handle = gather_op(x_in, group, 0, async_op=True)
        dx = _dgrad(dy2, weight, transposed_weight) if ctx.needs_input_grad[0] else None
        reduce_handle = None
        if dx is not None and mode == "output" and group is not None:
            if sequence_parallel:
                dx, reduce_handle = reduce_scatter_op(dx, group, dim=0, async_op=True)
            else:
                dx, reduce_handle = reduce_op(dx, group, async_op=True)
        if gather_handle is not None:
            gather_handle.wait()
        dw = weight_grad(dy2, x2, weight, transposed_weight) if weight.requires_grad or getattr(weight, "grad_buffer", None) is not None else None
        if reduce_handle is not None:
            reduce_handle.wait()
        return dx, dw, db, None, None, None, None


def _backward_fused(ctx, fused, dy2, x_in, weight, transposed_weight, mode, db):
    """Backward of a sequence-parallel linear layer with every collective folded into a GEMM."""
    has_buffer = weight.requires_grad or getattr(weight, "grad_buffer", None) is not None
    buf, accumulate = wgrad_target(weight) if has_buffer else (None, False)
    out = buf.view(weight.shape) if buf is not None else (torch.empty(weight.shape, dtype=weight.dtype, device=weight.device) if has_buffer else None)
    if mode == "output":
        # dy holds all tokens (local output features); x is sharded over tokens
        pending = fused.start_gather(x_in) if (out is not None and fused.single_launch) else None  # crosses NVLink under the dgrad
        dx = fused.matmul_reduce_scatter(dy2, weight, not transposed_weight) if ctx.needs_input_grad[0] else None
        if pending is not None:  # dW = dy^T gather(x)   (or gather(x)^T dy for a transposed weight): one GEMM over all tokens
            fused.wgrad_from_gathered(dy2, fused.finish_gather(pending), out, accumulate, gathered_is_a=transposed_weight)
        elif out is not None:
            fused.gathered_wgrad(dy2, x_in, out, accumulate, shard_is_a=transposed_weight)
    elif fused.single_launch:
        # dy is sharded over tokens; x holds all tokens (local input features).  dy is gathered once: the dgrad GEMM takes the
        # rows as they arrive, the weight gradient reads the same landing zone afterwards.
        pending = fused.start_gather(dy2)
        dx = fused.matmul_gathered(pending, weight, not transposed_weight) if ctx.needs_input_grad[0] else None
        if out is not None:  # dW = gather(dy)^T x   (or x^T gather(dy))
            fused.wgrad_from_gathered(x_in, fused.finish_gather(pending), out, accumulate, gathered_is_a=not transposed_weight)
    else:
        dx = fused.all_gather_matmul(dy2, weight, not transposed_weight) if ctx.needs_input_grad[0] else None
        if out is not None:
            fused.gathered_wgrad(x_in, dy2, out, accumulate, shard_is_a=not transposed_weight)
    dw = None if buf is not None else out
    return dx, dw, db, None, None, None, None


_Linear._backward_fused = staticmethod(_backward_fused)


def linear(x, weight, bias=None, *, transposed_weight: bool = False, mode: str = "none", group=None,
           sequence_parallel: bool = False):
    """Differentiable linear layer; see the module docstring for `mode`."""
    # Flatten outside the autograd node so its output is a fresh tensor (rotary later rotates it in place).
    lead = x.shape[:-1]
    y = _Linear.apply(x.reshape(-1, x.shape[-1]), weight, bias, transposed_weight, mode, group, sequence_parallel)
    if len(lead) != 1 and y.shape[0] == lead.numel():
        y = y.view(*lead, y.shape[-1])
    return y
