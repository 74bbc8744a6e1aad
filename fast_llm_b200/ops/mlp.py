"""Two-layer MLP as one autograd node with a hand-written backward and activation recomputation.

    h = x W1^T (+ b1)          [tokens, (2 if gated) * ffn]     gate columns first, then up columns
    a = act(gate) * up         (or act(h))
    y = a W2 (+ b2)            W2 stored transposed: [ffn, hidden]

Under tensor parallelism W1 is split by rows of each of its two halves and W2 by rows, so `h` and `a` hold ffn/tp
columns; the input is all-gathered (sequence parallel) and the output reduce-scattered or all-reduced.
Recompute levels follow `fast_llm/functional/config.py:31-47`: none keeps `a`; activation recomputes `a` in backward
(default here: the recompute rides along in the activation-backward kernel for free); activation_and_input also
re-gathers / recomputes the layer input; full recomputes `h` as well.  Parity: `fast_llm/functional/triton/mlp.py:207-418`.
"""

import enum

import torch

from fast_llm_b200.ops.activation import ActivationType, _native as _act_native, act_bwd_native, act_fwd_native, mlp_activation_reference
from fast_llm_b200.ops.gemm import gated_ok, matmul_nn, matmul_nt, matmul_nt_gated
from fast_llm_b200.ops.linear import bias_grad, weight_grad
from fast_llm_b200.parallel import fused_tp
from fast_llm_b200.parallel.ops import gather_op, reduce_op, reduce_scatter_op


class MLPRecomputeLevel(str, enum.Enum):
    none = "none"
    activation = "activation"
    activation_and_input = "activation_and_input"
    full = "full"

    @property
    def recompute_layer_1(self) -> bool:
        return self == MLPRecomputeLevel.full

    @property
    def recompute_activation(self) -> bool:
        return self != MLPRecomputeLevel.none

    @property
    def recompute_sparse_input(self) -> bool:
        return self in (MLPRecomputeLevel.full, MLPRecomputeLevel.activation_and_input)


def _act_fwd(h, gated, act):
    if _act_native(h):
        return act_fwd_native(h, gated, act)
    return mlp_activation_reference(h, gated, act)


def _act_bwd(da, h, gated, act, recompute):
    if _act_native(h):
        return act_bwd_native(da.contiguous(), h, gated, act, recompute)
    with torch.enable_grad():
        h_ = h.detach().requires_grad_()
        a = mlp_activation_reference(h_, gated, act)
    (dh,) = torch.autograd.grad(a, h_, da)
    return dh, (a.detach() if recompute else None)


class _MLP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, gated, act, group, sequence_parallel, recompute):
        shape = x.shape
        x_in = x.reshape(-1, shape[-1])
        fused = _fused_context(x_in, w1, b1, w2, b2, group, sequence_parallel)
        if fused is not None:
            # both collectives ride in the GEMMs: the token shards arrive inside the layer-1 GEMM (peers push, the GEMM waits per
            # row block), the partial outputs of layer 2 leave for their owners from its epilogue
            if gated and w1.shape[0] % 16 == 0:
                h, a = fused.matmul_gathered_gated(fused.start_gather(x_in), w1, act.code)  # and the activation in its epilogue
            else:
                h = fused.matmul_gathered(fused.start_gather(x_in), w1, False)
                a = _act_fwd(h, gated, act)
            y = fused.matmul_reduce_scatter(a, w2, True)
            ctx.save_for_backward(x_in, None if recompute.recompute_layer_1 else h, None if recompute.recompute_activation else a)
            ctx.params = (w1, b1, w2, b2)
            ctx.args = (gated, act, group, sequence_parallel, recompute, shape)
            ctx.fused = fused
            return y if len(shape) == 2 else y.view(*shape[:-1], y.shape[-1])
        ctx.fused = None
        x2 = gather_op(x_in, group, 0) if (sequence_parallel and group is not None) else x_in
        if gated and b1 is None and gated_ok(x2, w1):
            h, a = matmul_nt_gated(x2, w1, act.code)  # the activation rides in the GEMM's epilogue
        else:
            h = matmul_nt(x2, w1)
            if b1 is not None:
                h = h + b1
            a = _act_fwd(h, gated, act)
        y = matmul_nn(a, w2)
        if group is not None:
            y = reduce_scatter_op(y, group, dim=0) if sequence_parallel else reduce_op(y, group)
        if b2 is not None:
            y = y + b2
        keep_input = x_in if (recompute.recompute_sparse_input or (sequence_parallel and group is not None)) else x2
        ctx.save_for_backward(keep_input, None if recompute.recompute_layer_1 else h, None if recompute.recompute_activation else a)
        ctx.params = (w1, b1, w2, b2)  # buffer views: kept outside autograd's version tracking (ZeRO-3 re-gathers them)
        ctx.args = (gated, act, group, sequence_parallel, recompute, shape)
        return y.view(*shape[:-1], y.shape[-1]) if y.shape[0] == x_in.shape[0] else y

    @staticmethod
    def backward(ctx, dy):
        x_saved, h, a = ctx.saved_tensors
        w1, b1, w2, b2 = ctx.params
        gated, act, group, sequence_parallel, recompute, shape = ctx.args
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.fused is not None:
            return _MLP._backward_fused(ctx, dy2, x_saved, h, a)
        db2 = bias_grad(dy2, b2) if b2 is not None else None
        sp = sequence_parallel and group is not None
        if sp:
            dy2 = gather_op(dy2, group, 0)
        x2 = gather_op(x_saved, group, 0) if sp else x_saved
        if h is None:
            h = matmul_nt(x2, w1)
            if b1 is not None:
                h = h + b1
        da = matmul_nt(dy2, w2)  # [tokens, ffn] = dy @ W2^T with W2 stored [ffn, hidden]
        dh, a_re = _act_bwd(da, h, gated, act, a is None)
        a = a_re if a is None else a
        dw2 = weight_grad(dy2, a, w2, transposed_weight=True)
        del a, da
        db1 = bias_grad(dh, b1) if b1 is not None else None
        dx = matmul_nn(dh, w1) if ctx.needs_input_grad[0] else None
        handle = None
        if dx is not None and group is not None:
            dx, handle = reduce_scatter_op(dx, group, dim=0, async_op=True) if sp else reduce_op(dx, group, async_op=True)
        dw1 = weight_grad(dh, x2, w1, transposed_weight=False)
        if handle is not None:
            handle.wait()
        if dx is not None and dx.numel() == x_saved.numel() and len(shape) != 2:
            dx = dx.view(shape)
        return dx, dw1, db1, dw2, db2, None, None, None, None, None


def _fused_context(x_in, w1, b1, w2, b2, group, sequence_parallel):
    """The tensor group's fused-collective context when it can serve this MLP (sequence parallel, no biases, single-launch
    gather, operands it accepts and a landing zone that is large enough), else None."""
    if not sequence_parallel or group is None or b1 is not None or b2 is not None:
        return None
    fused = fused_tp.usable(group, True, x_in, w1, w2)
    if fused is None or not fused.single_launch:
        return None
    return fused if fused.fits(x_in.shape[0] * group.size(), x_in.shape[1]) else None


def _backward_fused(ctx, dy2, x_saved, h, a):
    """Backward of the sequence-parallel MLP with every collective inside a GEMM: the output gradient and the layer input
    are each gathered once (their pushes cross NVLink under the first GEMM), the gathered output gradient feeds the layer-2
    dgrad as it arrives and the layer-2 weight gradient afterwards, the gathered input feeds the layer-1 weight gradient, and
    the input gradient is reduce-scattered from the epilogue of the layer-1 dgrad."""
    w1, b1, w2, b2 = ctx.params
    gated, act, group, sequence_parallel, recompute, shape = ctx.args
    fused = ctx.fused
    pending_dy = fused.start_gather(dy2)
    pending_x = fused.start_gather(x_saved)
    da = fused.matmul_gathered(pending_dy, w2, False)  # [tokens, ffn/tp] = gather(dy) @ W2^T
    if h is None:
        h = fused.matmul_gathered(pending_x, w1, False)
    dh, a_re = _act_bwd(da, h, gated, act, a is None)
    a = a_re if a is None else a
    del da
    dy_full = fused.finish_gather(pending_dy)
    dw2 = weight_grad(dy_full, a, w2, transposed_weight=True)
    del a
    dx = fused.matmul_reduce_scatter(dh, w1, True) if ctx.needs_input_grad[0] else None
    dw1 = weight_grad(dh, fused.finish_gather(pending_x), w1, transposed_weight=False)
    if dx is not None and len(shape) != 2:
        dx = dx.view(shape)
    return dx, dw1, None, dw2, None, None, None, None, None, None


_MLP._backward_fused = staticmethod(_backward_fused)


def mlp(x, w1, b1, w2, b2, *, gated: bool, activation: ActivationType, group=None, sequence_parallel: bool = False,
        recompute_level: MLPRecomputeLevel = MLPRecomputeLevel.activation):
    return _MLP.apply(x, w1, b1, w2, b2, gated, activation, group, sequence_parallel, recompute_level)
