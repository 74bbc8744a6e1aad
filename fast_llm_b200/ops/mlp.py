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


def mlp(x, w1, b1, w2, b2, *, gated: bool, activation: ActivationType, group=None, sequence_parallel: bool = False,
        recompute_level: MLPRecomputeLevel = MLPRecomputeLevel.activation):
    return _MLP.apply(x, w1, b1, w2, b2, gated, activation, group, sequence_parallel, recompute_level)
