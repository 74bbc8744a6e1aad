"""Differentiable tensor-parallel primitives (forward collective / backward collective pairs).

Parity: `fast_llm/core/ops.py:18-222`.  These are the plain (NCCL/Gloo) versions used on CPU, in tests and wherever no
fused compute+collective kernel applies.
"""

import torch
import torch.distributed as dist

from fast_llm_b200.parallel.collectives import all_gather_into_tensor, all_reduce, reduce_scatter_tensor


def reduce_op(x: torch.Tensor, group, op=dist.ReduceOp.SUM, async_op: bool = False):
    if group is None:
        return (x, None) if async_op else x
    handle = all_reduce(x, op=op, group=group, async_op=async_op)
    return (x, handle) if async_op else x


def split_op(x: torch.Tensor, group, dim: int = 0) -> torch.Tensor:
    if group is None:
        return x
    return x.chunk(group.size(), dim=dim)[group.rank()].contiguous()


def gather_op(x: torch.Tensor, group, dim: int = 0, async_op: bool = False, out: torch.Tensor | None = None):
    if group is None:
        return (x, None) if async_op else x
    x = x.contiguous()
    n = group.size()
    if dim == 0:
        out = x.new_empty([n * x.shape[0], *x.shape[1:]]) if out is None else out
        handle = all_gather_into_tensor(out, x, group, async_op=async_op)
        return (out, handle) if async_op else out
    tmp = x.new_empty([n * x.shape[0], *x.shape[1:]])
    all_gather_into_tensor(tmp, x, group)
    res = torch.cat(list(tmp.chunk(n, dim=0)), dim=dim)
    return (res, None) if async_op else res


def reduce_scatter_op(x: torch.Tensor, group, op=dist.ReduceOp.SUM, dim: int = 0, async_op: bool = False):
    if group is None:
        return (x, None) if async_op else x
    n = group.size()
    if dim != 0:
        x = torch.cat(x.chunk(n, dim=dim), dim=0)
    x = x.contiguous()
    out = x.new_empty([x.shape[0] // n, *x.shape[1:]])
    handle = reduce_scatter_tensor(out, x, op=op, group=group, async_op=async_op)
    return (out, handle) if async_op else out


class _ReduceForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return reduce_op(x.clone() if x.requires_grad else x, group)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _ReduceBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        return reduce_op(grad.contiguous().clone(), ctx.group), None


class _Split(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return split_op(x, group, dim)

    @staticmethod
    def backward(ctx, grad):
        return gather_op(grad, ctx.group, ctx.dim), None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, reduce_grads):
        ctx.group, ctx.dim, ctx.reduce_grads = group, dim, reduce_grads
        return gather_op(x, group, dim)

    @staticmethod
    def backward(ctx, grad):
        if ctx.reduce_grads:
            return reduce_scatter_op(grad, ctx.group, dim=ctx.dim), None, None, None
        return split_op(grad, ctx.group, ctx.dim), None, None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return reduce_scatter_op(x, group, dim=dim)

    @staticmethod
    def backward(ctx, grad):
        return gather_op(grad, ctx.group, ctx.dim), None, None


def reduce_forward(x, group):
    return x if group is None else _ReduceForward.apply(x, group)


def reduce_backward(x, group):
    return x if group is None else _ReduceBackward.apply(x, group)


def split(x, group, dim: int = 0):
    return x if group is None else _Split.apply(x, group, dim)


def gather(x, group, dim: int = 0, reduce_grads: bool = False):
    return x if group is None else _Gather.apply(x, group, dim, reduce_grads)


def reduce_scatter(x, group, dim: int = 0):
    return x if group is None else _ReduceScatter.apply(x, group, dim)
