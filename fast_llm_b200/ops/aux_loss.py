"""Attach an auxiliary scalar loss to an activation so its gradient flows without changing the forward value.

Parity: `fast_llm/functional/utils.py:63-80` (AuxiliaryLoss).
"""

import torch


class _AuxiliaryLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, activation, loss, grad_scale):
        ctx.grad = torch.full_like(loss, grad_scale) if not torch.is_tensor(grad_scale) else grad_scale.to(loss.dtype).reshape(loss.shape)
        return activation.view_as(activation)

    @staticmethod
    def backward(ctx, grad):
        return grad, ctx.grad, None


def attach_auxiliary_loss(activation: torch.Tensor, loss: torch.Tensor, grad_scale=1.0) -> torch.Tensor:
    return _AuxiliaryLoss.apply(activation, loss, grad_scale)
