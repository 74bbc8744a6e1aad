"""Parameter-gradient plumbing shared by the hand-written backward passes.

Parameters owned by a stage are views into a flat weight buffer and carry a `grad_buffer` attribute (a view into the
flat gradient buffer, fp32 or bf16) and a `param_grad_is_zero` flag.  Backward kernels add straight into that buffer
(parity: `fast_llm/tensor.py:351` accumulate_gradient, `fast_llm/functional/linear.py:27-69`), so parameter gradients
never materialise as `.grad`.  Parameters without a buffer (unit tests, plain modules) get ordinary autograd gradients.
"""

import torch


def has_grad_buffer(param: torch.Tensor) -> bool:
    return getattr(param, "grad_buffer", None) is not None


def accumulate_param_grad(param: torch.Tensor, grad: torch.Tensor) -> torch.Tensor | None:
    """Add `grad` into the parameter's gradient buffer, or hand it back to autograd if there is none."""
    if not has_grad_buffer(param):
        return grad
    buf = param.grad_buffer
    if getattr(param, "param_grad_is_zero", False):
        buf.copy_(grad.view_as(buf))
        param.param_grad_is_zero = False
    else:
        buf.add_(grad.view_as(buf))
    return None


def wgrad_target(param: torch.Tensor) -> tuple[torch.Tensor | None, bool]:
    """(buffer to accumulate a weight gradient into, whether to add to its current content)."""
    if not has_grad_buffer(param):
        return None, False
    # A joint view over several neighbouring parameters (fused QKV) tracks the state of its sources.
    sources = getattr(param, "_sources", None) or (param,)
    zero = [getattr(s, "param_grad_is_zero", False) for s in sources]
    assert all(zero) or not any(zero), "fused parameters must be accumulated together"
    for s in sources:
        s.param_grad_is_zero = False
    return param.grad_buffer, not zero[0]
