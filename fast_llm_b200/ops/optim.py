"""Optimizer kernels over flat fp32 shards (`csrc/optim.cu`): sum of squares, device-side clip coefficient, AdamW.

Replaces the apex multi-tensor kernels the reference calls from `fast_llm/core/kernels.py:20-91`.  Everything stays on
the device: the clip coefficient is computed by a one-thread kernel from the (all-reduced) squared norm and consumed by
the Adam kernel through a pointer, so the optimizer step needs no host synchronisation.
"""

import torch

from fast_llm_b200.ops import _lib


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[0] (+)= sum(x**2) for a flat fp32 tensor; deterministic two-stage reduction."""
    if x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.data_ptr() % 16 == 0:
        lib = _lib.get_lib()
        scratch = torch.empty(lib.flb_sumsq_scratch_floats(), dtype=torch.float32, device=x.device)
        _lib.check(lib.flb_sumsq(x.data_ptr(), x.numel(), scratch.data_ptr(), out.data_ptr(), int(accumulate),
                                 _lib.stream_ptr()), "flb_sumsq")
        _lib.count_launch(2)
        return out
    s = x.float().pow(2).sum()
    if accumulate:
        out.add_(s)
    else:
        out.fill_(s)
    return out


def sum_partials(partials: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[0] (+)= partials.sum() in a fixed order (one block); `partials` fp32 on the device."""
    if partials.is_cuda:
        _lib.check(_lib.get_lib().flb_sum_partials(partials.data_ptr(), partials.numel(), out.data_ptr(), int(accumulate),
                                                   _lib.stream_ptr()), "flb_sum_partials")
        _lib.count_launch()
        return out
    s = partials.float().sum()
    return out.add_(s) if accumulate else out.fill_(s)


def clip_coeff(normsq: torch.Tensor, max_norm: float, extra_scale: float, coeff_out: torch.Tensor,
               norm_out: torch.Tensor) -> None:
    """coeff = extra_scale * min(1, max_norm / (norm + 1e-6)), norm = sqrt(normsq) * extra_scale; max_norm <= 0 disables."""
    if normsq.is_cuda:
        _lib.check(_lib.get_lib().flb_clip_coeff(normsq.data_ptr(), float(max_norm), float(extra_scale),
                                                 coeff_out.data_ptr(), norm_out.data_ptr(), _lib.stream_ptr()), "flb_clip_coeff")
        _lib.count_launch()
        return
    norm = normsq.sqrt() * extra_scale
    c = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
    coeff_out.copy_(c * extra_scale)
    norm_out.copy_(norm)


def adamw_reference(w, g, m, v, w_lp, lr, beta1, beta2, eps, wd, step, gscale):
    g = g.float() * gscale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1**step, 1 - beta2**step
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + wd * w
    w.sub_(upd * lr)
    if w_lp is not None:
        w_lp.copy_(w)


def adamw(w, g, m, v, w_lp, lr: float, beta1: float, beta2: float, eps: float, wd: float, step: int,
          gscale: float = 1.0, gscale_tensor: torch.Tensor | None = None, noop_flag: torch.Tensor | None = None) -> None:
    """Fused decoupled-weight-decay Adam (apex `adam_w_mode`) on flat shards; `w_lp` gets the bf16 weights."""
    if w.numel() == 0:
        return
    if w.is_cuda and g.dtype == torch.float32 and (w_lp is None or w_lp.dtype == torch.bfloat16):
        _lib.check(
            _lib.get_lib().flb_adamw(w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _lib.ptr(w_lp), w.numel(),
                                     lr, beta1, beta2, eps, wd, step, gscale, _lib.ptr(gscale_tensor),
                                     _lib.ptr(noop_flag), _lib.stream_ptr()), "flb_adamw")
        _lib.count_launch()
        return
    if noop_flag is not None and bool(noop_flag.item()):
        return
    scale = gscale * (gscale_tensor.item() if gscale_tensor is not None else 1.0)
    adamw_reference(w, g, m, v, w_lp, lr, beta1, beta2, eps, wd, step, scale)
