"""Pointwise copy-cast / fill / add / bias+residual and the embedding gather / scatter-add (`csrc/elementwise.cu`).

Parity: `fast_llm/functional/triton/pointwise.py:14-120` (copy, fill, add) and the compiled embedding / bias-dropout-add
helpers (`fast_llm/layers/language_model/embedding.py:74`, `fast_llm/layers/decoder/block.py:140`).
"""

import torch

from fast_llm_b200.ops import _lib

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _ok(*ts):
    return all(t is None or (t.is_cuda and t.dtype in _DT and t.is_contiguous()) for t in ts)


def axpby_(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None = None, alpha: float = 1.0, beta: float = 1.0):
    """out = alpha * a (+ beta * b) with dtype casts (fp32 / bf16)."""
    if _ok(out, a, b):
        _lib.check(_lib.get_lib().flb_axpby(a.data_ptr(), _DT[a.dtype], _lib.ptr(b), _DT[b.dtype] if b is not None else 0,
                                            out.data_ptr(), _DT[out.dtype], out.numel(), alpha, beta, _lib.stream_ptr()), "flb_axpby")
        _lib.count_launch()
        return out
    res = a.float() * alpha
    if b is not None:
        res = res + b.float() * beta
    return out.copy_(res)


def copy_(out, a):
    return axpby_(out, a)


def add_(out, a, b):
    return axpby_(out, a, b)


def fill_(out: torch.Tensor, value: float):
    if _ok(out):
        _lib.check(_lib.get_lib().flb_fill(out.data_ptr(), _DT[out.dtype], out.numel(), float(value), _lib.stream_ptr()), "flb_fill")
        _lib.count_launch()
        return out
    return out.fill_(value)


def bias_residual(x: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor | None, scale: float = 1.0):
    """(x + bias) * scale + residual."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[-1] % 8 == 0 and not torch.is_grad_enabled():
        out = torch.empty_like(x)
        _lib.check(_lib.get_lib().flb_bias_residual(x.data_ptr(), _lib.ptr(bias), _lib.ptr(residual), out.data_ptr(),
                                                    x.numel() // x.shape[-1], x.shape[-1], scale, _lib.stream_ptr()), "flb_bias_residual")
        _lib.count_launch()
        return out
    out = x if bias is None else x + bias
    if scale != 1.0:
        out = out * scale
    return out if residual is None else out + residual


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_begin, vocab_end, scale):
        from fast_llm_b200.ops.param_grad import has_grad_buffer

        ids = ids.contiguous().long()
        out = torch.empty(*ids.shape, weight.shape[1], dtype=weight.dtype, device=weight.device)
        _lib.check(_lib.get_lib().flb_embedding_fwd(ids.data_ptr(), weight.data_ptr(), out.data_ptr(), ids.numel(),
                                                    weight.shape[1], vocab_begin, vocab_end, scale, _lib.stream_ptr()), "flb_embedding_fwd")
        _lib.count_launch()
        ctx.save_for_backward(ids)
        ctx.weight = weight
        ctx.args = (vocab_begin, vocab_end, scale)
        return out

    @staticmethod
    def backward(ctx, grad):
        from fast_llm_b200.ops.param_grad import has_grad_buffer

        (ids,) = ctx.saved_tensors
        weight = ctx.weight
        vocab_begin, vocab_end, scale = ctx.args
        grad = grad.contiguous()
        target = None
        if has_grad_buffer(weight) and weight.grad_buffer.dtype == torch.float32:
            target = weight.grad_buffer
            if getattr(weight, "param_grad_is_zero", False):
                target.zero_()
                weight.param_grad_is_zero = False
            ret = None
        else:
            target = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            ret = target
        _lib.check(_lib.get_lib().flb_embedding_bwd(ids.data_ptr(), grad.data_ptr(), target.data_ptr(), ids.numel(),
                                                    weight.shape[1], vocab_begin, vocab_end, scale, _lib.stream_ptr()), "flb_embedding_bwd")
        _lib.count_launch()
        if ret is not None:
            from fast_llm_b200.ops.param_grad import accumulate_param_grad

            ret = accumulate_param_grad(weight, ret.to(weight.dtype) if not has_grad_buffer(weight) else ret)
        return None, ret, None, None, None


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_begin: int = 0, vocab_end: int | None = None,
              scale: float = 1.0) -> torch.Tensor:
    """Token embedding lookup of a (possibly vocabulary-sharded) table; ids outside the shard give zero rows."""
    vocab_end = vocab_begin + weight.shape[0] if vocab_end is None else vocab_end
    if weight.is_cuda and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0 and weight.is_contiguous():
        return _Embedding.apply(ids, weight, vocab_begin, vocab_end, scale)
    mask = (ids >= vocab_begin) & (ids < vocab_end)
    out = torch.nn.functional.embedding((ids - vocab_begin).clamp(0, weight.shape[0] - 1), weight)
    out = out * mask.unsqueeze(-1)
    return out * scale if scale != 1.0 else out
