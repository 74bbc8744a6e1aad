"""RMSNorm / LayerNorm with the preceding residual add fused in (kernels: `csrc/norm.cu`).

Behavioural parity with `fast_llm/layers/common/normalization/normalization.py:176-316` and the Triton kernels
`fast_llm/functional/triton/normalization.py:12-254`: fp32 statistics, optional zero-centred weight, weight/bias
gradients accumulated into the gradient buffer.
"""

import torch

from fast_llm_b200.ops import _lib
from fast_llm_b200.ops.param_grad import accumulate_param_grad, has_grad_buffer


def norm_reference(x, weight, bias, eps: float, zero_centered: bool = False, layer_norm: bool = False):
    """Plain PyTorch restatement (fp32 math), used on CPU and as the test oracle."""
    xf = x.float()
    if layer_norm:
        xf = xf - xf.mean(-1, keepdim=True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (w + 1 if zero_centered else w)
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384


def _fwd_native(x2, delta2, weight, bias, eps, zero_centered, layer_norm):
    rows, cols = x2.shape
    y = torch.empty_like(x2)
    res = torch.empty_like(x2) if delta2 is not None else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x2.device) if layer_norm else None
    _lib.check(
        _lib.get_lib().flb_norm_fwd(
            x2.data_ptr(), _lib.ptr(delta2), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(res), y.data_ptr(),
            rstd.data_ptr(), _lib.ptr(mean), rows, cols, eps, int(zero_centered), int(layer_norm), _lib.stream_ptr(),
        ),
        "flb_norm_fwd",
    )
    _lib.count_launch()
    return res, y, rstd, mean


def _bwd_native(dy2, x2, weight, bias, rstd, mean, dres2, zero_centered, layer_norm, need_param_grads):
    rows, cols = x2.shape
    lib = _lib.get_lib()
    dx = torch.empty_like(x2)
    parts = lib.flb_norm_bwd_parts(rows, cols, int(layer_norm))
    dwp = torch.empty(parts, cols, dtype=torch.float32, device=x2.device) if need_param_grads and weight is not None else None
    dbp = torch.empty(parts, cols, dtype=torch.float32, device=x2.device) if need_param_grads and bias is not None else None
    _lib.check(
        lib.flb_norm_bwd(
            dy2.data_ptr(), x2.data_ptr(), _lib.ptr(weight), rstd.data_ptr(), _lib.ptr(mean), _lib.ptr(dres2),
            dx.data_ptr(), _lib.ptr(dwp), _lib.ptr(dbp), rows, cols, int(zero_centered), int(layer_norm),
            _lib.stream_ptr(),
        ),
        "flb_norm_bwd",
    )
    _lib.count_launch()
    return dx, dwp, dbp


def _reduce_param_grad(param, partial):
    """Column-sum the per-CTA partials into the gradient buffer (or a fresh tensor for autograd)."""
    parts, cols = partial.shape
    lib = _lib.get_lib()
    if has_grad_buffer(param):
        buf = param.grad_buffer
        accumulate = not getattr(param, "param_grad_is_zero", False)
        param.param_grad_is_zero = False
        _lib.check(
            lib.flb_colsum(partial.data_ptr(), buf.data_ptr(), parts, cols, int(accumulate),
                           int(buf.dtype == torch.bfloat16), _lib.stream_ptr()), "flb_colsum")
        _lib.count_launch()
        return None
    out = torch.empty(cols, dtype=torch.float32, device=partial.device)
    _lib.check(lib.flb_colsum(partial.data_ptr(), out.data_ptr(), parts, cols, 0, 0, _lib.stream_ptr()), "flb_colsum")
    _lib.count_launch()
    return out.to(param.dtype)


class _NormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, bias, eps, zero_centered, layer_norm):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        delta2 = None if delta is None else delta.reshape(-1, shape[-1])
        res, y, rstd, mean = _fwd_native(x2.contiguous(), None if delta2 is None else delta2.contiguous(), weight, bias,
                                         eps, zero_centered, layer_norm)
        ctx.save_for_backward(x2 if res is None else res, rstd, mean)
        ctx.params = (weight, bias)
        ctx.args = (zero_centered, layer_norm, shape, delta is not None)
        if delta is None:
            return y.view(shape)
        return res.view(shape), y.view(shape)

    @staticmethod
    def backward(ctx, *grads):
        x2, rstd, mean = ctx.saved_tensors
        weight, bias = ctx.params
        zero_centered, layer_norm, shape, has_delta = ctx.args
        if has_delta:
            dres, dy = grads
        else:
            dres, dy = None, grads[0]
        dy2 = dy.reshape(-1, shape[-1]).contiguous()
        dres2 = None if dres is None else dres.reshape(-1, shape[-1]).contiguous()
        need_w = weight is not None and (ctx.needs_input_grad[2] or has_grad_buffer(weight))
        dx, dwp, dbp = _bwd_native(dy2, x2, weight, bias, rstd, mean, dres2, zero_centered, layer_norm, need_w)
        dw = _reduce_param_grad(weight, dwp) if dwp is not None else None
        db = _reduce_param_grad(bias, dbp) if dbp is not None else None
        dx = dx.view(shape)
        return dx, (dx if has_delta else None), dw, db, None, None, None


def norm(x, weight=None, bias=None, eps: float = 1e-5, zero_centered: bool = False, layer_norm: bool = False):
    if _native(x):
        return _NormFunction.apply(x, None, weight, bias, eps, zero_centered, layer_norm)
    return norm_reference(x, weight, bias, eps, zero_centered, layer_norm)


def add_norm(x, delta, weight=None, bias=None, eps: float = 1e-5, zero_centered: bool = False, layer_norm: bool = False):
    """(x + delta, norm(x + delta)): the residual update and the pre-norm of the next sub-layer in one pass."""
    if _native(x):
        return _NormFunction.apply(x, delta, weight, bias, eps, zero_centered, layer_norm)
    res = x + delta
    return res, norm_reference(res, weight, bias, eps, zero_centered, layer_norm)
