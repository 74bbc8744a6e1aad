"""Grouped GEMMs and the grouped expert MLP of a dropless mixture-of-experts layer.

Token rows are sorted by expert and every expert's range is padded to a multiple of 256 rows (one tile of the CTA-pair
GEMM), `row_begin` (device, int32 `[experts + 1]`) holds the range starts.  One kernel launch serves all experts in
each of the six products of the layer - fprop and dgrad of both layers (`grouped_rows`) and both weight gradients
(`grouped_wgrad`) - and nothing about the routing result is needed on the host.
Parity: `fast_llm/functional/triton/sparse_linear.py:191-560` (output-sparse, input-inner-sparse and input-row-sparse
matmuls), `fast_llm/functional/triton/mlp.py:207-477` (`mlp_autograd` with a sparse map).
"""

import torch

from fast_llm_b200.ops import _lib
from fast_llm_b200.ops.activation import ActivationType, act_bwd_native, mlp_activation
from fast_llm_b200.ops.gemm import _EPI_STORE_BF16, _epilogue
from fast_llm_b200.ops.param_grad import wgrad_target

TILE_ROWS = 256


def grouped_available(x: torch.Tensor, ffn: int, gated: bool) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and ffn % TILE_ROWS == 0 and x.shape[-1] % 8 == 0)


def grouped_rows(a: torch.Tensor, b: torch.Tensor, row_begin: torch.Tensor, experts: int, n: int, k: int, b_mn: bool) -> torch.Tensor:
    """c[rows of e] = a[rows of e] @ B_e^T (b_mn False: b = [experts * n, k]) or @ B_e (b_mn True: b = [experts * k, n])."""
    rows = a.shape[0]
    out = torch.empty(rows, n, dtype=a.dtype, device=a.device)
    _lib.check(_lib.get_lib().flb_grouped_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), row_begin.data_ptr(), experts, rows, 0, n, k,
                                                   a.stride(0), b.stride(0), out.stride(0), int(b_mn), _EPI_STORE_BF16, 1, _lib.stream_ptr()),
               "flb_grouped_gemm_bf16")
    _lib.count_launch()
    return out


def grouped_rows_gated(x: torch.Tensor, w1: torch.Tensor, row_begin: torch.Tensor, experts: int, ffn: int,
                       activation: ActivationType) -> tuple[torch.Tensor, torch.Tensor]:
    """First layer of gated experts with the activation in the GEMM's epilogue: h[rows of e] = x[rows of e] @ W1_e^T
    (W1_e = [gate rows; up rows], [2 ffn, hidden]) and act(gate) * up, both bf16, from one launch."""
    rows, hidden = x.shape
    h = torch.empty(rows, 2 * ffn, dtype=x.dtype, device=x.device)
    a = torch.empty(rows, ffn, dtype=x.dtype, device=x.device)
    _lib.check(_lib.get_lib().flb_grouped_gemm_gated_bf16(x.data_ptr(), w1.data_ptr(), h.data_ptr(), a.data_ptr(), row_begin.data_ptr(), experts, rows,
                                                         ffn, hidden, x.stride(0), w1.stride(0), h.stride(0), a.stride(0), activation.code,
                                                         _lib.stream_ptr()), "flb_grouped_gemm_gated_bf16")
    _lib.count_launch()
    return h, a


def grouped_wgrad(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, row_begin: torch.Tensor, experts: int, accumulate: bool) -> torch.Tensor:
    """out[e * m : (e + 1) * m] (+)= a[rows of e]^T @ b[rows of e];  a [rows, m], b [rows, n], out [experts * m, n]."""
    m, n = a.shape[1], b.shape[1]
    assert out.shape == (experts * m, n), (out.shape, experts, m, n)
    _lib.check(_lib.get_lib().flb_grouped_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), row_begin.data_ptr(), experts, a.shape[0], m, n, 0,
                                                   a.stride(0), b.stride(0), out.stride(0), 1, _epilogue(out, accumulate), 2, _lib.stream_ptr()),
               "flb_grouped_gemm_bf16")
    _lib.count_launch()
    return out


class _GroupedMLP(torch.autograd.Function):
    """y = act(x W1_e^T) W2_e for the expert e owning each row; W1 [experts * (1 + gated) * ffn, hidden], W2 [experts * ffn, hidden]."""

    @staticmethod
    def forward(ctx, x, row_begin, w1, w2, experts, gated, activation):
        hidden = x.shape[1]
        ffn = w2.shape[0] // experts
        if gated:
            h, a = grouped_rows_gated(x, w1, row_begin, experts, ffn, activation)  # the activation rides in the GEMM's epilogue
        else:
            h = grouped_rows(x, w1, row_begin, experts, w1.shape[0] // experts, hidden, b_mn=False)
            a = mlp_activation(h, gated, activation)
        y = grouped_rows(a, w2, row_begin, experts, hidden, ffn, b_mn=True)
        ctx.save_for_backward(x, h, row_begin)
        ctx.weights = (w1, w2)  # buffer views: kept outside autograd's version tracking
        ctx.args = (experts, gated, activation, ffn)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, h, row_begin = ctx.saved_tensors
        w1, w2 = ctx.weights
        experts, gated, activation, ffn = ctx.args
        hidden = x.shape[1]
        dy = dy.contiguous()
        da = grouped_rows(dy, w2, row_begin, experts, ffn, hidden, b_mn=False)
        dh, a = act_bwd_native(da, h, gated, activation, True)  # one kernel: the gradient and the recomputed activation
        del da
        grads = []
        for weight, lhs, rhs in ((w2, a, dy), (w1, dh, x)):
            needs = weight.requires_grad or getattr(weight, "grad_buffer", None) is not None
            if not needs:
                grads.append(None)
                continue
            buffer, accumulate = wgrad_target(weight)
            if buffer is not None:
                grouped_wgrad(lhs, rhs, buffer.view(weight.shape), row_begin, experts, accumulate)
                grads.append(None)
            else:
                grads.append(grouped_wgrad(lhs, rhs, torch.empty(weight.shape, dtype=weight.dtype, device=weight.device), row_begin, experts, False))
        dw2, dw1 = grads
        dx = grouped_rows(dh, w1, row_begin, experts, hidden, w1.shape[0] // experts, b_mn=True) if ctx.needs_input_grad[0] else None
        return dx, None, dw1, dw2, None, None, None


def grouped_mlp(x, row_begin, w1, w2, experts: int, gated: bool, activation: ActivationType) -> torch.Tensor:
    return _GroupedMLP.apply(x, row_begin, w1, w2, experts, gated, activation)


def _dispatch_raw(x, rows, scale, padded_rows: int) -> torch.Tensor:
    tokens, k = rows.shape
    out = torch.zeros(padded_rows, x.shape[1], dtype=x.dtype, device=x.device)  # padding rows stay zero
    _lib.check(_lib.get_lib().flb_moe_dispatch(x.data_ptr(), rows.data_ptr(), _lib.ptr(scale), out.data_ptr(), tokens, k, x.shape[1], _lib.stream_ptr()),
               "flb_moe_dispatch")
    _lib.count_launch()
    return out


def _combine_raw(y, rows, scores) -> torch.Tensor:
    tokens, k = rows.shape
    out = torch.empty(tokens, y.shape[1], dtype=y.dtype, device=y.device)
    _lib.check(_lib.get_lib().flb_moe_combine(y.data_ptr(), rows.data_ptr(), _lib.ptr(scores), out.data_ptr(), tokens, k, y.shape[1], _lib.stream_ptr()),
               "flb_moe_combine")
    _lib.count_launch()
    return out


class _Dispatch(torch.autograd.Function):
    """xs[rows[t, j]] = x[t]: copies every token to the row of each of its experts."""

    @staticmethod
    def forward(ctx, x, rows, padded_rows):
        ctx.save_for_backward(rows)
        return _dispatch_raw(x.contiguous(), rows, None, padded_rows)

    @staticmethod
    def backward(ctx, grad):
        (rows,) = ctx.saved_tensors
        return _combine_raw(grad.contiguous(), rows, None), None, None


class _Combine(torch.autograd.Function):
    """out[t] = sum_j scores[t, j] * y[rows[t, j]]"""

    @staticmethod
    def forward(ctx, y, rows, scores):
        scores = scores.float().contiguous()
        ctx.save_for_backward(y, rows, scores)
        return _combine_raw(y.contiguous(), rows, scores)

    @staticmethod
    def backward(ctx, grad):
        y, rows, scores = ctx.saved_tensors
        grad = grad.contiguous()
        tokens, k = rows.shape
        dy = _dispatch_raw(grad, rows, scores, y.shape[0])
        dscores = torch.empty(tokens, k, dtype=torch.float32, device=y.device)
        _lib.check(_lib.get_lib().flb_moe_score_grad(y.data_ptr(), rows.data_ptr(), grad.data_ptr(), dscores.data_ptr(), tokens, k, y.shape[1],
                                                     _lib.stream_ptr()), "flb_moe_score_grad")
        _lib.count_launch()
        return dy, None, dscores


def dispatch(x: torch.Tensor, rows: torch.Tensor, padded_rows: int) -> torch.Tensor:
    return _Dispatch.apply(x, rows, padded_rows)


def combine(y: torch.Tensor, rows: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
    return _Combine.apply(y, rows, scores)


def expert_rows(top_experts: torch.Tensor, experts: int) -> tuple[torch.Tensor, torch.Tensor, int]:
    """(rows int32 [tokens, k]: row of every (token, choice) in the expert-sorted padded space, row_begin, padded size)."""
    token_index, dest, row_begin, rows_upper_bound, order = expert_layout(top_experts, experts)
    rows = torch.empty(top_experts.numel(), dtype=torch.int32, device=top_experts.device)
    rows[order] = dest.to(torch.int32)
    return rows.view(top_experts.shape), row_begin, rows_upper_bound


def expert_layout(top_experts: torch.Tensor, experts: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """Device-side layout of the expert-sorted, padded row space.

    Returns (token_index [T*k]: source token of every sorted entry, dest [T*k]: its row in the padded space,
    row_begin int32 [experts + 1], rows_upper_bound: host-side size of the padded buffers)."""
    tokens, k = top_experts.shape
    flat = top_experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_experts = flat[order]
    counts = torch.bincount(flat, minlength=experts)
    padded = (counts + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS
    row_begin = torch.zeros(experts + 1, dtype=torch.int64, device=flat.device)
    row_begin[1:] = padded.cumsum(0)
    first_unpadded = counts.cumsum(0) - counts
    dest = row_begin[sorted_experts] + torch.arange(flat.numel(), device=flat.device) - first_unpadded[sorted_experts]
    rows_upper_bound = (tokens * k + experts * (TILE_ROWS - 1) + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS
    return torch.div(order, k, rounding_mode="floor"), dest, row_begin.to(torch.int32), rows_upper_bound, order
