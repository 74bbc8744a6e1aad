"""Top-k routing of a mixture-of-experts layer (`csrc/moe.cu`): the routing scores, the chosen experts, the load-balancing
and z-loss values and the gradient of the router logits in two kernels, and the layout of the expert-sorted, tile-padded row
space in one, with a PyTorch restatement for CPU tensors.

    scores, experts, aux, z = route_topk(logits, k, aux_weight, z_weight)

`aux = E * sum_e mean_t([e chosen for t]) * mean_t(softmax(logits)[t, e])`, `z = mean_t logsumexp(logits[t])^2`; their gradients
enter the backward of `scores` with weights `aux_weight` / `z_weight` (the values themselves are returned detached, for logging).
Parity: `fast_llm/layers/decoder/mlp/mixture_of_experts.py:237-262`, `fast_llm/functional/triton/sparse_copy.py:201-241`.
"""

import torch

from fast_llm_b200.ops import _lib

MAX_EXPERTS, MAX_TOP_K = 64, 8


def native_routing_available(logits: torch.Tensor, k: int) -> bool:
    return logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.shape[1] <= MAX_EXPERTS and k <= MAX_TOP_K


class _RouteTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, aux_weight, z_weight):
        logits = logits.contiguous()
        tokens, experts = logits.shape
        lib = _lib.get_lib()
        scores = torch.empty(tokens, k, dtype=torch.float32, device=logits.device)
        top = torch.empty(tokens, k, dtype=torch.int32, device=logits.device)
        partial = torch.empty(lib.flb_moe_route_blocks(tokens), experts, dtype=torch.float32, device=logits.device)
        lse = torch.empty(tokens, dtype=torch.float32, device=logits.device)
        _lib.check(lib.flb_moe_route(logits.data_ptr(), tokens, experts, k, scores.data_ptr(), top.data_ptr(), partial.data_ptr(), lse.data_ptr(),
                                     _lib.stream_ptr()), "flb_moe_route")
        _lib.count_launch()
        prob_mean = partial.sum(0) / tokens
        chosen_mean = torch.zeros(experts, dtype=torch.float32, device=logits.device).index_add_(
            0, top.reshape(-1).long(), torch.ones(tokens * k, dtype=torch.float32, device=logits.device)) / tokens
        aux = experts * (chosen_mean * prob_mean).sum()
        z = (lse * lse).mean()
        ctx.save_for_backward(logits, scores, top, chosen_mean)
        ctx.args = (k, float(aux_weight), float(z_weight))
        ctx.mark_non_differentiable(top)
        return scores, top, aux.detach(), z.detach()

    @staticmethod
    def backward(ctx, dscores, _dtop, _daux, _dz):
        logits, scores, top, chosen_mean = ctx.saved_tensors
        k, aux_weight, z_weight = ctx.args
        tokens, experts = logits.shape
        dlogits = torch.empty_like(logits)
        # d aux / d softmax[t, e] = E * chosen_mean[e] / tokens
        aux_grad = (chosen_mean * (aux_weight * experts / tokens)).contiguous() if aux_weight else None
        dscores = None if dscores is None else dscores.float().contiguous()
        _lib.check(_lib.get_lib().flb_moe_route_bwd(logits.data_ptr(), scores.data_ptr(), top.data_ptr(), _lib.ptr(dscores), _lib.ptr(aux_grad),
                                                    z_weight / tokens, tokens, experts, k, dlogits.data_ptr(), _lib.stream_ptr()), "flb_moe_route_bwd")
        _lib.count_launch()
        return dlogits, None, None, None


def route_topk_reference(logits: torch.Tensor, k: int, aux_weight: float = 0.0, z_weight: float = 0.0):
    """PyTorch restatement; the auxiliary losses are attached to the scores so that their gradients flow in backward."""
    from fast_llm_b200.ops.aux_loss import attach_auxiliary_loss

    logits = logits.float()
    z = torch.logsumexp(logits, dim=-1).pow(2).mean()
    if z_weight and logits.requires_grad:
        logits = attach_auxiliary_loss(logits, z, z_weight)
    top_logits, top = torch.topk(logits, k=k, dim=-1)
    scores = torch.softmax(top_logits, dim=-1, dtype=torch.float32)
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    mask = torch.zeros_like(probs).scatter_(1, top, 1.0)
    aux = logits.shape[1] * (mask.mean(0) * probs.mean(0)).sum()
    if aux_weight and logits.requires_grad:
        scores = attach_auxiliary_loss(scores, aux, aux_weight)
    return scores, top, aux.detach(), z.detach()


def route_topk(logits: torch.Tensor, k: int, aux_weight: float = 0.0, z_weight: float = 0.0):
    """(scores fp32 [T, k], experts [T, k] (int32 on the device path, int64 otherwise), aux value, z value)."""
    if native_routing_available(logits, k):
        return _RouteTopK.apply(logits, k, aux_weight, z_weight)
    return route_topk_reference(logits, k, aux_weight, z_weight)


def expert_rows_native(top: torch.Tensor, experts: int, tile_rows: int) -> tuple[torch.Tensor, torch.Tensor, int]:
    """(rows int32 [T, k], row_begin int32 [experts + 1], host-side upper bound of the padded row count) in one launch; rows of
    one expert are in token order (the same layout as a stable sort by expert gives)."""
    tokens, k = top.shape
    top = top.to(torch.int32).contiguous()
    rows = torch.empty(tokens, k, dtype=torch.int32, device=top.device)
    row_begin = torch.empty(experts + 1, dtype=torch.int32, device=top.device)
    _lib.check(_lib.get_lib().flb_moe_layout(top.data_ptr(), tokens * k, experts, tile_rows, rows.data_ptr(), row_begin.data_ptr(), None,
                                             _lib.stream_ptr()), "flb_moe_layout")
    _lib.count_launch()
    upper = (tokens * k + experts * (tile_rows - 1) + tile_rows - 1) // tile_rows * tile_rows
    return rows, row_begin, upper
