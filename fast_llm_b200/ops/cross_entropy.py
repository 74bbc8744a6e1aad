"""Fused cross-entropy forward + backward over (optionally vocabulary-parallel) logits (`csrc/loss.cu`).

Two kernels bracket the tensor-parallel exchange of per-token softmax statistics (max, sum-exp, target logit), matching
the structure of `fast_llm/functional/triton/entropy_loss.py:99-290,769-864`; the gradient overwrites the logits in
place, so the `[tokens, vocab]` matrix exists once.  A z-loss term (`fast_llm/functional/triton/z_loss.py:13`) rides on
the same softmax.
"""

import torch

from fast_llm_b200.ops import _lib


def cross_entropy_reference(logits, labels, grad_scale: float | None, logits_scale: float = 1.0, z_coef: float = 0.0,
                            group=None, vocab_begin: int = 0):
    """PyTorch restatement (fp32). Returns (per-token loss, per-token lse^2, grad or None). Ignores labels < 0."""
    x = logits.float() * logits_scale
    local_max = x.max(-1).values
    gmax = local_max.clone()
    if group is not None:
        torch.distributed.all_reduce(gmax, op=torch.distributed.ReduceOp.MAX, group=group)
    e = torch.exp(x - gmax[:, None])
    se = e.sum(-1)
    lab = labels - vocab_begin
    in_shard = (lab >= 0) & (lab < x.shape[-1]) & (labels >= 0)
    tgt = torch.where(in_shard, x.gather(-1, lab.clamp(0, x.shape[-1] - 1)[:, None])[:, 0], torch.zeros_like(se))
    if group is not None:
        torch.distributed.all_reduce(se, group=group)
        torch.distributed.all_reduce(tgt, group=group)
    valid = labels >= 0
    lse = gmax + se.log()
    loss = torch.where(valid, lse - tgt, torch.zeros_like(lse))
    z = torch.where(valid, lse * lse, torch.zeros_like(lse))
    grad = None
    if grad_scale is not None:
        g = grad_scale if torch.is_tensor(grad_scale) else torch.tensor(grad_scale, device=x.device)
        p = e / se[:, None] * (1 + 2 * z_coef * lse)[:, None]
        onehot = torch.zeros_like(p)
        onehot[in_shard, lab[in_shard]] = 1.0
        grad = ((p - onehot) * valid[:, None] * g * logits_scale).to(logits.dtype)
    return loss, z, grad


def cross_entropy_forward_backward(logits: torch.Tensor, labels: torch.Tensor, grad_scale, logits_scale: float = 1.0,
                                   z_coef: float = 0.0, group=None, vocab_begin: int = 0, in_place: bool = True):
    """Returns (loss_per_token fp32, z_per_token fp32, grad_logits).  `grad_scale` may be a float or a 1-element
    device tensor (kept on the device: no host sync); None skips the backward.  With `in_place` the gradient
    overwrites `logits`."""
    vec = 8 if logits.dtype == torch.bfloat16 else 4
    native = (logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(-1) == 1
              and logits.stride(0) % vec == 0 and logits.data_ptr() % 16 == 0)
    if not native:
        return cross_entropy_reference(logits, labels, grad_scale, logits_scale, z_coef, group, vocab_begin)
    lib = _lib.get_lib()
    rows, cols = logits.shape
    dtype_code = 1 if logits.dtype == torch.bfloat16 else 0
    labels = labels.contiguous()
    slots = 1
    fused = None
    if group is not None:
        from fast_llm_b200.parallel import fused_ce

        context = fused_ce.get(group)
        fused = context.slots(rows) if context is not None else None
    if fused is not None:
        # statistics go straight into every peer's buffer; the gradient kernel merges the shards
        stats, peer_ptrs = fused
        slots = context.world
        _lib.check(lib.flb_ce_stats_exchange(logits.data_ptr(), dtype_code, labels.data_ptr(), peer_ptrs, context.rank, context.world, rows, cols,
                                             logits.stride(0), vocab_begin, logits_scale, _lib.stream_ptr()), "flb_ce_stats_exchange")
        _lib.count_launch()
        context.barrier()
    else:
        stats = torch.empty(rows, 3, dtype=torch.float32, device=logits.device)
        _lib.check(lib.flb_ce_stats(logits.data_ptr(), dtype_code, labels.data_ptr(), stats.data_ptr(), rows, cols,
                                    logits.stride(0), vocab_begin, logits_scale, _lib.stream_ptr()), "flb_ce_stats")
        _lib.count_launch()
        if group is not None:
            # Merge shards: global max, rescaled sum-exp, summed target logit.
            local_max = stats[:, 0].clone()
            gmax = local_max.clone()
            torch.distributed.all_reduce(gmax, op=torch.distributed.ReduceOp.MAX, group=group)
            packed = torch.stack([stats[:, 1] * torch.exp(local_max - gmax), stats[:, 2]], 0)
            torch.distributed.all_reduce(packed, group=group)
            stats = torch.stack([gmax, packed[0], packed[1]], 1).contiguous()
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    z = torch.empty(rows, dtype=torch.float32, device=logits.device)
    grad = None
    gs_val, gs_ptr = 1.0, None
    if grad_scale is not None:
        if in_place:
            grad = logits
        else:
            pad = 8 if logits.dtype == torch.bfloat16 else 4
            grad = torch.empty(rows, (cols + pad - 1) // pad * pad, dtype=logits.dtype, device=logits.device)[:, :cols]
        if torch.is_tensor(grad_scale):
            gs_ptr = grad_scale.float().contiguous()
        else:
            gs_val = float(grad_scale)
    _lib.check(
        lib.flb_ce_grad_slots(logits.data_ptr(), dtype_code, labels.data_ptr(), stats.data_ptr(), slots, _lib.ptr(grad),
                        loss.data_ptr(), z.data_ptr(), rows, cols, logits.stride(0),
                        grad.stride(0) if grad is not None else logits.stride(0), vocab_begin, logits_scale, gs_val,
                        _lib.ptr(gs_ptr), z_coef, _lib.stream_ptr()), "flb_ce_grad_slots")
    _lib.count_launch()
    return loss, z, grad
