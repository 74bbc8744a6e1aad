"""Language-model losses over one shared softmax (`csrc/loss.cu`).

Two families, both vocabulary-parallel aware and both written so that the `[tokens, vocab]` logits are read twice and
written once, with no fp32 copy of them:

* **from labels**: every loss whose dependence on a token's logits goes through `lse = logsumexp(s)` and the target logit
  `s_label` only (cross-entropy, z-loss, KL against one-hot targets, the log-probability ratios of GRPO / GSPO / DPO).
  `softmax_statistics` returns `lse` and `s_label` per token; the losses are functions of these `[tokens]` vectors, their
  derivatives `a = dL/dlse`, `b = dL/ds_label` come from autograd on the vectors, and `softmax_coeff_grad` writes
  `a_t softmax_j + b_t [j = label_t]` for the sum of all of them in one pass.
  Parity: `fast_llm/functional/triton/monolithic_loss.py:14-353`, `grpo_loss.py:13`, `gspo_loss.py:12`, `z_loss.py:13`.
* **from a distribution** (distillation): cross-entropy, forward KL and reverse KL against teacher logits with a
  temperature and a loss mask: `distribution_loss_forward_backward`.
  Parity: `fast_llm/functional/triton/entropy_loss.py:294-700`, `fast_llm/functional/entropy_loss.py:123-215`.

On CPU (and for dtypes / layouts the kernels do not take) the same arithmetic runs as PyTorch ops on fp32 without autograd
over the logits.
"""

import torch

from fast_llm_b200.ops import _lib


def _native(logits: torch.Tensor) -> bool:
    vec = 8 if logits.dtype == torch.bfloat16 else 4
    return (logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.dim() == 2 and logits.stride(-1) == 1
            and logits.stride(0) % vec == 0 and logits.data_ptr() % 16 == 0)


def _all_reduce(t, group, op=None):
    if group is not None:
        torch.distributed.all_reduce(t, op=op or torch.distributed.ReduceOp.SUM, group=group)
    return t


class SoftmaxStatistics:
    """Per-token statistics of softmax(logits * scale) over the whole (possibly sharded) vocabulary.

    `lse` and `target` are fp32 `[tokens]` tensors (target = scaled logit at the label, 0 for labels < 0).
    `raw` / `slots` are the kernel's `[slots, tokens, 3]` buffer, consumed again by `softmax_coeff_grad`."""

    def __init__(self, lse, target, raw=None, slots=1, scale=1.0, vocab_begin=0):
        self.lse, self.target, self.raw, self.slots, self.scale, self.vocab_begin = lse, target, raw, slots, scale, vocab_begin


def softmax_statistics(logits: torch.Tensor, labels: torch.Tensor | None, logits_scale: float = 1.0, group=None,
                       vocab_begin: int = 0) -> SoftmaxStatistics:
    rows, cols = logits.shape
    if labels is None:
        labels = torch.full((rows,), -1, dtype=torch.int64, device=logits.device)
    labels = labels.contiguous()
    if _native(logits):
        lib = _lib.get_lib()
        dtype_code = 1 if logits.dtype == torch.bfloat16 else 0
        fused = context = None
        if group is not None:
            from fast_llm_b200.parallel import fused_ce

            context = fused_ce.get(group)
            fused = context.slots(rows) if context is not None else None
        if fused is not None:
            raw, peer_ptrs = fused
            slots = context.world
            _lib.check(lib.flb_ce_stats_exchange(logits.data_ptr(), dtype_code, labels.data_ptr(), peer_ptrs, context.rank, context.world, rows,
                                                 cols, logits.stride(0), vocab_begin, logits_scale, _lib.stream_ptr()), "flb_ce_stats_exchange")
            _lib.count_launch()
            context.barrier()
            view = raw  # [slots, rows, 3]
            gmax = view[:, :, 0].max(0).values
            se = (view[:, :, 1] * torch.exp(view[:, :, 0] - gmax)).sum(0)
            target = view[:, :, 2].sum(0)
        else:
            raw = torch.empty(rows, 3, dtype=torch.float32, device=logits.device)
            _lib.check(lib.flb_ce_stats(logits.data_ptr(), dtype_code, labels.data_ptr(), raw.data_ptr(), rows, cols, logits.stride(0),
                                        vocab_begin, logits_scale, _lib.stream_ptr()), "flb_ce_stats")
            _lib.count_launch()
            slots = 1
            if group is not None:
                local_max = raw[:, 0]
                gmax = _all_reduce(local_max.clone(), group, torch.distributed.ReduceOp.MAX)
                packed = _all_reduce(torch.stack([raw[:, 1] * torch.exp(local_max - gmax), raw[:, 2]], 0), group)
                raw = torch.stack([gmax, packed[0], packed[1]], 1).contiguous()
            gmax, se, target = raw[:, 0], raw[:, 1], raw[:, 2]
        return SoftmaxStatistics(gmax + se.log(), target, raw, slots, logits_scale, vocab_begin)
    # PyTorch path (fp32, chunk-free: CPU tests and odd layouts)
    x = logits.float() * logits_scale
    gmax = _all_reduce(x.max(-1).values, group, torch.distributed.ReduceOp.MAX)
    se = _all_reduce(torch.exp(x - gmax[:, None]).sum(-1), group)
    lab = labels - vocab_begin
    in_shard = (lab >= 0) & (lab < cols) & (labels >= 0)
    target = torch.where(in_shard, x.gather(-1, lab.clamp(0, cols - 1)[:, None])[:, 0], torch.zeros_like(se))
    target = _all_reduce(target, group)
    return SoftmaxStatistics(gmax + se.log(), target, None, 1, logits_scale, vocab_begin)


def softmax_coeff_grad(logits: torch.Tensor, labels: torch.Tensor | None, stats: SoftmaxStatistics, prob_coeff: torch.Tensor,
                       label_coeff: torch.Tensor, *, accumulate_into: torch.Tensor | None = None, in_place: bool = True) -> torch.Tensor:
    """Gradient wrt the (unscaled) logits of a loss with `dL/dlse = prob_coeff`, `dL/ds_label = label_coeff` per token.
    Written over `logits` when `in_place`, added to `accumulate_into` when given, else into a new tensor."""
    rows, cols = logits.shape
    scale = stats.scale
    a = (prob_coeff.float() * scale).contiguous()
    b = (label_coeff.float() * scale).contiguous()
    if _native(logits) and stats.raw is not None and (accumulate_into is None or _native(accumulate_into)):
        if accumulate_into is not None:
            grad, accumulate = accumulate_into, 1
        elif in_place:
            grad, accumulate = logits, 0
        else:
            pad = 8 if logits.dtype == torch.bfloat16 else 4
            grad, accumulate = torch.empty(rows, (cols + pad - 1) // pad * pad, dtype=logits.dtype, device=logits.device)[:, :cols], 0
        lab = None if labels is None else labels.contiguous()
        _lib.check(_lib.get_lib().flb_softmax_coeff_grad(
            logits.data_ptr(), 1 if logits.dtype == torch.bfloat16 else 0, _lib.ptr(lab), stats.raw.data_ptr(), stats.slots, a.data_ptr(),
            b.data_ptr(), grad.data_ptr(), rows, cols, logits.stride(0), grad.stride(0), stats.vocab_begin, scale, accumulate,
            _lib.stream_ptr()), "flb_softmax_coeff_grad")
        _lib.count_launch()
        return grad
    p = torch.exp(logits.float() * scale - stats.lse[:, None])
    grad = p * a[:, None]
    if labels is not None:
        lab = labels - stats.vocab_begin
        in_shard = (lab >= 0) & (lab < cols) & (labels >= 0)
        grad[in_shard, lab[in_shard]] += b[in_shard]
    grad = grad.to(logits.dtype)
    if accumulate_into is not None:
        return accumulate_into.add_(grad)
    if in_place:
        return logits.copy_(grad)
    return grad


def label_coefficients(per_token_fn, stats: SoftmaxStatistics, weight: "float | torch.Tensor | None"):
    """Evaluate `per_token_fn(lse, target) -> scalar` and return (value, dL/dlse, dL/dtarget) scaled by `weight`;
    the derivatives are None when `weight` is None (no backward)."""
    if weight is None:
        with torch.no_grad():
            return per_token_fn(stats.lse, stats.target), None, None
    with torch.enable_grad():
        lse = stats.lse.detach().requires_grad_()
        target = stats.target.detach().requires_grad_()
        value = per_token_fn(lse, target)
        a, b = torch.autograd.grad(value * weight, (lse, target), allow_unused=True)
    zeros = torch.zeros_like(stats.lse)
    return value.detach(), zeros if a is None else a, zeros if b is None else b


# ---------------------------------------------------------------------------------------------------------------------
# from a distribution
def _merge_distribution_stats(raw: torch.Tensor, group):
    """raw [T, 7] of this shard -> merged (lse_s, se_s, C, lse_t, se_t, A, B) over the vocabulary group."""
    m_s, se_s, c = raw[:, 0], raw[:, 1], raw[:, 2]
    m_t, se_t, a, b = raw[:, 3], raw[:, 4], raw[:, 5], raw[:, 6]
    if group is not None:
        gm_s = _all_reduce(m_s.clone(), group, torch.distributed.ReduceOp.MAX)
        gm_t = _all_reduce(m_t.clone(), group, torch.distributed.ReduceOp.MAX)
        rs, rt = torch.exp(m_s - gm_s), torch.exp(m_t - gm_t)
        packed = _all_reduce(torch.stack([se_s * rs, c * rs, se_t * rt, a * rt, b * rt], 0), group)
        se_s, c, se_t, a, b = packed.unbind(0)
        m_s, m_t = gm_s, gm_t
    return m_s + se_s.log(), se_s, c, m_t + se_t.log(), se_t, a, b


def distribution_loss_forward_backward(logits: torch.Tensor, teacher: torch.Tensor, loss_mask: torch.Tensor | None, grad_output,
                                       kind: str, *, logits_scale: float = 1.0, teacher_scale: float = 1.0, group=None,
                                       accumulate_into: torch.Tensor | None = None, in_place: bool = False,
                                       normalize_teacher: bool = True):
    """Per-token loss (fp32 `[tokens]`, mask applied) and the gradient wrt `logits` of `sum_t grad_output_t * loss_t`.

    `kind`: "cross_entropy" (-sum q log p), "forward_kl" (KL(q || p)) or "reverse_kl" (KL(p || q)) with
    p = softmax(logits * logits_scale), q = softmax(teacher * teacher_scale).  `grad_output`: None (no backward), a float
    or a `[tokens]` / one-element tensor; the mask multiplies it.  `teacher` holds this rank's vocabulary shard.
    `normalize_teacher=False` takes `teacher * teacher_scale` as log-probabilities as they are (log q_j, not renormalised)."""
    rows, cols = logits.shape
    assert teacher.shape == logits.shape, (teacher.shape, logits.shape)
    mask = None if loss_mask is None else loss_mask.float()
    native = _native(logits) and teacher.is_cuda
    if native and (teacher.dtype != logits.dtype or not _native(teacher)):
        teacher = teacher.to(logits.dtype).contiguous()
        native = _native(teacher)
    if native:
        lib = _lib.get_lib()
        dtype_code = 1 if logits.dtype == torch.bfloat16 else 0
        raw = torch.empty(rows, 7, dtype=torch.float32, device=logits.device)
        _lib.check(lib.flb_dist_stats(logits.data_ptr(), teacher.data_ptr(), dtype_code, raw.data_ptr(), rows, cols, logits.stride(0),
                                      teacher.stride(0), logits_scale, teacher_scale, _lib.stream_ptr()), "flb_dist_stats")
        _lib.count_launch()
    else:
        s = logits.float() * logits_scale
        t = teacher.float() * teacher_scale
        m_s, m_t = s.max(-1).values, t.max(-1).values
        es, et = torch.exp(s - m_s[:, None]), torch.exp(t - m_t[:, None])
        raw = torch.stack([m_s, es.sum(-1), (es * (s - t)).sum(-1), m_t, et.sum(-1), (et * s).sum(-1), (et * t).sum(-1)], 1)
    lse_s, se_s, c_sum, lse_t, se_t, a_sum, b_sum = _merge_distribution_stats(raw, group)
    if not normalize_teacher:
        # q_j = exp(t_j): sums weighted by e^(t - max t) become sums weighted by q after multiplying by e^(max t)
        rescale = torch.exp(lse_t) / se_t
        a_sum, b_sum, se_t, lse_t = a_sum * rescale, b_sum * rescale, torch.ones_like(se_t), torch.zeros_like(lse_t)
    if kind == "cross_entropy":
        per_token = lse_s - a_sum / se_t
    elif kind == "forward_kl":
        per_token = lse_s - a_sum / se_t + b_sum / se_t - lse_t
    elif kind == "reverse_kl":
        per_token = c_sum / se_s - lse_s + lse_t
    else:
        raise NotImplementedError(kind)
    loss = per_token if mask is None else per_token * mask
    if grad_output is None:
        return loss, None
    g = torch.as_tensor(grad_output, dtype=torch.float32, device=logits.device)
    g = (g.expand(rows) if g.dim() == 0 or g.numel() == 1 else g).reshape(-1) * logits_scale
    if mask is not None:
        g = g * mask
    zeros = torch.zeros_like(g)
    if kind == "reverse_kl":
        ca, cb, cc = g * (lse_t - lse_s - per_token), zeros, g
    else:
        ca, cb, cc = g, -g, zeros
    if native and (accumulate_into is None or _native(accumulate_into)):
        if accumulate_into is not None:
            grad, accumulate = accumulate_into, 1
        elif in_place:
            grad, accumulate = logits, 0
        else:
            pad = 8 if logits.dtype == torch.bfloat16 else 4
            grad, accumulate = torch.empty(rows, (cols + pad - 1) // pad * pad, dtype=logits.dtype, device=logits.device)[:, :cols], 0
        _lib.check(_lib.get_lib().flb_dist_grad(
            logits.data_ptr(), teacher.data_ptr(), dtype_code, lse_s.contiguous().data_ptr(), lse_t.contiguous().data_ptr(),
            ca.contiguous().data_ptr(), cb.contiguous().data_ptr(), cc.contiguous().data_ptr(), grad.data_ptr(), rows, cols, logits.stride(0),
            teacher.stride(0), grad.stride(0), logits_scale, teacher_scale, accumulate, _lib.stream_ptr()), "flb_dist_grad")
        _lib.count_launch()
        return loss, grad
    s = logits.float() * logits_scale
    t = teacher.float() * teacher_scale
    p = torch.exp(s - lse_s[:, None])
    grad = p * (ca[:, None] + cc[:, None] * (s - t)) + cb[:, None] * torch.exp(t - lse_t[:, None])
    grad = grad.to(logits.dtype)
    if accumulate_into is not None:
        return loss, accumulate_into.add_(grad)
    if in_place:
        return loss, logits.copy_(grad)
    return loss, grad
