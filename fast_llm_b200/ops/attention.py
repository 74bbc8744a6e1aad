"""Variable-length (packed documents) causal attention with GQA and sliding window.

`packed_attention(qkv, ...)` takes the fused projection output `[tokens, (heads + 2*kv_heads) * head_dim]` and returns
`[tokens, heads * head_dim]`; its backward writes dq, dk, dv into one packed gradient so the fused QKV projection's
backward is a single GEMM.  `attention(q, k, v, ...)` is the general form (keys may include a prefix from earlier
micro-sequences or other sequence-data-parallel ranks; causal masks are bottom-right aligned).

On B200 both forms run this package's tcgen05 kernels (`csrc/attention_fwd.cu`, `csrc/attention_bwd.cu`: bf16, head size
128, key segments at least as long as the query segments); smaller head sizes are zero-padded to 128.  Dropout, heads
wider than 128, fp16 and a window without causality go through PyTorch's `scaled_dot_product_attention` per document.  On
CPU a per-document PyTorch restatement, which doubles as the test oracle (math of `fast_llm/layers/attention/
attention.py:209-256`).
"""

import torch

from fast_llm_b200.ops import _lib


def attention_reference(q, k, v, cu_seqlens_q, cu_seqlens_k, causal: bool, window_size: int | None, scale: float):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] -> [Tq, Hq, D]; fp32 math, differentiable."""
    hq, hkv = q.shape[1], k.shape[1]
    rep = hq // hkv
    outs = []
    cq = cu_seqlens_q.tolist()
    ck = cu_seqlens_k.tolist()
    for i in range(len(cq) - 1):
        qs = q[cq[i] : cq[i + 1]].float()
        ks = k[ck[i] : ck[i + 1]].float().repeat_interleave(rep, dim=1)
        vs = v[ck[i] : ck[i + 1]].float().repeat_interleave(rep, dim=1)
        lq, lk = qs.shape[0], ks.shape[0]
        if lq == 0:
            continue
        scores = torch.einsum("qhd,khd->hqk", qs, ks) * scale
        qi = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
        ki = torch.arange(lk, device=q.device)[None, :]
        mask = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
        if causal:
            mask &= ki <= qi
        if window_size is not None:
            mask &= ki > qi - window_size if causal else (ki - qi).abs() < window_size
        scores = scores.masked_fill(~mask[None], float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        probs = torch.nan_to_num(probs)
        outs.append(torch.einsum("hqk,khd->qhd", probs, vs))
    return torch.cat(outs, 0).to(q.dtype) if outs else q.new_zeros(q.shape)


def _native_dtype_ok(t: torch.Tensor, dropout_p: float) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and dropout_p == 0.0


def attention_forward_native(q2d, q_col0, kv2d, k_col0, v_col0, cu_q, cu_k, max_seqlen_q, heads, kv_heads, head_dim, causal, window_size, scale):
    """tcgen05 forward (`csrc/attention_fwd.cu`).  q2d / kv2d: 2-D row views ([tokens, row_stride]) holding the heads at the
    given column offsets.  Returns (out [tokens, heads, head_dim], lse [heads, tokens] fp32)."""
    total_q, total_k = q2d.shape[0], kv2d.shape[0]
    out = torch.empty(total_q, heads, head_dim, dtype=q2d.dtype, device=q2d.device)
    lse = torch.empty(heads, total_q, dtype=torch.float32, device=q2d.device)
    _lib.check(
        _lib.get_lib().flb_attention_fwd(
            q2d.data_ptr(), q2d.stride(0), q_col0, kv2d.data_ptr(), kv2d.stride(0), k_col0, v_col0, cu_q.data_ptr(), cu_k.data_ptr(),
            cu_q.numel() - 1, max_seqlen_q, total_q, total_k, heads, kv_heads, head_dim, out.data_ptr(), lse.data_ptr(), int(causal),
            int(window_size or 0), float(scale), _lib.stream_ptr()), "flb_attention_fwd")
    _lib.count_launch()
    return out, lse


def attention_backward_native(q2d, q_col0, kv2d, k_col0, v_col0, out, dout, lse, cu_q, cu_k, max_seqlen_k, heads, kv_heads, head_dim,
                              dq2d, dkv2d, causal, window_size, scale):
    """tcgen05 backward (`csrc/attention_bwd.cu`).  Writes dq into `dq2d` and dk / dv into `dkv2d` at the column offsets the
    forward inputs have in `q2d` / `kv2d` (the gradient buffers mirror the input layout)."""
    total_q, total_k = q2d.shape[0], kv2d.shape[0]
    delta = torch.empty(heads, total_q, dtype=torch.float32, device=q2d.device)
    dq_accum = torch.empty(heads * ((total_q + 31) // 32) * 32 * head_dim, dtype=torch.float32, device=q2d.device)
    dout = dout.contiguous()
    _lib.check(
        _lib.get_lib().flb_attention_bwd(
            q2d.data_ptr(), q2d.stride(0), q_col0, kv2d.data_ptr(), kv2d.stride(0), k_col0, v_col0, out.data_ptr(), dout.data_ptr(),
            lse.data_ptr(), cu_q.data_ptr(), cu_k.data_ptr(), cu_q.numel() - 1, max_seqlen_k, total_q, total_k, heads, kv_heads, head_dim,
            dq2d.data_ptr(), dq2d.stride(0), dkv2d.data_ptr(), dkv2d.stride(0), delta.data_ptr(), dq_accum.data_ptr(), int(causal),
            int(window_size or 0), float(scale), _lib.stream_ptr()), "flb_attention_bwd")
    _lib.count_launch(3)


_NATIVE_HEAD = 128  # head size of the tcgen05 kernels; smaller heads are zero-padded to it
_MIN_ROWS = 128  # fewer query or key rows than one tile are padded with rows of no document


def _joint_key_value_rows(k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """[Tk, 2 * kv_heads * 128] rows holding the keys of every head followed by the values: a view when k and v already sit
    side by side in one buffer (slices of a fused projection or of a gathered key/value tensor), else a copy."""
    tk, kv_heads, d = k.shape
    width = kv_heads * d
    side_by_side = (k.stride(2) == 1 and v.stride(2) == 1 and k.stride(1) == d and v.stride(1) == d and k.stride(0) == v.stride(0)
                    and k.stride(0) >= 2 * width and v.data_ptr() - k.data_ptr() == width * k.element_size()
                    and k.untyped_storage().data_ptr() == v.untyped_storage().data_ptr())
    if side_by_side and k.data_ptr() % 16 == 0 and k.stride(0) % 8 == 0:
        return torch.as_strided(k, (tk, 2 * width), (k.stride(0), 1))
    return torch.cat([k.reshape(tk, width), v.reshape(tk, width)], dim=1)


class _NativeAttention(torch.autograd.Function):
    """q [Tq, heads, 128], k / v [Tk, kv_heads, 128]; the key segments may be longer than the query segments (a prefix from
    earlier micro-sequences or other sequence-data ranks): masks are bottom-right aligned."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, window_size, scale):
        tq, heads, d = q.shape
        kv_heads = k.shape[1]
        q2d = q.reshape(tq, heads * d)
        if q2d.data_ptr() % 16 or q2d.stride(0) % 8 or q2d.stride(1) != 1:
            q2d = q2d.contiguous()
        kv2d = _joint_key_value_rows(k, v)
        out, lse = attention_forward_native(q2d, 0, kv2d, 0, kv_heads * d, cu_q, cu_k, max_q, heads, kv_heads, d, causal, window_size, scale)
        ctx.save_for_backward(q2d, kv2d, out, lse, cu_q, cu_k)
        ctx.args = (max_k, heads, kv_heads, causal, window_size, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q2d, kv2d, out, lse, cu_q, cu_k = ctx.saved_tensors
        max_k, heads, kv_heads, causal, window_size, scale = ctx.args
        d = _NATIVE_HEAD
        tq, tk, width = q2d.shape[0], kv2d.shape[0], kv_heads * d
        dq = torch.empty(tq, heads * d, dtype=q2d.dtype, device=q2d.device)
        # key rows outside every `cu_k` segment (another sequence-data rank's later tokens) are attended by no query here
        # and are written by no CTA: they must read as zero
        dkv = torch.zeros(tk, 2 * width, dtype=kv2d.dtype, device=kv2d.device)
        attention_backward_native(q2d, 0, kv2d, 0, width, out, dout.reshape(tq, heads * d), lse, cu_q, cu_k, max_k, heads, kv_heads, d, dq, dkv,
                                  causal, window_size, scale)
        return dq.view(tq, heads, d), dkv[:, :width].view(tk, kv_heads, d), dkv[:, width:].view(tk, kv_heads, d), None, None, None, None, None, None, None


class _PackedNativeAttention(torch.autograd.Function):
    """Self-attention over the fused projection output [tokens, (heads + 2 kv_heads) x 128]; the backward writes dq, dk and
    dv into one packed gradient, so the projection's backward is one GEMM."""

    @staticmethod
    def forward(ctx, qkv, cu, max_len, heads, kv_heads, causal, window_size, scale):
        d = _NATIVE_HEAD
        nq, nkv = heads * d, kv_heads * d
        out, lse = attention_forward_native(qkv, 0, qkv, nq, nq + nkv, cu, cu, max_len, heads, kv_heads, d, causal, window_size, scale)
        ctx.save_for_backward(qkv, out, lse, cu)
        ctx.args = (max_len, heads, kv_heads, causal, window_size, scale)
        return out.view(qkv.shape[0], nq)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, cu = ctx.saved_tensors
        max_len, heads, kv_heads, causal, window_size, scale = ctx.args
        d = _NATIVE_HEAD
        nq, nkv = heads * d, kv_heads * d
        dqkv = torch.empty_like(qkv)
        attention_backward_native(qkv, 0, qkv, nq, nq + nkv, out, dout.reshape(qkv.shape[0], nq), lse, cu, cu, max_len, heads, kv_heads, d,
                                  dqkv, dqkv, causal, window_size, scale)
        return dqkv, None, None, None, None, None, None, None


def _kernel_supports(causal: bool, window_size) -> bool:
    return causal or window_size is None


def _sdpa_fallback(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, window_size, scale, dropout_p):
    """Per-document `scaled_dot_product_attention` for what the tcgen05 kernels do not take (dropout, heads wider than 128,
    fp16, a window without causality): correct and differentiable, quadratic in memory per document."""
    rep = q.shape[1] // k.shape[1]
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    outs = []
    for i in range(len(cq) - 1):
        qs = q[cq[i] : cq[i + 1]].transpose(0, 1)
        ks = k[ck[i] : ck[i + 1]].transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[ck[i] : ck[i + 1]].transpose(0, 1).repeat_interleave(rep, dim=0)
        lq, lk = qs.shape[1], ks.shape[1]
        if lq == 0:
            continue
        qi = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
        ki = torch.arange(lk, device=q.device)[None, :]
        mask = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
        if causal:
            mask &= ki <= qi
        if window_size is not None:
            mask &= ki > qi - window_size if causal else (ki - qi).abs() < window_size
        out = torch.nn.functional.scaled_dot_product_attention(qs[None], ks[None], vs[None], attn_mask=mask, dropout_p=dropout_p, scale=scale)
        outs.append(out[0].transpose(0, 1))
    return torch.cat(outs, 0) if outs else q.new_zeros(q.shape)


def attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, *, causal: bool = True,
              window_size: int | None = None, scale: float | None = None, dropout_p: float = 0.0):
    """q [Tq, Hq, D], k / v [Tk, Hkv, D] -> [Tq, Hq, D]."""
    d = q.shape[-1]
    scale = d**-0.5 if scale is None else scale
    if not q.is_cuda:
        return attention_reference(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, window_size, scale)
    if not (_native_dtype_ok(q, dropout_p) and d <= _NATIVE_HEAD and d % 8 == 0 and _kernel_supports(causal, window_size)):
        return _sdpa_fallback(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, window_size, scale, dropout_p)
    tq = q.shape[0]
    # generation steps hold a few rows only: the tensor maps always cover at least one full 128-row tile (rows past the last
    # `cu_seqlens` entry belong to no document: nothing reads or writes them)
    rows_q, rows_k = max(_MIN_ROWS - tq, 0), max(_MIN_ROWS - k.shape[0], 0)
    if d < _NATIVE_HEAD or rows_q or rows_k:
        # zero columns change neither the scores nor the first d output columns
        q = torch.nn.functional.pad(q, (0, _NATIVE_HEAD - d, 0, 0, 0, rows_q))
        k, v = (torch.nn.functional.pad(t, (0, _NATIVE_HEAD - d, 0, 0, 0, rows_k)) for t in (k, v))
    out = _NativeAttention.apply(q, k, v, cu_seqlens_q.int(), cu_seqlens_k.int(), max_seqlen_q, max_seqlen_k, causal, window_size, scale)
    return out[:tq, :, :d] if (d < _NATIVE_HEAD or rows_q) else out


def packed_attention(qkv, cu_seqlens, max_seqlen: int, heads: int, kv_heads: int, head_dim: int, *, causal: bool = True,
                     window_size: int | None = None, scale: float | None = None, dropout_p: float = 0.0):
    scale = head_dim**-0.5 if scale is None else scale
    t = qkv.shape[0]
    nq, nkv = heads * head_dim, kv_heads * head_dim
    if qkv.is_cuda and _native_dtype_ok(qkv, dropout_p) and head_dim == _NATIVE_HEAD and _kernel_supports(causal, window_size) \
            and qkv.stride(-1) == 1 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
        return _PackedNativeAttention.apply(qkv, cu_seqlens.int(), max_seqlen, heads, kv_heads, causal, window_size, scale)
    q = qkv[:, :nq].reshape(t, heads, head_dim)
    k = qkv[:, nq : nq + nkv].reshape(t, kv_heads, head_dim)
    v = qkv[:, nq + nkv :].reshape(t, kv_heads, head_dim)
    if qkv.is_cuda:
        return attention(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=causal, window_size=window_size, scale=scale,
                         dropout_p=dropout_p).reshape(t, nq)
    return attention_reference(q, k, v, cu_seqlens, cu_seqlens, causal, window_size, scale).reshape(t, nq)
