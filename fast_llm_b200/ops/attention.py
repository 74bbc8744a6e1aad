"""Variable-length (packed documents) causal attention with GQA and sliding window.

`packed_attention(qkv, ...)` takes the fused projection output `[tokens, (heads + 2*kv_heads) * head_dim]` and returns
`[tokens, heads * head_dim]`; its backward writes dq, dk, dv into one packed gradient so the fused QKV projection's
backward is a single GEMM.  `attention(q, k, v, ...)` is the general form (keys may include a prefix from earlier
micro-sequences or other sequence-data-parallel ranks; causal masks are bottom-right aligned).

On B200 the packed path runs this package's tcgen05 kernels (`csrc/attention_fwd.cu`, `csrc/attention_bwd.cu`; bf16, head
size 128); other shapes, dropout and the prefix form use the flash-attention 2 library kernel (a library call, like
cuBLAS for a plain GEMM); on CPU a per-document PyTorch restatement, which doubles as the test oracle (math of `fast_llm/layers/attention/
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


def _window(window_size, causal):
    if window_size is None:
        return (-1, 0 if causal else -1)
    # a window of w tokens = the current token plus w - 1 earlier ones
    return (window_size - 1, 0 if causal else window_size - 1)


def _use_flash(q):
    return q.is_cuda and q.dtype in (torch.bfloat16, torch.float16)


def _use_native_forward(t: torch.Tensor, head_dim: int, dropout_p: float) -> bool:
    import os

    return (t.is_cuda and t.dtype == torch.bfloat16 and head_dim == 128 and dropout_p == 0.0 and t.stride(-1) == 1
            and os.environ.get("FLB_ATTENTION", "tcgen05") == "tcgen05")


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


def _use_native_backward() -> bool:
    import os

    return os.environ.get("FLB_ATTENTION_BWD", "tcgen05") == "tcgen05"


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


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, window_size, scale, dropout_p):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward

        wl, wr = _window(window_size, causal)
        out, lse, _, rng_state = _flash_attn_varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, dropout_p, scale, causal,
                                                            window_size_left=wl, window_size_right=wr)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k, rng_state)
        ctx.args = (max_q, max_k, causal, wl, wr, scale, dropout_p)
        return out

    @staticmethod
    def backward(ctx, dout):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        q, k, v, out, lse, cu_q, cu_k, rng_state = ctx.saved_tensors
        max_q, max_k, causal, wl, wr, scale, dropout_p = ctx.args
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_varlen_backward(dout.contiguous(), q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max_q, max_k, dropout_p,
                                    scale, causal, wl, wr, 0.0, None, False, rng_state)
        # Key rows past the last `cu_k` segment (another sequence-data rank's later tokens) are attended by no query here;
        # the library leaves them unwritten (with grouped heads it sums an uninitialised staging buffer into them).
        uncovered = torch.arange(k.shape[0], device=k.device) >= cu_k[-1]
        dk.masked_fill_(uncovered[:, None, None], 0)
        dv.masked_fill_(uncovered[:, None, None], 0)
        return dq, dk, dv, None, None, None, None, None, None, None, None


def attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, *, causal: bool = True,
              window_size: int | None = None, scale: float | None = None, dropout_p: float = 0.0):
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if _use_flash(q):
        return _FlashAttention.apply(q, k, v, cu_seqlens_q.int(), cu_seqlens_k.int(), max_seqlen_q, max_seqlen_k, causal,
                                     window_size, scale, dropout_p)
    return attention_reference(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, window_size, scale)


class _PackedFlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cu, max_len, heads, kv_heads, head_dim, causal, window_size, scale, dropout_p):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward

        t = qkv.shape[0]
        nq, nkv = heads * head_dim, kv_heads * head_dim
        q = qkv[:, :nq].view(t, heads, head_dim)
        k = qkv[:, nq : nq + nkv].view(t, kv_heads, head_dim)
        v = qkv[:, nq + nkv :].view(t, kv_heads, head_dim)
        wl, wr = _window(window_size, causal)
        if _use_native_forward(qkv, head_dim, dropout_p) and (causal or window_size is None):
            out, lse = attention_forward_native(qkv, 0, qkv, nq, nq + nkv, cu, cu, max_len, heads, kv_heads, head_dim, causal, window_size, scale)
            rng_state = None
        else:
            out, lse, _, rng_state = _flash_attn_varlen_forward(q, k, v, cu, cu, max_len, max_len, dropout_p, scale, causal,
                                                                window_size_left=wl, window_size_right=wr)
        ctx.save_for_backward(qkv, out, lse, cu, rng_state)
        ctx.args = (max_len, heads, kv_heads, head_dim, causal, wl, wr, scale, dropout_p)
        ctx.native = rng_state is None and _use_native_backward()
        ctx.window_size = window_size
        return out.view(t, nq)

    @staticmethod
    def backward(ctx, dout):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        qkv, out, lse, cu, rng_state = ctx.saved_tensors
        max_len, heads, kv_heads, head_dim, causal, wl, wr, scale, dropout_p = ctx.args
        t = qkv.shape[0]
        nq, nkv = heads * head_dim, kv_heads * head_dim
        dqkv = torch.empty_like(qkv)
        if ctx.native:
            attention_backward_native(qkv, 0, qkv, nq, nq + nkv, out, dout.view(t, nq), lse, cu, cu, max_len, heads, kv_heads, head_dim,
                                      dqkv, dqkv, causal, ctx.window_size, scale)
            return dqkv, None, None, None, None, None, None, None, None, None
        views = lambda x: (x[:, :nq].view(t, heads, head_dim), x[:, nq : nq + nkv].view(t, kv_heads, head_dim),
                           x[:, nq + nkv :].view(t, kv_heads, head_dim))
        q, k, v = views(qkv)
        dq, dk, dv = views(dqkv)
        _flash_attn_varlen_backward(dout.contiguous().view(t, heads, head_dim), q, k, v, out, lse, dq, dk, dv, cu, cu,
                                    max_len, max_len, dropout_p, scale, causal, wl, wr, 0.0, None, False, rng_state)
        return dqkv, None, None, None, None, None, None, None, None, None


def packed_attention(qkv, cu_seqlens, max_seqlen: int, heads: int, kv_heads: int, head_dim: int, *, causal: bool = True,
                     window_size: int | None = None, scale: float | None = None, dropout_p: float = 0.0):
    scale = head_dim**-0.5 if scale is None else scale
    if _use_flash(qkv):
        return _PackedFlashAttention.apply(qkv, cu_seqlens.int(), max_seqlen, heads, kv_heads, head_dim, causal,
                                           window_size, scale, dropout_p)
    t = qkv.shape[0]
    nq, nkv = heads * head_dim, kv_heads * head_dim
    q = qkv[:, :nq].reshape(t, heads, head_dim)
    k = qkv[:, nq : nq + nkv].reshape(t, kv_heads, head_dim)
    v = qkv[:, nq + nkv :].reshape(t, kv_heads, head_dim)
    return attention_reference(q, k, v, cu_seqlens, cu_seqlens, causal, window_size, scale).reshape(t, nq)
