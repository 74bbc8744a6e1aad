"""State-space / linear-attention recurrences over packed documents: Mamba selective scan, gated delta rule (scalar decay)
and Kimi delta attention (per-channel decay).

All three are linear recurrences `state_t = decay_t * state_{t-1} + write_t` evaluated chunk by chunk: inside a chunk the
contributions are combined with pairwise decays `exp(c_t - c_s)`, `s <= t` (always <= 1, so no overflow however strong the
decay), and the state is carried from chunk to chunk.  `chunked_scan` runs the chunk loop without building an autograd
graph, keeps only the state at each chunk boundary and re-evaluates one chunk at a time in the backward pass, so memory
stays at one chunk of intermediates plus `chunks x state`.  Documents never share state: the loop restarts at every
document boundary given by `cu_seqlens`.

Each op has a token-by-token restatement (`*_reference`) used as the test oracle.
Parity (semantics): `fast_llm/layers/ssm/mamba.py:183-236` (selective scan call), `fast_llm/layers/ssm/gdn.py:41-210`
(gated delta rule), `fast_llm/layers/ssm/kda.py:33-203` (KDA and its gate).
"""

import typing

import torch


# ----------------------------------------------------------------------------------------------------------------------
# chunk loop with boundary-state checkpointing
# ----------------------------------------------------------------------------------------------------------------------
class _ChunkedScan(torch.autograd.Function):
    """forward(step, n_seq, n_shared, chunk, boundaries, state0, *seq_inputs, *shared_inputs) -> (outputs, final_state)

    `step(state, seq_chunk_tuple, shared_tuple) -> (out_chunk, new_state)` must be differentiable torch code.
    `boundaries` is the sorted list of document starts + total length; chunks never straddle a boundary and the state is
    reset to zero at each document start.
    """

    @staticmethod
    def forward(ctx, step, n_seq, chunk, boundaries, state_shape, *tensors):
        seq, shared = tensors[:n_seq], tensors[n_seq:]
        ctx.step, ctx.n_seq, ctx.spans = step, n_seq, []
        outs, states = [], []
        ref = seq[0]
        with torch.no_grad():
            for begin, end in zip(boundaries[:-1], boundaries[1:]):
                state = torch.zeros(state_shape, dtype=torch.float32, device=ref.device)
                for lo in range(begin, end, chunk):
                    hi = min(lo + chunk, end)
                    states.append(state)
                    ctx.spans.append((lo, hi, lo == begin))
                    out, state = step(state, tuple(t[lo:hi] for t in seq), shared)
                    outs.append(out)
        ctx.save_for_backward(*tensors, *states)
        ctx.n_tensors = len(tensors)
        if not outs:
            return ref.new_zeros((0,) + tuple(state_shape[:0]))
        return torch.cat(outs, 0)

    @staticmethod
    def backward(ctx, grad_out):
        saved = ctx.saved_tensors
        tensors, states = saved[: ctx.n_tensors], saved[ctx.n_tensors :]
        seq, shared = tensors[: ctx.n_seq], tensors[ctx.n_seq :]
        seq_grads = [torch.zeros_like(t) if t.is_floating_point() else None for t in seq]
        shared_grads = [torch.zeros_like(t, dtype=torch.float32) if t.is_floating_point() else None for t in shared]
        grad_state = None
        for index in range(len(ctx.spans) - 1, -1, -1):
            lo, hi, first = ctx.spans[index]
            with torch.enable_grad():
                state_in = states[index].detach().requires_grad_(not first)
                chunk_in = tuple(t[lo:hi].detach().requires_grad_(t.is_floating_point()) for t in seq)
                shared_in = tuple(t.detach().requires_grad_(t.is_floating_point()) for t in shared)
                out, state_out = ctx.step(state_in, chunk_in, shared_in)
                targets = [out] if grad_state is None else [out, state_out]
                grads_in = [grad_out[lo:hi]] if grad_state is None else [grad_out[lo:hi], grad_state]
                wanted = [t for t in (*chunk_in, *shared_in, state_in) if t.requires_grad]
                grads = torch.autograd.grad(targets, wanted, grads_in, allow_unused=True)
            it = iter(grads)
            for i, t in enumerate(chunk_in):
                if t.requires_grad:
                    g = next(it)
                    if g is not None:
                        seq_grads[i][lo:hi] = g
            for i, t in enumerate(shared_in):
                if t.requires_grad:
                    g = next(it)
                    if g is not None:
                        shared_grads[i] += g
            grad_state = None if first else next(it)
        shared_grads = [None if g is None else g.to(t.dtype) for g, t in zip(shared_grads, shared)]
        return (None, None, None, None, None, *seq_grads, *shared_grads)


def chunked_scan(step: typing.Callable, state_shape, seq_inputs, shared_inputs, cu_seqlens, chunk: int) -> torch.Tensor:
    total = seq_inputs[0].shape[0]
    boundaries = [0, total] if cu_seqlens is None else [int(b) for b in cu_seqlens.tolist()]
    if boundaries[-1] < total:  # trailing padding forms its own document
        boundaries.append(total)
    return _ChunkedScan.apply(step, len(seq_inputs), chunk, boundaries, tuple(state_shape), *seq_inputs, *shared_inputs)


# ----------------------------------------------------------------------------------------------------------------------
# depthwise causal convolution
# ----------------------------------------------------------------------------------------------------------------------
def causal_conv1d_reference(x, weight, bias, document_index, activation) -> torch.Tensor:
    """x [tokens, channels]; weight [channels, k]; out[t] = act(bias + sum_j weight[:, j] * x[t - (k - 1 - j)]) within a document."""
    from fast_llm_b200.ops.activation import activation_reference

    tokens = x.shape[0]
    k = weight.shape[-1]
    xf = x.float()
    out = torch.zeros_like(xf)
    for j in range(k):
        shift = k - 1 - j
        if shift >= tokens:
            continue
        shifted = torch.zeros_like(xf)
        shifted[shift:] = xf[: tokens - shift]
        if document_index is not None and shift > 0:
            same = torch.zeros(tokens, dtype=torch.bool, device=x.device)
            same[shift:] = document_index[shift:] == document_index[: tokens - shift]
            shifted = shifted * same[:, None]
        out = out + shifted * weight[:, j].float()[None, :]
    if bias is not None:
        out = out + bias.float()[None, :]
    return activation_reference(out, activation).to(x.dtype)


class _CausalConv1d(torch.autograd.Function):
    TOKENS_PER_BLOCK = 64

    @staticmethod
    def forward(ctx, x, weight, bias, document_index, activation):
        from fast_llm_b200.ops import _lib

        x = x.contiguous()
        w32 = weight.float().contiguous()
        b32 = None if bias is None else bias.float().contiguous()
        doc = None if document_index is None else document_index.to(torch.int32).contiguous()
        out = torch.empty_like(x)
        tokens, channels = x.shape
        _lib.check(_lib.get_lib().flb_causal_conv1d_fwd(x.data_ptr(), w32.data_ptr(), _lib.ptr(b32), _lib.ptr(doc), out.data_ptr(), tokens, channels,
                                                       w32.shape[1], activation.code, _lib.stream_ptr()), "flb_causal_conv1d_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x, w32, b32, doc)
        ctx.activation, ctx.has_bias, ctx.dtypes = activation, bias is not None, (weight.dtype, None if bias is None else bias.dtype)
        return out

    @staticmethod
    def backward(ctx, grad):
        from fast_llm_b200.ops import _lib

        x, w32, b32, doc = ctx.saved_tensors
        tokens, channels = x.shape
        width = w32.shape[1]
        grad = grad.contiguous()
        dpre, dx = torch.empty_like(x), torch.empty_like(x)
        blocks = (tokens + _CausalConv1d.TOKENS_PER_BLOCK - 1) // _CausalConv1d.TOKENS_PER_BLOCK
        partial = torch.empty(blocks, channels, width + 1, dtype=torch.float32, device=x.device)
        _lib.check(_lib.get_lib().flb_causal_conv1d_bwd(x.data_ptr(), w32.data_ptr(), _lib.ptr(b32), _lib.ptr(doc), grad.data_ptr(), dpre.data_ptr(),
                                                       dx.data_ptr(), partial.data_ptr(), tokens, channels, width, ctx.activation.code,
                                                       _CausalConv1d.TOKENS_PER_BLOCK, _lib.stream_ptr()), "flb_causal_conv1d_bwd")
        _lib.count_launch(2)
        sums = partial.sum(0)  # fixed order: deterministic
        dw = sums[:, :width].to(ctx.dtypes[0])
        db = sums[:, width].to(ctx.dtypes[1]) if ctx.has_bias else None
        return dx, dw, db, None, None


def causal_conv1d(x, weight, bias, document_index, activation) -> torch.Tensor:
    """Depthwise causal convolution with fused bias and activation; weight [channels, k] (k <= 8)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and weight.shape[-1] <= 8:
        return _CausalConv1d.apply(x, weight, bias, document_index, activation)
    return causal_conv1d_reference(x, weight, bias, document_index, activation)


def _lower_mask(n: int, device, strict: bool) -> torch.Tensor:
    return torch.ones(n, n, dtype=torch.bool, device=device).tril(-1 if strict else 0)


# ----------------------------------------------------------------------------------------------------------------------
# Mamba selective scan
# ----------------------------------------------------------------------------------------------------------------------
def _selective_scan_step(state, chunk_in, shared):
    """state [d, n]; x, dt, z [L, d]; b, c [L, groups, n] (each group serves d / groups adjacent channels); a [d, n]; skip [d]."""
    x, dt, b, c, z = chunk_in
    a, skip, dt_bias = shared
    if b.shape[1] != x.shape[1]:
        b = b.repeat_interleave(x.shape[1] // b.shape[1], dim=1)
    if c.shape[1] != x.shape[1]:
        c = c.repeat_interleave(x.shape[1] // c.shape[1], dim=1)
    xf, dtf = x.float(), dt.float()
    if dt_bias is not None:
        dtf = dtf + dt_bias.float()
    dtf = torch.nn.functional.softplus(dtf)
    log_decay = dtf[:, :, None] * a.float()[None]  # [L, d, n], <= 0
    cum = log_decay.cumsum(0)
    write = (dtf * xf)[:, :, None] * b.float()  # [L, d, n]
    length = x.shape[0]
    mask = _lower_mask(length, x.device, strict=False)[:, :, None, None]
    pair = torch.where(mask, (cum[:, None] - cum[None, :]).clamp(max=0.0).exp(), torch.zeros((), device=x.device))
    states = cum.exp() * state[None] + torch.einsum("tsdn,sdn->tdn", pair, write)
    y = (states * c.float()).sum(-1) + skip.float()[None] * xf
    if z is not None:
        y = y * torch.nn.functional.silu(z.float())
    return y.to(x.dtype), states[-1]


class _SelectiveScan(torch.autograd.Function):
    """Chunk-parallel CUDA scan (`csrc/ssm.cu`): three launches forward, four backward; the only saved state beyond the
    inputs is the [chunks, state, channels] start state and decay product of every 64-token chunk."""

    @staticmethod
    def forward(ctx, x, dt, a, b, c, skip, z, dt_bias, starts):
        from fast_llm_b200.ops import _lib

        lib = _lib.get_lib()
        x, dt, b, c = x.contiguous(), dt.contiguous(), b.contiguous(), c.contiguous()
        z = None if z is None else z.contiguous()
        a32, skip32 = a.float().contiguous(), skip.float().contiguous()
        bias32 = None if dt_bias is None else dt_bias.float().contiguous()
        tokens, channels = x.shape
        state = a32.shape[1]
        chunks = lib.flb_selective_scan_chunks(tokens)
        chunk_state = torch.empty(chunks, state, channels, dtype=torch.float32, device=x.device)
        chunk_decay = torch.empty_like(chunk_state)
        y = torch.empty_like(x)
        _lib.check(lib.flb_selective_scan_fwd(x.data_ptr(), dt.data_ptr(), a32.data_ptr(), b.data_ptr(), c.data_ptr(), skip32.data_ptr(), _lib.ptr(z),
                                              _lib.ptr(bias32), _lib.ptr(starts), tokens, channels, state, b.shape[1], c.shape[1],
                                              chunk_state.data_ptr(), chunk_decay.data_ptr(), y.data_ptr(), _lib.stream_ptr()), "flb_selective_scan_fwd")
        _lib.count_launch(3)
        ctx.save_for_backward(x, dt, a32, b, c, skip32, z, bias32, starts, chunk_state, chunk_decay)
        ctx.dtypes = (a.dtype, skip.dtype, None if dt_bias is None else dt_bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        from fast_llm_b200.ops import _lib

        lib = _lib.get_lib()
        x, dt, a32, b, c, skip32, z, bias32, starts, chunk_state, chunk_decay = ctx.saved_tensors
        tokens, channels = x.shape
        state, chunks = a32.shape[1], chunk_state.shape[0]
        checkpoints = torch.empty(lib.flb_selective_scan_checkpoints(tokens, state), state, channels, dtype=torch.float32, device=x.device)
        dy = dy.contiguous()
        dx, ddt = torch.empty_like(x), torch.empty_like(dt)
        dz = None if z is None else torch.empty_like(z)
        db = torch.zeros(b.shape, dtype=torch.float32, device=x.device)
        dc = torch.zeros(c.shape, dtype=torch.float32, device=x.device)
        adjoint = torch.empty_like(chunk_state)
        da_partial = torch.empty_like(chunk_state)
        dskip_partial = torch.empty(chunks, channels, dtype=torch.float32, device=x.device)
        dbias_partial = torch.empty_like(dskip_partial)
        _lib.check(lib.flb_selective_scan_bwd(x.data_ptr(), dt.data_ptr(), a32.data_ptr(), b.data_ptr(), c.data_ptr(), skip32.data_ptr(), _lib.ptr(z),
                                              _lib.ptr(bias32), _lib.ptr(starts), tokens, channels, state, b.shape[1], c.shape[1],
                                              chunk_state.data_ptr(), chunk_decay.data_ptr(), adjoint.data_ptr(), checkpoints.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                              ddt.data_ptr(), _lib.ptr(dz), db.data_ptr(), dc.data_ptr(), da_partial.data_ptr(),
                                              dskip_partial.data_ptr(), dbias_partial.data_ptr(), _lib.stream_ptr()), "flb_selective_scan_bwd")
        _lib.count_launch(4)
        da = da_partial.sum(0).t().to(ctx.dtypes[0])
        dskip = dskip_partial.sum(0).to(ctx.dtypes[1])
        dbias = None if bias32 is None else dbias_partial.sum(0).to(ctx.dtypes[2])
        return dx, ddt, da, db.to(b.dtype), dc.to(c.dtype), dskip, dz, dbias, None


def _scan_kernel_applies(x, dt, a, b, c, z) -> bool:
    if not (x.is_cuda and all(t is None or t.dtype == torch.bfloat16 for t in (x, dt, b, c, z))):
        return False
    channels, state = a.shape
    return state in (4, 8, 16, 32) and channels % b.shape[1] == 0 and channels % c.shape[1] == 0


def document_starts(cu_seqlens, tokens: int, device) -> torch.Tensor | None:
    """uint8 [tokens], 1 at the first token of every document (None for one document)."""
    if cu_seqlens is None or cu_seqlens.numel() <= 2:
        return None
    starts = torch.zeros(tokens, dtype=torch.uint8, device=device)
    starts[cu_seqlens[:-1].to(device=device, dtype=torch.long)] = 1
    return starts


def selective_scan(x, dt, a, b, c, skip, z=None, dt_bias=None, cu_seqlens=None, chunk: int = 16) -> torch.Tensor:
    """y_t = C_t . h_t + D x_t (times silu(z_t)), h_t = exp(softplus(dt_t + bias) A) h_{t-1} + softplus(.) B_t x_t.

    x, dt, z: [tokens, channels]; a: [channels, state] (negative); b, c: [tokens, groups, state] with `groups` dividing
    `channels` (group i serves channels [i * channels / groups, (i + 1) * channels / groups)); skip: [channels].
    bf16 CUDA inputs run the chunk-parallel kernels; everything else the chunked PyTorch restatement below.
    """
    if _scan_kernel_applies(x, dt, a, b, c, z):
        return _SelectiveScan.apply(x, dt, a, b, c, skip, z, dt_bias, document_starts(cu_seqlens, x.shape[0], x.device))

    def step(state, chunk_in, shared):
        xs, dts, bs, cs, *rest = chunk_in
        zs = rest[0] if z is not None else None
        a_, skip_, *bias_ = shared
        return _selective_scan_step(state, (xs, dts, bs, cs, zs), (a_, skip_, bias_[0] if bias_ else None))

    seq = [x, dt, b, c] + ([z] if z is not None else [])
    shared = [a, skip] + ([dt_bias] if dt_bias is not None else [])
    return chunked_scan(step, a.shape, seq, shared, cu_seqlens, chunk)


def selective_scan_reference(x, dt, a, b, c, skip, z=None, dt_bias=None, cu_seqlens=None) -> torch.Tensor:
    total = x.shape[0]
    starts = {0} if cu_seqlens is None else set(int(s) for s in cu_seqlens.tolist())
    dtf = dt.float() + (0 if dt_bias is None else dt_bias.float())
    dtf = torch.nn.functional.softplus(dtf)
    h = torch.zeros_like(a, dtype=torch.float32)
    ys = []
    for t in range(total):
        if t in starts:
            h = torch.zeros_like(h)
        bt = b[t].float().repeat_interleave(x.shape[1] // b.shape[1], dim=0)
        ct = c[t].float().repeat_interleave(x.shape[1] // c.shape[1], dim=0)
        h = (dtf[t][:, None] * a.float()).exp() * h + (dtf[t] * x[t].float())[:, None] * bt
        y = (h * ct).sum(-1) + skip.float() * x[t].float()
        if z is not None:
            y = y * torch.nn.functional.silu(z[t].float())
        ys.append(y)
    return torch.stack(ys).to(x.dtype)


# ----------------------------------------------------------------------------------------------------------------------
# Delta rule with scalar (gated DeltaNet) or per-channel (KDA) decay
# ----------------------------------------------------------------------------------------------------------------------
def l2_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def _chunk_layout(boundaries: list[int], chunk: int, device):
    """Cut every document into chunks of `chunk` tokens (the last one padded).  Returns the [chunks, chunk] token index of
    every slot (-1: padding) and, per chunk, whether it starts a document."""
    import numpy as np

    rows, first = [], []
    for begin, end in zip(boundaries[:-1], boundaries[1:]):
        for lo in range(begin, end, chunk):
            row = np.full(chunk, -1, dtype=np.int64)
            row[: min(chunk, end - lo)] = np.arange(lo, min(lo + chunk, end))
            rows.append(row)
            first.append(lo == begin)
    index = torch.from_numpy(np.stack(rows)) if rows else torch.zeros(0, chunk, dtype=torch.int64)
    return index.to(device), first


class _DeltaStateScan(torch.autograd.Function):
    """State entering every chunk of S_{c+1} = decay_c o S_c - mix_c S_c + write_c (zero at document starts): one CUDA kernel
    walks the chunks (`flb_delta_state_scan`), a second one the adjoint recurrence; the gradients of mix, write and decay are
    batched products of the two results."""

    @staticmethod
    def applies(mix: torch.Tensor, write: torch.Tensor) -> bool:
        dk, dv = write.shape[-2:]
        return mix.is_cuda and mix.dtype == torch.float32 and dv % 32 == 0 and dk in (32, 64, 128)

    @staticmethod
    def _scan(decay, mix, add, first, reverse: bool) -> torch.Tensor:
        from fast_llm_b200.ops import _lib

        chunks, heads, dk, dv = add.shape
        per_row = decay.shape[-2] == dk
        out = torch.empty_like(add)
        _lib.check(_lib.get_lib().flb_delta_state_scan(decay.data_ptr(), mix.data_ptr(), add.data_ptr(), first.data_ptr(), out.data_ptr(), chunks, heads,
                                                       dk, dv, int(per_row), int(reverse), _lib.stream_ptr()), "flb_delta_state_scan")
        _lib.count_launch()
        return out

    @staticmethod
    def forward(ctx, decay, mix, write, first):
        decay, mix, write = decay.contiguous(), mix.contiguous(), write.contiguous()
        states = _DeltaStateScan._scan(decay, mix, write, first, False)
        ctx.save_for_backward(decay, mix, first, states)
        return states

    @staticmethod
    def backward(ctx, grad_states):
        decay, mix, first, states = ctx.saved_tensors
        leaving = _DeltaStateScan._scan(decay, mix, grad_states.contiguous(), first, True)  # adjoint of the state leaving every chunk
        grad_mix = -(leaving @ states.transpose(-1, -2))
        weighted = leaving * states
        grad_decay = weighted.sum(-1, keepdim=True) if decay.shape[-2] == states.shape[-2] else weighted.sum((-1, -2), keepdim=True)
        return grad_decay, grad_mix, leaving, None


def _delta_rule_all_chunks(q, k, v, g, beta, boundaries: list[int], chunk: int) -> torch.Tensor:
    """Delta rule with everything that does not depend on the carried state computed for ALL chunks at once.

    With S the state entering a chunk, the corrected values are U = U0 - W S where (I + Lmat) [U0 | W] = [V | K o Gamma]
    (one batched unit-triangular solve), so
        out   = QK (beta U0) + (Q o Gamma - QK (beta W)) S
        S_out = decay S - (Kout^T beta W) S + Kout^T beta U0
    and only the last line is sequential: one [dk, dk] x [dk, dv] product per head and chunk."""
    device, out_dtype = q.device, v.dtype
    index, first = _chunk_layout(boundaries, chunk, device)
    chunks = index.shape[0]
    valid = index >= 0
    gather = index.clamp(min=0)

    def cut(t):  # [tokens, heads, ...] -> [chunks, heads, chunk, ...], zero in the padding
        picked = t.float()[gather]
        picked = picked * valid.view(chunks, chunk, *([1] * (picked.dim() - 2)))
        return picked.transpose(1, 2)

    qc, kc, vc = cut(q), cut(k), cut(v)  # [C, h, L, d]
    gc, bc = cut(g), cut(beta)  # [C, h, L] (or [C, h, L, dk] for a per-channel decay), [C, h, L]
    per_channel = gc.dim() == 4
    cum = gc.cumsum(2)
    low = _lower_mask(chunk, device, strict=False)
    strict = _lower_mask(chunk, device, strict=True)
    zero = torch.zeros((), device=device)
    if per_channel:
        # decay between two tokens differs per key channel: weight every product k_t[d] k_s[d] separately
        pair = torch.where(low[:, :, None], (cum[:, :, :, None] - cum[:, :, None, :]).clamp(max=0.0).exp(), zero)  # [C, h, t, s, d]
        keys = kc[:, :, None, :, :] * pair  # k_s[d] * decay(t, s)[d]; plain products and sums: einsum maps this to tiny GEMMs
        kk = (keys * kc[:, :, :, None, :]).sum(-1)
        qk = (keys * qc[:, :, :, None, :]).sum(-1)
        grow = cum.exp()
        carry = (cum[:, :, -1:] - cum).exp()
        decay = cum[:, :, -1].exp()[..., None]  # [C, h, dk, 1]
    else:
        pair = torch.where(low, (cum[..., :, None] - cum[..., None, :]).clamp(max=0.0).exp(), zero)  # [C, h, t, s]
        kk = (kc @ kc.transpose(-1, -2)) * pair
        qk = (qc @ kc.transpose(-1, -2)) * pair
        grow = cum.exp()[..., None]
        carry = (cum[..., -1:] - cum).exp()[..., None]
        decay = cum[..., -1].exp()[..., None, None]  # [C, h, 1, 1]
    system = torch.eye(chunk, device=device) + torch.where(strict, kk * bc[..., None, :], zero)
    solved = torch.linalg.solve_triangular(system, torch.cat([vc, kc * grow], dim=-1), upper=False, unitriangular=True)
    dv = vc.shape[-1]
    values = solved[..., :dv] * bc[..., None]  # beta U0
    reads = solved[..., dv:] * bc[..., None]  # beta W
    out_local = qk @ values
    q_state = qc * grow - qk @ reads
    k_out = (kc * carry).transpose(-1, -2)  # [C, h, dk, L]
    write = k_out @ values  # [C, h, dk, dv]
    mix = k_out @ reads  # [C, h, dk, dk]
    heads, dk = qc.shape[1], qc.shape[-1]
    state = torch.zeros(heads, dk, dv, dtype=torch.float32, device=device)
    if chunks and _DeltaStateScan.applies(mix, write):
        entering = _DeltaStateScan.apply(decay, mix, write, torch.tensor(first, dtype=torch.uint8).to(device, non_blocking=True))
    else:
        states = []
        # unbind once: indexing inside the loop would make autograd build a full-size zero tensor per chunk and operand
        for c, (decay_c, mix_c, write_c) in enumerate(zip(decay.unbind(0), mix.unbind(0), write.unbind(0))):
            if first[c]:
                state = torch.zeros_like(state)
            states.append(state)
            state = torch.baddbmm(state * decay_c, mix_c, state, alpha=-1.0) + write_c
        entering = torch.stack(states) if chunks else None
    out = out_local + q_state @ entering if chunks else out_local
    return out.transpose(1, 2)[valid].to(out_dtype)


def chunk_delta_rule(q, k, v, g, beta, cu_seqlens=None, chunk: int = 64, normalize_qk: bool = True, scale: float | None = None) -> torch.Tensor:
    """q, k [tokens, heads, dk]; v [tokens, heads, dv]; g [tokens, heads(, dk)] log decay; beta [tokens, heads] -> [tokens, heads, dv]."""
    if normalize_qk:
        q, k = l2_normalize(q.float()), l2_normalize(k.float())
    q = q * (q.shape[-1] ** -0.5 if scale is None else scale)
    heads, dk, dv = q.shape[1], q.shape[2], v.shape[2]
    if g.dim() == 3:
        chunk = min(chunk, 32)  # the pairwise per-channel decay tensor is [chunks, heads, L, L, dk]
    total = q.shape[0]
    boundaries = [0, total] if cu_seqlens is None else [int(b) for b in cu_seqlens.tolist()]
    if boundaries[-1] < total:  # trailing padding forms its own document
        boundaries.append(total)
    return _delta_rule_all_chunks(q, k, v, g, beta, boundaries, chunk)


def delta_rule_reference(q, k, v, g, beta, cu_seqlens=None, normalize_qk: bool = True, scale: float | None = None) -> torch.Tensor:
    if normalize_qk:
        q, k = l2_normalize(q.float()), l2_normalize(k.float())
    q = q.float() * (q.shape[-1] ** -0.5 if scale is None else scale)
    k, vf, gf, bf = k.float(), v.float(), g.float(), beta.float()
    total, heads, dk = q.shape
    starts = {0} if cu_seqlens is None else set(int(s) for s in cu_seqlens.tolist())
    state = torch.zeros(heads, dk, v.shape[2], dtype=torch.float32, device=q.device)
    outs = []
    for t in range(total):
        if t in starts:
            state = torch.zeros_like(state)
        decay = gf[t].exp()
        state = state * (decay[:, :, None] if gf.dim() == 3 else decay[:, None, None])
        read = torch.einsum("hd,hde->he", k[t], state)
        state = state + bf[t][:, None, None] * torch.einsum("hd,he->hde", k[t], vf[t] - read)
        outs.append(torch.einsum("hd,hde->he", q[t], state))
    return torch.stack(outs).to(v.dtype)


def gdn_log_decay(alpha: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    """g = -exp(A_log) * softplus(alpha + dt_bias); alpha [tokens, heads]."""
    return -a_log.float().exp() * torch.nn.functional.softplus(alpha.float() + dt_bias.float())


def kda_gate(g: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor | None = None) -> torch.Tensor:
    """Per-channel log decay: -exp(A_log[head]) * softplus(g + dt_bias); g [tokens, heads, head_dim]."""
    heads, dim = g.shape[-2:]
    g = g.float()
    if dt_bias is not None:
        g = g + dt_bias.float().view(heads, dim)
    return -a_log.float().view(heads, 1).exp() * torch.nn.functional.softplus(g)
