"""Rotary position embedding applied in place on packed [tokens, heads*head_dim] projections (`csrc/elementwise.cu`).

Frequencies come from a host-built fp64 table, so every scaling scheme (default, llama3, yarn, proportional) shares one
kernel.  Pairing is element i with i + rot_dim/2 inside a head, the "real/imaginary halves" layout of
`fast_llm/functional/triton/rotary.py:10-67` and of Hugging Face Llama checkpoints.
"""

import torch

from fast_llm_b200.ops import _lib


def rope_reference(x: torch.Tensor, table: torch.Tensor, positions: torch.Tensor | None, n_heads: int, head_dim: int,
                   rot_dim: int, conj: bool = False) -> torch.Tensor:
    """Out-of-place PyTorch restatement. x: [tokens, >= n_heads*head_dim]; table: [max_pos, rot_dim] (cos | sin)."""
    tokens = x.shape[0]
    half = rot_dim // 2
    pos = torch.arange(tokens, device=x.device) if positions is None else positions.long()
    cos = table[pos, :half].unsqueeze(1)
    sin = table[pos, half:rot_dim].unsqueeze(1)
    if conj:
        sin = -sin
    out = x.clone()
    h = x[:, : n_heads * head_dim].reshape(tokens, n_heads, head_dim).float()
    a, b = h[..., :half], h[..., half:rot_dim]
    rot = torch.cat([a * cos - b * sin, b * cos + a * sin, h[..., rot_dim:]], dim=-1)
    out[:, : n_heads * head_dim] = rot.reshape(tokens, n_heads * head_dim).to(x.dtype)
    return out


def rope_(x: torch.Tensor, table: torch.Tensor, positions: torch.Tensor | None, n_heads: int, head_dim: int,
          rot_dim: int, conj: bool = False) -> torch.Tensor:
    """In place on the first n_heads*head_dim columns of every row of x."""
    if x.is_cuda and x.dtype == torch.bfloat16 and rot_dim % 16 == 0 and x.stride(-1) == 1 and x.stride(0) % 8 == 0:
        if positions is not None and positions.dtype != torch.int32:
            positions = positions.to(torch.int32)
        _lib.check(
            _lib.get_lib().flb_rope(x.data_ptr(), table.data_ptr(), _lib.ptr(positions), x.shape[0], x.stride(0),
                                    n_heads, head_dim, rot_dim, int(conj), _lib.stream_ptr()),
            "flb_rope",
        )
        _lib.count_launch()
        return x
    x.copy_(rope_reference(x, table, positions, n_heads, head_dim, rot_dim, conj))
    return x


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, table, positions, n_heads, head_dim, rot_dim):
        ctx.save_for_backward(table, positions)
        ctx.args = (n_heads, head_dim, rot_dim)
        ctx.mark_dirty(x)
        return rope_(x, table, positions, n_heads, head_dim, rot_dim)

    @staticmethod
    def backward(ctx, grad):
        table, positions = ctx.saved_tensors
        # The incoming gradient may be shared with other consumers: rotate a private copy.
        return rope_(grad.clone(memory_format=torch.contiguous_format), table, positions, *ctx.args, conj=True), None, None, None, None, None


def rope(x, table, positions, n_heads, head_dim, rot_dim):
    """Differentiable in-place rotary (the rotation is orthogonal, so backward is the inverse rotation of the gradient)."""
    return _Rope.apply(x, table, positions, n_heads, head_dim, rot_dim)
