"""MLP activations, gated (SwiGLU & friends) or plain (`csrc/elementwise.cu`).

Parity: `fast_llm/functional/triton/mlp.py:30-204` — input `[rows, 2n]` holds gate columns then up columns,
`out = act(gate) * up`; backward can recompute the forward output so it need not be stored.
"""

import enum

import torch

from fast_llm_b200.ops import _lib


class ActivationType(str, enum.Enum):
    identity = "identity"
    silu = "silu"
    gelu = "gelu"
    relu = "relu"
    squared_relu = "squared_relu"
    sigmoid = "sigmoid"
    gelu_erf = "gelu_erf"

    @property
    def code(self) -> int:
        return _CODES[self]

    @property
    def hf_name(self) -> str:
        return {"gelu": "gelu_pytorch_tanh", "squared_relu": "relu2", "gelu_erf": "gelu"}.get(self.value, self.value)

    @classmethod
    def from_hf_name(cls, name: str) -> "ActivationType":
        return {"gelu_pytorch_tanh": cls.gelu, "gelu_new": cls.gelu, "relu2": cls.squared_relu, "gelu": cls.gelu_erf,
                "swish": cls.silu}.get(name) or cls(name)


_CODES = {ActivationType.identity: 0, ActivationType.silu: 1, ActivationType.gelu: 2, ActivationType.relu: 3,
          ActivationType.squared_relu: 4, ActivationType.sigmoid: 5, ActivationType.gelu_erf: 6}


def activation_reference(x: torch.Tensor, act: ActivationType) -> torch.Tensor:
    f = torch.nn.functional
    return {
        ActivationType.identity: lambda t: t,
        ActivationType.silu: f.silu,
        ActivationType.gelu: lambda t: f.gelu(t, approximate="tanh"),
        ActivationType.relu: f.relu,
        ActivationType.squared_relu: lambda t: f.relu(t).pow(2),
        ActivationType.sigmoid: torch.sigmoid,
        ActivationType.gelu_erf: f.gelu,
    }[act](x)


def mlp_activation_reference(x: torch.Tensor, gated: bool, act: ActivationType) -> torch.Tensor:
    if gated:
        gate, up = x.chunk(2, dim=-1)
        return (activation_reference(gate.float(), act) * up.float()).to(x.dtype)
    return activation_reference(x.float(), act).to(x.dtype)


def _native(x):
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0


def act_fwd_native(x2: torch.Tensor, gated: bool, act: ActivationType) -> torch.Tensor:
    rows = x2.shape[0]
    n = x2.shape[1] // 2 if gated else x2.shape[1]
    out = torch.empty(rows, n, dtype=x2.dtype, device=x2.device)
    _lib.check(_lib.get_lib().flb_act_fwd(x2.data_ptr(), out.data_ptr(), rows, n, int(gated), act.code, _lib.stream_ptr()), "flb_act_fwd")
    _lib.count_launch()
    return out


def act_bwd_native(grad_out2, x2, gated: bool, act: ActivationType, recompute: bool):
    rows = x2.shape[0]
    n = x2.shape[1] // 2 if gated else x2.shape[1]
    grad_in = torch.empty_like(x2)
    out = torch.empty(rows, n, dtype=x2.dtype, device=x2.device) if recompute else None
    _lib.check(
        _lib.get_lib().flb_act_bwd(grad_out2.data_ptr(), x2.data_ptr(), grad_in.data_ptr(), _lib.ptr(out), rows, n,
                                   int(gated), act.code, _lib.stream_ptr()), "flb_act_bwd")
    _lib.count_launch()
    return grad_in, out


class _MLPActivation(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gated, act):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        ctx.save_for_backward(x2)
        ctx.args = (gated, act, shape)
        out = act_fwd_native(x2, gated, act)
        return out.view(*shape[:-1], out.shape[-1])

    @staticmethod
    def backward(ctx, grad):
        (x2,) = ctx.saved_tensors
        gated, act, shape = ctx.args
        grad_in, _ = act_bwd_native(grad.reshape(-1, grad.shape[-1]).contiguous(), x2, gated, act, False)
        return grad_in.view(shape), None, None


def mlp_activation(x: torch.Tensor, gated: bool, act: ActivationType) -> torch.Tensor:
    if _native(x):
        return _MLPActivation.apply(x, gated, act)
    return mlp_activation_reference(x, gated, act)
