"""Rotary position embeddings: none, default, llama3, yarn, proportional (partial rotary), default_2d (vision patches).

Each variant only differs in its inverse-frequency vector; a host-built fp64 table of cos/sin per position feeds the
one in-place kernel of `fast_llm_b200.ops.rotary`.  Parity: `fast_llm/layers/attention/rotary/config.py:25-163`,
`rotary.py:96-353`.
"""

import math

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.parameter import ModuleConfig
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.ops.rotary import rope
from fast_llm_b200.utils import Assert


@config_class(registry=True)
class RotaryConfig(ModuleConfig):
    @classmethod
    def _get_default_subclass(cls):
        return NoRotaryConfig if cls is RotaryConfig else cls

    def get_layer(self, head_size: int) -> "Rotary":
        return self._rotary_class(self, head_size)

    @property
    def enabled(self) -> bool:
        return True


@config_class(dynamic_type={RotaryConfig: "none"})
class NoRotaryConfig(RotaryConfig):
    _abstract = False

    @property
    def enabled(self) -> bool:
        return False

    @property
    def _rotary_class(self):
        return NoRotary


@config_class(dynamic_type={RotaryConfig: "default"})
class DefaultRotaryConfig(RotaryConfig):
    _abstract = False
    theta: float = Field(default=10000, desc="Base of the frequency geometric progression.", hint=FieldHint.architecture)

    @property
    def _rotary_class(self):
        return DefaultRotary


@config_class(dynamic_type={RotaryConfig: "llama3"})
class Llama3RotaryConfig(DefaultRotaryConfig):
    scale_factor: float = Field(default=8.0, hint=FieldHint.architecture)
    low_frequency_factor: float = Field(default=1.0, hint=FieldHint.architecture)
    high_frequency_factor: float = Field(default=4.0, hint=FieldHint.architecture)
    original_context_length: int = Field(default=8192, hint=FieldHint.architecture)

    def _validate(self):
        super()._validate()
        Assert.gt(self.high_frequency_factor, self.low_frequency_factor)

    @property
    def _rotary_class(self):
        return Llama3Rotary


@config_class(dynamic_type={RotaryConfig: "yarn"})
class YarnRotaryConfig(DefaultRotaryConfig):
    scale_factor: float = Field(default=8.0, hint=FieldHint.architecture)
    attention_factor: None | float = Field(default=None, hint=FieldHint.architecture)
    beta_fast: float = Field(default=32.0, hint=FieldHint.architecture)
    beta_slow: float = Field(default=1.0, hint=FieldHint.architecture)
    original_context_length: int = Field(default=8192, hint=FieldHint.architecture)

    def _validate(self):
        if self.attention_factor is None:
            self.attention_factor = 0.1 * math.log(self.scale_factor) + 1.0
        super()._validate()

    @property
    def _rotary_class(self):
        return YarnRotary


@config_class(dynamic_type={RotaryConfig: "default_2d"})
class Rotary2DConfig(DefaultRotaryConfig):
    @property
    def _rotary_class(self):
        return Rotary2D


@config_class(dynamic_type={RotaryConfig: "proportional"})
class ProportionalRotaryConfig(DefaultRotaryConfig):
    _abstract = False
    partial_rotary_factor: float = Field(default=1.0, desc="Fraction of each head that is rotated.", hint=FieldHint.architecture, valid=check_field(Assert.in_range_incl, 0, 1.0))

    @property
    def _rotary_class(self):
        return ProportionalRotary


class Rotary:
    def __init__(self, config: RotaryConfig, head_size: int):
        self._config = config
        self._head_size = head_size
        self._table = None
        self._table_length = 0

    @property
    def rot_dim(self) -> int:
        return self._head_size

    def _inverse_frequencies(self, device) -> torch.Tensor:
        raise NotImplementedError

    def _attention_scale(self) -> float:
        return 1.0

    def get_table(self, length: int, device) -> torch.Tensor:
        """[length, rot_dim] fp32: cos in the first half of each row, sin in the second."""
        if self._table is None or self._table_length < length or self._table.device != torch.device(device):
            length = max(length, 2 * self._table_length)
            inv = self._inverse_frequencies("cpu")
            ang = torch.arange(length, dtype=torch.float64)[:, None] * inv[None, :]
            scale = self._attention_scale()
            self._table = torch.cat([ang.cos() * scale, ang.sin() * scale], -1).float().contiguous().to(device)
            self._table_length = length
        return self._table

    def preprocess(self, kwargs: dict) -> None:
        pass

    def forward(self, x: torch.Tensor, n_heads: int, kwargs: dict) -> torch.Tensor:
        """Rotate, in place, the first n_heads heads of the packed rows of x ([tokens, >= n_heads*head_size])."""
        positions = kwargs.get(BlockKwargs.position_ids)
        max_pos = kwargs.get("max_position", None)
        if max_pos is None:
            max_pos = x.shape[0] if positions is None else kwargs.get(BlockKwargs.max_seqlen_k, x.shape[0])
        table = self.get_table(int(max_pos) + 1, x.device)
        return rope(x, table, positions, n_heads, self._head_size, self.rot_dim)


class NoRotary(Rotary):
    def forward(self, x, n_heads, kwargs):
        return x


class DefaultRotary(Rotary):
    def _inverse_frequencies(self, device):
        d = self.rot_dim
        return self._config.theta ** (-torch.arange(0, d, 2, dtype=torch.float64, device=device) / d)


class ProportionalRotary(DefaultRotary):
    @property
    def rot_dim(self) -> int:
        return int(self._head_size * self._config.partial_rotary_factor) // 2 * 2


class Llama3Rotary(DefaultRotary):
    def _inverse_frequencies(self, device):
        c = self._config
        inv = super()._inverse_frequencies(device)
        wavelen = 2 * math.pi / inv
        low_wavelen = c.original_context_length / c.low_frequency_factor
        high_wavelen = c.original_context_length / c.high_frequency_factor
        smooth = (c.original_context_length / wavelen - c.low_frequency_factor) / (c.high_frequency_factor - c.low_frequency_factor)
        blended = (1 - smooth) * inv / c.scale_factor + smooth * inv
        out = torch.where(wavelen > low_wavelen, inv / c.scale_factor, inv)
        mid = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
        return torch.where(mid, blended, out)


class YarnRotary(DefaultRotary):
    def _attention_scale(self) -> float:
        return self._config.attention_factor

    def _correction_dim(self, rotations: float) -> float:
        c = self._config
        return self.rot_dim * math.log(c.original_context_length / (rotations * 2 * math.pi)) / (2 * math.log(c.theta))

    def _inverse_frequencies(self, device):
        c = self._config
        d = self.rot_dim
        extrapolation = super()._inverse_frequencies(device)
        interpolation = extrapolation / c.scale_factor
        low = max(math.floor(self._correction_dim(c.beta_fast)), 0)
        high = min(math.ceil(self._correction_dim(c.beta_slow)), d - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(d // 2, dtype=torch.float64, device=device) - low) / (high - low)).clamp(0, 1)
        extrapolation_factor = 1 - ramp
        return interpolation * (1 - extrapolation_factor) + extrapolation * extrapolation_factor


class Rotary2D(DefaultRotary):
    """Image patches: the first half of the frequency pairs follows the patch row, the second half the column.
    `kwargs["patch_positions"]` holds [tokens, 2] (row, column)."""

    def forward(self, x, n_heads, kwargs):
        pos = kwargs["patch_positions"].to(x.device)
        d = self.rot_dim
        inv = self._config.theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
        # alternate frequencies between rows and columns
        inv_h, inv_w = inv[0::2], inv[1::2]
        ang = torch.cat([pos[:, :1].double().cpu() * inv_h[None], pos[:, 1:2].double().cpu() * inv_w[None]], -1)
        table = torch.cat([ang.cos(), ang.sin()], -1).float().contiguous().to(x.device)
        return rope(x, table, None, n_heads, self._head_size, d)
