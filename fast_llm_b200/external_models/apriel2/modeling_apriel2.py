"""Apriel2 (text) in plain PyTorch for `transformers`: attention, Mamba, gated DeltaNet, Kimi delta attention and
stochastic mixers (which run their main mixer), one mixer per block as named by the configuration.

`Apriel2Model` / `Apriel2ForConditionalGeneration` add the vision encoder of the multimodal format (patch embeddings,
non-causal blocks with 2-D rotary positions, adapter MLP); its features replace the embeddings of the `image_token_index`
placeholders, one per placeholder in order.

Stand-alone file: it is copied next to exported checkpoints and loaded with `trust_remote_code`.  It favours clarity
over speed: the recurrent mixers step through the sequence token by token.  During generation every mixer keeps what it
needs of the prefix in an `Apriel2Cache` (rotated keys and values, the last inputs of each causal convolution, the
recurrent state), so a step runs the new tokens only.
Same role as `fast_llm_external_models/apriel2/modeling_apriel2.py`.
"""

import math

import torch
import torch.nn.functional as F
from torch import nn
from transformers import GenerationMixin, PreTrainedModel
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast

try:
    from .configuration_apriel2 import Apriel2Config, Apriel2TextConfig
except ImportError:  # loaded as a top-level module
    from configuration_apriel2 import Apriel2Config, Apriel2TextConfig

_ACTIVATIONS = {"silu": F.silu, "gelu": F.gelu, "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh"), "relu": F.relu,
                "relu2": lambda x: F.relu(x) ** 2, "sigmoid": torch.sigmoid, "identity": lambda x: x}


class RMSNorm(nn.Module):
    def __init__(self, size: int, epsilon: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size))
        self.epsilon = epsilon

    def forward(self, x: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
        xf = x.float()
        out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.epsilon) * self.weight.float()
        if gate is not None:
            out = out * F.silu(gate.float())
        return out.to(x.dtype)


def _linear(in_features: int, out_features: int, bias: bool) -> nn.Linear:
    return nn.Linear(in_features, out_features, bias=bias)


def _bias_enabled(section: dict, layer: str, default: bool) -> bool:
    enabled = section.get(layer, {}).get("bias", {}).get("enabled")
    return default if enabled is None else enabled


class CausalConv1d(nn.Module):
    """Depthwise causal convolution over [batch, tokens, channels] followed by SiLU."""

    def __init__(self, channels: int, kernel_size: int, bias: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(channels, 1, kernel_size))
        self.bias = nn.Parameter(torch.zeros(channels)) if bias else None

    def forward(self, x: torch.Tensor, state: dict | None = None, key: str = "conv") -> torch.Tensor:
        """`state[key]` holds the last kernel_size - 1 inputs of the prefix ([batch, channels, kernel_size - 1], fp32)."""
        k = self.weight.shape[-1]
        inputs = x.transpose(1, 2).float()
        if state is not None and key in state:
            inputs = torch.cat([state[key], inputs], dim=-1)
        else:
            inputs = F.pad(inputs, (k - 1, 0))
        if state is not None:
            state[key] = inputs[..., inputs.shape[-1] - (k - 1):]
        y = F.conv1d(inputs, self.weight.float(), None if self.bias is None else self.bias.float(), groups=self.weight.shape[0])
        return F.silu(y).transpose(1, 2).to(x.dtype)


# ------------------------------------------------------------------------------------------------------------ attention
def _rotary_frequencies(rotary: dict, head_size: int, device) -> torch.Tensor:
    theta = rotary.get("theta", 10000.0)
    inv = theta ** (-torch.arange(0, head_size, 2, dtype=torch.float64, device=device) / head_size)
    kind = rotary.get("type", "mistral_1d")
    if kind in ("mistral_1d", "default", "pixtral_2d"):
        return inv
    if kind == "llama3":
        factor, low, high = rotary["scale_factor"], rotary["low_frequency_factor"], rotary["high_frequency_factor"]
        original = rotary["original_context_length"]
        wavelength = 2 * math.pi / inv
        smooth = ((original / wavelength - low) / (high - low)).clamp(0, 1)
        return (1 - smooth) * inv / factor + smooth * inv
    raise NotImplementedError(f"rotary type {kind} is not available in this stand-alone model")


def _apply_rotary(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x [batch, tokens, heads, head_size]; pairs are (i, i + head_size / 2)."""
    cos, sin = angles.cos()[None, :, None, :], angles.sin()[None, :, None, :]
    x1, x2 = x.float().chunk(2, dim=-1)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, hidden: int, c: dict):
        super().__init__()
        self.heads, self.groups, self.head_size = c["heads"], c["head_groups"], c["head_size"]
        default = c.get("add_linear_biases", True)
        self.q_proj = _linear(hidden, self.heads * self.head_size, _bias_enabled(c, "query_layer", default))
        self.k_proj = _linear(hidden, self.groups * self.head_size, _bias_enabled(c, "key_layer", default))
        self.v_proj = _linear(hidden, self.groups * self.head_size, _bias_enabled(c, "value_layer", _bias_enabled(c, "key_layer", default)))
        self.o_proj = _linear(self.heads * self.head_size, hidden, _bias_enabled(c, "dense_layer", default))
        self.rotary = c.get("rotary", {"type": "mistral_1d"})
        self.window = c.get("window_size")
        self.causal = c.get("causal", True)

    def _angles(self, positions: torch.Tensor, device) -> torch.Tensor:
        """positions [tokens] (text) or [tokens, 2] = (row, column) of an image patch: there the even frequencies follow
        the row and fill the first half of the pairs, the odd ones follow the column."""
        frequencies = _rotary_frequencies(self.rotary, self.head_size, device)
        positions = positions.to(device=device, dtype=torch.float64)
        if positions.dim() == 1:
            return (positions[:, None] * frequencies[None, :]).float()
        return torch.cat([positions[:, :1] * frequencies[None, 0::2], positions[:, 1:2] * frequencies[None, 1::2]], dim=-1).float()

    def forward(self, x: torch.Tensor, state: dict | None = None, positions: torch.Tensor | None = None,
                segments: torch.Tensor | None = None) -> torch.Tensor:
        """`state`: rotated keys and values of the prefix and its length.  `segments` [tokens]: tokens attend within their
        own segment only (the patches of one image)."""
        batch, tokens, _ = x.shape
        q = self.q_proj(x).view(batch, tokens, self.heads, self.head_size)
        k = self.k_proj(x).view(batch, tokens, self.groups, self.head_size)
        v = self.v_proj(x).view(batch, tokens, self.groups, self.head_size)
        past = 0 if state is None else state.get("length", 0)
        index = torch.arange(past, past + tokens, device=x.device)
        angles = self._angles(index if positions is None else positions, x.device)
        q, k = _apply_rotary(q, angles), _apply_rotary(k, angles)
        key_index = index
        if state is not None:
            if "k" in state:
                k, v = torch.cat([state["k"], k], dim=1), torch.cat([state["v"], v], dim=1)
                key_index = torch.arange(past + tokens - k.shape[1], past + tokens, device=x.device)
            keep = k.shape[1] if self.window is None else min(k.shape[1], self.window - 1)  # what later tokens can still see
            state["k"], state["v"], state["length"] = k[:, k.shape[1] - keep:], v[:, v.shape[1] - keep:], past + tokens
        repeat = self.heads // self.groups
        k, v = k.repeat_interleave(repeat, dim=2), v.repeat_interleave(repeat, dim=2)
        if self.causal:
            mask = index[:, None] >= key_index[None, :]
        else:
            mask = torch.ones(tokens, key_index.shape[0], dtype=torch.bool, device=x.device)
        if self.window is not None:  # the current token plus window - 1 earlier ones
            mask = mask & (index[:, None] - key_index[None, :] < self.window)
        if segments is not None:
            mask = mask & (segments[:, None] == segments[None, :])
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask)
        return self.o_proj(out.transpose(1, 2).reshape(batch, tokens, self.heads * self.head_size))


class MLP(nn.Module):
    def __init__(self, hidden: int, c: dict):
        super().__init__()
        default = c.get("add_linear_biases", True)
        size = c["intermediate_size"]
        self.gated = c.get("gated", False)
        self.activation = _ACTIVATIONS[c.get("activation", "silu" if self.gated else "gelu")]
        if self.gated:
            self.gate_proj = _linear(hidden, size, _bias_enabled(c, "layer_1", default))
        self.up_proj = _linear(hidden, size, _bias_enabled(c, "layer_1", default))
        self.down_proj = _linear(size, hidden, _bias_enabled(c, "layer_2", default))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.gated:
            return self.down_proj(self.activation(self.gate_proj(x)) * self.up_proj(x))
        return self.down_proj(self.activation(self.up_proj(x)))


# ------------------------------------------------------------------------------------------------------- recurrent mixers
class Mamba(nn.Module):
    """in_proj -> [z | x | B | C]; x through a causal convolution; h_t = exp(dt A) h_{t-1} + dt B_t x_t per channel with
    `state_size` states; y = <C_t, h_t> + D x, gated by silu(z).  B is shared by the channels of a head group, C by the
    `state_size` channels of a head."""

    def __init__(self, hidden: int, c: dict):
        super().__init__()
        self.state, self.inner, self.xb = c["state_size"], c["d_inner"], c["d_xb"]
        self.repeat_before_conv = c.get("repeat_kv_before_conv", True)
        bias = c.get("add_linear_biases", False)
        self.in_proj = _linear(hidden, 2 * self.inner + 2 * self.xb, bias)
        self.dt_in_proj = _linear(hidden, c["dt_rank"], bias)
        self.dt_proj = _linear(c["dt_rank"], self.inner, c.get("dt_proj_bias", True))
        self.conv1d = CausalConv1d(self.inner if self.repeat_before_conv else self.xb, c.get("d_conv", 4), c.get("conv_bias", True))
        self.out_proj = _linear(self.inner, hidden, bias)
        self.A_log = nn.Parameter(torch.zeros(self.inner, self.state))
        self.D = nn.Parameter(torch.ones(self.inner))

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        cache = state
        batch, tokens, _ = x.shape
        n, groups, heads = self.state, self.xb // self.state, self.inner // self.state
        z, xs, b, c = torch.split(self.in_proj(x), [self.inner, self.xb, self.xb, self.inner], dim=-1)
        dt = F.linear(self.dt_in_proj(x), self.dt_proj.weight).float()
        if self.dt_proj.bias is not None:
            dt = dt + self.dt_proj.bias.float()
        dt = F.softplus(dt)

        def expand(t):  # [.., groups * n] -> [.., heads * n]
            return t.reshape(batch, tokens, groups, 1, n).expand(-1, -1, -1, heads // groups, -1).reshape(batch, tokens, self.inner)

        xs = self.conv1d(expand(xs), cache) if self.repeat_before_conv else expand(self.conv1d(xs, cache))
        a = -torch.exp(self.A_log.float())
        b = b.float().reshape(batch, tokens, groups, 1, n).expand(-1, -1, -1, self.inner // groups, -1).reshape(batch, tokens, self.inner, n)
        c = c.float().reshape(batch, tokens, heads, 1, n).expand(-1, -1, -1, n, -1).reshape(batch, tokens, self.inner, n)
        xf = xs.float()
        state = cache["ssm"] if cache is not None and "ssm" in cache else torch.zeros(batch, self.inner, n, dtype=torch.float32, device=x.device)
        outputs = []
        for t in range(tokens):
            state = torch.exp(dt[:, t, :, None] * a) * state + (dt[:, t] * xf[:, t])[:, :, None] * b[:, t]
            outputs.append((state * c[:, t]).sum(-1) + self.D.float() * xf[:, t])
        if cache is not None:
            cache["ssm"] = state
        y = torch.stack(outputs, dim=1) * F.silu(z.float())
        return self.out_proj(y.to(x.dtype))


def _l2_normalize(x: torch.Tensor) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def _delta_rule(q, k, v, log_decay, beta, cache: dict | None = None):
    """q, k [batch, tokens, heads, dk]; v [batch, tokens, heads, dv]; log_decay [batch, tokens, heads] or [.., heads, dk];
    beta [batch, tokens, heads].  S_t = decay S_{t-1} + beta k (v - k^T decay S_{t-1});  o_t = q^T S_t.
    `cache["delta"]` carries S over from the prefix."""
    q, k = _l2_normalize(q.float()) * q.shape[-1] ** -0.5, _l2_normalize(k.float())
    v, beta = v.float(), beta.float()
    batch, tokens, heads, dk = q.shape
    if cache is not None and "delta" in cache:
        state = cache["delta"]
    else:
        state = torch.zeros(batch, heads, dk, v.shape[-1], dtype=torch.float32, device=q.device)
    outputs = []
    for t in range(tokens):
        decay = log_decay[:, t].float().exp()
        state = state * (decay[..., None] if decay.dim() == 3 else decay[..., None, None])
        read = torch.einsum("bhd,bhde->bhe", k[:, t], state)
        state = state + beta[:, t, :, None, None] * torch.einsum("bhd,bhe->bhde", k[:, t], v[:, t] - read)
        outputs.append(torch.einsum("bhd,bhde->bhe", q[:, t], state))
    if cache is not None:
        cache["delta"] = state
    return torch.stack(outputs, dim=1)


class GatedDeltaNet(nn.Module):
    def __init__(self, hidden: int, c: dict, epsilon: float):
        super().__init__()
        self.value_heads, self.key_heads = c["value_heads"], c["key_heads"]
        self.key_dim, self.value_dim = c["key_head_dim"], c["value_head_dim"]
        key_size, value_size = self.key_heads * self.key_dim, self.value_heads * self.value_dim
        self.in_proj_qkvz = _linear(hidden, 2 * key_size + 2 * value_size, False)
        self.in_proj_ba = _linear(hidden, 2 * self.value_heads, False)
        self.convolution = CausalConv1d(2 * key_size + value_size, c.get("convolution_layer", {}).get("kernel_size", 4), False)
        self.out_proj = _linear(value_size, hidden, False)
        self.dt_bias = nn.Parameter(torch.ones(self.value_heads))
        self.A_log = nn.Parameter(torch.zeros(self.value_heads))
        self.norm = RMSNorm(self.value_dim, epsilon)

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        batch, tokens, _ = x.shape
        key_size, value_size = self.key_heads * self.key_dim, self.value_heads * self.value_dim
        qkv, z = torch.split(self.in_proj_qkvz(x), [2 * key_size + value_size, value_size], dim=-1)
        q, k, v = torch.split(self.convolution(qkv, state), [key_size, key_size, value_size], dim=-1)
        repeat = self.value_heads // self.key_heads
        q = q.reshape(batch, tokens, self.key_heads, self.key_dim).repeat_interleave(repeat, dim=2)
        k = k.reshape(batch, tokens, self.key_heads, self.key_dim).repeat_interleave(repeat, dim=2)
        v = v.reshape(batch, tokens, self.value_heads, self.value_dim)
        beta, alpha = torch.split(self.in_proj_ba(x), [self.value_heads, self.value_heads], dim=-1)
        log_decay = -self.A_log.float().exp() * F.softplus(alpha.float() + self.dt_bias.float())
        out = _delta_rule(q, k, v, log_decay, beta.float().sigmoid(), state).to(x.dtype)
        out = self.norm(out, z.reshape(batch, tokens, self.value_heads, self.value_dim))
        return self.out_proj(out.reshape(batch, tokens, value_size))


class KimiDeltaAttention(nn.Module):
    def __init__(self, hidden: int, c: dict):
        super().__init__()
        self.heads, self.head_dim = c["heads"], c["head_dim"]
        size = self.heads * self.head_dim
        kernel = c.get("convolution_layer", {}).get("kernel_size", 4)
        self.q_proj, self.k_proj, self.v_proj = _linear(hidden, size, False), _linear(hidden, size, False), _linear(hidden, size, False)
        self.q_conv, self.k_conv, self.v_conv = CausalConv1d(size, kernel, False), CausalConv1d(size, kernel, False), CausalConv1d(size, kernel, False)
        self.f_a_proj, self.f_b_proj = _linear(hidden, self.head_dim, False), _linear(self.head_dim, size, False)
        self.g_a_proj, self.g_b_proj = _linear(hidden, self.head_dim, False), _linear(self.head_dim, size, False)
        self.beta_proj = _linear(hidden, self.heads, False)
        self.o_proj = _linear(size, hidden, False)
        self.dt_bias = nn.Parameter(torch.ones(size))
        self.A_log = nn.Parameter(torch.zeros(self.heads))
        self.norm = RMSNorm(self.head_dim, c.get("normalization", {}).get("epsilon", 1e-5))

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        batch, tokens, _ = x.shape
        shape = (batch, tokens, self.heads, self.head_dim)
        q = self.q_conv(self.q_proj(x), state, "q_conv").reshape(shape)
        k = self.k_conv(self.k_proj(x), state, "k_conv").reshape(shape)
        v = self.v_conv(self.v_proj(x), state, "v_conv").reshape(shape)
        gate = self.f_b_proj(self.f_a_proj(x)).reshape(shape).float() + self.dt_bias.float().view(self.heads, self.head_dim)
        log_decay = -self.A_log.float().view(self.heads, 1).exp() * F.softplus(gate)
        out = _delta_rule(q, k, v, log_decay, self.beta_proj(x).float().sigmoid(), state).to(x.dtype)
        out = self.norm(out, self.g_b_proj(self.g_a_proj(x)).reshape(shape))
        return self.o_proj(out.reshape(batch, tokens, self.heads * self.head_dim))


class StochasticMixer(nn.Module):
    """All the candidate mixers are loaded; inference runs the main one."""

    def __init__(self, hidden: int, c: dict, epsilon: float):
        super().__init__()
        self.mixers = nn.ModuleDict({name: build_mixer(hidden, sub, epsilon) for name, sub in c["mixers"].items()})
        self.main = c.get("main_mixer_name") or next(iter(c["mixers"]))

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        return self.mixers[self.main](x, state)


def build_mixer(hidden: int, c: dict, epsilon: float) -> nn.Module:
    kind = c.get("type", "attention")
    if kind == "attention":
        return Attention(hidden, c)
    if kind == "mamba":
        return Mamba(hidden, c)
    if kind == "gdn":
        return GatedDeltaNet(hidden, c, epsilon)
    if kind == "kda":
        return KimiDeltaAttention(hidden, c)
    if kind == "stochastic":
        return StochasticMixer(hidden, c, epsilon)
    raise NotImplementedError(f"mixer type {kind}")


# ------------------------------------------------------------------------------------------------------------------ model
class Block(nn.Module):
    def __init__(self, hidden: int, c: dict):
        super().__init__()
        epsilon = c["normalization"].get("epsilon", 1e-5)
        self.input_layernorm = RMSNorm(hidden, epsilon)
        self.post_attention_layernorm = RMSNorm(hidden, epsilon)
        self.mixer = build_mixer(hidden, c["mixer"], epsilon)
        self.mlp = MLP(hidden, c["mlp"])

    def forward(self, x: torch.Tensor, state: dict | None = None, **mixer_arguments) -> torch.Tensor:
        x = x + self.mixer(self.input_layernorm(x), state, **mixer_arguments)
        return x + self.mlp(self.post_attention_layernorm(x))


class Decoder(nn.Module):
    def __init__(self, config: Apriel2TextConfig):
        super().__init__()
        self.blocks = nn.ModuleList(Block(config.hidden_size, c) for c in config.block_configs())


class Apriel2Cache:
    """What each block's mixer keeps of the prefix: one dictionary per block (attention: rotated keys and values,
    trimmed to the window; recurrent mixers: convolution inputs and the state), filled by the mixers themselves."""

    def __init__(self, blocks: int):
        self.layers: list[dict] = [{} for _ in range(blocks)]
        self.length = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.length

    def reorder_cache(self, beam_idx: torch.Tensor) -> None:
        """Beam search: row i continues from row beam_idx[i]."""
        for layer in self.layers:
            for name, value in layer.items():
                if torch.is_tensor(value):
                    layer[name] = value.index_select(0, beam_idx.to(value.device))


class Apriel2PreTrainedModel(PreTrainedModel):
    config_class = Apriel2TextConfig
    base_model_prefix = "model"
    _no_split_modules = ["Block"]
    _is_stateful = True  # recurrent states cannot be rolled back to a shorter prefix

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        return False  # `forward` makes its own `Apriel2Cache`


class Apriel2TextModel(Apriel2PreTrainedModel):
    def __init__(self, config: Apriel2TextConfig):
        super().__init__(config)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.decoder = Decoder(config)
        self.norm = RMSNorm(config.hidden_size, config.head.get("normalization", {}).get("epsilon", 1e-5))
        self.post_init()

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_input_embeddings(self, value):
        self.embed_tokens = value

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values: Apriel2Cache | None = None, use_cache: bool = False,
                output_hidden_states: bool = False, **kwargs):
        """With `past_key_values` the inputs are the tokens that follow the cached prefix."""
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        if use_cache and past_key_values is None:
            past_key_values = Apriel2Cache(len(self.decoder.blocks))
        states = [hidden] if output_hidden_states else None
        for index, block in enumerate(self.decoder.blocks):
            hidden = block(hidden, None if past_key_values is None else past_key_values.layers[index])
            if states is not None:
                states.append(hidden)
        if past_key_values is not None:
            past_key_values.length += hidden.shape[1]
        return BaseModelOutputWithPast(last_hidden_state=self.norm(hidden), past_key_values=past_key_values,
                                       hidden_states=tuple(states) if states is not None else None)


def _causal_lm_loss(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1), ignore_index=-100)


class Apriel2ForCausalLM(Apriel2PreTrainedModel, GenerationMixin):
    _tied_weights_keys = ["lm_head.weight"]

    def __init__(self, config: Apriel2TextConfig):
        super().__init__(config)
        self.model = Apriel2TextModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, value):
        self.lm_head = value

    def prepare_inputs_for_generation(self, input_ids, past_key_values: Apriel2Cache | None = None, use_cache: bool = True, **kwargs):
        if past_key_values is not None:
            input_ids = input_ids[:, past_key_values.get_seq_length():]  # the cache holds the rest
        return {"input_ids": input_ids, "past_key_values": past_key_values, "use_cache": use_cache}

    def forward(self, input_ids=None, inputs_embeds=None, labels=None, past_key_values: Apriel2Cache | None = None,
                use_cache: bool = False, output_hidden_states: bool = False, **kwargs):
        outputs = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, past_key_values=past_key_values, use_cache=use_cache,
                             output_hidden_states=output_hidden_states)
        logits = self.lm_head(outputs.last_hidden_state)
        loss = None if labels is None else _causal_lm_loss(logits, labels)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values, hidden_states=outputs.hidden_states)


# ------------------------------------------------------------------------------------------------------------ multimodal
class PatchEmbeddings(nn.Module):
    """A linear layer over each flattened patch ([channels, patch height, patch width]) and a normalization."""

    def __init__(self, hidden: int, c: dict):
        super().__init__()
        self.patch_height, self.patch_width = c["patch_height"], c["patch_width"]
        self.patch_embeddings = nn.Conv2d(c.get("input_channels", 3), hidden, (self.patch_height, self.patch_width),
                                          stride=(self.patch_height, self.patch_width), bias=False)
        self.normalization = RMSNorm(hidden, c.get("normalization", {}).get("epsilon", 1e-5))

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        """image [channels, height, width] -> [rows * columns, hidden], row-major."""
        features = self.patch_embeddings(image[None].to(self.patch_embeddings.weight.dtype))[0]
        return self.normalization(features.flatten(1).transpose(0, 1))


class VisionEncoderBlocks(nn.Module):
    def __init__(self, hidden: int, c: dict):
        super().__init__()
        assert c.get("type", "fixed") == "fixed", "the vision encoder uses one block description"
        self.blocks = nn.ModuleList(Block(hidden, c["block"]) for _ in range(c["num_blocks"]))


class VisionAdapter(nn.Module):
    def __init__(self, vision_hidden: int, hidden: int, c: dict):
        super().__init__()
        if c.get("gated", False):
            raise NotImplementedError("gated vision adapter")
        bias = c.get("add_linear_biases", True)
        self.linear_1 = _linear(vision_hidden, c["intermediate_size"], bias)
        self.linear_2 = _linear(c["intermediate_size"], hidden, bias)
        self.activation = _ACTIVATIONS[c.get("activation", "gelu")]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear_2(self.activation(self.linear_1(x)))


class Apriel2VisionEncoder(nn.Module):
    """All patches of all images form one sequence; a patch attends to the patches of its own image, with rotary
    positions from its (row, column) in the patch grid."""

    def __init__(self, c: dict, hidden: int):
        super().__init__()
        self.embeddings = PatchEmbeddings(c["hidden_size"], c["embeddings"])
        self.encoder = VisionEncoderBlocks(c["hidden_size"], c["encoder"])
        self.adapter = VisionAdapter(c["hidden_size"], hidden, c["adapter"])

    def forward(self, pixel_values, image_sizes=None) -> torch.Tensor:
        """`pixel_values`: [images, channels, height, width] (normalised; with `image_sizes` = (height, width) per image
        when the images were padded to a common size) or a list of [channels, height, width].  Returns
        [patches of all images, text hidden size] in image order, row-major within an image."""
        embeddings = self.embeddings
        features, positions, segments = [], [], []
        for index, image in enumerate(pixel_values):
            if image_sizes is not None:
                height, width = (int(v) for v in image_sizes[index])
                image = image[:, :height, :width]
            rows, columns = image.shape[1] // embeddings.patch_height, image.shape[2] // embeddings.patch_width
            features.append(embeddings(image[:, :rows * embeddings.patch_height, :columns * embeddings.patch_width]))
            grid = torch.stack(torch.meshgrid(torch.arange(rows), torch.arange(columns), indexing="ij"), dim=-1).reshape(-1, 2)
            positions.append(grid)
            segments.append(torch.full((rows * columns,), index))
        hidden = torch.cat(features)[None]
        positions, segments = torch.cat(positions).to(hidden.device), torch.cat(segments).to(hidden.device)
        for block in self.encoder.blocks:
            hidden = block(hidden, None, positions=positions, segments=segments)
        return self.adapter(hidden[0])


class Apriel2Model(Apriel2TextModel):
    """The text model plus the vision encoder (no output layer)."""

    config_class = Apriel2Config

    def __init__(self, config: Apriel2Config):
        super().__init__(config)
        self.vision_encoder = Apriel2VisionEncoder(config.vision_encoder, config.hidden_size) if config.vision_encoder else None
        self.post_init()

    def get_image_features(self, pixel_values, image_sizes=None) -> torch.Tensor:
        return self.vision_encoder(pixel_values, image_sizes)

    def merge(self, input_ids: torch.Tensor, pixel_values, image_sizes=None) -> torch.Tensor:
        embeddings = self.embed_tokens(input_ids)
        if pixel_values is None:
            return embeddings
        features = self.get_image_features(pixel_values, image_sizes).to(embeddings.dtype)
        mask = input_ids == self.config.image_token_index
        if int(mask.sum()) != features.shape[0]:
            raise ValueError(f"{int(mask.sum())} image placeholder tokens but {features.shape[0]} image features")
        return embeddings.masked_scatter(mask.unsqueeze(-1), features)

    def forward(self, input_ids=None, pixel_values=None, image_sizes=None, inputs_embeds=None, **kwargs):
        if inputs_embeds is None:
            inputs_embeds = self.merge(input_ids, pixel_values, image_sizes)
        return super().forward(inputs_embeds=inputs_embeds, **kwargs)


class Apriel2ForConditionalGeneration(Apriel2PreTrainedModel, GenerationMixin):
    config_class = Apriel2Config
    _tied_weights_keys = ["lm_head.weight"]

    def __init__(self, config: Apriel2Config):
        super().__init__(config)
        self.model = Apriel2Model(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def set_input_embeddings(self, value):
        self.model.embed_tokens = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, value):
        self.lm_head = value

    def prepare_inputs_for_generation(self, input_ids, past_key_values: Apriel2Cache | None = None, use_cache: bool = True,
                                      pixel_values=None, image_sizes=None, **kwargs):
        if past_key_values is not None and past_key_values.get_seq_length() > 0:
            # the images went in with the prompt
            return {"input_ids": input_ids[:, past_key_values.get_seq_length():], "past_key_values": past_key_values, "use_cache": use_cache}
        return {"input_ids": input_ids, "pixel_values": pixel_values, "image_sizes": image_sizes, "past_key_values": past_key_values,
                "use_cache": use_cache}

    def forward(self, input_ids=None, pixel_values=None, image_sizes=None, inputs_embeds=None, labels=None,
                past_key_values: Apriel2Cache | None = None, use_cache: bool = False, output_hidden_states: bool = False, **kwargs):
        outputs = self.model(input_ids=input_ids, pixel_values=pixel_values, image_sizes=image_sizes, inputs_embeds=inputs_embeds,
                             past_key_values=past_key_values, use_cache=use_cache, output_hidden_states=output_hidden_states)
        logits = self.lm_head(outputs.last_hidden_state)
        loss = None if labels is None else _causal_lm_loss(logits, labels)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values, hidden_states=outputs.hidden_states)


__all__ = ["Apriel2Cache", "Apriel2ForCausalLM", "Apriel2ForConditionalGeneration", "Apriel2Model", "Apriel2PreTrainedModel", "Apriel2TextModel"]
