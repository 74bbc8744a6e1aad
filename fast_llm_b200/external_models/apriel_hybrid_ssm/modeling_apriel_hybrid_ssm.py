"""Apriel hybrid SSM in plain PyTorch for `transformers`: a Mistral-style decoder whose layers are attention ("t"),
Mamba ("m2") or gated DeltaNet ("gdn") as listed in `hybrid_block_layout`.

Stand-alone file: it is copied next to exported checkpoints and loaded with `trust_remote_code`.  It favours clarity
over speed: the recurrent mixers step through the sequence token by token.  During generation every mixer keeps what it
needs of the prefix in a `HybridCache` (rotated keys and values, the last inputs of the causal convolution, the
recurrent state), so a step runs the new tokens only.
"""

import math

import torch
import torch.nn.functional as F
from torch import nn
from transformers import GenerationMixin, PreTrainedModel
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast

try:
    from .configuration_apriel_hybrid_ssm import AprielHybridSSMConfig
except ImportError:  # loaded as a top-level module
    from configuration_apriel_hybrid_ssm import AprielHybridSSMConfig

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


def _rotary_frequencies(rotary: dict, head_size: int, device) -> torch.Tensor:
    theta = rotary.get("theta", 10000.0)
    inv = theta ** (-torch.arange(0, head_size, 2, dtype=torch.float64, device=device) / head_size)
    kind = rotary.get("type", "mistral_1d")
    if kind in ("mistral_1d", "default"):
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

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        """`state`: rotated keys and values of the prefix (trimmed to the window) and its length."""
        batch, tokens, _ = x.shape
        q = self.q_proj(x).view(batch, tokens, self.heads, self.head_size)
        k = self.k_proj(x).view(batch, tokens, self.groups, self.head_size)
        v = self.v_proj(x).view(batch, tokens, self.groups, self.head_size)
        past = 0 if state is None else state.get("length", 0)
        index = torch.arange(past, past + tokens, device=x.device)
        angles = (index.double()[:, None] * _rotary_frequencies(self.rotary, self.head_size, x.device)[None, :]).float()
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
        mask = index[:, None] >= key_index[None, :]
        if self.window is not None:  # the current token plus window - 1 earlier ones
            mask = mask & (index[:, None] - key_index[None, :] < self.window)
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
    beta [batch, tokens, heads].  S_t = decay S_{t-1} + beta k (v - k^T decay S_{t-1});  o_t = q^T S_t."""
    q, k = _l2_normalize(q.float()) * q.shape[-1] ** -0.5, _l2_normalize(k.float())
    v, beta = v.float(), beta.float()
    batch, tokens, heads, dk = q.shape
    if cache is not None and "delta" in cache:  # S carried over from the prefix
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
        self.conv1d = CausalConv1d(2 * key_size + value_size, c.get("convolution_layer", {}).get("kernel_size", 4), False)
        self.out_proj = _linear(value_size, hidden, False)
        self.dt_bias = nn.Parameter(torch.ones(self.value_heads))
        self.A_log = nn.Parameter(torch.zeros(self.value_heads))
        self.norm = RMSNorm(self.value_dim, epsilon)

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        batch, tokens, _ = x.shape
        key_size, value_size = self.key_heads * self.key_dim, self.value_heads * self.value_dim
        qkv, z = torch.split(self.in_proj_qkvz(x), [2 * key_size + value_size, value_size], dim=-1)
        q, k, v = torch.split(self.conv1d(qkv, state), [key_size, key_size, value_size], dim=-1)
        repeat = self.value_heads // self.key_heads
        q = q.reshape(batch, tokens, self.key_heads, self.key_dim).repeat_interleave(repeat, dim=2)
        k = k.reshape(batch, tokens, self.key_heads, self.key_dim).repeat_interleave(repeat, dim=2)
        v = v.reshape(batch, tokens, self.value_heads, self.value_dim)
        beta, alpha = torch.split(self.in_proj_ba(x), [self.value_heads, self.value_heads], dim=-1)
        log_decay = -self.A_log.float().exp() * F.softplus(alpha.float() + self.dt_bias.float())
        out = _delta_rule(q, k, v, log_decay, beta.float().sigmoid(), state).to(x.dtype)
        out = self.norm(out, z.reshape(batch, tokens, self.value_heads, self.value_dim))
        return self.out_proj(out.reshape(batch, tokens, value_size))




# ------------------------------------------------------------------------------------------------------------------ model
def _rotary_section(config) -> dict:
    scaling = getattr(config, "rope_scaling", None)
    theta = getattr(config, "rope_theta", 10000.0)
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        return {"type": "llama3", "theta": theta, "scale_factor": scaling["factor"], "low_frequency_factor": scaling["low_freq_factor"],
                "high_frequency_factor": scaling["high_freq_factor"], "original_context_length": scaling["original_max_position_embeddings"]}
    return {"type": "mistral_1d", "theta": theta}


class Layer(nn.Module):
    def __init__(self, config: AprielHybridSSMConfig, kind: str):
        super().__init__()
        hidden, epsilon = config.hidden_size, config.rms_norm_eps
        self.kind = kind
        self.input_layernorm = RMSNorm(hidden, epsilon)
        self.post_attention_layernorm = RMSNorm(hidden, epsilon)
        if kind == "t":
            heads = config.num_attention_heads
            self.self_attn = Attention(hidden, {
                "heads": heads, "head_groups": config.num_key_value_heads, "head_size": getattr(config, "head_dim", None) or hidden // heads,
                "add_linear_biases": False, "rotary": _rotary_section(config), "window_size": getattr(config, "sliding_window", None)})
        elif kind == "m2":
            ssm = config.ssm_cfg
            dt_rank = ssm.get("dt_rank", "auto")
            self.mixer = Mamba(hidden, {
                "state_size": ssm.get("d_state", 16), "d_inner": ssm.get("d_inner") or hidden * ssm.get("expand", 1), "d_xb": ssm.get("d_xb") or hidden,
                "dt_rank": -(-hidden // 16) if dt_rank == "auto" else dt_rank, "add_linear_biases": ssm.get("bias", False),
                "repeat_kv_before_conv": ssm.get("repeat_kv_before_conv", True), "d_conv": ssm.get("d_conv", 4),
                "conv_bias": ssm.get("conv_bias", True), "dt_proj_bias": ssm.get("dt_proj_bias", True)})
        elif kind == "gdn":
            linear = config.linear_attn_config
            self.mixer = GatedDeltaNet(hidden, {
                "value_heads": linear["gdn_num_value_heads"], "key_heads": linear["gdn_num_key_heads"], "key_head_dim": linear["gdn_key_head_dim"],
                "value_head_dim": linear["gdn_value_head_dim"], "convolution_layer": {"kernel_size": linear.get("gdn_linear_conv_kernel_size", 4)}}, epsilon)
        else:
            raise NotImplementedError(f"layer type {kind}")
        self.mlp = MLP(hidden, {"intermediate_size": config.intermediate_size, "gated": True, "activation": config.hidden_act, "add_linear_biases": False})

    def forward(self, x: torch.Tensor, state: dict | None = None) -> torch.Tensor:
        mixer = self.self_attn if self.kind == "t" else self.mixer
        x = x + mixer(self.input_layernorm(x), state)
        return x + self.mlp(self.post_attention_layernorm(x))


class HybridCache:
    """What each layer's mixer keeps of the prefix: one dictionary per layer, filled by the mixers themselves."""

    def __init__(self, layers: int):
        self.layers: list[dict] = [{} for _ in range(layers)]
        self.length = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.length

    def reorder_cache(self, beam_idx: torch.Tensor) -> None:
        """Beam search: row i continues from row beam_idx[i]."""
        for layer in self.layers:
            for name, value in layer.items():
                if torch.is_tensor(value):
                    layer[name] = value.index_select(0, beam_idx.to(value.device))


class AprielHybridSSMPreTrainedModel(PreTrainedModel):
    config_class = AprielHybridSSMConfig
    base_model_prefix = "model"
    _no_split_modules = ["Layer"]
    _is_stateful = True  # recurrent states cannot be rolled back to a shorter prefix

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        return False  # `forward` makes its own `HybridCache`


class AprielHybridSSMModel(AprielHybridSSMPreTrainedModel):
    def __init__(self, config: AprielHybridSSMConfig):
        super().__init__(config)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(Layer(config, kind) for kind in config.hybrid_block_layout)
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_init()

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_input_embeddings(self, value):
        self.embed_tokens = value

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values: HybridCache | None = None, use_cache: bool = False,
                output_hidden_states: bool = False, **kwargs):
        """With `past_key_values` the inputs are the tokens that follow the cached prefix."""
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        if use_cache and past_key_values is None:
            past_key_values = HybridCache(len(self.layers))
        states = [hidden] if output_hidden_states else None
        for index, layer in enumerate(self.layers):
            hidden = layer(hidden, None if past_key_values is None else past_key_values.layers[index])
            if states is not None:
                states.append(hidden)
        if past_key_values is not None:
            past_key_values.length += hidden.shape[1]
        return BaseModelOutputWithPast(last_hidden_state=self.norm(hidden), past_key_values=past_key_values,
                                       hidden_states=tuple(states) if states is not None else None)


class AprielHybridSSMForCausalLM(AprielHybridSSMPreTrainedModel, GenerationMixin):
    _tied_weights_keys = ["lm_head.weight"]

    def __init__(self, config: AprielHybridSSMConfig):
        super().__init__(config)
        self.model = AprielHybridSSMModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, value):
        self.lm_head = value

    def prepare_inputs_for_generation(self, input_ids, past_key_values: HybridCache | None = None, use_cache: bool = True, **kwargs):
        if past_key_values is not None:
            input_ids = input_ids[:, past_key_values.get_seq_length():]  # the cache holds the rest
        return {"input_ids": input_ids, "past_key_values": past_key_values, "use_cache": use_cache}

    def forward(self, input_ids=None, inputs_embeds=None, labels=None, past_key_values: HybridCache | None = None, use_cache: bool = False,
                output_hidden_states: bool = False, **kwargs):
        outputs = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, past_key_values=past_key_values, use_cache=use_cache,
                             output_hidden_states=output_hidden_states)
        logits = self.lm_head(outputs.last_hidden_state)
        loss = None
        if labels is not None:
            loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1), ignore_index=-100)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values, hidden_states=outputs.hidden_states)
