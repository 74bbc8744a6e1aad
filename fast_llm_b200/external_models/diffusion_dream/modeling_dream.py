"""Dream in plain PyTorch for `transformers`: a decoder with bidirectional attention whose logits at position i
predict token i + 1, sampled by iterative unmasking (`diffusion_generate`).

Stand-alone file: it is copied next to exported checkpoints and loaded with `trust_remote_code`.
"""

import math

import torch
import torch.nn.functional as F
from torch import nn
from transformers import PreTrainedModel
from transformers.modeling_outputs import MaskedLMOutput

try:
    from .configuration_dream import DreamConfig
except ImportError:  # loaded as a top-level module
    from configuration_dream import DreamConfig

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



def _rotary_section(config) -> dict:
    scaling = getattr(config, "rope_scaling", None)
    theta = getattr(config, "rope_theta", None) or (getattr(config, "rope_parameters", None) or {}).get("rope_theta", 10000.0)
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        return {"type": "llama3", "theta": theta, "scale_factor": scaling["factor"], "low_frequency_factor": scaling["low_freq_factor"],
                "high_frequency_factor": scaling["high_freq_factor"], "original_context_length": scaling["original_max_position_embeddings"]}
    return {"type": "mistral_1d", "theta": theta}


class Attention(nn.Module):
    def __init__(self, config: DreamConfig):
        super().__init__()
        hidden = config.hidden_size
        self.heads, self.groups = config.num_attention_heads, config.num_key_value_heads
        self.head_size = getattr(config, "head_dim", None) or hidden // self.heads
        qkv_bias = True
        self.q_proj = nn.Linear(hidden, self.heads * self.head_size, bias=qkv_bias)
        self.k_proj = nn.Linear(hidden, self.groups * self.head_size, bias=qkv_bias)
        self.v_proj = nn.Linear(hidden, self.groups * self.head_size, bias=qkv_bias)
        self.o_proj = nn.Linear(self.heads * self.head_size, hidden, bias=getattr(config, "attention_bias", False))
        self.rotary = _rotary_section(config)
        self.bidirectional = config.bidirectional

    def forward(self, x: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        batch, tokens, _ = x.shape
        q = self.q_proj(x).view(batch, tokens, self.heads, self.head_size)
        k = self.k_proj(x).view(batch, tokens, self.groups, self.head_size)
        v = self.v_proj(x).view(batch, tokens, self.groups, self.head_size)
        positions = torch.arange(tokens, device=x.device, dtype=torch.float64)
        angles = (positions[:, None] * _rotary_frequencies(self.rotary, self.head_size, x.device)[None, :]).float()
        q, k = _apply_rotary(q, angles), _apply_rotary(k, angles)
        repeat = self.heads // self.groups
        k, v = k.repeat_interleave(repeat, dim=2), v.repeat_interleave(repeat, dim=2)
        mask = torch.ones(tokens, tokens, dtype=torch.bool, device=x.device)
        if not self.bidirectional:
            mask = mask.tril()
        mask = mask[None, None]
        if attention_mask is not None:  # [batch, tokens], 0 for padding
            mask = mask & attention_mask.bool()[:, None, None, :]
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



class Layer(nn.Module):
    def __init__(self, config: DreamConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.self_attn = Attention(config)
        self.mlp = MLP(config.hidden_size, {"intermediate_size": config.intermediate_size, "gated": True, "activation": config.hidden_act,
                                            "add_linear_biases": getattr(config, "mlp_bias", False)})

    def forward(self, x: torch.Tensor, attention_mask=None) -> torch.Tensor:
        x = x + self.self_attn(self.input_layernorm(x), attention_mask)
        return x + self.mlp(self.post_attention_layernorm(x))


class Decoder(nn.Module):
    def __init__(self, config: DreamConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(Layer(config) for _ in range(config.num_hidden_layers))
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)


class DreamModel(PreTrainedModel):
    config_class = DreamConfig
    base_model_prefix = "model"
    _no_split_modules = ["Layer"]
    _tied_weights_keys = ["lm_head.weight"]

    def __init__(self, config: DreamConfig):
        super().__init__(config)
        self.model = Decoder(config)
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

    def forward(self, input_ids=None, attention_mask=None, inputs_embeds=None, **kwargs):
        hidden = self.model.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        for layer in self.model.layers:
            hidden = layer(hidden, attention_mask)
        return MaskedLMOutput(logits=self.lm_head(self.model.norm(hidden)))

    @torch.no_grad()
    def diffusion_generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, steps: int = 8, temperature: float = 0.0,
                           generator: torch.Generator | None = None) -> torch.Tensor:
        """Append `max_new_tokens` mask tokens to the prompt and reveal them over `steps` rounds: every round predicts all
        masked positions at once (position i is predicted by the logits at i - 1) and keeps the most confident ones."""
        mask_id = self.config.mask_token_id
        batch, prompt = input_ids.shape
        tokens = torch.cat([input_ids, input_ids.new_full((batch, max_new_tokens), mask_id)], dim=1)
        for step in range(steps):
            masked = tokens == mask_id
            remaining = int(masked.sum(1).max())
            if remaining == 0:
                break
            logits = self(input_ids=tokens).logits.float()
            logits = torch.cat([logits[:, :1], logits[:, :-1]], dim=1)  # align: entry i now scores token i
            logits[..., mask_id] = -float("inf")
            if temperature > 0:
                probabilities = F.softmax(logits / temperature, dim=-1)
                choice = torch.multinomial(probabilities.view(-1, probabilities.shape[-1]), 1, generator=generator).view(batch, -1)
                confidence = probabilities.gather(-1, choice[..., None])[..., 0]
            else:
                confidence, choice = F.softmax(logits, dim=-1).max(-1)
            confidence = confidence.masked_fill(~masked, -1.0)
            reveal = math.ceil(remaining / (steps - step))
            keep = confidence.topk(min(reveal, confidence.shape[1]), dim=1).indices
            selected = torch.zeros_like(masked).scatter_(1, keep, True) & masked
            tokens = torch.where(selected, choice, tokens)
        return tokens
