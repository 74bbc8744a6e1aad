"""Megatron-LM compatible parameter initialisation (single process, for bit-matching comparisons).

Megatron creates, per layer and from ONE random stream, the attention output projection, then a fused
`[groups, heads_per_group + 2, head_size, hidden]` query-key-value block, then the MLP weights with the second layer
stored `[hidden, ffn]`.  To reproduce its values with this framework's layout (separate `query` / `key_value` weights
visited before `dense`, second MLP layer stored `[ffn, hidden]`), each parameter replays the relevant part of that stream:
`query` and `key_value` draw (dense, qkv) from the current stream state, keep their slice of qkv and REWIND the stream;
`dense` draws the same pair and leaves the stream advanced.  Position embeddings and MoE routers come from the default
CPU generator like in Megatron.  Parity: `fast_llm/models/gpt/megatron.py:17-167`.
"""

import torch

from fast_llm_b200.utils import Assert, div


def set_megatron_distributed_seeds(config) -> None:
    """Seed offsets under which the generators line up with Megatron's."""
    config.dp_seed_shift = 0
    config.pp_seed_shift = 100
    config.pp_gen_init_seed_shift = 0
    config.tp_seed_shift = 1
    config.tp_gen_init_seed_shift = 2718
    config.reproducible_init = False


def get_init_megatron(meta, block_config, hidden_size: int):
    """Initialiser `(tensor, distributed) -> None` for one parameter of a decoder block (or embedding)."""
    name = meta.tensor_name
    base = meta.param_init_method
    mixer, mlp = block_config.mixer, block_config.mlp
    experts = getattr(mlp, "experts", 1)

    def draw(shape, generator, like: torch.Tensor) -> torch.Tensor:
        out = torch.empty(shape, dtype=torch.float32, device=generator.device)
        base(meta, out, generator)
        return out.to(like.device)

    def init(tensor: torch.Tensor, distributed) -> None:
        Assert.eq(distributed.config.world_size, 1)
        generator = distributed.tp_init_generator
        if "bias" in name:
            value = draw(tensor.shape, generator, tensor)
        elif any(part in name for part in ("mixer.query", "mixer.key_value", "mixer.dense")):
            state = generator.get_state()
            heads_per_group = div(mixer.heads, mixer.head_groups)
            dense = draw((mixer.heads * mixer.head_size, hidden_size), generator, tensor)
            qkv = draw((mixer.head_groups, heads_per_group + 2, mixer.head_size, hidden_size), generator, tensor)
            if "dense" in name:
                value = dense
            else:
                generator.set_state(state)
                value = qkv[:, :heads_per_group] if "query" in name else qkv[:, heads_per_group:].transpose(0, 1)
        elif "position_embeddings" in name:
            cpu = distributed.default_cpu_generator
            draw(tensor.shape, cpu, tensor)  # Megatron draws (and discards) once before the values it keeps
            value = draw(tensor.shape, cpu, tensor)
        elif "mlp.router.weight" in name:
            value = draw(tensor.shape, distributed.default_cpu_generator, tensor)
        elif experts > 1 and "mlp.layer_" in name:
            gen = generator if meta.is_tensor_parallel else distributed.pp_init_generator
            state = gen.get_state()
            ffn = mlp.intermediate_size
            first, second = [], []
            for _ in range(experts):  # per expert: first layer, then the second one drawn as [hidden, ffn]
                first.append(draw(((1 + mlp.gated) * ffn, hidden_size), gen, tensor))
                second.append(draw((hidden_size, ffn), gen, tensor).t())
            if "layer_1" in name:
                gen.set_state(state)
                value = torch.cat(first, 0)
            else:
                value = torch.cat(second, 0)
        elif "mlp.layer_2" in name:
            value = draw((meta.shape[1], meta.shape[0]), generator, tensor).t()
        else:
            value = draw(tensor.shape, generator, tensor)
        tensor.copy_(value.reshape(tensor.shape))

    return init
