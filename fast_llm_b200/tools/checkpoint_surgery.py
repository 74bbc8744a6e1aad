"""Checkpoint surgery on Hugging Face checkpoints (safetensors + config.json), without instantiating the model:

    python -m fast_llm_b200.tools.checkpoint_surgery add_experts hf_checkpoint=... output_dir=... num_new_experts=2 ...
        MoE upcycling: append experts (copies of existing ones plus optional noise, or noise only) and router rows to a
        Mixtral-style checkpoint.
    python -m fast_llm_b200.tools.checkpoint_surgery add_mtp_heads hf_checkpoint=... output_dir=... num_prediction_heads=3
        Turn a Llama / Mistral checkpoint into an `mtp_llama` one: every extra head starts as a copy of the last
        transformer layer, every head gets its own copy of the final norm.

Parity: `tools/moe_add_experts.py`, `tools/transformer_add_mtp_heads.py`.
"""

import enum
import json
import logging
import pathlib
import shutil
import typing

import torch
import yaml

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.config.runnable import RunnableConfig

logger = logging.getLogger(__name__)


class InitMethod(str, enum.Enum):
    from_existing = "from_existing"
    from_scratch = "from_scratch"


def load_hf_state(path: pathlib.Path) -> tuple[dict, dict[str, torch.Tensor]]:
    import safetensors.torch

    config = json.loads((path / "config.json").read_text())
    state: dict[str, torch.Tensor] = {}
    for file in sorted(path.glob("*.safetensors")):
        state.update(safetensors.torch.load_file(str(file)))
    if not state:
        raise FileNotFoundError(f"No safetensors file in {path}")
    return config, state


def save_hf_state(path: pathlib.Path, source: pathlib.Path, config: dict, state: dict[str, torch.Tensor], surgery: dict) -> None:
    import safetensors.torch

    path.mkdir(parents=True, exist_ok=True)
    safetensors.torch.save_file({k: v.contiguous() for k, v in state.items()}, str(path / "model.safetensors"), metadata={"format": "pt"})
    (path / "config.json").write_text(json.dumps(config, indent=2))
    for extra in source.iterdir():  # tokenizer, generation config, ...
        if extra.is_file() and extra.suffix not in (".safetensors",) and extra.name not in ("config.json", "model.safetensors.index.json"):
            shutil.copy(extra, path / extra.name)
    (path / "surgery_config.yaml").write_text(yaml.safe_dump(surgery))


@config_class(registry=True, dynamic_type={RunnableConfig: "checkpoint_surgery"})
class CheckpointSurgeryConfig(RunnableConfig):
    _abstract: typing.ClassVar[bool] = True
    hf_checkpoint: pathlib.Path = Field(default=None, desc="Source checkpoint directory.", hint=FieldHint.core)
    output_dir: pathlib.Path = Field(default=None, desc="Where the modified checkpoint is written.", hint=FieldHint.core)
    seed: int = Field(default=0, desc="Seed of the noise.", hint=FieldHint.optional)


@config_class(dynamic_type={RunnableConfig: "moe_add_experts", CheckpointSurgeryConfig: "add_experts"})
class AddExpertsConfig(CheckpointSurgeryConfig):
    _abstract: typing.ClassVar[bool] = False
    num_new_experts: int = Field(default=1, desc="Experts to append to every layer.", hint=FieldHint.core)
    expert_init_method: InitMethod = Field(default=InitMethod.from_existing, hint=FieldHint.core)
    router_init_method: InitMethod = Field(default=InitMethod.from_existing, hint=FieldHint.core)
    expert_init_std: float = Field(default=0.0, desc="Standard deviation of the noise added to (or used as) new experts.", hint=FieldHint.core)
    router_init_std: float = Field(default=0.0, hint=FieldHint.core)

    def run(self) -> None:
        config, state = load_hf_state(self.hf_checkpoint)
        experts, layers = config["num_local_experts"], config["num_hidden_layers"]
        generator = torch.Generator().manual_seed(self.seed)

        def noise(like: torch.Tensor, std: float) -> torch.Tensor:
            return (torch.randn(like.shape, generator=generator) * std).to(like.dtype)

        for layer in range(layers):
            base = f"model.layers.{layer}.block_sparse_moe"
            for new in range(self.num_new_experts):
                source = new % experts
                for w in ("w1", "w2", "w3"):
                    old = state[f"{base}.experts.{source}.{w}.weight"]
                    extra = noise(old, self.expert_init_std)
                    state[f"{base}.experts.{experts + new}.{w}.weight"] = old + extra if self.expert_init_method == InitMethod.from_existing else extra
            router = state[f"{base}.gate.weight"]
            assert router.shape == (experts, config["hidden_size"]), router.shape
            rows = router[torch.arange(self.num_new_experts) % experts].clone()
            extra = noise(rows, self.router_init_std)
            rows = rows + extra if self.router_init_method == InitMethod.from_existing else extra
            state[f"{base}.gate.weight"] = torch.cat([router, rows], 0)
        config["num_local_experts"] = experts + self.num_new_experts
        save_hf_state(self.output_dir, self.hf_checkpoint, config, state, self.to_dict())
        logger.info(f"Wrote {self.output_dir}: {experts} -> {experts + self.num_new_experts} experts per layer")


@config_class(dynamic_type={RunnableConfig: "transformer_add_mtp_heads", CheckpointSurgeryConfig: "add_mtp_heads"})
class AddPredictionHeadsConfig(CheckpointSurgeryConfig):
    _abstract: typing.ClassVar[bool] = False
    num_prediction_heads: int = Field(default=2, desc="Total prediction heads (the original model counts as the first).", hint=FieldHint.core)
    prediction_head_init_std: float = Field(default=0.0, desc="Noise added to the copied layers.", hint=FieldHint.core)

    def run(self) -> None:
        config, state = load_hf_state(self.hf_checkpoint)
        if config.get("model_type") not in ("llama", "mistral", "apriel"):
            raise ValueError(f"Model type {config.get('model_type')} is not supported")
        if config.get("model_type") == "mistral" and config.get("sliding_window") is not None:
            raise ValueError("mtp_llama has no sliding window: the source must not use one")
        generator = torch.Generator().manual_seed(self.seed)
        last = f"model.layers.{config['num_hidden_layers'] - 1}."
        last_keys = [k for k in state if k.startswith(last)]
        for head in range(self.num_prediction_heads - 1):
            for key in last_keys:
                tensor = state[key].clone()
                if self.prediction_head_init_std > 0 and tensor.dim() > 1:
                    tensor = tensor + (torch.randn(tensor.shape, generator=generator) * self.prediction_head_init_std).to(tensor.dtype)
                state[f"model.mtp_heads.{head}.{key[len(last):]}"] = tensor
        norm = state.pop("model.norm.weight")
        for head in range(self.num_prediction_heads):
            state[f"model.mtp_norms.{head}.weight"] = norm.clone()
        config.update(model_type="mtp_llama", architectures=["MTPLlamaForCausalLM"], prediction_heads=self.num_prediction_heads,
                      auto_map={"AutoConfig": "configuration_mtp_llama.MTPLlamaConfig", "AutoModel": "modeling_mtp_llama.MTPLlamaModel",
                                "AutoModelForCausalLM": "modeling_mtp_llama.MTPLlamaForCausalLM"})
        config.setdefault("mlp_bias", False)
        save_hf_state(self.output_dir, self.hf_checkpoint, config, state, self.to_dict())
        logger.info(f"Wrote {self.output_dir} with {self.num_prediction_heads} prediction heads")


if __name__ == "__main__":
    CheckpointSurgeryConfig.parse_and_run()
