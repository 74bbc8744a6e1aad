"""Configuration of Llava around an Apriel hybrid (attention / Mamba / gated DeltaNet) language model.

Stand-alone file: it is copied next to exported checkpoints, together with the language model's own two files, and loaded by
`transformers` with `trust_remote_code`.  Same role as `fast_llm_external_models/llava_hybrid/configuration_llava_hybrid.py`.
"""

from transformers.configuration_utils import PretrainedConfig
from transformers.models.auto import CONFIG_MAPPING

try:  # inside the package / next to an exported checkpoint
    from fast_llm_b200.external_models.apriel_hybrid_ssm.configuration_apriel_hybrid_ssm import AprielHybridSSMConfig
except ImportError:  # pragma: no cover - the flat directory of an exported checkpoint
    from .configuration_apriel_hybrid_ssm import AprielHybridSSMConfig


class LlavaHybridConfig(PretrainedConfig):
    model_type = "llava_hybrid"
    sub_configs = {"text_config": AprielHybridSSMConfig}

    def __init__(self, vision_config=None, text_config=None, image_token_index: int = 32000, projector_hidden_act: str = "gelu",
                 vision_feature_select_strategy: str = "full", vision_feature_layer: int = -1, multimodal_projector_bias: bool = True,
                 **kwargs):
        if vision_feature_select_strategy not in ("default", "full"):
            raise ValueError(f"vision_feature_select_strategy must be 'default' or 'full', got {vision_feature_select_strategy!r}")
        if isinstance(vision_config, dict):
            vision_config = CONFIG_MAPPING[vision_config.get("model_type", "pixtral")](**{k: v for k, v in vision_config.items() if k != "model_type"})
        elif vision_config is None:
            vision_config = CONFIG_MAPPING["pixtral"]()
        if isinstance(text_config, dict):
            text_config = AprielHybridSSMConfig(**{k: v for k, v in text_config.items() if k != "model_type"})
        elif text_config is None:
            text_config = AprielHybridSSMConfig()
        self.vision_config = vision_config
        self.text_config = text_config
        self.image_token_index = image_token_index
        self.projector_hidden_act = projector_hidden_act
        self.vision_feature_select_strategy = vision_feature_select_strategy
        self.vision_feature_layer = vision_feature_layer
        self.multimodal_projector_bias = multimodal_projector_bias
        super().__init__(**kwargs)

    def to_dict(self):
        out = super().to_dict()
        out["vision_config"] = self.vision_config.to_dict()
        out["text_config"] = self.text_config.to_dict()
        return out


__all__ = ["LlavaHybridConfig"]
