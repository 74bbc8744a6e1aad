"""Configuration of the Apriel hybrid SSM model: Mistral fields plus a per-layer layout of mixer kinds.

Stand-alone file: it is copied next to exported checkpoints and loaded by `transformers` with `trust_remote_code`.
"""

from transformers.models.mistral.configuration_mistral import MistralConfig


class AprielHybridSSMConfig(MistralConfig):
    model_type = "apriel_ssm_thinker_hybrid"

    def __init__(self, hybrid_block_layout: list[str] | None = None, ssm_cfg: dict | None = None, linear_attn_config: dict | None = None, **kwargs):
        super().__init__(**kwargs)
        # "t": attention, "m2": Mamba, "gdn": gated DeltaNet
        self.hybrid_block_layout = hybrid_block_layout or ["t"] * self.num_hidden_layers
        self.ssm_cfg = ssm_cfg or {}
        self.linear_attn_config = linear_attn_config or {}
