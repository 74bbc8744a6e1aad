"""Configuration of Apriel2: a decoder whose blocks name their mixer by type; the multimodal variant adds a vision encoder.

Stand-alone file: it is copied next to exported checkpoints and loaded by `transformers` with `trust_remote_code`.

    decoder  {"type": "fixed", "num_blocks": n, "block": BLOCK} or
             {"type": "pattern", "num_blocks": n, "pattern": [names...], "blocks": {name: BLOCK}}
    BLOCK    {"mixer": MIXER, "mlp": {"type": "mlp", "intermediate_size", "gated", "activation", "add_linear_biases"},
              "normalization": {"type": "rms_norm", "epsilon"}}
    MIXER    {"type": "attention" | "mamba" | "gdn" | "kda" | "stochastic", ...}

`Apriel2Config` (model type `apriel2`) adds `image_token_index` and
    vision_encoder {"hidden_size", "embeddings": {"patch_height", "patch_width", "normalization"},
                    "encoder": {"type": "fixed", "num_blocks", "block": BLOCK (non-causal attention, `pixtral_2d` rotary)},
                    "adapter": {"type": "mlp", "intermediate_size", "activation", "add_linear_biases"}}
"""

from transformers import PretrainedConfig


class Apriel2TextConfig(PretrainedConfig):
    model_type = "apriel2_text"

    def __init__(self, hidden_size: int = 4096, vocab_size: int = 32000, decoder: dict | None = None, head: dict | None = None,
                 tie_word_embeddings: bool = False, initializer_range: float = 0.02, **kwargs):
        self.hidden_size = hidden_size
        self.initializer_range = initializer_range
        self.vocab_size = vocab_size
        self.decoder = decoder or {
            "type": "fixed", "num_blocks": 2,
            "block": {"mixer": {"type": "attention", "heads": 32, "head_groups": 8, "head_size": 128, "add_linear_biases": False,
                                "rotary": {"type": "mistral_1d", "theta": 10000.0}},
                      "mlp": {"type": "mlp", "intermediate_size": 14336, "gated": True, "activation": "silu", "add_linear_biases": False},
                      "normalization": {"type": "rms_norm", "epsilon": 1e-5}}}
        self.head = head or {"normalization": {"type": "rms_norm", "epsilon": 1e-5}}
        super().__init__(tie_word_embeddings=tie_word_embeddings, **kwargs)

    def get_text_config(self, *args, **kwargs):
        # `decoder` here is a plain dict describing the blocks, not a nested model configuration
        return self

    @property
    def num_hidden_layers(self) -> int:
        return self.decoder["num_blocks"]

    def block_configs(self) -> list[dict]:
        """One block description per layer, in order."""
        decoder = self.decoder
        if decoder.get("type", "fixed") == "fixed":
            return [decoder["block"]] * decoder["num_blocks"]
        pattern = decoder["pattern"]
        return [decoder["blocks"][pattern[i % len(pattern)]] for i in range(decoder["num_blocks"])]


class Apriel2Config(Apriel2TextConfig):
    model_type = "apriel2"

    def __init__(self, vision_encoder: dict | None = None, image_token_index: int | None = None, **kwargs):
        self.vision_encoder = vision_encoder
        self.image_token_index = image_token_index
        super().__init__(**kwargs)
