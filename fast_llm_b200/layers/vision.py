"""Vision encoder for multimodal models: patch embeddings -> non-causal encoder blocks (2-D rotary) -> adapter MLP.

Image patches travel as `kwargs[namespace]["patches"]` ([patches, channels, height, width], already normalised) with
their (row, column) coordinates; the encoder's attention is variable-length over images (`cu_seqlens` in the same
namespace).  The adapter output is handed to the language model's embedding layer, which adds it at the token positions
given by `embedding_map`.
Parity: `fast_llm/layers/vision/config.py:22-112`, `embeddings.py:15-75`, `vision_encoder.py:18-135`.
"""

import torch

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import Layer, LayerWithNamespace
from fast_llm_b200.engine.initialization import init_normal_
from fast_llm_b200.engine.parameter import combine_lr_scales
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.linear import AffineLinearConfig
from fast_llm_b200.layers.mixer import BlockConfig, MLPBaseConfig
from fast_llm_b200.layers.normalization import NormalizationConfig
from fast_llm_b200.tensor import TensorDim
from fast_llm_b200.utils import Assert


class VisionKwargs(BlockKwargs):
    patches = "patches"
    patch_positions = "patch_positions"


@config_class()
class ImageNormalizationConfig(Config):
    """Pixel preprocessing: `(pixel / rescale_factor - mean) / std` per channel."""

    mean_r: float = Field(default=0.48145466, desc="Mean of the red channel.", hint=FieldHint.optional)
    mean_g: float = Field(default=0.4578275, desc="Mean of the green channel.", hint=FieldHint.optional)
    mean_b: float = Field(default=0.40821073, desc="Mean of the blue channel.", hint=FieldHint.optional)
    std_r: float = Field(default=0.26862954, desc="Standard deviation of the red channel.", hint=FieldHint.optional)
    std_g: float = Field(default=0.26130258, desc="Standard deviation of the green channel.", hint=FieldHint.optional)
    std_b: float = Field(default=0.27577711, desc="Standard deviation of the blue channel.", hint=FieldHint.optional)
    rescale_factor: float = Field(default=255.0, desc="Pixel values are divided by this first.", hint=FieldHint.optional)

    def normalize(self, patches: torch.Tensor) -> torch.Tensor:
        mean = torch.tensor([self.mean_r, self.mean_g, self.mean_b], dtype=torch.float32, device=patches.device).view(1, 3, 1, 1)
        std = torch.tensor([self.std_r, self.std_g, self.std_b], dtype=torch.float32, device=patches.device).view(1, 3, 1, 1)
        return (patches.float() / self.rescale_factor - mean) / std


@config_class()
class PatchEmbeddingsConfig(BlockConfig):
    _abstract = False
    patch_embeddings: AffineLinearConfig = Field(desc="Linear layer over the flattened patch.", hint=FieldHint.architecture)
    normalization: NormalizationConfig = Field(desc="Normalization after the projection.", hint=FieldHint.architecture)
    patch_height: int = Field(default=16, desc="Patch height in pixels.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    patch_width: int = Field(default=16, desc="Patch width in pixels.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    full_precision_residual: bool = Field(default=False, desc="Keep the residual stream in the optimisation dtype.", hint=FieldHint.stability)

    @property
    def input_channels(self) -> int:
        return 3

    def get_layer(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None):
        return PatchEmbeddings(self, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft)


class PatchEmbeddings(Layer):
    def __init__(self, config: PatchEmbeddingsConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        self._residual_dtype = (distributed_config.optimization_dtype if config.full_precision_residual else distributed_config.compute_dtype).torch
        patch_dim = TensorDim("patch", config.input_channels * config.patch_height * config.patch_width)
        self.patch_embeddings = config.patch_embeddings.get_layer(patch_dim, hidden_dim, default_weight_initialization=init_normal_(),
                                                                  default_bias_initialization=init_normal_(), default_add_bias=False,
                                                                  lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.normalization = config.normalization.get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)

    def get_preprocessing_config(self, phase=None) -> dict:
        c = self._config
        return {"patch_shape": (c.input_channels, c.patch_height, c.patch_width)}

    def forward(self, input_, kwargs, losses=None, metrics=None):
        patches = kwargs[VisionKwargs.patches]
        dc = self._distributed_config
        if dc.sequence_tensor_parallel and dc.tensor_parallel > 1:
            # the layers that follow hold their rank's share of the patch sequence (the batch was padded to a multiple)
            patches = patches.chunk(dc.tensor_parallel)[dc.tensor_rank]
        weight = self.patch_embeddings.weight
        flat = patches.flatten(1).to(weight.dtype if torch.is_tensor(weight) else patches.dtype)
        return self.normalization(self.patch_embeddings(flat)).to(self._residual_dtype)

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        c = self._config
        patches = kwargs.get(VisionKwargs.patches)
        count = 0 if patches is None else patches.shape[0]
        return 2 * count * c.input_channels * c.patch_height * c.patch_width * self._hidden_dim.global_size


class VisionAdapter(Layer):
    """The adapter MLP as a layer of its own (vision width -> language model width)."""

    def __init__(self, mlp, distributed_config):
        super().__init__(mlp._config, distributed_config)
        self.mlp = mlp

    def set_names(self, prefix: str = "") -> None:
        self.module_name = prefix.rstrip(".")
        self.mlp.set_names(prefix)

    def forward(self, input_, kwargs, losses=None, metrics=None):
        return self.mlp.forward(input_, {**kwargs, BlockKwargs.num_tokens: input_.shape[0]}, losses, metrics)

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        patches = kwargs.get(VisionKwargs.patches)
        return self.mlp.get_compute_usage(input_meta, {**kwargs, BlockKwargs.num_tokens: 0 if patches is None else patches.shape[0]}, config)


@config_class(registry=True)
class VisionEncoderConfig(BlockConfig):
    _abstract = False
    embeddings: PatchEmbeddingsConfig = Field(desc="Patch embeddings.", hint=FieldHint.architecture)
    encoder: "BlockSequenceConfig" = Field(desc="Encoder blocks (non-causal attention with 2-D rotary).", hint=FieldHint.architecture)
    adapter: MLPBaseConfig = Field(desc="Adapter MLP into the language model's hidden size.", hint=FieldHint.architecture)
    normalization: ImageNormalizationConfig = Field(desc="Pixel normalisation applied while preprocessing a batch.", hint=FieldHint.feature)
    hidden_size: int = Field(default=1024, desc="Hidden size of the encoder.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))

    @classmethod
    def _get_default_subclass(cls):
        return cls

    def get_layers(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None, namespace: str = "vision_encoder") -> list[Layer]:
        """[patch embeddings, encoder blocks..., adapter], each reading its kwargs from `kwargs[namespace]`."""
        lr_scale = combine_lr_scales(lr_scale, self.lr_scale)
        vision_dim = TensorDim("hidden", self.hidden_size)
        embeddings = self.embeddings.get_layer(distributed_config, vision_dim, lr_scale=lr_scale, peft=peft)
        blocks = self.encoder.get_layers(distributed_config, vision_dim, lr_scale=lr_scale, peft=peft)
        adapter = VisionAdapter(self.adapter.get_layer(distributed_config, vision_dim, lr_scale=lr_scale, peft=peft, output_dim=hidden_dim), distributed_config)
        embeddings.set_names(f"{namespace}.embeddings.")
        for i, block in enumerate(blocks):
            block.set_names(f"{namespace}.encoder.{i}.")
        adapter.set_names(f"{namespace}.adapter.")
        return [_Namespaced(layer, namespace) for layer in (embeddings, *blocks, adapter)]


from fast_llm_b200.layers.block import BlockSequenceConfig  # noqa: E402

VisionEncoderConfig.__annotations__["encoder"] = BlockSequenceConfig


class _Namespaced(LayerWithNamespace):
    """Namespace wrapper that keeps the wrapped layer's parameters, names and hooks visible to the engine."""

    def __init__(self, layer: Layer, namespace: str):
        super().__init__(layer, namespace)
        self.module_name = layer.module_name

    def set_names(self, prefix: str = "") -> None:
        pass

    def setup(self, distributed) -> None:
        self._distributed, self._is_setup = distributed, True
        if not self._layer._is_setup:
            self._layer.setup(distributed)

    def preprocess(self, kwargs: dict) -> None:
        if self._namespace in kwargs:
            self._layer.preprocess(kwargs[self._namespace])

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        return self._layer.get_compute_usage(input_meta, {**kwargs, **kwargs.get(self._namespace, {})}, config)
