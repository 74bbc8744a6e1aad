"""Layer and model base classes.

A model is a flat list of `Layer`s (the unit of pipeline/stage splitting).  Layers declare their parameters as
`ParameterMeta`s; memory is bound later, either by a `Stage` (views into the flat ZeRO buffers) or by `materialize`
(stand-alone tensors, for unit tests and tools).  `forward(input, kwargs, losses, metrics)` matches the contract of
`fast_llm/engine/base_model/base_model.py:19-165`; the implementation does not build on `torch.nn.Module`.
"""

import abc
import dataclasses
import typing

import torch

from fast_llm_b200.config import Config, Field, FieldHint, config_class
from fast_llm_b200.engine.parameter import ModuleConfig
from fast_llm_b200.parallel.topology import DistributedConfig, PhaseType
from fast_llm_b200.tensor import ParameterMeta


class ReductionType(str):
    sum = "sum"
    average = "average"
    minimum = "minimum"
    maximum = "maximum"


@dataclasses.dataclass
class LossDef:
    """A named scalar a model reports; `count` micro-batch contributions are averaged, then reduced over ranks."""

    name: str
    formatted_name: str
    count: int = 1
    dtype: torch.dtype = torch.float32
    reduction: str = ReductionType.average

    def reduce(self, values: list[torch.Tensor], distributed) -> float | None:
        from fast_llm_b200.parallel.collectives import all_reduce

        if values:
            total = torch.stack([v.detach().to(self.dtype).reshape(()) for v in values]).sum()
            if self.reduction == ReductionType.average:
                total = total / self.count
        else:
            total = torch.zeros((), dtype=self.dtype, device=distributed.device)
        if self.reduction in (ReductionType.sum, ReductionType.average):
            op = torch.distributed.ReduceOp.SUM
        elif self.reduction == ReductionType.minimum:
            op = torch.distributed.ReduceOp.MIN
        else:
            op = torch.distributed.ReduceOp.MAX
        if distributed.data_group is not None:
            all_reduce(total, op=op, group=distributed.data_group)
            if self.reduction == ReductionType.average:
                total = total / distributed.config.data_parallel
        if distributed.pipeline_group is not None:
            all_reduce(total, op=op, group=distributed.pipeline_group)
        return total.item()


@config_class()
class BaseModelConfig(ModuleConfig):
    """Architecture of a model; `get_base_model` builds the layers."""

    def get_base_model(self, distributed_config: DistributedConfig) -> "BaseModel":
        raise NotImplementedError

    def compare_architecture(self, other: "BaseModelConfig", log_fn=ValueError):
        """Compare only the fields hinted as architecture (checkpoint compatibility)."""
        from fast_llm_b200.utils import compare_nested

        errors = compare_nested(architecture_dict(self), architecture_dict(other))
        if errors:
            message = "Architecture mismatch:\n  " + "\n  ".join(errors)
            if isinstance(log_fn, type) and issubclass(log_fn, BaseException):
                raise log_fn(message)
            return log_fn(message)
        return None


def architecture_dict(config: Config) -> dict:
    out = {}
    for name, field in config.fields().items():
        value = getattr(config, name)
        if isinstance(value, Config):
            sub = architecture_dict(value)
            if sub:
                out[name] = sub
        elif isinstance(value, dict) and any(isinstance(v, Config) for v in value.values()):
            out[name] = {k: architecture_dict(v) for k, v in value.items()}
        elif field.hint == FieldHint.architecture:
            from fast_llm_b200.config.core import _serialize

            out[name] = _serialize(value, None, True, True)
    return out


class LayerBase:
    """Owns parameter metas and sub-layers; knows nothing about how memory is provided."""

    def __init__(self, config: Config | None, distributed_config: DistributedConfig, *, lr_scale=None, peft=None):
        object.__setattr__(self, "_param_metas", {})
        object.__setattr__(self, "_sublayers", {})
        self._config = config
        self._distributed_config = distributed_config
        self._lr_scale = lr_scale
        self._peft = peft
        self._distributed = None
        self._is_setup = False
        self.module_name = ""

    # ---- registration through attribute assignment
    def __setattr__(self, key, value):
        if isinstance(value, ParameterMeta):
            self._param_metas[key] = value
            return
        if isinstance(value, LayerBase):
            self._sublayers[key] = value
        elif key in self._sublayers:
            del self._sublayers[key]
        object.__setattr__(self, key, value)

    def __getattr__(self, key):
        metas = self.__dict__.get("_param_metas")
        if metas is not None and key in metas:
            meta = metas[key]
            return meta.tensor if meta.tensor is not None else meta
        raise AttributeError(f"{type(self).__name__} has no attribute {key}")

    def parameter_meta(self, name: str) -> ParameterMeta:
        return self._param_metas[name]

    def named_parameter_metas(self, prefix: str = "") -> typing.Iterator[tuple[str, ParameterMeta]]:
        for name, meta in self._param_metas.items():
            yield prefix + name, meta
        for name, sub in self._sublayers.items():
            yield from sub.named_parameter_metas(f"{prefix}{name}.")

    def named_sublayers(self, prefix: str = "") -> typing.Iterator[tuple[str, "LayerBase"]]:
        yield prefix.rstrip("."), self
        for name, sub in self._sublayers.items():
            yield from sub.named_sublayers(f"{prefix}{name}.")

    def set_names(self, prefix: str = "") -> None:
        self.module_name = prefix.rstrip(".")
        for name, meta in self._param_metas.items():
            meta.tensor_name = prefix + name
        for name, sub in self._sublayers.items():
            sub.set_names(f"{prefix}{name}.")

    # ---- lifecycle
    def setup(self, distributed) -> None:
        assert not self._is_setup
        self._distributed = distributed
        self._is_setup = True
        for sub in self._sublayers.values():
            if not sub._is_setup:
                sub.setup(distributed)

    def materialize(self, distributed=None, device=None, dtype: torch.dtype | None = None, requires_grad: bool = True):
        """Stand-alone allocation + initialisation of every parameter (no stage, no ZeRO buffers)."""
        from fast_llm_b200.parallel.distributed import Distributed

        distributed = distributed or self._distributed or Distributed(self._distributed_config)
        if not self._is_setup:
            self.setup(distributed)
        device = device or distributed.device
        dtype = dtype or self._distributed_config.compute_dtype.torch
        for name, meta in self.named_parameter_metas():
            t = torch.empty(meta.shape, device=device, dtype=dtype)
            meta.init_parameter(t, distributed)
            t.requires_grad_(requires_grad and meta.requires_grad)
            meta.tensor = t
        return self

    def parameters(self) -> list[torch.Tensor]:
        return [m.tensor for _, m in self.named_parameter_metas() if m.tensor is not None]

    def get_layers(self) -> list["Layer"]:
        raise NotImplementedError

    def get_compute_usage(self, input_meta, kwargs: dict, config) -> int:
        """Forward FLOPs for one micro-batch described by kwargs (used for throughput accounting)."""
        return sum(sub.get_compute_usage(input_meta, kwargs, config) for sub in self._sublayers.values())

    def get_recompute_usage(self, kwargs: dict) -> int:
        """FLOPs of forward work that the backward pass repeats instead of keeping its result (activation recomputation):
        the difference between the FLOPs the hardware executes and the model's."""
        return sum(sub.get_recompute_usage(kwargs) for sub in self._sublayers.values() if hasattr(sub, "get_recompute_usage"))

    def get_loss_definitions(self, count: int = 1) -> list[LossDef]:
        out = []
        for sub in self._sublayers.values():
            out += sub.get_loss_definitions(count)
        return out

    def get_preprocessing_config(self, phase: PhaseType) -> dict:
        out = {}
        for sub in self._sublayers.values():
            out.update(sub.get_preprocessing_config(phase))
        return out

    def preprocess(self, kwargs: dict) -> None:
        for sub in self._sublayers.values():
            sub.preprocess(kwargs)

    def unwrap(self):
        return self


class Layer(LayerBase):
    """A unit of the model's layer list: `forward(input, kwargs, losses, metrics) -> output`."""

    layer_count: float = 1.0  # weight when splitting layers into stages

    def get_layers(self) -> list["Layer"]:
        return [self]

    @abc.abstractmethod
    def forward(self, input_: torch.Tensor, kwargs: dict, losses: dict | None = None, metrics: dict | None = None) -> torch.Tensor:
        pass

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)


class LayerWithNamespace(Layer):
    """Gives a wrapped layer its own kwargs namespace (e.g. the vision encoder inside a multimodal model)."""

    def __init__(self, layer: Layer, namespace: str | None = None):
        super().__init__(layer._config, layer._distributed_config)
        self._layer = layer
        self._namespace = namespace
        self.layer_count = layer.layer_count

    def forward(self, input_, kwargs, losses=None, metrics=None):
        if self._namespace is not None and self._namespace in kwargs:
            kwargs = {**kwargs, **kwargs[self._namespace]}
        return self._layer.forward(input_, kwargs, losses, metrics)

    def unwrap(self):
        return self._layer.unwrap()


class BaseModel(LayerBase):
    """Root of a model: a sequence of layers plus batch preprocessing and tied-parameter declarations."""

    def __init__(self, config: BaseModelConfig, distributed_config: DistributedConfig):
        super().__init__(config, distributed_config)
        self._reference_models = {}

    def get_layers(self) -> list[Layer]:
        raise NotImplementedError

    def preprocess_batch(self, batch, *, phase: PhaseType, iteration: int, metrics: dict | None = None, device=None):
        raise NotImplementedError

    def get_tied_parameters(self) -> dict[str, tuple[ParameterMeta, ...]]:
        """name -> metas that share one tensor (first is the owner)."""
        return {}

    def get_activation_shape(self, layer_index: int, kwargs: dict) -> tuple[int, int] | None:
        """Shape of the activation that enters layer `layer_index` on this rank, for pipeline transfers; None: the default
        `[tokens (/ tensor ranks with sequence parallelism), hidden]`."""
        return None

    def add_reference_model(self, name: str, inference_runner) -> None:
        assert name not in self._reference_models
        self._reference_models[name] = inference_runner
