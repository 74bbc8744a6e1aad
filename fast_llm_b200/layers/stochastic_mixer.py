"""Stochastic mixer: each decoder layer owns several candidate mixers and runs ONE of them per training step (supernet
training).  Evaluation and export use the main mixer.

Sampling is reproducible and identical on every rank: a CPU generator seeded from (global seed, `seed_shift`, iteration)
is created when the micro-batch is preprocessed and consumed in layer order.  Strategies: `uniform` / `weighted` draw
independently per layer; `full_layout` draws a whole layer->mixer assignment in which every split of the layers between
mixers is equally likely; `predefined_layouts` are drawn first with their own probabilities.
Parity: `fast_llm/layers/decoder/config.py:133-260`, `fast_llm/layers/decoder/stochastic_mixer.py:27-292`.
"""

import enum
import logging

import torch

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.engine.base_model import LayerBase, LossDef
from fast_llm_b200.engine.parameter import combine_lr_scales
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.mixer import MixerConfig
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)

MAX_SEED = 2**31 - 1


class StochasticMixerSamplingStrategy(str, enum.Enum):
    uniform = "uniform"
    weighted = "weighted"
    full_layout = "full_layout"


class StochasticMixerKwargs:
    generator = "stochastic_mixer_generator"
    layout = "stochastic_mixer_layout"
    layout_counter = "stochastic_mixer_layout_counter"
    num_layers = "stochastic_mixer_num_layers"


def normalize_probabilities(values: list[float]) -> list[float]:
    Assert.custom(lambda v: all(x >= 0 for x in v), values)
    total = float(sum(values))
    Assert.gt(total, 0)
    return [v / total for v in values]


@config_class(dynamic_type={MixerConfig: "stochastic"})
class StochasticMixerConfig(MixerConfig):
    _abstract = False
    mixers: dict[str, MixerConfig] | None = Field(default=None, desc="Candidate mixers by name (at least one).", hint=FieldHint.architecture)
    sampling_strategy: StochasticMixerSamplingStrategy = Field(default=StochasticMixerSamplingStrategy.uniform, desc="How a mixer is drawn during training.", hint=FieldHint.feature)
    sampling_weights: dict[str, float] | None = Field(default=None, desc="Per-mixer probability for `weighted` (normalised).", hint=FieldHint.feature)
    main_mixer_name: str | None = Field(default=None, desc="Mixer used for evaluation, inference and export (default: the first).", hint=FieldHint.architecture)
    predefined_layouts: list[list[str]] = Field(default_factory=list, desc="Whole-model layouts (one mixer name per layer) to oversample.", hint=FieldHint.feature)
    predefined_layout_probabilities: list[float] = Field(default_factory=list, desc="Probability of each predefined layout; the rest goes to the strategy.", hint=FieldHint.feature)
    seed_shift: int = Field(default=200560490131, desc="Offset of the sampling seed.", hint=FieldHint.optional)

    def _validate(self):
        super()._validate()
        if not self.mixers:
            raise ValueError("A stochastic mixer needs at least one candidate in `mixers`")
        if self.main_mixer_name is None:
            with self._set_implicit_default():
                self.main_mixer_name = next(iter(self.mixers))
        if self.main_mixer_name not in self.mixers:
            raise ValueError(f"main_mixer_name '{self.main_mixer_name}' is not one of {list(self.mixers)}")
        if self.sampling_strategy == StochasticMixerSamplingStrategy.full_layout and self.sampling_weights is not None:
            raise ValueError("sampling_weights cannot be combined with the full_layout strategy")
        if self.sampling_weights is not None:
            Assert.eq(set(self.sampling_weights), set(self.mixers))
            with self._set_implicit_default():
                self.sampling_weights = dict(zip(self.sampling_weights, normalize_probabilities(list(self.sampling_weights.values()))))
        if self.predefined_layouts:
            Assert.eq(len(self.predefined_layouts), len(self.predefined_layout_probabilities))
            length = len(self.predefined_layouts[0])
            for layout, probability in zip(self.predefined_layouts, self.predefined_layout_probabilities):
                Assert.eq(len(layout), length)
                Assert.custom(lambda names: all(n in self.mixers for n in names), layout)
                Assert.in_range_incl(probability, 0, 1)
            Assert.leq(sum(self.predefined_layout_probabilities), 1 + 1e-6)
        else:
            Assert.eq(len(self.predefined_layout_probabilities), 0)

    @property
    def layer_class(self):
        return StochasticMixer


class LayerDict(LayerBase):
    """Named sub-layers (parameters appear as `<name>.<...>`)."""

    def __init__(self, layers: dict[str, LayerBase], distributed_config):
        super().__init__(None, distributed_config)
        for name, layer in layers.items():
            setattr(self, name, layer)

    def items(self):
        return self._sublayers.items()

    def values(self):
        return self._sublayers.values()

    def keys(self):
        return self._sublayers.keys()

    def __getitem__(self, name):
        return self._sublayers[name]

    def __len__(self):
        return len(self._sublayers)


class StochasticMixer(LayerBase):
    def __init__(self, config: StochasticMixerConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None, return_bias: bool = False):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self.mixers = LayerDict({name: mixer.get_layer(distributed_config, hidden_dim, lr_scale=self._lr_scale, peft=peft, return_bias=return_bias)
                                 for name, mixer in config.mixers.items()}, distributed_config)
        names = list(config.mixers)
        strategy = config.sampling_strategy
        if strategy == StochasticMixerSamplingStrategy.full_layout:
            self._probabilities = None
        elif strategy == StochasticMixerSamplingStrategy.uniform:
            self._probabilities = torch.full((len(names),), 1.0 / len(names))
        else:
            if config.sampling_weights is None:
                raise ValueError("The weighted strategy needs `sampling_weights`")
            self._probabilities = torch.tensor([config.sampling_weights[n] for n in names], dtype=torch.float32)
        self._layout_probabilities = (
            torch.tensor([*config.predefined_layout_probabilities, max(1.0 - sum(config.predefined_layout_probabilities), 0.0)], dtype=torch.float32)
            if config.predefined_layouts else None)
        # only the sampled mixer sees gradients in a given step
        for _, meta in self.mixers.named_parameter_metas():
            meta.allow_no_grad = True
        self.selection_counts = {name: 0 for name in names}
        self.last_selected = None

    # ---- sampling
    def sample_allocation(self, num_layers: int, generator: torch.Generator) -> list[int]:
        """Layers per mixer, every composition of `num_layers` into len(mixers) non-negative parts equally likely
        (stars and bars: choose the bar positions among num_layers + mixers - 1 slots)."""
        count = len(self.mixers)
        if count == 1:
            return [num_layers]
        bars = torch.randperm(num_layers + count - 1, generator=generator)[: count - 1].sort().values.tolist()
        edges = [-1, *bars, num_layers + count - 1]
        return [hi - lo - 1 for lo, hi in zip(edges[:-1], edges[1:])]

    def sample_layout(self, num_layers: int, generator: torch.Generator) -> list[str]:
        counts = self.sample_allocation(num_layers, generator)
        ordered = [name for name, n in zip(self.mixers.keys(), counts) for _ in range(n)]
        return [ordered[i] for i in torch.randperm(num_layers, generator=generator).tolist()]

    def preprocess(self, kwargs: dict) -> None:
        c = self._config
        kwargs[StochasticMixerKwargs.num_layers] = kwargs.get(StochasticMixerKwargs.num_layers, 0) + 1
        if StochasticMixerKwargs.generator not in kwargs:
            generator = torch.Generator(device="cpu")
            generator.manual_seed((self._distributed_config.seed + c.seed_shift + int(kwargs.get(BlockKwargs.iteration, 0))) % MAX_SEED)
            kwargs[StochasticMixerKwargs.generator] = generator
        for mixer in self.mixers.values():
            mixer.preprocess(kwargs)

    def _draw_layout(self, kwargs: dict) -> None:
        """First stochastic layer of the micro-batch decides whether a whole-model layout applies."""
        c = self._config
        kwargs[StochasticMixerKwargs.layout] = None
        generator = kwargs[StochasticMixerKwargs.generator]
        num_layers = kwargs[StochasticMixerKwargs.num_layers]
        layout = None
        if self._layout_probabilities is not None:
            Assert.eq(len(c.predefined_layouts[0]), num_layers)
            index = torch.multinomial(self._layout_probabilities, 1, generator=generator).item()
            if index < len(c.predefined_layouts):
                layout = c.predefined_layouts[index]
        if layout is None and c.sampling_strategy == StochasticMixerSamplingStrategy.full_layout:
            layout = self.sample_layout(num_layers, generator)
        kwargs[StochasticMixerKwargs.layout] = layout
        kwargs[StochasticMixerKwargs.layout_counter] = [0]

    def _sample_mixer_name(self, kwargs: dict) -> str:
        if not kwargs.get("training", True) or StochasticMixerKwargs.generator not in kwargs:
            return self._config.main_mixer_name
        if StochasticMixerKwargs.layout not in kwargs:
            self._draw_layout(kwargs)
        layout = kwargs[StochasticMixerKwargs.layout]
        if layout is not None:
            counter = kwargs[StochasticMixerKwargs.layout_counter]
            name = layout[counter[0] % len(layout)]
            counter[0] += 1
            return name
        index = torch.multinomial(self._probabilities, 1, generator=kwargs[StochasticMixerKwargs.generator]).item()
        return list(self.mixers.keys())[index]

    def forward(self, x: torch.Tensor, kwargs: dict, losses=None, metrics=None) -> torch.Tensor:
        name = self._sample_mixer_name(kwargs)
        if kwargs.get("training", True):
            self.selection_counts[name] += 1
            self.last_selected = name
            if metrics is not None:
                prefix = f"{self.module_name}/stochastic"
                total = sum(self.selection_counts.values())
                metrics[f"{prefix}/last_selected"] = name
                for n, count in self.selection_counts.items():
                    metrics[f"{prefix}/{n}_count_total"] = count
                    metrics[f"{prefix}/{n}_proportion_total"] = count / total
        return self.mixers[name].forward(x, kwargs, losses, metrics)

    def get_compute_usage(self, input_meta, kwargs=None, config=None) -> int:
        """Expected FLOPs under the sampling distribution."""
        c = self._config
        usages = {name: mixer.get_compute_usage(input_meta, kwargs, config) for name, mixer in self.mixers.items()}
        if self._probabilities is not None:
            expected = sum(u * p for u, p in zip(usages.values(), self._probabilities.tolist()))
        else:
            expected = sum(usages.values()) / len(usages)
        if c.predefined_layouts:
            fixed = sum(p * sum(usages[n] for n in layout) / len(layout) for p, layout in zip(c.predefined_layout_probabilities, c.predefined_layouts))
            expected = fixed + (1.0 - sum(c.predefined_layout_probabilities)) * expected
        return int(expected)

    def get_loss_definitions(self, count: int = 1) -> list[LossDef]:
        out = []
        for name, mixer in self.mixers.items():
            for definition in mixer.get_loss_definitions(count):
                out.append(LossDef(name=f"{name}/{definition.name}", formatted_name=f"{name} {definition.formatted_name}",
                                   count=definition.count, dtype=definition.dtype))
        return out
