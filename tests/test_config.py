import enum
import pathlib

import pytest
import yaml

from fast_llm_b200.config import Config, Field, FieldHint, FieldUpdate, FieldVerboseLevel, UpdateType, ValidationError, check_field, config_class
from fast_llm_b200.utils import Assert


class Color(str, enum.Enum):
    red = "red"
    blue = "blue"


@config_class(registry=True)
class ShapeConfig(Config):
    _abstract = True
    size: int = Field(default=1, hint=FieldHint.core, valid=check_field(Assert.gt, 0))

    @classmethod
    def _get_default_subclass(cls):
        return CircleConfig if cls is ShapeConfig else cls


@config_class(dynamic_type={ShapeConfig: "circle"})
class CircleConfig(ShapeConfig):
    _abstract = False
    radius: float = Field(default=2.0, hint=FieldHint.optional)
    color: Color = Field(default=Color.red, hint=FieldHint.feature)
    path: pathlib.Path | None = Field(default=None)


@config_class(dynamic_type={ShapeConfig: "square"})
class SquareConfig(ShapeConfig):
    _abstract = False
    size = FieldUpdate(default=4)
    side: float = Field(default=1.0)


@config_class()
class SceneConfig(Config):
    main: ShapeConfig = Field(hint=FieldHint.core)
    extras: dict[str, ShapeConfig] = Field(default_factory=dict)
    numbers: list[int] = Field(default_factory=list)
    pair: tuple[float, float] = Field(default=(0.0, 1.0))
    derived: int = Field(default=None, init=False, hint=FieldHint.derived)

    def _validate(self):
        self.derived = len(self.numbers)
        super()._validate()


def test_from_dict_dynamic_type_and_coercion():
    c = SceneConfig.from_dict({"main": {"type": "circle", "radius": 3, "color": "blue", "path": "/tmp/x"},
                               "extras": {"a": {"type": "square"}}, "numbers": [1, 2], "pair": [1, 2]}).validate()
    assert isinstance(c.main, CircleConfig) and c.main.radius == 3.0 and isinstance(c.main.radius, float)
    assert c.main.color is Color.blue and c.main.path == pathlib.Path("/tmp/x")
    assert isinstance(c.extras["a"], SquareConfig) and c.extras["a"].size == 4
    assert c.pair == (1.0, 2.0) and c.derived == 2


def test_defaults_and_default_subclass():
    c = SceneConfig().validate()
    assert isinstance(c.main, CircleConfig) and c.main.size == 1


def test_updates_override_and_merge():
    base = {"main": {"type": "circle", "radius": 3, "size": 2}}
    c = SceneConfig.from_dict(base, {("main", "radius"): 5, "numbers": [7]}).validate()
    assert c.main.radius == 5 and c.main.size == 2 and c.numbers == [7]
    c2 = SceneConfig.from_dict(base, {"main": {"size": 9}}, update_type=UpdateType.update).validate()
    assert c2.main.size == 9 and c2.main.radius == 3
    c3 = SceneConfig.from_dict(base, {"main": {"size": 9}}).validate()
    assert c3.main.radius == 2.0


def test_explicit_fields_round_trip():
    c = SceneConfig.from_dict({"main": {"type": "square", "side": 2.5}}).validate()
    d = c.to_dict()
    assert d == {"main": {"type": "square", "side": 2.5}}
    assert SceneConfig.from_dict(d).validate().to_dict(FieldVerboseLevel.everything) == c.to_dict(FieldVerboseLevel.everything)
    full = c.to_dict(FieldVerboseLevel.everything)
    assert full["main"]["size"] == 4 and "derived" not in full
    yaml.safe_dump(full)


def test_frozen_after_validation():
    c = SceneConfig().validate()
    with pytest.raises(RuntimeError):
        c.numbers = [1]
    with pytest.raises(RuntimeError):
        c.main.size = 3


@pytest.mark.parametrize("bad", [{"unknown": 1}, {"main": {"size": "a"}}, {"main": {"size": -1}}, {"main": {"type": "hexagon"}},
                                 {"numbers": [1.5]}, {"main": {"color": "green"}}, {"pair": [1]}])
def test_validation_errors(bad):
    with pytest.raises((ValidationError, KeyError)):
        SceneConfig.from_dict(bad).validate()


def test_derived_field_cannot_be_set():
    with pytest.raises((TypeError, ValidationError)):
        SceneConfig.from_dict({"derived": 3}).validate()


def test_compare():
    a = SceneConfig.from_dict({"numbers": [1]}).validate()
    b = SceneConfig.from_dict({"numbers": [2]}).validate()
    with pytest.raises(ValueError):
        a.compare(b)
    a.compare(SceneConfig.from_dict({"numbers": [1]}).validate())


def test_reference_example_configs_load():
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.models.gpt.trainer import GPTTrainerConfig

    root = pathlib.Path(__file__).resolve().parent.parent
    for name in ("mistral.yaml", "tiny_llama.yaml"):
        config = GPTTrainerConfig.from_dict(yaml.safe_load((root / "examples" / name).read_text())).validate()
        assert config.model.base_model.decoder.block.mlp.gated
    mistral = GPTTrainerConfig.from_dict(yaml.safe_load((root / "examples" / "mistral.yaml").read_text()),
                                         {("model", "distributed", "tensor_parallel"): 1}).validate()
    assert mistral.model.multi_stage.num_grad_buffers == 2
    assert mistral.model.base_model.decoder.block.mixer.window_size == 4096


def test_cli_validate_only(tmp_path):
    from fast_llm_b200.cli import fast_llm_main

    root = pathlib.Path(__file__).resolve().parent.parent
    config = fast_llm_main(["train", "gpt", "-v", "-c", str(root / "examples" / "tiny_llama.yaml"), "training.train_iters=3",
                            "model.base_model.decoder.block.mixer.heads=4"])
    assert config.training.train_iters == 3 and config.model.base_model.decoder.block.mixer.heads == 4


def test_hydra_style_composition_and_override_grammar(tmp_path):
    """`--hydra-path DIR --hydra-config NAME`: the base file's `defaults` list pulls in group files under their group's key, a
    group is re-selected on the command line, and the override grammar (`k=v` existing key, `+k=v` new key, `++k=v` either,
    `~k` delete) applies to the composed dictionary."""
    import yaml

    from fast_llm_b200.cli import fast_llm_main
    from fast_llm_b200.config.compose import apply_overrides, compose_config

    conf = tmp_path / "conf"
    (conf / "model").mkdir(parents=True)
    (conf / "data").mkdir()
    (conf / "base.yaml").write_text(yaml.safe_dump({"defaults": [{"model": "tiny"}, {"data": "random"}, "_self_"],
                                                    "training": {"train_iters": 2, "num_workers": 0}}))
    block = {"mixer": {"type": "attention", "heads": 4, "head_groups": 2, "head_size": 8}, "mlp": {"intermediate_size": 64}}
    distributed = {"compute_dtype": "float32", "use_cuda": False}
    (conf / "model/tiny.yaml").write_text(yaml.safe_dump({"base_model": {"hidden_size": 32, "decoder": {"num_blocks": 2, "block": block}}, "distributed": distributed}))
    (conf / "model/wide.yaml").write_text(yaml.safe_dump({"base_model": {"hidden_size": 64, "decoder": {"num_blocks": 1, "block": block}}, "distributed": distributed}))
    (conf / "data/random.yaml").write_text(yaml.safe_dump({"datasets": {"training": {"type": "random"}}, "micro_batch_size": 64}))

    composed, remaining = compose_config(conf, "base", {}, ["model=wide", "training.train_iters=3"])
    assert composed["model"]["base_model"]["hidden_size"] == 64 and composed["data"]["micro_batch_size"] == 64 and remaining == ["training.train_iters=3"]
    (conf / "optimizer").mkdir()
    with pytest.raises(ValueError):
        compose_config(conf, "base", {}, ["optimizer=adam"])  # a group that no defaults list mentions

    config = fast_llm_main(["train", "gpt", "-v", "--hydra-path", str(conf), "--hydra-config", "base", "model=wide", "training.train_iters=3",
                            "+optimizer.weight_decay=0.0", "~training.num_workers"])
    assert config.model.base_model.hidden_size == 64 and config.training.train_iters == 3 and config.optimizer.weight_decay == 0.0
    assert config.training.num_workers == 2  # deleted from the composed dictionary: the class default again

    data = {"a": {"b": 1}}
    assert apply_overrides(data, ["a.b=2", "+a.c=3", "++a.d.e=4", "~a.b"]) == {"a": {"c": 3, "d": {"e": 4}}}
    with pytest.raises(KeyError):
        apply_overrides({"a": {}}, ["a.x=1"])  # changing a key that does not exist needs `+`
    with pytest.raises(KeyError):
        apply_overrides({"a": {}}, ["~a.x"])
