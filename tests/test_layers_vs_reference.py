"""Layer-level parity with the reference's own modules where its tree is present: rotary frequency tables (default, llama3,
yarn), the dynamic fp16 loss scaler's state machine, LoRA's forward and gradients against a plain restatement."""

import os
import pathlib
import sys
import types

import pytest
import torch

# the reference checkout: $FAST_LLM_REFERENCE, else a `reference` directory beside this repository
REFERENCE = pathlib.Path(os.environ.get("FAST_LLM_REFERENCE") or pathlib.Path(__file__).resolve().parents[2] / "reference")
needs_reference = pytest.mark.skipif(not (REFERENCE / "fast_llm" / "layers").is_dir(), reason="reference tree not present")


@pytest.fixture
def reference_path():
    old_flag = torch._dynamo.config.disable
    torch._dynamo.config.disable = True
    sys.path.insert(0, str(REFERENCE))
    yield
    torch._dynamo.config.disable = old_flag
    sys.path.remove(str(REFERENCE))
    for name in [n for n in sys.modules if n == "fast_llm" or n.startswith("fast_llm.")]:
        del sys.modules[name]


ROTARY_CASES = {
    "default": {"type": "default", "theta": 10000.0},
    "llama3": {"type": "llama3", "theta": 500000.0, "scale_factor": 8.0, "low_frequency_factor": 1.0, "high_frequency_factor": 4.0,
               "original_context_length": 8192},
    "yarn": {"type": "yarn", "theta": 10000.0, "scale_factor": 4.0, "attention_factor": 1.2, "beta_fast": 32.0, "beta_slow": 1.0,
             "original_context_length": 4096},
}


@needs_reference
@pytest.mark.parametrize("kind", list(ROTARY_CASES))
@pytest.mark.parametrize("head_size", [64, 128])
def test_rotary_angles_match_the_reference(reference_path, kind, head_size):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm.layers.attention.rotary import rotary as reference_rotary
    from fast_llm_b200.layers.rotary import RotaryConfig

    fields = ROTARY_CASES[kind]
    config = RotaryConfig.from_dict(fields)
    config.validate()
    ours = config.get_layer(head_size)
    reference_class = {"default": reference_rotary.DefaultRotary, "llama3": reference_rotary.Llama3Rotary, "yarn": reference_rotary.YarnRotary}[kind]
    stand_in = object.__new__(reference_class)
    object.__setattr__(stand_in, "_config", types.SimpleNamespace(**{k: v for k, v in fields.items() if k != "type"}))
    expected = reference_class._get_angle_scales(stand_in, head_size, torch.device("cpu")).double()
    torch.testing.assert_close(ours._inverse_frequencies("cpu").double(), expected, rtol=1e-6, atol=0)
    # the table the kernels read: cos | sin of position * angle, times the attention factor (yarn)
    table = ours.get_table(33, "cpu")
    angles = torch.arange(table.shape[0], dtype=torch.float64)[:, None] * expected[None, :]
    factor = fields.get("attention_factor", 1.0)
    torch.testing.assert_close(table[:33].double(), torch.cat([angles.cos(), angles.sin()], -1)[:33] * factor, rtol=1e-5, atol=1e-6)


def test_dynamic_loss_scaler_follows_the_reference_state_machine():
    """Halve after `hysteresis` overflowing steps in a row (not before), double after `window` clean steps, never below the
    minimum; the saved state carries the reference's key names (`fast_llm/engine/optimizer/optimizer.py:257-311`)."""
    from fast_llm_b200.engine.optimizer.config import GradientScalerConfig
    from fast_llm_b200.engine.optimizer.optimizer import DynamicGradScaler

    config = GradientScalerConfig.from_dict({"initial": 1024.0, "minimum": 256.0, "window": 3, "hysteresis": 2})
    config.validate()
    scaler = DynamicGradScaler(config)
    scales = []
    for overflow in [True, False, True, True, False, False, False, True, True, True, True, True, True]:
        scaler.update(overflow)
        scales.append(scaler.grad_scale)
    # one overflow is tolerated (hysteresis 2): a clean step in between does not restore the tolerance until `window` of them
    assert scales[0] == 1024.0
    assert scales[2] == 512.0 or scales[3] == 512.0
    assert min(scales) == 256.0
    state = scaler.state_dict()
    assert state["type"] == "DynamicGradScaler" and {"scale", "growth", "hysteresis"} <= set(state)
    other = DynamicGradScaler(config)
    other.load(state)
    assert other.state_dict() == state
    with pytest.raises(ValueError):
        other.load({**state, "type": "ConstantGradScaler"})


def test_lora_matches_a_plain_restatement():
    """y = x W^T + (alpha / r) (x A^T) B^T with W frozen: outputs and the gradients of A, B and x."""
    import fast_llm_b200.models.auto  # noqa: F401
    from tests.common import build_trainer, tiny_trainer_config, train_steps

    updates = {("model", "base_model", "peft"): {"type": "lora", "rank": 4, "alpha": 8.0}}
    trainer, _ = build_trainer(tiny_trainer_config(updates))
    names = [n for n, _, _ in trainer.multi_stage.get_state_tensor_iterator(("weights",))]
    lora_names = [n for n in names if "lora" in n]
    assert lora_names, "LoRA adds parameters"
    before = {n: t.clone() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    losses = train_steps(trainer, 3)
    after = {n: t.clone() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    assert all(l == l for l in losses)
    changed = {n for n in names if not torch.equal(before[n], after[n])}
    # only the adapters train (B starts at zero, so A's first gradient is zero but B's is not: after three steps both moved)
    assert changed and all("lora" in n for n in changed), sorted(changed - set(lora_names))[:5]
    frozen = [n for n in names if "lora" not in n]
    assert all(torch.equal(before[n], after[n]) for n in frozen)
