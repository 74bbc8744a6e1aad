"""State-space / linear-attention mixers: chunked scans against token-by-token restatements, and hybrid models training."""

import copy

import pytest
import torch

from tests.common import TINY_BASE_MODEL, build_trainer, tiny_trainer_config, train_steps


def _grads(fn, inputs, weight):
    out = fn(*inputs)
    return out, torch.autograd.grad((out * weight).sum(), [i for i in inputs if torch.is_tensor(i) and i.requires_grad])


@pytest.mark.parametrize("chunk", [4, 16])
def test_selective_scan_matches_sequential(chunk):
    from fast_llm_b200.ops.ssm import selective_scan, selective_scan_reference

    torch.manual_seed(0)
    tokens, channels, state, groups = 50, 12, 4, 3
    x, dt, z = (torch.randn(tokens, channels, requires_grad=True) for _ in range(3))
    a = (-torch.rand(channels, state) * 4).requires_grad_()
    b = torch.randn(tokens, groups, state, requires_grad=True)
    c = torch.randn(tokens, channels // 2, state, requires_grad=True)
    skip, bias = torch.randn(channels, requires_grad=True), torch.randn(channels, requires_grad=True)
    cu = torch.tensor([0, 7, 30, 50])
    inputs = [x, dt, a, b, c, skip, z, bias]
    weight = torch.randn(tokens, channels)
    out, grads = _grads(lambda *t: selective_scan(*t, cu, chunk=chunk), inputs, weight)
    ref, ref_grads = _grads(lambda *t: selective_scan_reference(*t, cu), inputs, weight)
    torch.testing.assert_close(out, ref, atol=1e-4, rtol=1e-4)
    for g, r in zip(grads, ref_grads):
        torch.testing.assert_close(g, r, atol=5e-4, rtol=1e-3)


def test_selective_scan_strong_decay_is_finite():
    """Decays far beyond exp(-88) per chunk neither overflow nor lose the token's own write."""
    from fast_llm_b200.ops.ssm import selective_scan, selective_scan_reference

    torch.manual_seed(1)
    tokens, channels, state = 40, 4, 2
    x = torch.randn(tokens, channels)
    dt = torch.full((tokens, channels), 30.0)
    a = -torch.full((channels, state), 16.0)
    b, c = torch.randn(tokens, 1, state), torch.randn(tokens, 1, state)
    out = selective_scan(x, dt, a, b, c, torch.zeros(channels), chunk=16)
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out, selective_scan_reference(x, dt, a, b, c, torch.zeros(channels)), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("per_channel", [False, True])
def test_chunk_delta_rule_matches_recurrence(per_channel):
    from fast_llm_b200.ops.ssm import chunk_delta_rule, delta_rule_reference

    torch.manual_seed(0)
    tokens, heads, dk, dv = 50, 3, 8, 6
    q, k = (torch.randn(tokens, heads, dk, requires_grad=True) for _ in range(2))
    v = torch.randn(tokens, heads, dv, requires_grad=True)
    g = (-torch.rand(tokens, heads, dk) * 2 if per_channel else -torch.rand(tokens, heads) * 2).requires_grad_()
    beta = torch.rand(tokens, heads, requires_grad=True)
    cu = torch.tensor([0, 7, 30, 50])
    weight = torch.randn(tokens, heads, dv)
    out, grads = _grads(lambda *t: chunk_delta_rule(*t, cu, chunk=8), [q, k, v, g, beta], weight)
    ref, ref_grads = _grads(lambda *t: delta_rule_reference(*t, cu), [q, k, v, g, beta], weight)
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-4)
    for a, r in zip(grads, ref_grads):
        torch.testing.assert_close(a, r, atol=1e-5, rtol=1e-3)


def test_documents_do_not_share_state():
    from fast_llm_b200.ops.ssm import chunk_delta_rule

    torch.manual_seed(0)
    q, k, v = torch.randn(20, 2, 4), torch.randn(20, 2, 4), torch.randn(20, 2, 4)
    g, beta = -torch.rand(20, 2), torch.rand(20, 2)
    packed = chunk_delta_rule(q, k, v, g, beta, torch.tensor([0, 12, 20]), chunk=8)
    alone = chunk_delta_rule(q[12:], k[12:], v[12:], g[12:], beta[12:], None, chunk=8)
    torch.testing.assert_close(packed[12:], alone)


def test_mamba_initializers():
    from fast_llm_b200.layers.ssm import init_a_log_, init_dt_bias_

    generator = torch.Generator().manual_seed(0)
    bias = torch.empty(1000)
    init_dt_bias_(0.001, 0.1)(None, bias, generator)
    steps = torch.nn.functional.softplus(bias)
    assert steps.min() >= 0.001 - 1e-6 and steps.max() <= 0.1 + 1e-6
    a = torch.empty(6, 4)
    init_a_log_(4, 6)(None, a, generator)
    torch.testing.assert_close(a.exp(), torch.arange(1.0, 5.0).expand(6, 4))


MIXERS = {
    "mamba": {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False},
    "mamba_docs": {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "repeat_kv_before_conv": False,
                   "cross_document_attention": False},
    "gdn": {"type": "gdn", "value_heads": 4, "key_heads": 2, "key_head_dim": 8, "value_head_dim": 8},
    "kda": {"type": "kda", "heads": 4, "head_dim": 8},
}


@pytest.mark.parametrize("name", list(MIXERS))
def test_hybrid_model_trains(name):
    """A two-block pattern (attention block, SSM block) runs through the engine and its loss goes down."""
    base = copy.deepcopy(TINY_BASE_MODEL)
    attention_block = base["decoder"]["block"]
    ssm_block = copy.deepcopy(attention_block)
    ssm_block["mixer"] = MIXERS[name]
    base["decoder"] = {"type": "pattern", "blocks": {"t": attention_block, "m": ssm_block}, "pattern": ["t", "m"], "num_blocks": 2}
    config = tiny_trainer_config({("model", "base_model"): base, ("data", "micro_batch_size"): 64,
                                  ("optimizer", "learning_rate", "base"): 3e-3})
    trainer, _ = build_trainer(config)
    losses = train_steps(trainer, 6)
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0]


def _stochastic_config(**kwargs):
    base = copy.deepcopy(TINY_BASE_MODEL)
    attention = base["decoder"]["block"]["mixer"]
    base["decoder"]["block"]["mixer"] = {"type": "stochastic", "mixers": {"attention": attention, "gdn": MIXERS["gdn"]}, **kwargs}
    base["decoder"]["num_blocks"] = 4
    return tiny_trainer_config({("model", "base_model"): base, ("data", "micro_batch_size"): 64})


def _stochastic_layers(trainer):
    from fast_llm_b200.layers.stochastic_mixer import StochasticMixer

    return [layer for _, layer in trainer._multi_stage.base_model.named_sublayers() if isinstance(layer, StochasticMixer)]


@pytest.mark.parametrize("strategy", ["uniform", "full_layout"])
def test_stochastic_mixer_trains_and_samples(strategy):
    trainer, _ = build_trainer(_stochastic_config(sampling_strategy=strategy))
    losses = train_steps(trainer, 8)
    assert all(torch.isfinite(torch.tensor(losses)))
    layers = _stochastic_layers(trainer)
    assert len(layers) == 4
    totals = {"attention": 0, "gdn": 0}
    for layer in layers:
        assert sum(layer.selection_counts.values()) == 8
        for name, count in layer.selection_counts.items():
            totals[name] += count
    assert totals["attention"] > 0 and totals["gdn"] > 0


def test_stochastic_mixer_predefined_layout_and_eval():
    layout = ["gdn", "attention", "attention", "gdn"]
    trainer, _ = build_trainer(_stochastic_config(predefined_layouts=[layout], predefined_layout_probabilities=[1.0]))
    train_steps(trainer, 3)
    for layer, expected in zip(_stochastic_layers(trainer), layout):
        assert layer.selection_counts[expected] == 3
    # outside training the main mixer (the first one) runs
    layer = _stochastic_layers(trainer)[0]
    assert layer._sample_mixer_name({"training": False}) == "attention"


def test_stochastic_allocation_is_a_composition():
    trainer, _ = build_trainer(_stochastic_config(sampling_strategy="full_layout"))
    layer = _stochastic_layers(trainer)[0]
    generator = torch.Generator().manual_seed(0)
    seen = set()
    for _ in range(200):
        counts = layer.sample_allocation(4, generator)
        assert sum(counts) == 4 and all(c >= 0 for c in counts)
        seen.add(tuple(counts))
    assert seen == {(i, 4 - i) for i in range(5)}
