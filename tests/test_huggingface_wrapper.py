"""The Hugging Face wrapper: logits match the engine's own forward, left padding is inert, `generate` runs greedy decoding."""

import pytest
import torch

from tests.common import build_trainer, tiny_trainer_config


def _wrapped():
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    trainer, _ = build_trainer(tiny_trainer_config())
    return HuggingfaceGPTModelForCausalLM(trainer._multi_stage), trainer


def test_forward_matches_engine_and_ignores_left_padding():
    model, trainer = _wrapped()
    torch.manual_seed(0)
    ids = torch.randint(0, 512, (2, 12))
    out = model(input_ids=ids)
    assert out.logits.shape == (2, 12, 512)
    from fast_llm_b200.engine.inference.runner import InferenceRunner

    runner = InferenceRunner(trainer._multi_stage)
    runner.setup()
    for row in range(2):
        torch.testing.assert_close(out.logits[row], runner.forward_tokens(ids[row]), atol=1e-5, rtol=1e-5)
    # left padding: same logits on the real tokens
    padded = torch.cat([torch.zeros(2, 3, dtype=torch.long), ids], 1)
    mask = torch.cat([torch.zeros(2, 3, dtype=torch.long), torch.ones(2, 12, dtype=torch.long)], 1)
    out_padded = model(input_ids=padded, attention_mask=mask, output_hidden_states=True)
    torch.testing.assert_close(out_padded.logits[:, 3:], out.logits, atol=1e-5, rtol=1e-5)
    assert len(out_padded.hidden_states) == 2 and out_padded.hidden_states[0].shape == (2, 15, 64)


def test_generate_is_greedy_decoding():
    model, trainer = _wrapped()
    torch.manual_seed(1)
    prompt = torch.randint(0, 512, (1, 6))
    generated = model.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=4, do_sample=False, pad_token_id=0)
    assert generated.shape == (1, 10)
    expected = prompt.clone()
    for _ in range(4):
        logits = model(input_ids=expected).logits
        expected = torch.cat([expected, logits[:, -1].argmax(-1, keepdim=True)], 1)
    assert torch.equal(generated, expected)


def test_generation_with_the_key_value_cache_matches_generation_without():
    """An attention-only decoder keeps keys and values between steps: the prompt runs once, then one token per row per step,
    and the result equals re-running the prefix (left-padded batch, greedy and beam search)."""
    model, trainer = _wrapped()
    assert model.config.use_cache and model.generation_config.use_cache
    torch.manual_seed(2)
    prompt = torch.randint(1, 512, (3, 9))
    mask = torch.ones_like(prompt)
    mask[0, :4], mask[2, :1] = 0, 0  # rows of 5, 9 and 8 real tokens
    prompt = prompt * mask
    sizes = []
    runner = model._inference_runner
    original = runner.forward_rows
    runner.forward_rows = lambda tokens, cache, names=None: (sizes.append(tuple(tokens.shape)), original(tokens, cache, names))[1]
    cached = model.generate(prompt, attention_mask=mask, max_new_tokens=5, do_sample=False, pad_token_id=0)
    assert sizes == [(3, 9)] + [(3, 1)] * 4, sizes
    plain = model.generate(prompt, attention_mask=mask, max_new_tokens=5, do_sample=False, pad_token_id=0, use_cache=False)
    assert len(sizes) == 5  # the run without the cache went through the packed path
    assert torch.equal(cached, plain)
    beams = model.generate(prompt, attention_mask=mask, max_new_tokens=4, do_sample=False, num_beams=3, pad_token_id=0)
    beams_plain = model.generate(prompt, attention_mask=mask, max_new_tokens=4, do_sample=False, num_beams=3, pad_token_id=0, use_cache=False)
    assert torch.equal(beams, beams_plain)
    # logits of a cached step against the packed forward pass
    out = model(input_ids=prompt, attention_mask=mask, use_cache=True)
    step = model(input_ids=cached[:, 9:11], past_key_values=out.past_key_values)
    full = model(input_ids=cached[:, :11], attention_mask=torch.cat([mask, torch.ones(3, 2, dtype=mask.dtype)], 1))
    torch.testing.assert_close(step.logits, full.logits[:, 9:], atol=1e-5, rtol=1e-5)
    assert step.past_key_values.get_seq_length() == 11


def test_recurrent_decoders_generate_without_a_cache():
    import copy

    from tests.common import TINY_BASE_MODEL
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    base = copy.deepcopy(TINY_BASE_MODEL)
    block = base["decoder"]["block"]
    mamba = copy.deepcopy(block)
    mamba["mixer"] = {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False}
    base["decoder"] = {"type": "pattern", "blocks": {"t": block, "m": mamba}, "pattern": ["t", "m"], "num_blocks": 2}
    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base}))
    model = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    assert not model.config.use_cache
    prompt = torch.randint(1, 512, (1, 6))
    out = model.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=3, do_sample=False, pad_token_id=0)
    assert out.shape == (1, 9) and model(input_ids=prompt, use_cache=True).past_key_values is None


def _tensor_parallel_generation(rank, world_size, prompt, mask):
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    updates = {("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
               ("model", "distributed", "tensor_parallel"): world_size, ("model", "distributed", "reproducible_init"): True}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    model = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    out = None
    if rank == 0:
        prompt, mask = torch.from_numpy(prompt), torch.from_numpy(mask)
        cached = model.generate(prompt, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0)
        plain = model.generate(prompt, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0, use_cache=False)
        beams = model.generate(prompt, attention_mask=mask, max_new_tokens=3, do_sample=False, num_beams=2, pad_token_id=0)
        model.stop_workers()
        out = (cached.numpy(), plain.numpy(), beams.numpy())
    else:
        model.worker_forward()
    distributed.shutdown()
    return out


def test_tensor_parallel_workers_follow_cached_generation():
    """Two tensor-parallel ranks: the coordinator generates, the worker mirrors every pass and keeps its own heads' cache
    (beam search reorders both).  The result equals the single-process model with the same initial weights."""
    from tests.distributed_utils import run_distributed

    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    torch.manual_seed(3)
    prompt = torch.randint(1, 512, (2, 7))
    mask = torch.ones_like(prompt)
    mask[1, :2] = 0
    prompt = prompt * mask
    results = run_distributed(_tensor_parallel_generation, 2, prompt.numpy(), mask.numpy())
    cached, plain, beams = results[0]
    assert (cached == plain).all()
    trainer, _ = build_trainer(tiny_trainer_config({("model", "distributed", "reproducible_init"): True}))
    single = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    expected = single.generate(prompt, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0)
    assert (torch.from_numpy(cached) == expected).all()
    expected_beams = single.generate(prompt, attention_mask=mask, max_new_tokens=3, do_sample=False, num_beams=2, pad_token_id=0)
    assert (torch.from_numpy(beams) == expected_beams).all()


@pytest.mark.gpu
def test_cached_generation_on_the_gpu():
    """bf16 on the device: a cached step (a few query rows against the cached keys, through the tcgen05 attention kernel)
    gives the logits of the packed forward pass over the whole sequence, and `generate` runs with the cache."""
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM
    from fast_llm_b200.utils.device_errors import check_device_errors

    trainer, _ = build_trainer(tiny_trainer_config({("model", "distributed", "use_cuda"): True, ("model", "distributed", "compute_dtype"): "bf16"}))
    model = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    assert model.config.use_cache
    torch.manual_seed(4)
    prompt = torch.randint(1, 512, (3, 40), device="cuda")
    mask = torch.ones_like(prompt)
    mask[0, :7], mask[2, :1] = 0, 0
    prompt = prompt * mask
    more = torch.randint(1, 512, (3, 3), device="cuda")
    out = model(input_ids=prompt, attention_mask=mask, use_cache=True)
    first = model(input_ids=more[:, :1], past_key_values=out.past_key_values)
    second = model(input_ids=more[:, 1:], past_key_values=first.past_key_values)
    full = model(input_ids=torch.cat([prompt, more], 1), attention_mask=torch.cat([mask, torch.ones_like(more)], 1), use_cache=False)
    torch.cuda.synchronize()
    check_device_errors()
    assert second.past_key_values.get_seq_length() == 43
    cached = torch.cat([out.logits, first.logits, second.logits], 1).float()
    real = torch.cat([mask, torch.ones_like(more)], 1).bool()
    assert torch.isfinite(cached[real]).all()
    torch.testing.assert_close(cached[real], full.logits.float()[real], atol=0.06, rtol=0.05)
    generated = model.generate(prompt, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0)
    assert generated.shape == (3, 44)
