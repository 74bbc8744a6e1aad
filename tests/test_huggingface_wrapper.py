"""The Hugging Face wrapper: logits match the engine's own forward, left padding is inert, `generate` runs greedy decoding."""

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
