"""The evaluation-harness adapter, without the harness: scores and generations against direct computation."""

import torch

from tests.common import build_trainer, tiny_trainer_config
from tests.test_preparation import tokenizer_path  # noqa: F401  (fixture)


def test_loglikelihood_and_generation(tokenizer_path):  # noqa: F811
    from fast_llm_b200.data.config import TokenizerConfig
    from fast_llm_b200.engine.evaluation.evaluators import FastLLMLmEvalWrapper
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    trainer, _ = build_trainer(tiny_trainer_config())
    model = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    tokenizer = TokenizerConfig.from_dict({"path": str(tokenizer_path)}).get_tokenizer()
    wrapper = FastLLMLmEvalWrapper(model, tokenizer, batch_size=2, max_new_tokens=5)
    requests = [("the quick brown", " fox jumps"), ("hello", " world"), ("pack my box with", " five"), ("", "hello world")]
    scores = wrapper.loglikelihood(requests)
    assert len(scores) == 4
    for (context, continuation), (score, greedy) in zip(requests, scores):
        context_tokens, continuation_tokens = wrapper._encode_pair(context, continuation)
        ids = torch.tensor([context_tokens + continuation_tokens])
        log_probs = torch.log_softmax(model(input_ids=ids).logits[0].float(), -1)
        n = len(continuation_tokens)
        expected = sum(log_probs[len(context_tokens) - 1 + i, t].item() for i, t in enumerate(continuation_tokens))
        assert abs(score - expected) < 1e-3, (context, continuation)
        assert isinstance(greedy, bool) and n > 0
    rolling = wrapper.loglikelihood_rolling([("the quick brown fox",)])
    tokens = wrapper.tok_encode("the quick brown fox")
    assert abs(rolling[0] - wrapper._score([([tokenizer.bod_id], tokens)])[0][0]) < 1e-4
    text = wrapper.generate_until([("the quick", {"until": ["\n"], "max_gen_toks": 4})])
    assert isinstance(text[0], str)


def test_evaluate_command(tmp_path, capsys):
    """`fast-llm evaluate gpt ...` runs the configured evaluators once without training."""
    from fast_llm_b200.cli import fast_llm_main

    args = ["evaluate", "gpt", "model.base_model.embeddings.vocab_size=512", "model.base_model.hidden_size=64",
            "model.base_model.decoder.num_blocks=1", "model.base_model.decoder.block.mixer.heads=4", "model.base_model.decoder.block.mixer.head_groups=2",
            "model.base_model.decoder.block.mixer.head_size=16", "model.base_model.decoder.block.mixer.rotary.type=default",
            "model.base_model.decoder.block.mlp.intermediate_size=128", "model.distributed.use_cuda=false", "model.distributed.compute_dtype=float32",
            "data.datasets.validation.type=random", "data.micro_batch_size=64", "training.evaluators.validation.iterations=2",
            "training.evaluators.validation.interval=1", "training.num_workers=0"]
    fast_llm_main(args)
    captured = capsys.readouterr()
    assert "validation @ validation" in captured.out + captured.err and "lm loss" in captured.out + captured.err


def test_batched_generation_matches_one_by_one_and_harness_arguments_parse(tokenizer_path):  # noqa: F811
    from fast_llm_b200.data.config import TokenizerConfig
    from fast_llm_b200.engine.evaluation.evaluators import FastLLMLmEvalWrapper, parse_harness_arguments
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    trainer, _ = build_trainer(tiny_trainer_config())
    model = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    tokenizer = TokenizerConfig.from_dict({"path": str(tokenizer_path)}).get_tokenizer()
    requests = [("the quick brown fox", {"until": ["\n"], "max_gen_toks": 4}), ("hello", {"until": ["\n"], "max_gen_toks": 4}),
                ("pack my box", {"max_gen_toks": 3}), ("a", {"until": "\n", "max_gen_toks": 4})]
    batched = FastLLMLmEvalWrapper(model, tokenizer, batch_size=3).generate_until(requests)
    single = FastLLMLmEvalWrapper(model, tokenizer, batch_size=1).generate_until(requests)
    # prompts of different lengths share a left-padded batch: padding must not change what is generated
    assert batched == single and all(isinstance(t, str) for t in batched)
    wrapper = FastLLMLmEvalWrapper(model, tokenizer, batch_size=2, max_length=64)
    ids, mask = wrapper.tok_batch_encode(["the quick brown fox", "hello"])
    assert ids.shape == mask.shape and mask[1].sum() < mask[0].sum() and mask[1, 0] == 0 and mask[0, 0] == 1
    assert wrapper.max_length == 64 and wrapper.prefix_token_id == tokenizer.bod_id
    rendered = wrapper.apply_chat_template([{"role": "user", "content": "hi"}])
    assert "hi" in rendered and rendered != "hi"  # the tokenizer's own template when it has one, else a plain "role: content" form

    parsed = parse_harness_arguments(["--tasks", "hellaswag,arc_easy", "--num_fewshot", "5", "--limit=0.25", "--apply_chat_template",
                                      "--gen_kwargs", "temperature=0,top_p=1", "bootstrap_iters=0", "--log-samples"])
    assert parsed == {"tasks": ["hellaswag", "arc_easy"], "num_fewshot": 5, "limit": 0.25, "apply_chat_template": True,
                      "gen_kwargs": {"temperature": 0, "top_p": 1}, "bootstrap_iters": 0, "log_samples": True}


def _replica_rank(rank, world_size, tokenizer_file):
    """Two data-parallel replicas of the same model share the harness' requests."""
    from fast_llm_b200.data.config import TokenizerConfig
    from fast_llm_b200.engine.evaluation.evaluators import FastLLMLmEvalWrapper
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    trainer, distributed = build_trainer(tiny_trainer_config({
        ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank, ("model", "distributed", "local_world_size"): world_size,
        ("model", "distributed", "backend"): "gloo", ("model", "distributed", "reproducible_init"): True}))
    model = HuggingfaceGPTModelForCausalLM(trainer._multi_stage)
    tokenizer = TokenizerConfig.from_dict({"path": tokenizer_file}).get_tokenizer()
    requests = [("the quick brown", " fox jumps"), ("hello", " world"), ("pack my box with", " five"), ("", "hello world"), ("a b c", " d")]
    prompts = [("the quick", {"max_gen_toks": 3}), ("hello there", {"max_gen_toks": 3}), ("pack", {"max_gen_toks": 3})]
    shared = FastLLMLmEvalWrapper(model, tokenizer, batch_size=2, data_group=distributed.batch_data_group)
    alone = FastLLMLmEvalWrapper(model, tokenizer, batch_size=2)
    counted = {"forwards": 0}
    original = model.forward

    def counting_forward(*args, **kwargs):
        counted["forwards"] += 1
        return original(*args, **kwargs)

    model.forward = counting_forward
    together = (shared.loglikelihood(requests), shared.loglikelihood_rolling([("the quick brown fox",), ("hello world",)]), shared.generate_until(prompts))
    shared_forwards = counted["forwards"]
    counted["forwards"] = 0
    separately = (alone.loglikelihood(requests), alone.loglikelihood_rolling([("the quick brown fox",), ("hello world",)]), alone.generate_until(prompts))
    alone_forwards = counted["forwards"]
    distributed.shutdown()
    return together, separately, shared_forwards, alone_forwards


def test_replicas_share_the_requests(tokenizer_path):  # noqa: F811
    from tests.distributed_utils import run_distributed

    results = run_distributed(_replica_rank, 2, str(tokenizer_path))
    for together, separately, shared_forwards, alone_forwards in results:
        for a, b in zip(together[0], separately[0]):
            assert abs(a[0] - b[0]) < 1e-4 and a[1] == b[1]
        assert all(abs(a - b) < 1e-4 for a, b in zip(together[1], separately[1]))
        assert together[2] == separately[2]
        assert shared_forwards < alone_forwards  # each replica ran only its share
    assert results[0][0] == results[1][0]
