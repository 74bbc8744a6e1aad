"""Shared helpers for tests: tiny model configs and trainers on CPU."""

import copy

TINY_BASE_MODEL = {
    "embeddings": {"vocab_size": 512},
    "decoder": {"num_blocks": 2, "block": {
        "mixer": {"type": "attention", "rotary": {"type": "default"}, "heads": 4, "head_groups": 2, "head_size": 16, "add_linear_biases": False},
        "mlp": {"intermediate_size": 128, "gated": True, "activation": "silu", "add_linear_biases": False},
        "normalization": {"type": "rms_norm"}}},
    "head": {"normalization": {"type": "rms_norm"}},
    "hidden_size": 64,
}


def tiny_trainer_config(updates: dict | None = None):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.models.gpt.trainer import GPTTrainerConfig

    config = {
        "training": {"train_iters": 4, "num_workers": 0, "logs": {"interval": 1}},
        "data": {"datasets": {"training": {"type": "random"}}, "micro_batch_size": 128, "seed": 0},
        "optimizer": {"learning_rate": {"base": 1e-3}, "weight_decay": 0.01},
        "model": {"base_model": copy.deepcopy(TINY_BASE_MODEL),
                  "distributed": {"compute_dtype": "float32", "use_cuda": False, "seed": 0, "world_size": 1, "rank": 0, "local_world_size": 1}},
    }
    return GPTTrainerConfig.from_dict(config, updates or {})


def build_trainer(config):
    from fast_llm_b200.parallel.distributed import Distributed

    config.validate()
    distributed = Distributed(config.model.distributed)
    run = config.get_run(distributed)
    trainer = config.get_trainer_class()(config=config)
    trainer.setup(distributed, run)
    trainer._prepare_training_state()
    return trainer, distributed


def train_steps(trainer, steps: int, start: int = 0):
    from fast_llm_b200.parallel.topology import PhaseType

    schedule = trainer._schedules[PhaseType.training]
    iterator = trainer._data.get_iterator("training", consumed_samples=start * schedule.samples_per_batch, num_workers=0)
    losses = []
    for i in range(steps):
        out, ok, _ = trainer.runner.run_step(iterator, schedule, iteration=start + i + 1)
        losses.append(out["lm_loss"])
    return losses
