"""Parallel layouts on CPU ranks (Gloo): every layout must reproduce the single-process run on the same global batch."""

import pytest
import torch

from tests.common import build_trainer, tiny_trainer_config, train_steps
from tests.distributed_utils import run_distributed

STEPS = 2


def _single(updates: dict, steps: int = STEPS):
    trainer, _ = build_trainer(tiny_trainer_config(updates))
    losses = train_steps(trainer, steps)
    weights = {n: t.clone() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    return losses, weights


def _rank_main(rank, world_size, updates, steps):
    updates = {**updates, ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo"}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    losses = train_steps(trainer, steps)
    # numpy arrays travel by value through the result queue (torch tensors would be shared-memory handles)
    weights = {n: t.clone().numpy() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    distributed.shutdown()
    return losses, weights


LAYOUTS = {
    "dp2": (2, {}, {("schedule", "depth_first_micro_batches"): 2}),
    "dp2_z2": (2, {("model", "multi_stage", "zero_stage"): 2}, {("schedule", "depth_first_micro_batches"): 2}),
    "dp2_z3": (2, {("model", "multi_stage", "zero_stage"): 3}, {("schedule", "depth_first_micro_batches"): 2}),
    "dp2_df2": (2, {("schedule", "depth_first_micro_batches"): 2}, {("schedule", "depth_first_micro_batches"): 4}),
    "tp2": (2, {("model", "distributed", "tensor_parallel"): 2}, {}),
    "stp2": (2, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True}, {}),
    "stp2_novp": (2, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True,
                      ("model", "base_model", "embeddings", "vocab_parallel"): False}, {}),
    "sdp2": (2, {("model", "distributed", "sequence_data_parallel"): 2}, {}),
    "pp2": (2, {("model", "distributed", "pipeline_parallel"): 2, ("schedule", "breadth_first_micro_batches"): 2},
            {("schedule", "breadth_first_micro_batches"): 2}),
    "pp2_tied": (2, {("model", "distributed", "pipeline_parallel"): 2, ("schedule", "breadth_first_micro_batches"): 2,
                     ("model", "base_model", "tied_embedding_weight"): True},
                 {("schedule", "breadth_first_micro_batches"): 2, ("model", "base_model", "tied_embedding_weight"): True}),
    "dp2_stp2": (4, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True},
                 {("schedule", "depth_first_micro_batches"): 2}),
    # combinations (the reference's `tests/utils/distributed_configs.py:212-463` runs the same families)
    "dp2_z2_df4": (2, {("model", "multi_stage", "zero_stage"): 2, ("schedule", "depth_first_micro_batches"): 4},
                   {("schedule", "depth_first_micro_batches"): 8}),
    "stp2_ce4": (2, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True,
                     ("model", "base_model", "head", "cross_entropy_splits"): 4},
                 {("model", "base_model", "head", "cross_entropy_splits"): 4}),
    "sdp2_stp2": (4, {("model", "distributed", "sequence_data_parallel"): 2, ("model", "distributed", "tensor_parallel"): 2,
                      ("model", "distributed", "sequence_tensor_parallel"): True}, {}),
    "pp2_ms4": (2, {("model", "distributed", "pipeline_parallel"): 2, ("schedule", "breadth_first_micro_batches"): 2,
                    ("schedule", "micro_batch_splits"): 4},
                {("schedule", "breadth_first_micro_batches"): 2, ("schedule", "micro_batch_splits"): 4}),
    "tp2_pp2": (4, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "pipeline_parallel"): 2,
                    ("schedule", "breadth_first_micro_batches"): 2}, {("schedule", "breadth_first_micro_batches"): 2}),
    "dp2_stp2_pp2": (8, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True,
                         ("model", "distributed", "pipeline_parallel"): 2, ("schedule", "breadth_first_micro_batches"): 2},
                     {("schedule", "breadth_first_micro_batches"): 2, ("schedule", "depth_first_micro_batches"): 2}),
}


@pytest.mark.parametrize("name", list(LAYOUTS))
def test_layout_matches_single_process(name):
    world_size, parallel_updates, single_updates = LAYOUTS[name]
    # reproducible_init makes the initial weights independent of the layout
    common = {("model", "distributed", "reproducible_init"): True}
    ref_losses, ref_weights = _single({**common, **single_updates})
    results = run_distributed(_rank_main, world_size, {**common, **parallel_updates}, STEPS)
    for losses, weights in results:
        assert losses == pytest.approx(ref_losses, rel=2e-4), name
        for key, value in weights.items():
            # a copy of a tied weight on another pipeline rank is exported under its own name: compare with the owner
            reference = ref_weights[key if key in ref_weights else {"head.output_weights": "embeddings.word_embeddings_weight"}[key]]
            torch.testing.assert_close(torch.from_numpy(value), reference, rtol=2e-3, atol=2e-5, msg=lambda m: f"{name} {key}: {m}")


def _debug_rank(rank, world_size):
    import logging

    records = []

    class _Collect(logging.Handler):
        def emit(self, record):
            records.append(record.getMessage())

    logging.getLogger("fast_llm_b200").addHandler(_Collect())
    updates = {("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
               ("model", "distributed", "tensor_parallel"): 2, ("model", "multi_stage", "debug_tensor_parallel"): True,
               ("model", "multi_stage", "debug_activation_memory"): True}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    train_steps(trainer, 1)
    # make the ranks disagree on a replicated tensor: the check must notice
    from fast_llm_b200.parallel.collectives import check_parallel_match

    matched = check_parallel_match(torch.full((4,), float(rank)), distributed.tensor_group, "planted")
    distributed.shutdown()
    return [m for m in records if "MISMATCH" in m], any("fw: " in m for m in records), matched


def test_debug_hooks_check_replicated_tensors_and_log_memory():
    """`debug_tensor_parallel` compares every replicated layer output and gradient across the tensor group (silent when they
    agree, loud when they do not); `debug_activation_memory` logs the allocator after every layer."""
    results = run_distributed(_debug_rank, 2)
    for mismatches, logged_memory, planted_matched in results:
        assert mismatches == ["MISMATCH planted: 4 of 4 entries differ between ranks"]
        assert not planted_matched
    assert results[0][1], "rank 0 logs memory after every layer"


def _tensor_log_rank(rank, world_size, parallel_updates):
    from fast_llm_b200.utils.tensor_logs import TensorLogs

    updates = {("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
               ("model", "distributed", "reproducible_init"): True, ("model", "multi_stage", "debug_layer_outputs"): 2,
               ("model", "multi_stage", "debug_layer_gradients"): 2, **parallel_updates}
    config = tiny_trainer_config(updates)
    config.validate()
    from fast_llm_b200.parallel.distributed import Distributed

    distributed = Distributed(config.model.distributed)
    run = config.get_run(distributed)
    trainer = config.get_trainer_class()(config=config)
    with run:
        TensorLogs.reset(save=True, show=False)  # keep the records in memory (storing them as artifacts needs an experiment directory)
        trainer.setup(distributed, run)
        trainer._prepare_training_state()
        train_steps(trainer, 1)
        records = [{k: v for k, v in r.items() if k in ("name", "shape", "mu", "std", "min", "max")} for r in TensorLogs.get()]
    distributed.shutdown()
    return records


@pytest.mark.parametrize("name,world_size,updates", [
    ("tp2", 2, {("model", "distributed", "tensor_parallel"): 2}),
    ("stp2", 2, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True}),
])
def test_tensor_logs_of_a_parallel_layout_match_the_single_process_run(name, world_size, updates):
    """Every layer output and every gradient reaching it, reconstructed to the global tensor and logged once: the records of a
    tensor-parallel run (replicated activations) and of a sequence-parallel run (token shards gathered) must be those of the
    single-process run, name by name (the reference's way of comparing layouts: `tests/utils/compare_tensor_logs.py`)."""
    reference = run_distributed(_tensor_log_rank, 1, {})[0]
    records = run_distributed(_tensor_log_rank, world_size, updates)
    assert len(reference) >= 6
    assert records[1] == [], "only the first rank of the groups logs the global tensors"
    assert [r["name"] for r in records[0]] == [r["name"] for r in reference]
    for got, expected in zip(records[0], reference):
        assert got["shape"] == expected["shape"], got["name"]
        for key in ("mu", "std", "min", "max"):
            assert got[key] == pytest.approx(expected[key], rel=2e-4, abs=2e-6), (name, got["name"], key)


# ---- save in one layout, load in another (reference: `tests/utils/save_load_configs.py:76-157`, `tests/models/test_checkpoint.py`)
_SHARDS = ("weights", "exp_avgs", "exp_avgs_sq")
_CROSS_LAYOUTS = {
    "dp2": (2, {}),
    "tp2": (2, {("distributed", "tensor_parallel"): 2}),
    "stp2": (2, {("distributed", "tensor_parallel"): 2, ("distributed", "sequence_tensor_parallel"): True}),
    "pp2": (2, {("distributed", "pipeline_parallel"): 2}),
    "dp2_z3": (2, {("multi_stage", "zero_stage"): 3}),
}


def _global_state(model):
    return {f"{shard}/{name}": tensor.clone().numpy() for name, shard, tensor in model.get_state_tensor_iterator(_SHARDS)}


def _save_rank(rank, world_size, model_updates, path):
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig

    updates = {("model", *key): value for key, value in model_updates.items()}
    if ("model", "distributed", "pipeline_parallel") in updates:
        updates[("schedule", "breadth_first_micro_batches")] = 2
    updates.update({("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
                    ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
                    ("model", "distributed", "reproducible_init"): True})
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    train_steps(trainer, 2)  # two optimizer steps: both Adam moments are non-trivial
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="distributed", optimizer_state=True))
    state = _global_state(trainer.multi_stage)
    distributed.shutdown()
    return state


def _load_rank(rank, world_size, model_updates, path):
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.models.gpt.model import GPTModel

    updates = {("distributed", "tensor_parallel"): 1, ("distributed", "sequence_tensor_parallel"): False,
               ("distributed", "pipeline_parallel"): 1, ("multi_stage", "zero_stage"): 1, **model_updates,
               ("distributed", "world_size"): world_size, ("distributed", "rank"): rank, ("distributed", "local_world_size"): world_size,
               ("distributed", "backend"): "gloo", ("distributed", "use_cuda"): False}
    model = GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format="distributed", optimizer_state=True), updates, use_cpu=True)
    state = _global_state(model)
    model.distributed.shutdown()
    return state


@pytest.mark.parametrize("saved,loaded", [("dp2", "tp2"), ("tp2", "pp2"), ("stp2", "dp2_z3"), ("pp2", "stp2"), ("dp2_z3", "pp2")])
def test_checkpoint_saved_in_one_layout_loads_in_another(saved, loaded, tmp_path):
    """Weights and both Adam moments written by the ranks of one layout are read back bit for bit by the ranks of another
    (every rank's shard is assembled from the overlapping pieces of the saved shards)."""
    save_world, save_updates = _CROSS_LAYOUTS[saved]
    load_world, load_updates = _CROSS_LAYOUTS[loaded]
    path = str(tmp_path / "ckpt")
    written = {}
    for state in run_distributed(_save_rank, save_world, save_updates, path):
        written.update(state)
    assert any(k.startswith("exp_avgs_sq/") and v.any() for k, v in written.items())
    seen = set()
    for state in run_distributed(_load_rank, load_world, load_updates, path):
        for key, value in state.items():
            reference_key = key if key in written else key.replace("head.output_weights", "embeddings.word_embeddings_weight")
            assert (value == written[reference_key]).all(), f"{saved}->{loaded}: {key}"
            seen.add(reference_key)
    assert seen == set(written)


def _load_external_rank(rank, world_size, model_updates, path):
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.models.gpt.model import GPTModel

    updates = {**model_updates, ("distributed", "world_size"): world_size, ("distributed", "rank"): rank,
               ("distributed", "local_world_size"): world_size, ("distributed", "backend"): "gloo", ("distributed", "use_cuda"): False}
    model = GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format="llama"), updates, use_cpu=True)
    state = {name: tensor.clone().numpy() for name, _, tensor in model.get_state_tensor_iterator(("weights",))}
    model.distributed.shutdown()
    return state


@pytest.mark.parametrize("layout", ["tp2", "stp2", "pp2", "dp2_z3"])
def test_hugging_face_checkpoint_loads_in_every_layout(layout, tmp_path):
    """A Hugging Face checkpoint read by the ranks of a parallel layout: every rank fills its own shards from the global tensors
    (a pipeline rank reports nothing for the stages it does not hold, which the completeness check must accept), and together
    the ranks hold exactly the weights a single process reads."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.models.gpt.model import GPTModel

    trainer, _ = build_trainer(tiny_trainer_config())
    path = tmp_path / "hf"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="llama"))
    single = GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format="llama"), use_cpu=True)
    expected = {name: tensor.clone() for name, _, tensor in single.get_state_tensor_iterator(("weights",))}
    world, updates = _CROSS_LAYOUTS[layout]
    seen = set()
    for state in run_distributed(_load_external_rank, world, updates, str(path)):
        for name, value in state.items():
            torch.testing.assert_close(torch.from_numpy(value), expected[name], rtol=0, atol=0, msg=lambda m: f"{layout} {name}: {m}")
            seen.add(name)
    assert seen == set(expected)


def _multimodal_rank(rank, world_size, updates, steps):
    from tests.test_multimodal import _config

    updates = {**updates, ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
               ("model", "distributed", "reproducible_init"): True}
    trainer, distributed = build_trainer(_config(updates))
    losses = train_steps(trainer, steps)
    weights = {n: t.clone().numpy() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    distributed.shutdown()
    return losses, weights


_MULTIMODAL_LAYOUTS = {
    "tp2": (2, {("model", "distributed", "tensor_parallel"): 2}, {}),
    # 3 images of 1 x 3 patches: 9 patches, padded to 10 for the two sequence-parallel ranks
    "stp2_odd_patches": (2, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True,
                             ("data", "datasets", "training", "image_patch_grid"): [1, 3]},
                         {("data", "datasets", "training", "image_patch_grid"): [1, 3]}),
    "pp2": (2, {("model", "distributed", "pipeline_parallel"): 2, ("schedule", "breadth_first_micro_batches"): 2},
            {("schedule", "breadth_first_micro_batches"): 2}),
    "stp2_pp2": (4, {("model", "distributed", "tensor_parallel"): 2, ("model", "distributed", "sequence_tensor_parallel"): True,
                     ("model", "distributed", "pipeline_parallel"): 2, ("schedule", "breadth_first_micro_batches"): 2},
                 {("schedule", "breadth_first_micro_batches"): 2}),
}


@pytest.mark.parametrize("name", list(_MULTIMODAL_LAYOUTS))
def test_multimodal_layout_matches_single_process(name):
    """The vision encoder under the parallel layouts: with sequence parallelism the patch sequence is split over the tensor
    ranks (padded with blank patches to a multiple) and the embedding layer gathers the encoder outputs for its share of the
    tokens; with pipeline parallelism the activations sent between vision stages are `[patches, vision width]`, not
    `[tokens, hidden]`.  Losses and final weights equal the single-process run (the reference runs `llava` through the same
    layouts: `tests/utils/model_configs.py:690-703`)."""
    from tests.test_multimodal import _config

    world_size, parallel_updates, single_updates = _MULTIMODAL_LAYOUTS[name]
    common = {("model", "distributed", "reproducible_init"): True}
    trainer, _ = build_trainer(_config({**common, **single_updates}))
    reference_losses = train_steps(trainer, STEPS)
    reference_weights = {n: t.clone() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    results = run_distributed(_multimodal_rank, world_size, {**common, **parallel_updates}, STEPS)
    seen = set()
    for losses, weights in results:
        assert losses == pytest.approx(reference_losses, rel=2e-4), name
        for key, value in weights.items():
            # Adam divides by the root of the second moment: where a gradient is next to zero, a different summation order
            # moves the update by a fraction of the learning rate (1e-3); a wrong gradient would move it by all of it
            torch.testing.assert_close(torch.from_numpy(value), reference_weights[key], rtol=2e-3, atol=3e-4, msg=lambda m: f"{name} {key}: {m}")
            seen.add(key)
    assert seen == set(reference_weights)


def _tied_pipeline_rank(rank, world_size, path_out, path_in):
    """Train a model with tied embeddings on two pipeline ranks, export it as Llama; then load `path_in` (a Llama checkpoint)."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig

    updates = {("model", "base_model", "tied_embedding_weight"): True, ("model", "distributed", "pipeline_parallel"): 2,
               ("schedule", "breadth_first_micro_batches"): 2, ("model", "distributed", "world_size"): world_size,
               ("model", "distributed", "rank"): rank, ("model", "distributed", "local_world_size"): world_size,
               ("model", "distributed", "backend"): "gloo", ("model", "distributed", "reproducible_init"): True}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    train_steps(trainer, 1)
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path_out, format="llama"))
    trainer.multi_stage.load_checkpoint(CheckpointLoadConfig(path=path_in, format="llama"))
    state = {name: tensor.clone().numpy() for name, _, tensor in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    distributed.shutdown()
    return state


def test_tied_embeddings_across_pipeline_ranks_in_hugging_face_formats(tmp_path):
    """With the embedding table on the first pipeline rank and the output layer on the last, the last rank keeps a copy under the
    name `head.output_weights`.  A Hugging Face checkpoint holds the tensor once: the export writes the owner's only (and
    `transformers` ties it again), the import gives the same tensor to the owner and to the copy."""
    import safetensors.torch
    import transformers

    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig

    single, _ = build_trainer(tiny_trainer_config({("model", "base_model", "tied_embedding_weight"): True}))
    single.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "source", format="llama"))
    source = {}
    for file in (tmp_path / "source").glob("*.safetensors"):
        source.update(safetensors.torch.load_file(str(file)))
    assert "lm_head.weight" not in source
    states = run_distributed(_tied_pipeline_rank, 2, str(tmp_path / "exported"), str(tmp_path / "source"))
    exported = {}
    for file in (tmp_path / "exported").glob("*.safetensors"):
        exported.update(safetensors.torch.load_file(str(file)))
    assert sorted(exported) == sorted(source)
    hf = transformers.AutoModelForCausalLM.from_pretrained(tmp_path / "exported", dtype=torch.float32)
    assert hf.lm_head.weight.data_ptr() == hf.model.embed_tokens.weight.data_ptr()
    # after the import both holders have the checkpoint's embedding table
    embedding = source["model.embed_tokens.weight"].float()
    holders = {name: value for state in states for name, value in state.items() if name in ("embeddings.word_embeddings_weight", "head.output_weights")}
    assert set(holders) == {"embeddings.word_embeddings_weight", "head.output_weights"}
    for name, value in holders.items():
        torch.testing.assert_close(torch.from_numpy(value), embedding, rtol=0, atol=0, msg=lambda m: f"{name}: {m}")
