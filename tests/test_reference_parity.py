"""Trajectory parity with the reference implementation on CPU: the same YAML, the same memmap dataset file and the same initial
distributed checkpoint (both written by this framework, both read by the unmodified reference through its own CLI) must give
the same losses and gradient norms step after step.  Skipped when the reference tree is not present.

The reference's optimizer without apex (`fast_llm/core/kernels.py:74-91`) calls `torch.optim.adamw.adamw` with the step count
it has already advanced, and that function advances it once more, so its bias correction runs one step ahead of the rule its
apex path implements.  With `beta_1 = beta_2 = 0` the bias correction is 1 at every step and the two agree exactly; that
configuration carries the step-by-step comparison, the default betas are compared on the first step (identical forward,
backward and data) and loosely afterwards."""

import os
import pathlib
import re
import subprocess
import sys

import numpy as np
import pytest
import torch
import yaml

# the reference checkout: $FAST_LLM_REFERENCE, else a `reference` directory beside this repository
REFERENCE = pathlib.Path(os.environ.get("FAST_LLM_REFERENCE") or pathlib.Path(__file__).resolve().parents[2] / "reference")
pytestmark = pytest.mark.skipif(not (REFERENCE / "fast_llm" / "cli.py").exists(), reason="reference tree not present")

CONFIG = {
    "training": {"train_iters": 5, "num_workers": 0, "logs": {"interval": 1}, "checkpoint": {"interval": 5}},
    "data": {"datasets": {"training": {"type": "memmap", "path": None}}, "micro_batch_size": 128, "shuffle": "disabled", "seed": 0},
    "optimizer": {"learning_rate": {"base": 1.0e-3}, "weight_decay": 0.01},
    "model": {
        "base_model": {
            "embeddings": {"vocab_size": 512},
            "decoder": {"num_blocks": 2, "block": {
                "mixer": {"type": "attention", "rotary": {"type": "default"}, "heads": 4, "head_groups": 2, "head_size": 16, "add_linear_biases": False},
                "mlp": {"intermediate_size": 128, "gated": True, "activation": "silu", "add_linear_biases": False},
                "normalization": {"type": "rms_norm"}}},
            "head": {"normalization": {"type": "rms_norm"}},
            "hidden_size": 64,
        },
        "distributed": {"compute_dtype": "float32", "use_cuda": False, "seed": 0},
    },
}


@pytest.fixture(scope="module")
def workspace(tmp_path_factory):
    """Dataset with documents shorter and longer than a sample (samples hold one document, several, and the middle of one),
    the YAML, and the initial checkpoint."""
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.data.document import LanguageModelDocument
    from fast_llm_b200.data.memmap import MemmapDataset
    from fast_llm_b200.models.gpt.trainer import GPTTrainerConfig
    from fast_llm_b200.parallel.distributed import Distributed

    root = tmp_path_factory.mktemp("parity")
    rng = np.random.RandomState(0)
    documents = [LanguageModelDocument(tokens=torch.from_numpy(rng.randint(0, 512, size=int(rng.randint(20, 300))).astype(np.int32)))
                 for _ in range(200)]
    data_path = root / "data" / "shard_0.fast_llm_dataset"
    data_path.parent.mkdir()
    MemmapDataset.write_dataset(data_path, documents)
    config = yaml.safe_load(yaml.safe_dump(CONFIG))
    config["data"]["datasets"]["training"]["path"] = str(data_path)
    (root / "config.yaml").write_text(yaml.safe_dump(config))
    trainer_config = GPTTrainerConfig.from_dict(config, {("run", "experiment_dir"): str(root / "init"), ("model", "distributed", "world_size"): 1,
                                                        ("model", "distributed", "rank"): 0, ("model", "distributed", "local_world_size"): 1})
    trainer_config.validate()
    distributed = Distributed(trainer_config.model.distributed)
    run = trainer_config.get_run(distributed)
    trainer = trainer_config.get_trainer_class()(config=trainer_config)
    with run:
        trainer.setup(distributed, run)
        trainer._prepare_training_state()
        trainer._save_checkpoint(trainer_config.training.checkpoint, {}, 0)
    return root


def _overrides(root, name, extra):
    return [f"run.experiment_dir={root / name}", f"pretrained.path={root / 'init' / 'checkpoint' / '0'}", "pretrained.format=distributed",
            "pretrained.model_weights=true", *extra]


def _trajectory(text: str, loss_name: str):
    losses = [float(x) for x in re.findall(rf"{loss_name}:? ([0-9.]+)", text)]
    norms = [float(x) for x in re.findall(r"grad norm:? ([0-9.]+)", text)]
    return losses, norms


def _run_ours(root, name, extra=()):
    repo = pathlib.Path(__file__).resolve().parent.parent
    out = subprocess.run([sys.executable, "-m", "fast_llm_b200.cli", "train", "gpt", "-c", str(root / "config.yaml"), *_overrides(root, name, extra)],
                         cwd=repo, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return _trajectory(out.stdout + out.stderr, "lm loss")


def _run_reference(root, name, extra=()):
    env = {**os.environ, "PYTHONPATH": str(REFERENCE), "TORCHDYNAMO_DISABLE": "1", "PYTHONHASHSEED": "0"}
    out = subprocess.run([sys.executable, "-m", "fast_llm.cli", "train", "gpt", "--config", str(root / "config.yaml"),
                          *_overrides(root, name, ["run.torch_dynamo_enable=false", "run.enable_triton_kernels=false", "model.distributed.backend=gloo",
                                                   "data.gpu=false", *extra])],
                         cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    return _trajectory(out.stdout + out.stderr, "lm_head_loss")


def test_same_trajectory_as_the_reference(workspace):
    betas = ["optimizer.beta_1=0", "optimizer.beta_2=0"]
    ours, reference = _run_ours(workspace, "ours", betas), _run_reference(workspace, "reference", betas)
    assert len(ours[0]) == len(reference[0]) == 5
    # five printed digits each
    assert ours[0] == pytest.approx(reference[0], abs=2e-5)
    assert ours[1] == pytest.approx(reference[1], abs=2e-4)
    # and the weights the two frameworks end with (both in the distributed checkpoint layout)
    from safetensors import safe_open

    def shard(path):
        with safe_open(path, "pt") as f:
            return f.get_tensor("weights_shard").float()

    mine = shard(workspace / "ours" / "checkpoint" / "5" / "rank_0.safetensors")
    theirs = shard(workspace / "reference" / "checkpoint" / "5" / "rank_0.safetensors")
    # with beta_2 = 0 the update of an element is lr * sign(g) unless |g| is of the order of epsilon: a few such elements differ
    close = (mine - theirs).abs() <= 1e-6
    assert close.float().mean().item() > 0.999
    assert (mine - theirs).abs().max().item() <= 2.5e-3


def test_default_betas_first_step_is_identical_and_the_rest_close(workspace):
    ours, reference = _run_ours(workspace, "ours_default"), _run_reference(workspace, "reference_default")
    assert ours[0][0] == pytest.approx(reference[0][0], abs=1e-5) and ours[1][0] == pytest.approx(reference[1][0], abs=1e-4)
    # later steps: the reference's no-apex optimizer is one step ahead in its bias correction (see the module docstring)
    assert ours[0] == pytest.approx(reference[0], rel=1e-2)


def _save_in_layout(rank, world_size, model_updates, path, hf_path):
    """Ranks of one layout train two steps and save a distributed checkpoint; rank 0 also exports Hugging Face tensors."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from tests.common import build_trainer, tiny_trainer_config, train_steps

    updates = {("model", *key): value for key, value in model_updates.items()}
    if ("model", "distributed", "pipeline_parallel") in updates:
        updates[("schedule", "breadth_first_micro_batches")] = 2
    updates.update({("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
                    ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
                    ("model", "distributed", "reproducible_init"): True})
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    train_steps(trainer, 2)
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="distributed"))
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=hf_path, format="llama"))
    distributed.shutdown()
    return True


@pytest.mark.parametrize("layout,updates", [
    ("tp2", {("distributed", "tensor_parallel"): 2}),
    ("pp2", {("distributed", "pipeline_parallel"): 2}),
    ("dp2_z3", {("multi_stage", "zero_stage"): 3}),
])
def test_the_reference_reads_checkpoints_written_by_two_ranks_of_this_framework(layout, updates, tmp_path):
    """A distributed checkpoint written by two ranks here (tensor-, pipeline- or data-parallel shards) is converted to
    Hugging Face tensors by the unmodified reference CLI in one process, i.e. through the reference's own cross-layout
    loader; the tensors equal this framework's own export of the same model bit for bit."""
    import safetensors

    from tests.distributed_utils import run_distributed

    path, ours = tmp_path / "distributed", tmp_path / "ours_hf"
    run_distributed(_save_in_layout, 2, updates, str(path), str(ours))
    theirs = tmp_path / "reference_hf"
    env = {**os.environ, "PYTHONPATH": str(REFERENCE), "TORCHDYNAMO_DISABLE": "1", "PYTHONHASHSEED": "0"}
    out = subprocess.run([sys.executable, "-m", "fast_llm.cli", "convert", "gpt", f"input.path={path}", "input.format=distributed",
                          f"output.path={theirs}", "output.format=llama", "use_cpu=true"],
                         cwd=tmp_path, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, "\n".join(line for line in (out.stdout + out.stderr).splitlines() if "Warning" not in line and "warnings.warn" not in line)[-3000:]

    def tensors(directory):
        found = {}
        for file in sorted(pathlib.Path(directory).glob("*.safetensors")):
            with safetensors.safe_open(str(file), framework="pt") as f:
                for key in f.keys():
                    found[key] = f.get_tensor(key)
        return found

    a, b = tensors(ours), tensors(theirs)
    assert set(a) == set(b) and len(a) > 10
    for key in a:
        assert torch.equal(a[key].float(), b[key].float()), f"{layout}: {key}"
