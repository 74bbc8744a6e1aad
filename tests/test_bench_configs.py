"""The benchmark's configurations build and validate on a machine without a GPU (the benchmark itself needs one)."""

import importlib.util
import pathlib
import sys

import pytest
import yaml

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("arguments,world,expect", [
    ([], 1, {"zero": 1, "tp": 1, "pp": 1, "depth": 32}),
    (["--gpus", "8"], 8, {"zero": 1, "tp": 1, "pp": 1, "depth": 4}),
    (["--gpus", "8", "--config", "llama3_8b_tp4"], 8, {"zero": 2, "tp": 4, "pp": 1, "depth": 4}),
    (["--gpus", "8", "--config", "mixtral_8x7b_z3"], 8, {"zero": 3, "tp": 1, "pp": 1, "depth": 4}),
    (["--gpus", "8", "--config", "llama3_70b_pp2_tp4", "--layers", "48"], 8, {"zero": 1, "tp": 4, "pp": 2, "breadth": 8}),
])
def test_benchmark_configurations_validate(arguments, world, expect, monkeypatch):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.models.gpt.trainer import GPTTrainerConfig

    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py", *arguments])
    args = bench.parse_args()
    base = yaml.safe_load((ROOT / "examples" / "mistral.yaml").read_text())
    updates = bench.config_updates(args, world)
    updates.update({("model", "distributed", "world_size"): world, ("model", "distributed", "rank"): 0,
                    ("model", "distributed", "local_world_size"): world, ("model", "distributed", "use_cuda"): False})
    config = GPTTrainerConfig.from_dict(base, updates)
    config.validate()
    distributed = config.model.distributed
    assert config.model.multi_stage.zero_stage == expect["zero"]
    assert (distributed.tensor_parallel, distributed.pipeline_parallel) == (expect["tp"], expect["pp"])
    if "depth" in expect:
        assert config.schedule.depth_first_micro_batches == expect["depth"]
    else:
        assert config.schedule.breadth_first_micro_batches == expect["breadth"]
    if "--layers" in arguments:
        assert config.model.base_model.decoder.num_blocks == 48
    # the line the driver parses: metric, config and parallelism strings exist for every configuration
    line = bench.result_line(args, world, 1000.0, {"sm_mhz": 1.0, "sm_max_mhz": 1.0, "reasons": []}, 1, None, "ours", {})
    assert line["n_gpus"] == world and line["value"] > 0 and line["config"]["parallelism"] and line["higher_is_better"] is True
