"""The static plan: step order, restore / reduce placement, early receives in a common transfer order, the stream-order
deadlock proof and the simulated timeline - on stub models, no process group needed.
Model of the cases: `tests/test_schedule.py`-style checks of `fast_llm/engine/schedule/schedule.py:264-371` in the reference."""

import types

import pytest

from fast_llm_b200.engine.schedule.config import ScheduleConfig, StepType
from fast_llm_b200.engine.schedule.schedule import Schedule
from fast_llm_b200.parallel.topology import DistributedConfig, PhaseType


def _schedule(pp, rank, stages, breadth=1, depth=1, splits=1, weight_buffers=None, grad_buffers=None, delay=0.0):
    multi_stage_config = types.SimpleNamespace(num_weight_buffers=weight_buffers, num_grad_buffers=grad_buffers, pipeline_delay=delay)
    local = {s: object() for s in range(stages) if s % pp == rank}
    multi_stage = types.SimpleNamespace(stages=[object()] * stages, stages_on_device=local,
                                        config=types.SimpleNamespace(multi_stage=multi_stage_config))
    config = ScheduleConfig.from_dict({"breadth_first_micro_batches": breadth, "depth_first_micro_batches": depth, "micro_batch_splits": splits})
    distributed = DistributedConfig.from_dict({"world_size": pp, "rank": rank, "local_world_size": pp, "pipeline_parallel": pp, "use_cuda": False})
    distributed.validate()
    return Schedule(multi_stage, config, distributed, PhaseType.training)


GRID = [(2, 2, 1, 1, 1), (2, 2, 4, 1, 1), (2, 4, 4, 1, 1), (2, 4, 2, 3, 1), (2, 4, 3, 2, 2), (4, 4, 8, 1, 1), (4, 8, 4, 2, 1), (4, 8, 8, 1, 2),
        (3, 6, 5, 1, 1), (8, 8, 8, 1, 1), (8, 16, 16, 1, 1)]


def _transfers(schedule, rank, peer):
    """Transfers between `rank` and `peer` in the order `rank` issues them: ("send" / "recv", key of the consuming step)."""
    consumers = {schedule._producer(s): (s.type_, *s.key) for s in schedule.global_steps if s.recv_from is not None}
    out = []
    for step in schedule._per_rank_steps()[rank]:
        for receiver in step.recv_launch:
            if receiver.recv_from == peer:
                out.append(("recv", (receiver.type_, *receiver.key)))
        if step.send_to == peer:
            out.append(("send", consumers[(step.type_, *step.key)]))
    return out


@pytest.mark.parametrize("pp,stages,breadth,depth,splits", GRID)
def test_both_sides_issue_the_transfers_of_a_pair_in_one_order(pp, stages, breadth, depth, splits):
    schedule = _schedule(pp, 0, stages, breadth, depth, splits)  # building it runs the deadlock proof for all ranks
    for a in range(pp):
        for b in range(a + 1, pp):
            mine, theirs = _transfers(schedule, a, b), _transfers(schedule, b, a)
            assert len(mine) == len(theirs)
            flipped = [("recv" if op == "send" else "send", key) for op, key in theirs]
            assert mine == flipped, f"ranks {a} and {b} disagree on the order of their transfers"
    # every rank derives the same placement
    for rank in range(1, min(pp, 3)):
        other = _schedule(pp, rank, stages, breadth, depth, splits)
        for r in range(pp):
            assert [[(x.type_, *x.key) for x in s.recv_launch] for s in schedule._per_rank_steps()[r]] == \
                   [[(x.type_, *x.key) for x in s.recv_launch] for s in other._per_rank_steps()[r]]


@pytest.mark.parametrize("pp,stages,breadth,depth,splits", GRID)
def test_receives_are_posted_no_later_than_their_use_and_each_exactly_once(pp, stages, breadth, depth, splits):
    for rank in range(pp):
        schedule = _schedule(pp, rank, stages, breadth, depth, splits)
        posted = {}
        for index, step in enumerate(schedule.steps):
            for receiver in step.recv_launch:
                assert (receiver.type_, *receiver.key) not in posted
                posted[(receiver.type_, *receiver.key)] = index
        for index, step in enumerate(schedule.steps):
            if step.recv_from is not None:
                assert posted[(step.type_, *step.key)] <= index
        assert len(posted) == sum(s.recv_from is not None for s in schedule.steps)


def test_a_receive_in_front_of_a_needed_send_is_reported_as_a_deadlock():
    schedule = _schedule(2, 0, 4, breadth=2)
    # post rank 0's first receive before its second send: rank 1 will not send before it has received that
    steps = schedule._per_rank_steps()[0]
    receiver = next(s for s in steps if s.recv_from is not None)
    for s in steps:
        if receiver in s.recv_launch:
            s.recv_launch.remove(receiver)
    steps[1].recv_launch.insert(0, receiver)
    assert schedule._find_deadlock()
    with pytest.raises(RuntimeError, match="deadlock"):
        schedule._validate_send_recv()


def test_weight_gathers_are_issued_one_step_ahead():
    schedule = _schedule(1, 0, 4, breadth=2, weight_buffers=2)  # shared buffers: a gather per run of steps on a stage
    launched = {}
    for index, step in enumerate(schedule.steps):
        for target in step.restore_launch:
            launched[target.local_index] = index
    for index, step in enumerate(schedule.steps):
        if step.restore:
            assert launched[index] == max(index - 1, 0)
        else:
            assert index not in launched
    # first forward and first backward of a stage restore; the second micro-batch on the same stage does not
    restores = [(s.type_, s.stage, s.data_index) for s in schedule.steps if s.restore]
    assert (StepType.forward, 1, 0) in restores and (StepType.forward, 1, 1) not in restores


def test_simulated_timeline_gives_the_pipeline_bubble():
    # two stages on two ranks, b micro-batches: forward 1, backward 2 time units per stage and micro-batch;
    # rank 0 idles while rank 1 finishes its forwards and first backward: 3 b busy out of 3 b + 3
    for b in (1, 4, 16):
        schedule = _schedule(2, 0, 2, breadth=b)
        assert schedule._simulated_time == pytest.approx(3 * b + 3)
        assert schedule.simulated_idle_fraction == pytest.approx(3 / (3 * b + 3))
    # a communication delay stretches the critical path by one delay per hop (forward and backward)
    delayed = _schedule(2, 0, 2, breadth=4, delay=0.5)
    assert delayed._simulated_time == pytest.approx(3 * 4 + 3 + 2 * 0.5)


def test_schedule_profiler_writes_a_table_per_step(tmp_path):
    import yaml

    from tests.common import tiny_trainer_config
    from fast_llm_b200.parallel.distributed import Distributed

    config = tiny_trainer_config({("run", "experiment_dir"): str(tmp_path), ("training", "train_iters"): 2, ("schedule", "profile_schedule"): True,
                                  ("schedule", "depth_first_micro_batches"): 2})
    config.validate()
    distributed = Distributed(config.model.distributed)
    run = config.get_run(distributed)
    trainer = config.get_trainer_class()(config=config)
    with run:
        trainer.setup(distributed, run)
        trainer.run()
    files = sorted(tmp_path.glob("runs/*/artifacts/0/schedule_profile_rank_0_training_step_*.yaml"))
    assert len(files) == 2
    table = yaml.safe_load(files[-1].read_text())
    types_seen = {e["event_type"] for e in table["events"]}
    assert {"run", "restore", "reduce", "optimizer", "get_batch"} <= types_seen
    runs = [e for e in table["events"] if e["event_type"] == "run"]
    assert len(runs) == 2 * 2 * 4  # forward + backward, two micro-batches, four stages
    summary = table["summary"]
    assert summary["step_ms"] > 0 and summary["busy_ms_by_stream"]["compute"] > 0
    assert summary["compute_stream_idle_ms"] >= 0
    assert trainer.runner.last_profile["iteration"] == 2


def test_interval_arithmetic_of_the_profiler():
    from fast_llm_b200.engine.schedule.profiler import _subtract, _union_length

    assert _union_length([(0, 2), (1, 3), (5, 6)]) == 4
    # data-stream activity [0, 4] and [6, 8]; compute covers [1, 3] and [7, 9]: exposed = 1 + 1 + 1
    assert _subtract([(0, 4), (6, 8)], [(1, 3), (7, 9)]) == 3
