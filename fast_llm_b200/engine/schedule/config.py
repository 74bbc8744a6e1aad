"""Schedule configuration (parity: `fast_llm/engine/schedule/config.py:17-133`)."""

import enum

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.utils import Assert


@config_class()
class ScheduleConfig(Config):
    depth_first_micro_batches: int = Field(default=1, desc="Micro-batches processed one after the other (gradient accumulation).", hint=FieldHint.core, valid=check_field(Assert.gt, 0))
    breadth_first_micro_batches: int = Field(default=1, desc="Micro-batches in flight together: each stage runs all of them before the next stage.", hint=FieldHint.core, valid=check_field(Assert.gt, 0))
    micro_batch_splits: int = Field(default=1, desc="Split each micro-batch into this many sequential micro-sequences.", hint=FieldHint.performance, valid=check_field(Assert.gt, 0))
    pipeline_overlap: bool = Field(default=True, desc="Overlap pipeline transfers with compute.", hint=FieldHint.testing)
    data_overlap: bool = Field(default=True, desc="Overlap ZeRO gathers / reductions with compute.", hint=FieldHint.testing)
    throttle_cpu: bool = Field(default=True, desc="Keep the CPU from running too far ahead of the GPU.", hint=FieldHint.expert)
    throttle_cpu_rate: int = Field(default=1, hint=FieldHint.expert, valid=check_field(Assert.gt, 0))
    throttle_cpu_delay: int = Field(default=1, hint=FieldHint.expert, valid=check_field(Assert.geq, 0))
    debug_schedule: bool = Field(default=False, desc="Log the schedule.", hint=FieldHint.logging)
    debug_send_recv: bool = Field(default=False, desc="Send a header before each pipeline payload and check it.", hint=FieldHint.logging)
    profile_schedule: bool = Field(default=False, desc="Record device and host time of every schedule event.", hint=FieldHint.logging)
    skip_step: bool = Field(default=False, desc="Skip the optimizer step (testing).", hint=FieldHint.testing)

    @property
    def sequential_micro_batches(self) -> int:
        return self.depth_first_micro_batches * self.breadth_first_micro_batches

    @property
    def num_inputs(self) -> int:
        return self.sequential_micro_batches * self.micro_batch_splits


class StepType(str, enum.Enum):
    forward = "forward"
    backward = "backward"


class EventType(str, enum.Enum):
    batch_begin = "batch_begin"
    batch_end = "batch_end"
    run = "run"
    compute_wait_data = "compute_wait_data"
    compute_wait_pipe = "compute_wait_pipe"
    restore = "restore"
    reduce = "reduce"
    send = "send"
    recv = "recv"
    pipe_wait_compute = "pipe_wait_compute"
    data_wait_compute = "data_wait_compute"
    optimizer = "optimizer"
    get_batch = "get_batch"


class MockStream:
    """Stands in for a CUDA stream on CPU."""

    def wait_event(self, event):
        pass

    def wait_stream(self, stream):
        pass

    def synchronize(self):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        pass


class MockEvent:
    def record(self, stream=None):
        pass

    def wait(self, stream=None):
        pass

    def synchronize(self):
        pass

    def elapsed_time(self, other):
        return 0.0
