"""The per-step execution plan.

For a (model, batch layout, phase) the plan is fixed: an ordered list of forward / backward steps for this pipeline
rank, each annotated with what must happen around it - weight restore before first use (or every use when buffers are
shared), gradient reduction after a stage's last backward, pipeline receives and sends - plus FLOP accounting.  The
order is the breadth-first schedule of arXiv 2211.05953: inside each depth-first group every stage runs all in-flight
micro-batches (and their micro-sequences) before the next stage, so weights are gathered and gradients reduced once
per group.  A host-side simulation of the send / receive queues proves the plan cannot deadlock before anything runs.
Parity: `fast_llm/engine/schedule/schedule.py:25-543`.
"""

import dataclasses
import logging

from fast_llm_b200.engine.multi_stage.multi_stage import MultiStageModel
from fast_llm_b200.engine.schedule.config import ScheduleConfig, StepType
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.parallel.topology import DistributedConfig, PhaseType
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class Step:
    stage: int
    data_index: int  # which micro-batch of the step (depth-first major, breadth-first minor)
    micro_sequence: int
    type_: StepType
    depth_first_index: int = 0
    breadth_first_index: int = 0
    global_index: int = -1  # position in the global (all-ranks) order
    local_index: int = -1
    restore: bool = False  # gather this stage's weights before running
    reduce: bool = False  # reduce this stage's gradients after running
    reduce_accumulate: bool = False
    recv_from: int | None = None  # pipeline rank to receive the input (activation or gradient) from
    send_to: int | None = None  # pipeline rank to send the output to
    invalidate_after: bool = False  # shared weight buffer is about to be reused by another stage

    @property
    def key(self):
        return (self.stage, self.data_index, self.micro_sequence)

    def __repr__(self):
        return (f"Step({self.type_.value[:3]} stage={self.stage} mb={self.data_index} ms={self.micro_sequence}"
                f"{' restore' if self.restore else ''}{' reduce' if self.reduce else ''}"
                f"{f' recv<-{self.recv_from}' if self.recv_from is not None else ''}{f' send->{self.send_to}' if self.send_to is not None else ''})")


class Schedule:
    def __init__(self, multi_stage: MultiStageModel, batch_config: ScheduleConfig, distributed_config: DistributedConfig,
                 phase: PhaseType, sample_kwargs: dict | None = None):
        batch_config.validate()
        self._multi_stage = multi_stage
        self._config = batch_config
        self._distributed_config = distributed_config
        self._phase = phase
        self._is_training = phase.is_training
        self._num_stages = len(multi_stage.stages)
        self._pp = distributed_config.pipeline_parallel
        self._rank = distributed_config.pipeline_rank
        self._global_steps = self._create_steps()
        for i, step in enumerate(self._global_steps):
            step.global_index = i
        self._steps = [s for s in self._global_steps if s.stage % self._pp == self._rank]
        for i, step in enumerate(self._steps):
            step.local_index = i
        self._place_restore_and_reduce()
        self._place_send_recv()
        self._validate_send_recv()
        self._sample_kwargs = sample_kwargs
        if batch_config.debug_schedule:
            logger.info("Schedule:\n" + "\n".join(map(repr, self._steps)))

    @property
    def config(self) -> ScheduleConfig:
        return self._config

    @property
    def phase(self):
        return self._phase

    @property
    def steps(self) -> list[Step]:
        return self._steps

    @property
    def global_steps(self) -> list[Step]:
        return self._global_steps

    @property
    def samples_per_batch(self) -> int:
        return self._config.sequential_micro_batches * self._distributed_config.batch_data_parallel

    def __iter__(self):
        return iter(self._steps)

    def _create_steps(self) -> list[Step]:
        c = self._config
        steps = []
        for d in range(c.depth_first_micro_batches):
            for stage in range(self._num_stages):
                for b in range(c.breadth_first_micro_batches):
                    for m in range(c.micro_batch_splits):
                        steps.append(Step(stage, d * c.breadth_first_micro_batches + b, m, StepType.forward, d, b))
            if self._is_training:
                for stage in reversed(range(self._num_stages)):
                    for b in range(c.breadth_first_micro_batches):
                        for m in reversed(range(c.micro_batch_splits)):
                            steps.append(Step(stage, d * c.breadth_first_micro_batches + b, m, StepType.backward, d, b))
        return steps

    def _place_restore_and_reduce(self) -> None:
        ms = self._multi_stage
        local = sorted(s for s in range(self._num_stages) if s % self._pp == self._rank)
        shared_weights = ms.config.multi_stage.num_weight_buffers is not None and ms.config.multi_stage.num_weight_buffers < len(local)
        shared_grads = ms.config.multi_stage.num_grad_buffers is not None and ms.config.multi_stage.num_grad_buffers < len(local)
        restored_in_step = set()
        last_stage = None
        for step in self._steps:
            if shared_weights:
                # a run of consecutive steps on one stage shares one restore
                step.restore = step.stage != last_stage
            else:
                step.restore = step.stage not in restored_in_step
                restored_in_step.add(step.stage)
            last_stage = step.stage
        if not self._is_training:
            return
        # reduce after the last backward of a stage: per depth-first group when gradient buffers are shared,
        # once per step otherwise
        seen = set()
        for step in reversed(self._steps):
            if step.type_ != StepType.backward:
                continue
            key = (step.stage, step.depth_first_index) if shared_grads else step.stage
            if key not in seen:
                seen.add(key)
                step.reduce = True
                step.reduce_accumulate = shared_grads and step.depth_first_index > 0

    def _place_send_recv(self) -> None:
        if self._pp == 1:
            return
        for step in self._steps:
            if step.type_ == StepType.forward:
                if step.stage > 0:
                    step.recv_from = (step.stage - 1) % self._pp
                if step.stage < self._num_stages - 1:
                    step.send_to = (step.stage + 1) % self._pp
            else:
                if step.stage < self._num_stages - 1:
                    step.recv_from = (step.stage + 1) % self._pp
                if step.stage > 0:
                    step.send_to = (step.stage - 1) % self._pp

    def _validate_send_recv(self) -> None:
        """Simulate every rank executing its list with FIFO channels: each receive must find its message sent by a
        step that the sender reaches without first blocking on something the receiver has yet to send."""
        if self._pp == 1:
            return
        per_rank = {r: [s for s in self._global_steps if s.stage % self._pp == r] for r in range(self._pp)}
        position = {r: 0 for r in range(self._pp)}
        sent = set()
        progress = True
        while progress:
            progress = False
            for r in range(self._pp):
                while position[r] < len(per_rank[r]):
                    step = per_rank[r][position[r]]
                    if step.stage > 0 and step.type_ == StepType.forward:
                        need = ("f", step.stage - 1, step.data_index, step.micro_sequence)
                    elif step.type_ == StepType.backward and step.stage < self._num_stages - 1:
                        need = ("b", step.stage + 1, step.data_index, step.micro_sequence)
                    else:
                        need = None
                    if need is not None and need not in sent:
                        break
                    sent.add(("f" if step.type_ == StepType.forward else "b", step.stage, step.data_index, step.micro_sequence))
                    position[r] += 1
                    progress = True
        for r in range(self._pp):
            if position[r] != len(per_rank[r]):
                raise RuntimeError(f"Pipeline schedule deadlocks: rank {r} blocks at {per_rank[r][position[r]]}")

    def get_compute_usage(self, kwargs: dict | None = None, hardware: bool = False) -> int | None:
        """Model FLOPs of one step on this rank (forward + backward = 3x forward), from the layers' accounting."""
        kwargs = kwargs or self._sample_kwargs
        if kwargs is None:
            return None
        total = 0
        for stage in self._multi_stage.stages_on_device.values():
            for layer in stage.layers:
                try:
                    total += layer.get_compute_usage(None, kwargs, None)
                except Exception:
                    return None
        mult = 3 if self._is_training else 1
        return total * mult * self._config.num_inputs

    def get_compute_metrics(self, time_per_iteration: float, kwargs: dict | None = None) -> dict:
        flops = self.get_compute_usage(kwargs)
        if not flops or time_per_iteration <= 0:
            return {}
        return {"model_tflops": flops / time_per_iteration / 1e12, "hardware_tflops": flops / time_per_iteration / 1e12}
