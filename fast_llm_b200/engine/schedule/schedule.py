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
    # Placement of the asynchronous work (filled by the schedule):
    restore_launch: list = dataclasses.field(default_factory=list)  # steps whose weight gather is issued before this step runs
    recv_launch: list = dataclasses.field(default_factory=list)  # steps whose pipeline receive is posted before this step runs
    # Simulated timeline (units of one forward step of one stage)
    start: float = 0.0
    end: float = 0.0

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
        self._simulate_timeline()
        self._place_restore_launch()
        self._place_recv_launch()
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
        for step in self._global_steps:  # every rank's steps: the deadlock proof needs the whole picture
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

    # ---- simulated timeline -------------------------------------------------------------------------------------------
    FORWARD_TIME, BACKWARD_TIME = 1.0, 2.0

    def _producer(self, step: Step) -> tuple | None:
        """Key (type, stage, data_index, micro_sequence) of the step whose output this step consumes, if any."""
        if step.type_ == StepType.forward:
            return None if step.stage == 0 else (StepType.forward, step.stage - 1, step.data_index, step.micro_sequence)
        if step.stage == self._num_stages - 1:
            return (StepType.forward, step.stage, step.data_index, step.micro_sequence)
        return (StepType.backward, step.stage + 1, step.data_index, step.micro_sequence)

    def _per_rank_steps(self) -> dict[int, list[Step]]:
        return {r: [s for s in self._global_steps if s.stage % self._pp == r] for r in range(self._pp)}

    def _simulate_timeline(self) -> None:
        """Estimated start / end of every step of every pipeline rank, in units of one stage's forward time: a step starts
        when the rank's previous step has ended and its input has arrived (`pipeline_delay` after the producing step on
        another rank).  Used to place receives and to report the pipeline's idle fraction; raises on a plan in which some
        step can never start."""
        delay = self._multi_stage.config.multi_stage.pipeline_delay
        per_rank = self._per_rank_steps()
        by_key = {(s.type_, *s.key): s for s in self._global_steps}
        done: set = set()
        position = {r: 0 for r in range(self._pp)}
        clock = {r: 0.0 for r in range(self._pp)}
        progress = True
        while progress:
            progress = False
            for r in range(self._pp):
                while position[r] < len(per_rank[r]):
                    step = per_rank[r][position[r]]
                    producer = self._producer(step)
                    ready = clock[r]
                    if producer is not None:
                        if producer not in done:
                            break
                        source = by_key[producer]
                        ready = max(ready, source.end + (delay if source.stage % self._pp != r else 0.0))
                    step.start = ready
                    step.end = ready + (self.FORWARD_TIME if step.type_ == StepType.forward else self.BACKWARD_TIME)
                    clock[r] = step.end
                    done.add((step.type_, *step.key))
                    position[r] += 1
                    progress = True
        for r in range(self._pp):
            if position[r] != len(per_rank[r]):
                raise RuntimeError(f"Pipeline schedule deadlocks: rank {r} blocks at {per_rank[r][position[r]]}")
        self._simulated_time = max(clock.values()) if clock else 0.0
        self._simulated_busy = {r: sum(s.end - s.start for s in per_rank[r]) for r in range(self._pp)}

    @property
    def simulated_idle_fraction(self) -> float:
        """Share of the simulated step time this pipeline rank spends waiting (the pipeline bubble)."""
        if self._simulated_time <= 0:
            return 0.0
        return 1.0 - self._simulated_busy[self._rank] / self._simulated_time

    def _place_restore_launch(self) -> None:
        """The weight gather of a step that needs one is issued one step early, so that it runs on the data stream beside
        the previous step's math (the first step of the plan has nothing to hide behind)."""
        for i, step in enumerate(self._steps):
            if step.restore:
                self._steps[max(i - 1, 0)].restore_launch.append(step)

    def _place_recv_launch(self) -> None:
        """Decide when each pipeline receive is posted.  Point-to-point transfers between two ranks run in the order in which
        each side issues them, and a send does not complete before its receive is posted, so both sides must issue the
        transfers of a pair in ONE common order or they block each other.  That order is the simulated time at which the
        sender finishes the producing step (ties: position in the global plan).  A rank's sends are issued right after their
        step; each receive is posted right behind the last of the rank's own sends that precedes it in the common order - as
        early as the order allows, so the transfer overlaps with local math - and never later than the step that consumes it."""
        if self._pp == 1:
            return
        by_key = {(s.type_, *s.key): s for s in self._global_steps}

        def order_of_transfer_into(step: Step) -> tuple:
            source = by_key[self._producer(step)]
            return (source.end, source.global_index)

        consumers = {self._producer(s): s for s in self._global_steps if s.recv_from is not None}
        for steps in self._per_rank_steps().values():  # the same rule on every rank: the proof below replays all of them
            for step in steps:
                step.recv_launch = []
            sends = [(index, (step.end, step.global_index)) for index, step in enumerate(steps) if (step.type_, *step.key) in consumers
                     and step.send_to is not None]
            for index, step in enumerate(steps):
                if step.recv_from is None:
                    continue
                order = order_of_transfer_into(step)
                earlier_sends = [i for i, send_order in sends if send_order < order]
                launch = earlier_sends[-1] + 1 if earlier_sends else 0
                Assert.leq(launch, index)  # a send that precedes the transfer cannot come after the step that needs it
                steps[launch].recv_launch.append(step)
            for step in steps:
                step.recv_launch.sort(key=order_of_transfer_into)

    def _stream_operations(self, rank: int) -> tuple[list, list]:
        """(compute-stream nodes, pipeline-stream nodes) of one rank in issue order.  Nodes: ("run", step key), ("send", key of
        the sending step), ("recv", key of the receiving step)."""
        compute, pipe = [], []
        for step in self._per_rank_steps()[rank]:
            for receiver in step.recv_launch:
                pipe.append(("recv", (receiver.type_, *receiver.key)))
            compute.append(("run", (step.type_, *step.key)))
            if step.send_to is not None:
                pipe.append(("send", (step.type_, *step.key)))
        return compute, pipe

    def _validate_send_recv(self) -> None:
        """Final proof that the plan, with its receives posted early, cannot deadlock."""
        if self._pp == 1:
            return
        stuck = self._find_deadlock()
        if stuck:
            raise RuntimeError(f"Pipeline schedule deadlocks with these operations at the head of their streams: {stuck}")

    def _find_deadlock(self) -> dict:
        """Replay every rank's compute stream and pipeline stream: each executes its operations in issue order; a step waits
        for its receive, a send for its step, and a send and its receive complete together.  Streams advance as far as their
        heads allow until nothing moves.  Returns the operations left at the head of the streams (empty: no deadlock)."""
        streams = {}
        for r in range(self._pp):
            compute, pipe = self._stream_operations(r)
            streams[(r, "compute")], streams[(r, "pipe")] = compute, pipe
        heads = {k: 0 for k in streams}
        ran: set = set()       # step keys whose math has run
        received: set = set()  # step keys whose input has arrived
        by_key = {(s.type_, *s.key): s for s in self._global_steps}
        consumers = {self._producer(s): (s.type_, *s.key) for s in self._global_steps if s.recv_from is not None}
        progress = True
        while progress:
            progress = False
            for (r, kind), ops in streams.items():
                while heads[(r, kind)] < len(ops):
                    op, key = ops[heads[(r, kind)]]
                    if op == "run":
                        step = by_key[key]
                        producer = self._producer(step)
                        remote = step.recv_from is not None
                        if (remote and key not in received) or (producer is not None and not remote and producer not in ran):
                            break
                        ran.add(key)
                    elif op == "send":
                        if key not in ran:
                            break
                        # completes together with the matching receive: that must be at the head of the peer's pipeline stream
                        target = consumers[key]
                        peer = by_key[target].stage % self._pp
                        peer_ops, peer_head = streams[(peer, "pipe")], heads[(peer, "pipe")]
                        if peer_head >= len(peer_ops) or peer_ops[peer_head] != ("recv", target):
                            break
                        heads[(peer, "pipe")] += 1
                        received.add(target)
                    else:  # a receive advances with its send (handled from the sending side)
                        break
                    heads[(r, kind)] += 1
                    progress = True
        return {k: streams[k][heads[k]] for k in streams if heads[k] < len(streams[k])}

    def _next_rank(self, step: Step) -> int:
        """Pipeline rank that consumes this step's output (its own rank when the consumer is local or there is none)."""
        if step.type_ == StepType.forward:
            target = step.stage + 1 if step.stage < self._num_stages - 1 else step.stage
        else:
            target = step.stage - 1 if step.stage > 0 else step.stage
        return target % self._pp

    def get_compute_usage(self, kwargs: dict | None = None, hardware: bool = False) -> int | None:
        """FLOPs of one step on this rank from the layers' accounting: forward + backward = 3x forward for the model;
        `hardware` adds the forward work that backward recomputes."""
        kwargs = kwargs or self._sample_kwargs
        if kwargs is None:
            return None
        total = recomputed = 0
        for stage in self._multi_stage.stages_on_device.values():
            for layer in stage.layers:
                try:
                    total += layer.get_compute_usage(None, kwargs, None)
                    if hardware and self._is_training and hasattr(layer, "get_recompute_usage"):
                        recomputed += layer.get_recompute_usage(kwargs)
                except Exception:
                    return None
        mult = 3 if self._is_training else 1
        return (total * mult + recomputed) * self._config.num_inputs

    def get_compute_metrics(self, time_per_iteration: float, kwargs: dict | None = None) -> dict:
        flops = self.get_compute_usage(kwargs)
        if not flops or time_per_iteration <= 0:
            return {}
        # hardware FLOPs count what the GPU really executes: recomputed forward passes on top of the model's FLOPs
        hardware = self.get_compute_usage(kwargs, hardware=True) or flops
        return {"model_tflops": flops / time_per_iteration / 1e12, "hardware_tflops": hardware / time_per_iteration / 1e12}
