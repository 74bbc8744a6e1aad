"""Executes a `Schedule`: one optimizer step = every forward / backward step of the plan, gradient reduction,
optimizer update and loss reduction.

Streams: compute runs on the current stream; ZeRO weight gathers and gradient reductions run on a `data` stream and
pipeline transfers on a `pipeline` stream, ordered against compute with events, so they overlap with the neighbouring
stage's math.  Asynchronous work is issued where the schedule placed it: a stage's weight gather one step before its first
use (`Step.restore_launch`), a pipeline receive while the step runs during which the peer sends (`Step.recv_launch`), into
buffers allocated once per plan; the compute stream waits for each only at the point of use.  Shared weight / gradient
buffers (ZeRO-2/3) are guarded by events: a gather into a shared buffer waits for the last math that read it, a backward
that writes a shared gradient buffer waits for the reduction that last read it.  With `profile_schedule` every activity is
timed on its stream (`engine/schedule/profiler.py`).  On CPU the same code runs with mock streams.
Parity: `fast_llm/engine/schedule/runner.py:65-556`.
"""

import collections
import logging
import time
import typing

import torch

from fast_llm_b200.engine.multi_stage.config import StageMode
from fast_llm_b200.engine.multi_stage.multi_stage import MultiStageModel
from fast_llm_b200.engine.schedule.config import EventType, MockEvent, MockStream, ScheduleConfig, StepType
from fast_llm_b200.engine.schedule.profiler import NO_SPAN, ScheduleProfiler
from fast_llm_b200.engine.schedule.schedule import Schedule, Step
from fast_llm_b200.layers.kwargs import BlockKwargs, LanguageModelKwargs
from fast_llm_b200.parallel.collectives import all_reduce, recv, send
from fast_llm_b200.parallel.topology import DistributedConfig
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


class BatchContext:
    """Everything alive during one optimizer step."""

    def __init__(self, iteration: int, schedule: Schedule):
        self.iteration = iteration
        self.schedule = schedule
        self.data: dict[int, list] = {}  # data_index -> [(tokens, kwargs) per micro-sequence]
        self.contexts: dict[tuple, typing.Any] = {}
        self.outputs: dict[tuple, torch.Tensor] = {}
        self.grads: dict[tuple, torch.Tensor] = {}
        self.kv_leaves: dict[tuple, list] = {}  # (stage, data_index, micro_sequence) -> detached key/value prefixes
        self.losses: dict[str, list] = collections.defaultdict(list)
        self.metrics: dict = {}
        self.pending_sends: list = []
        self.data_iterator = None
        self.restore_events: dict[int, typing.Any] = {}  # local step index -> event recorded after its weight gather
        self.received: dict[tuple, tuple] = {}  # (step type, *step key) -> (buffer, event recorded after the receive)


class ScheduleRunner:
    def __init__(self, *, config: ScheduleConfig, multi_stage: MultiStageModel, distributed_config: DistributedConfig):
        config.validate()
        self._config = config
        self._multi_stage = multi_stage
        self._distributed_config = distributed_config
        self._is_setup = False
        self._num_stages = len(multi_stage.stages)

    def setup(self, distributed, optimizer=None) -> None:
        assert not self._is_setup
        self._is_setup = True
        self._distributed = distributed
        self._optimizer = optimizer
        self._stages_on_device = self._multi_stage.stages_on_device
        self._tied_remote_stages = self._multi_stage.tied_remote_stages
        self._use_cuda = distributed.device.type == "cuda"
        if self._use_cuda:
            self._compute_stream = torch.cuda.current_stream(distributed.device)
            overlap_data = self._config.data_overlap and self._distributed_config.data_parallel > 1
            self._data_stream = torch.cuda.Stream(distributed.device) if overlap_data else self._compute_stream
            overlap_pipe = self._config.pipeline_overlap and self._distributed_config.pipeline_parallel > 1
            self._pipeline_stream = torch.cuda.Stream(distributed.device) if overlap_pipe else self._compute_stream
            self._event = lambda: torch.cuda.Event()
        else:
            self._compute_stream = self._data_stream = self._pipeline_stream = MockStream()
            self._event = MockEvent
        self._loss_definitions = {d.name: d for d in self._multi_stage.base_model.get_loss_definitions()}
        self._throttle_events: collections.deque = collections.deque()
        self._stream_names = {id(self._compute_stream): "compute"}
        self._stream_names.setdefault(id(self._data_stream), "data")
        self._stream_names.setdefault(id(self._pipeline_stream), "pipeline")
        self._profiler = ScheduleProfiler(self._use_cuda, self._distributed_config.rank) if self._config.profile_schedule else None
        self.last_profile: dict | None = None
        # events guarding shared buffers: weight buffer index -> after the last math that read it (compute stream);
        # gradient buffer index -> after the last reduction that read it (data stream)
        self._weight_buffer_used: dict = {}
        self._grad_buffer_reduced: dict = {}
        self._recv_buffers: dict[tuple, torch.Tensor] = {}
        self._stage_ready: dict = {}  # stage -> event after which its updated weights are complete (overlapped update)
        self._run = None

    def wait_for_optimizer(self) -> None:
        """Make the compute stream wait for an optimizer step that is still running on the data stream; call before
        anything but the next training step reads the weights (evaluation, checkpoints, export)."""
        if self._stage_ready and self._data_stream is not self._compute_stream:
            self._compute_stream.wait_stream(self._data_stream)
        self._stage_ready = {}

    def set_run(self, run) -> None:
        """The run whose artifact directory receives the schedule profiles."""
        self._run = run

    def _span(self, type_: EventType, stream, step: Step | None = None):
        if self._profiler is None:
            return NO_SPAN
        return self._profiler.span(type_, self._stream_names.get(id(stream), "compute"), stream if self._use_cuda else None, step)

    def _stream_ctx(self, stream):
        if self._use_cuda and stream is not self._compute_stream:
            return torch.cuda.stream(stream)
        return MockStream()

    # ------------------------------------------------------------------------------------------------
    def run_step(self, data_iterator: typing.Iterator, schedule: Schedule, *, iteration: int = 1, return_metrics: bool = False,
                 preprocessed: bool = False) -> tuple[dict[str, float | int], bool, dict | None]:
        assert self._is_setup
        training = schedule.phase.is_training
        if training:
            assert self._multi_stage.stages_on_device is not None and self._optimizer is not None or self._config.skip_step
        if not training:
            self.wait_for_optimizer()
        context = BatchContext(iteration, schedule)
        context.data_iterator = data_iterator
        context.preprocessed = preprocessed
        metrics = context.metrics if return_metrics else None
        self._distributed.set_step(iteration, schedule.phase)
        if self._data_stream is not self._compute_stream:
            self._data_stream.wait_stream(self._compute_stream)
        if self._pipeline_stream is not self._compute_stream:
            self._pipeline_stream.wait_stream(self._compute_stream)
        if self._profiler is not None:
            self._profiler.begin(self._compute_stream if self._use_cuda else None)
        self._weight_buffer_used.clear()
        self._grad_buffer_reduced.clear()
        if training:
            for stage in self._stages_on_device.values():
                stage.reset_gradients()
        context.deferred_reduces = []
        for step in schedule.steps:
            self._run_one(context, step)
        for handle in context.pending_sends:
            if handle is not None:
                handle.wait()
        if training and context.deferred_reduces:
            # stages holding a copy of a parameter tied across pipeline ranks: first add the other holder's gradient
            if self._data_stream is not self._compute_stream:
                self._data_stream.wait_stream(self._compute_stream)
            with self._stream_ctx(self._data_stream):
                self._multi_stage.exchange_tied_gradients()
                for stage, accumulate in context.deferred_reduces:
                    with self._span(EventType.reduce, self._data_stream):
                        stage.reduce_gradients(accumulate)
        fused = training and getattr(self._optimizer, "pushes_weights_to_peers", False)
        # With the fused update (Adam stores the new weights into every data rank's buffers, stage by stage) the optimizer runs
        # on the data stream right behind the reductions and the compute stream is not held back: the next step's first
        # forward of a stage waits only for that stage's weights (`_stage_ready`), so the weight push overlaps with it.
        overlap_update = fused and not self._config.skip_step and self._data_stream is not self._compute_stream
        if self._data_stream is not self._compute_stream and not overlap_update:
            self._compute_stream.wait_stream(self._data_stream)
        if self._pipeline_stream is not self._compute_stream:
            self._compute_stream.wait_stream(self._pipeline_stream)
        Assert.empty(context.contexts)

        update_successful = True
        if training and not self._config.skip_step:
            update_stream = self._data_stream if overlap_update else self._compute_stream
            with self._stream_ctx(update_stream), self._span(EventType.optimizer, update_stream):
                update_successful = self._optimizer.step(context.metrics if return_metrics else None)
            if overlap_update:
                self._stage_ready = dict(self._optimizer.stage_ready_events)
            # Adam wrote the new weights into this rank's slice of the weight buffers.  With one data rank that is the
            # whole buffer; otherwise the next restore all-gathers the other slices.
            if (self._distributed_config.data_parallel > 1 and not fused) or self._multi_stage._num_weight_buffers < len(self._stages_on_device):
                self._multi_stage.invalidate_buffers()
        losses = self._reduce_losses(context, schedule)
        if self._profiler is not None:
            self.last_profile = self._profiler.finish(iteration, schedule.phase.value)
            if self._run is not None and self._run.experiment_directory is not None:
                import yaml

                name = f"schedule_profile_rank_{self._distributed_config.rank}_{schedule.phase.value}_step_{iteration}.yaml"
                with self._run.open_artifact(name, verbose=False) as f:
                    yaml.safe_dump(self.last_profile, f, sort_keys=False)
            logger.info(ScheduleProfiler.format_summary(self.last_profile))
        return losses, update_successful, (context.metrics if return_metrics else None)

    # ------------------------------------------------------------------------------------------------
    def _get_data(self, context: BatchContext, data_index: int):
        if data_index not in context.data:
            t0 = time.perf_counter()
            with self._span(EventType.get_batch, self._compute_stream):
                batch = next(context.data_iterator)
                t1 = time.perf_counter()
                if context.preprocessed:
                    inputs = batch
                else:
                    inputs = self._multi_stage.base_model.preprocess_batch(
                        batch, phase=context.schedule.phase, iteration=context.iteration, metrics=context.metrics,
                        device=self._distributed.device)
            Assert.eq(len(inputs), self._config.micro_batch_splits)
            # Gradients are averaged over the whole data group, but the sequence-data ranks of one sample hold
            # partial gradients that must be summed: pre-multiply by their number.
            grad_output = ((self._optimizer.grad_scale if self._optimizer is not None else 1.0) / self._config.sequential_micro_batches
                           * self._distributed_config.sequence_data_parallel)
            for _, kwargs in inputs:
                kwargs[BlockKwargs.grad_output] = grad_output
            context.data[data_index] = inputs
            context.metrics["data_wait_ms"] = context.metrics.get("data_wait_ms", 0.0) + (t1 - t0) * 1e3
            context.metrics["preprocess_ms"] = context.metrics.get("preprocess_ms", 0.0) + (time.perf_counter() - t1) * 1e3
        return context.data[data_index]

    def _run_one(self, context: BatchContext, step: Step) -> None:
        if self._config.throttle_cpu and self._use_cuda:
            self._throttle()
        stage = self._stages_on_device[step.stage]
        # ---- asynchronous work the schedule placed at this step
        deferred = []
        for target in step.restore_launch:
            # a gather into the very buffer this step's math reads can only go behind that math
            if target is not step and self._stages_on_device[target.stage].weight_buffer_index == stage.weight_buffer_index:
                deferred.append(target)
            else:
                self._launch_restore(context, target)
        for target in step.recv_launch:
            self._launch_recv(context, target)
        # ---- this step
        if step.restore:
            event = context.restore_events.pop(step.local_index)
            if self._data_stream is not self._compute_stream:
                with self._span(EventType.compute_wait_data, self._compute_stream, step):
                    self._compute_stream.wait_event(event)
        ready = self._stage_ready.pop(step.stage, None)
        if ready is not None:
            self._compute_stream.wait_event(ready)  # the previous step's update of this stage, still running when we got here
        if step.type_ == StepType.backward:
            reduced = self._grad_buffer_reduced.pop(stage.grad_buffer_index, None)
            if reduced is not None and self._data_stream is not self._compute_stream:
                self._compute_stream.wait_event(reduced)  # the reduction that last read this (shared) gradient buffer
        with self._span(EventType.run, self._compute_stream, step):
            if step.type_ == StepType.forward:
                self._forward(context, step, stage)
            else:
                self._backward(context, step, stage)
        if self._shared_weight_buffers and self._data_stream is not self._compute_stream:
            used = self._event()
            used.record(self._compute_stream)
            self._weight_buffer_used[stage.weight_buffer_index] = used
        for target in deferred:
            self._launch_restore(context, target)
        if step.reduce:
            if self._data_stream is not self._compute_stream:
                self._data_stream.wait_stream(self._compute_stream)
            if step.stage in self._tied_remote_stages:
                # its gradient buffer is still missing the contribution of the other pipeline rank: reduce at the end
                Assert.custom(lambda ok: ok, not step.reduce_accumulate and self._multi_stage._num_grad_buffers >= len(self._stages_on_device))
                context.deferred_reduces.append((stage, step.reduce_accumulate))
                return
            with self._stream_ctx(self._data_stream):
                with self._span(EventType.reduce, self._data_stream, step):
                    stage.reduce_gradients(step.reduce_accumulate)
                if step.reduce_accumulate or self._multi_stage._num_grad_buffers < len(self._stages_on_device):
                    stage.reset_gradients()
                    if self._data_stream is not self._compute_stream:
                        reduced = self._event()
                        reduced.record(self._data_stream)
                        self._grad_buffer_reduced[stage.grad_buffer_index] = reduced

    @property
    def _shared_weight_buffers(self) -> bool:
        return self._multi_stage._num_weight_buffers < len(self._stages_on_device)

    def _launch_restore(self, context: BatchContext, target: Step) -> None:
        """Issue the weight gather of `target` on the data stream and remember the event its math will wait for."""
        stage = self._stages_on_device[target.stage]
        with self._stream_ctx(self._data_stream):
            used = self._weight_buffer_used.pop(stage.weight_buffer_index, None)
            if used is not None and self._data_stream is not self._compute_stream:
                self._data_stream.wait_event(used)  # the last math that read the buffer about to be overwritten
            with self._span(EventType.restore, self._data_stream, target):
                stage.restore_parameters()
            event = self._event()
            event.record(self._data_stream if self._use_cuda else None)
        context.restore_events[target.local_index] = event

    def _throttle(self) -> None:
        event = torch.cuda.Event()
        event.record()
        self._throttle_events.append(event)
        limit = self._config.throttle_cpu_delay + 8
        while len(self._throttle_events) > limit:
            self._throttle_events.popleft().synchronize()

    def _forward(self, context: BatchContext, step: Step, stage) -> None:
        inputs = self._get_data(context, step.data_index)
        tokens, kwargs = inputs[step.micro_sequence]
        if step.stage == 0:
            input_ = tokens
        elif step.recv_from is not None:
            input_ = self._received(context, step)
        else:
            input_ = context.outputs.pop((step.stage - 1, step.data_index, step.micro_sequence))
        splits = self._config.micro_batch_splits
        if splits > 1:
            kwargs = dict(kwargs)
            if step.micro_sequence > 0:
                leaves = context.kv_leaves[(step.stage, step.data_index, step.micro_sequence - 1)]
                kwargs[BlockKwargs.past_key_values] = list(leaves)
            if step.micro_sequence < splits - 1:
                kwargs[BlockKwargs.presents] = []
        output, ctx = stage.forward(input_, kwargs, context.losses, context.metrics)
        presents = kwargs.get(BlockKwargs.presents) if splits > 1 else None
        if presents is not None:
            training = context.schedule.phase.is_training
            context.kv_leaves[step.key] = [kv.detach().requires_grad_(training) for kv in presents]
        if context.schedule.phase.is_training:
            context.contexts[step.key] = (ctx, presents)
        if step.stage < self._num_stages - 1:
            if step.send_to is not None:
                self._send(context, step, output)
            else:
                context.outputs[step.key] = output

    def _backward(self, context: BatchContext, step: Step, stage) -> None:
        if step.stage == self._num_stages - 1:
            output_grad = None
        elif step.recv_from is not None:
            output_grad = self._received(context, step)
        else:
            output_grad = context.grads.pop((step.stage + 1, step.data_index, step.micro_sequence))
        ctx, presents = context.contexts.pop(step.key)
        if presents:
            leaves = context.kv_leaves.pop(step.key)
            input_, output = ctx
            tensors, grads = [output], [output_grad]
            for kv, leaf in zip(presents, leaves):
                if leaf.grad is not None:
                    tensors.append(kv)
                    grads.append(leaf.grad)
            torch.autograd.backward(tensors, grads)
            input_grad = None
            if torch.is_tensor(input_) and input_.is_floating_point() and input_.requires_grad:
                input_grad, input_.grad = input_.grad, None
        else:
            context.kv_leaves.pop(step.key, None)
            input_grad = stage.backward(output_grad, ctx)
        if step.stage > 0:
            if step.send_to is not None:
                self._send(context, step, input_grad)
            else:
                context.grads[step.key] = input_grad
        if step.stage == 0 and step.micro_sequence == 0:
            last_use = all(s.data_index != step.data_index or s.local_index <= step.local_index for s in context.schedule.steps)
            if last_use:
                context.data.pop(step.data_index, None)

    # ---- pipeline transfers (NCCL / Gloo point to point on the pipeline stream)
    def _hidden_shape(self, kwargs, layer_index: int | None = None) -> tuple[int, int]:
        if layer_index is not None:  # models whose layers do not all work on [tokens, hidden] (a vision encoder in front)
            shape = self._multi_stage.base_model.get_activation_shape(layer_index, kwargs)
            if shape is not None:
                return tuple(shape)
        tokens = kwargs[BlockKwargs.num_tokens]
        dc = self._distributed_config
        if dc.sequence_tensor_parallel:
            tokens //= dc.tensor_parallel
        return (tokens, self._multi_stage.base_model._hidden_dim.size)

    def _launch_recv(self, context: BatchContext, target: Step) -> None:
        """Post the receive of `target`'s input (forward) or output gradient (backward) on the pipeline stream, into a buffer
        that belongs to this step of the plan and is reused by every later optimizer step."""
        kwargs = self._get_data(context, target.data_index)[target.micro_sequence][1]
        # forward: what enters the target stage; backward: the gradient of what leaves it (= what enters the next stage)
        stage = self._multi_stage.stages[target.stage]
        shape = self._hidden_shape(kwargs, stage._begin if target.type_ == StepType.forward else stage._end)
        dtype = self._distributed_config.compute_dtype.torch
        key = (id(context.schedule), target.type_, *target.key)
        buffer = self._recv_buffers.get(key)
        if buffer is None or tuple(buffer.shape) != tuple(shape) or buffer.dtype != dtype:
            buffer = self._recv_buffers[key] = torch.empty(shape, dtype=dtype, device=self._distributed.device)
        with self._stream_ctx(self._pipeline_stream):
            with self._span(EventType.recv, self._pipeline_stream, target):
                if self._config.debug_send_recv:
                    header = torch.empty(2, dtype=torch.int64, device=self._distributed.device)
                    recv(header, target.recv_from, self._distributed.pipeline_group)
                    Assert.eq(header.tolist(), [target.data_index * 1000 + target.micro_sequence, buffer.numel()])
                recv(buffer, target.recv_from, self._distributed.pipeline_group)
            event = self._event()
            event.record(self._pipeline_stream if self._use_cuda else None)
        context.received[(target.type_, *target.key)] = (buffer, event)

    def _received(self, context: BatchContext, step: Step) -> torch.Tensor:
        buffer, event = context.received.pop((step.type_, *step.key))
        if self._pipeline_stream is not self._compute_stream:
            with self._span(EventType.compute_wait_pipe, self._compute_stream, step):
                self._compute_stream.wait_event(event)
        # the buffer is reused by the same step of the next optimizer step: hand out a tensor of its own when autograd may
        # keep it (a stage's input is saved for its backward) and the next step could overwrite it first
        return buffer

    def _send(self, context: BatchContext, step: Step, tensor: torch.Tensor) -> None:
        if self._pipeline_stream is not self._compute_stream:
            self._pipeline_stream.wait_stream(self._compute_stream)
        with self._stream_ctx(self._pipeline_stream), self._span(EventType.send, self._pipeline_stream, step):
            tensor = tensor.contiguous()
            if self._config.debug_send_recv:
                header = torch.tensor([step.data_index * 1000 + step.micro_sequence, tensor.numel()], dtype=torch.int64, device=tensor.device)
                context.pending_sends.append(send(header, step.send_to, self._distributed.pipeline_group, async_op=True))
            context.pending_sends.append(send(tensor, step.send_to, self._distributed.pipeline_group, async_op=True))
            if self._use_cuda:
                tensor.record_stream(self._pipeline_stream) if self._pipeline_stream is not self._compute_stream else None

    # ---- losses
    def _reduce_losses(self, context: BatchContext, schedule: Schedule) -> dict[str, float]:
        out = {}
        count = self._config.sequential_micro_batches
        for name, definition in self._loss_definitions.items():
            definition.count = count
            values = context.losses.get(name, [])
            # micro-sequences of one micro-batch are already normalised by the whole micro-batch's label count
            out[name] = definition.reduce(values, self._distributed)
        for name, values in context.losses.items():
            if name not in out and values:
                out[name] = (torch.stack([v.float().reshape(()) for v in values]).sum() / count).item()
        return out
