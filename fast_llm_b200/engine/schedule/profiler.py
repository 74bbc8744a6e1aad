"""Schedule profiler: device and host time of every event of one optimizer step, and what of it is exposed.

`ScheduleConfig.profile_schedule` makes the runner bracket every activity (a stage's forward or backward, a weight gather, a
gradient reduction, a pipeline send or receive, fetching a batch, the optimizer) with a pair of CUDA events on the stream it
runs on, plus host timestamps.  At the end of the step the events are resolved into one table per rank:

  * `events`: type, stage / micro-batch / micro-sequence, stream, start and duration on the device and on the host;
  * `summary`: device time per event type, busy time per stream, and for the data and pipeline streams the *exposed* time - the
    part of their activity during which the compute stream had nothing to run, i.e. what the step really pays for the
    collectives - and the time the compute stream sat idle between its own events.

The table is written as a YAML artifact of the run (`schedule_profile_rank_<r>_<phase>_step_<i>.yaml`) and its summary is
logged.  On CPU the same code runs with host timestamps only.
Parity: `fast_llm/engine/schedule/runner.py:481-536` (event recording and the YAML artifact); the exposed-time analysis has no
counterpart there.
"""

import dataclasses
import logging
import time

import torch

from fast_llm_b200.engine.schedule.config import EventType

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class _Span:
    type_: EventType
    stream: str
    stage: int | None
    data_index: int | None
    micro_sequence: int | None
    cpu_begin: float
    cpu_end: float = 0.0
    gpu_begin: "torch.cuda.Event | None" = None
    gpu_end: "torch.cuda.Event | None" = None


class _SpanContext:
    def __init__(self, profiler: "ScheduleProfiler", span: _Span, stream):
        self._profiler, self._span, self._stream = profiler, span, stream

    def __enter__(self):
        if self._profiler.use_cuda:
            # an NVTX range of the same name, so that a timeline viewer shows the schedule's events over the kernels
            label = self._span.type_.value if self._span.stage is None else f"{self._span.type_.value} s{self._span.stage} mb{self._span.data_index}"
            torch.cuda.nvtx.range_push(label)
            self._span.gpu_begin = torch.cuda.Event(enable_timing=True)
            self._span.gpu_begin.record(self._stream)
        self._span.cpu_begin = time.perf_counter()
        return self._span

    def __exit__(self, *exc):
        self._span.cpu_end = time.perf_counter()
        if self._profiler.use_cuda:
            self._span.gpu_end = torch.cuda.Event(enable_timing=True)
            self._span.gpu_end.record(self._stream)
            torch.cuda.nvtx.range_pop()
        self._profiler.spans.append(self._span)


class _NoSpan:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        pass


NO_SPAN = _NoSpan()


def _union_length(intervals: list[tuple[float, float]]) -> float:
    total, end = 0.0, float("-inf")
    for a, b in sorted(intervals):
        if b <= end:
            continue
        total += b - max(a, end)
        end = b
    return total


def _subtract(intervals: list[tuple[float, float]], cover: list[tuple[float, float]]) -> float:
    """Total length of `intervals` (united) not covered by `cover`."""
    both = _union_length(intervals + cover)
    return both - _union_length(cover)


class ScheduleProfiler:
    def __init__(self, use_cuda: bool, rank: int):
        self.use_cuda = use_cuda
        self.rank = rank
        self.spans: list[_Span] = []
        self._origin_event = None
        self._origin_cpu = 0.0

    def begin(self, compute_stream) -> None:
        self.spans = []
        self._origin_cpu = time.perf_counter()
        if self.use_cuda:
            self._origin_event = torch.cuda.Event(enable_timing=True)
            self._origin_event.record(compute_stream)

    def span(self, type_: EventType, stream_name: str, stream, step=None) -> _SpanContext:
        span = _Span(type_, stream_name, None if step is None else step.stage, None if step is None else step.data_index,
                     None if step is None else step.micro_sequence, 0.0)
        return _SpanContext(self, span, stream if self.use_cuda else None)

    def finish(self, iteration: int, phase: str) -> dict:
        """Resolve the events (synchronises the device) into the table described in the module docstring."""
        if self.use_cuda:
            torch.cuda.synchronize()
        events, by_stream = [], {}
        for span in self.spans:
            cpu_start = (span.cpu_begin - self._origin_cpu) * 1e3
            cpu_ms = (span.cpu_end - span.cpu_begin) * 1e3
            if self.use_cuda:
                gpu_start = self._origin_event.elapsed_time(span.gpu_begin)
                gpu_ms = span.gpu_begin.elapsed_time(span.gpu_end)
            else:
                gpu_start, gpu_ms = cpu_start, cpu_ms
            events.append({"event_type": span.type_.value, "stream": span.stream, "stage": span.stage, "micro_batch": span.data_index,
                           "micro_sequence": span.micro_sequence, "gpu_start_ms": round(gpu_start, 4), "gpu_ms": round(gpu_ms, 4),
                           "cpu_start_ms": round(cpu_start, 4), "cpu_ms": round(cpu_ms, 4)})
            by_stream.setdefault(span.stream, []).append((gpu_start, gpu_start + gpu_ms))
        per_type: dict[str, float] = {}
        host_per_type: dict[str, float] = {}
        for e in events:
            per_type[e["event_type"]] = per_type.get(e["event_type"], 0.0) + e["gpu_ms"]
            host_per_type[e["event_type"]] = host_per_type.get(e["event_type"], 0.0) + e["cpu_ms"]
        compute = by_stream.get("compute", [])
        step_ms = max((b for spans in by_stream.values() for _, b in spans), default=0.0)
        summary = {
            "step_ms": round(step_ms, 3),
            "gpu_ms_by_event_type": {k: round(v, 3) for k, v in sorted(per_type.items())},
            # host time spent queueing the work of each event type: close to the device time means the host is the limiter
            "cpu_ms_by_event_type": {k: round(v, 3) for k, v in sorted(host_per_type.items())},
            "busy_ms_by_stream": {k: round(_union_length(v), 3) for k, v in sorted(by_stream.items())},
            "exposed_ms_by_stream": {k: round(_subtract(v, compute), 3) for k, v in sorted(by_stream.items()) if k != "compute"},
            "compute_stream_idle_ms": round(step_ms - _union_length(compute), 3),
        }
        return {"iteration": iteration, "phase": str(phase), "rank": self.rank, "summary": summary, "events": events}

    @staticmethod
    def format_summary(table: dict) -> str:
        s = table["summary"]
        lines = [f"Schedule profile, rank {table['rank']}, {table['phase']} step {table['iteration']}: {s['step_ms']:.2f} ms"]
        lines.append("  device ms by event:  " + ", ".join(f"{k} {v:.2f}" for k, v in s["gpu_ms_by_event_type"].items()))
        if "cpu_ms_by_event_type" in s:
            lines.append("  host ms by event:    " + ", ".join(f"{k} {v:.2f}" for k, v in s["cpu_ms_by_event_type"].items()))
        lines.append("  busy ms by stream:   " + ", ".join(f"{k} {v:.2f}" for k, v in s["busy_ms_by_stream"].items()))
        lines.append("  exposed (not under compute): " + (", ".join(f"{k} {v:.2f}" for k, v in s["exposed_ms_by_stream"].items()) or "-")
                     + f"; compute stream idle {s['compute_stream_idle_ms']:.2f}")
        return "\n".join(lines)
