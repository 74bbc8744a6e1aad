"""torch.profiler integration: skip / wait / warmup / active schedule, rank filter, tables and chrome traces written as
run artifacts (parity: `fast_llm/profile.py:29-180`).  The hot kernels are additionally profiled with ncu; see
`profiles/` for the summaries."""

import contextlib
import logging

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


@config_class()
class ProfilingConfig(Config):
    cpu: bool = Field(default=False, desc="Profile host activity.", hint=FieldHint.feature)
    cuda: bool = Field(default=False, desc="Profile device activity.", hint=FieldHint.core)
    skip: int = Field(default=1, desc="Iterations skipped first.", hint=FieldHint.optional, valid=check_field(Assert.geq, 0))
    wait: int = Field(default=0, desc="Idle iterations at the start of each cycle.", hint=FieldHint.optional, valid=check_field(Assert.geq, 0))
    warmup: int = Field(default=1, desc="Warm-up iterations of each cycle.", hint=FieldHint.optional, valid=check_field(Assert.geq, 0))
    cycles: int = Field(default=1, desc="Profiled iterations per cycle.", hint=FieldHint.optional, valid=check_field(Assert.gt, 0))
    averages: bool = Field(default=False, desc="Write the per-op averages table.", hint=FieldHint.logging)
    trace: bool = Field(default=False, desc="Write the chronological trace table.", hint=FieldHint.logging)
    table_width: int = Field(default=80, hint=FieldHint.logging, valid=check_field(Assert.geq, 40))
    ranks: set[int] = Field(default_factory=set, desc="Ranks to profile (empty: all).", hint=FieldHint.feature)
    log: bool = Field(default=False, desc="Print tables to the log.", hint=FieldHint.logging)
    export: bool = Field(default=False, desc="Export a chrome trace.", hint=FieldHint.logging)

    @property
    def enabled(self) -> bool:
        return self.cpu or self.cuda

    def get_profiler(self, *, distributed_config=None, start_step: int = 0, run=None):
        if not self.enabled or (self.ranks and distributed_config is not None and distributed_config.rank not in self.ranks):
            return NoProfiler()
        import torch

        activities = ([torch.profiler.ProfilerActivity.CPU] if self.cpu else []) + ([torch.profiler.ProfilerActivity.CUDA] if self.cuda and torch.cuda.is_available() else [])
        if not activities:
            return NoProfiler()
        schedule = torch.profiler.schedule(skip_first=self.skip, wait=self.wait, warmup=self.warmup, active=self.cycles)
        step_holder = {"step": start_step}

        def on_trace_ready(profiler):
            step = step_holder["step"]
            if self.averages:
                table = profiler.key_averages().table(sort_by="self_cuda_time_total" if self.cuda else "self_cpu_time_total", row_limit=100, max_name_column_width=self.table_width)
                if self.log:
                    logger.info(table)
                if run is not None:
                    with run.open_artifact(f"profile_averages_step_{step}") as f:
                        f.write(table)
            if self.trace:
                events = sorted(profiler.events(), key=lambda e: e.time_range.start)
                text = "\n".join(f"{e.time_range.start:>16} {e.time_range.elapsed_us():>10.1f}us {e.name[: self.table_width]}" for e in events)
                if run is not None:
                    with run.open_artifact(f"profile_trace_step_{step}") as f:
                        f.write(text)
            if self.export and run is not None and run.experiment_directory is not None:
                with run.open_artifact(f"profile_chrome_step_{step}.json") as f:
                    path = f.name
                profiler.export_chrome_trace(path)

        profiler = torch.profiler.profile(activities=activities, schedule=schedule, on_trace_ready=on_trace_ready, with_modules=True)
        return _StepCountingProfiler(profiler, step_holder)


class NoProfiler:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def step(self):
        pass


class _StepCountingProfiler:
    def __init__(self, profiler, holder):
        self._profiler, self._holder = profiler, holder

    def __enter__(self):
        self._profiler.__enter__()
        return self

    def __exit__(self, *exc):
        return self._profiler.__exit__(*exc)

    def step(self):
        self._holder["step"] += 1
        self._profiler.step()
