"""AdamW over flat shard slices with global-norm clipping and loss scaling, entirely on the device.

Per step: unscale check -> squared norm of every gradient-shard slice (deterministic two-stage reduction) ->
all-reduce over the world -> a one-thread kernel turns it into the clip coefficient -> one fused Adam launch per
parameter group reads the coefficient through a pointer and writes fp32 master weights, moments and the bf16 weight
buffer slice.  No `.item()` on the way.  Parity: `fast_llm/engine/optimizer/optimizer.py:53-311`.
"""

import logging

import torch

from fast_llm_b200.engine.optimizer.config import GradientScalerConfig, OptimizerConfig
from fast_llm_b200.engine.optimizer.learning_rate import create_schedule_from_config
from fast_llm_b200.ops.optim import adamw, clip_coeff, sum_partials, sumsq
from fast_llm_b200.parallel.collectives import all_reduce

logger = logging.getLogger(__name__)


class GradScaler:
    """No scaling."""

    def __init__(self, scale: float = 1.0, distributed=None):
        self._scale = scale
        self._distributed = distributed

    # Name written as `type` in the optimizer metadata; the reference writes its own class names there
    # (`fast_llm/engine/optimizer/optimizer.py:160-170`), so checkpoints resume in either framework.
    type_name = "NoopGradScaler"

    @property
    def grad_scale(self) -> float:
        return self._scale

    def state_dict(self) -> dict:
        return {"type": self.type_name}

    def load(self, state: dict, validate: bool = True) -> None:
        if validate and "type" in state and state["type"] != self.type_name:
            raise ValueError(f"Gradient scaler mismatch: checkpoint has {state['type']}, this run uses {self.type_name}")

    def check_overflow(self, grad_slices) -> bool:
        return False

    def update(self, found_overflow: bool) -> None:
        pass


class ConstantGradScaler(GradScaler):
    type_name = "ConstantGradScaler"

    def state_dict(self) -> dict:
        return {"type": self.type_name, "scale": self._scale}

    def load(self, state: dict, validate: bool = True) -> None:
        super().load(state, validate)
        self._scale = state.get("scale", self._scale)


class DynamicGradScaler(GradScaler):
    """fp16 loss scaling: halve after `hysteresis` overflowing steps, double after `window` clean ones."""

    def __init__(self, config: GradientScalerConfig, distributed=None):
        super().__init__(config.initial, distributed)
        self._config = config
        self._growth_tracker = 0
        self._hysteresis_tracker = config.hysteresis

    type_name = "DynamicGradScaler"

    def state_dict(self):
        return {"type": self.type_name, "scale": self._scale, "growth": self._growth_tracker, "hysteresis": self._hysteresis_tracker}

    def load(self, state, validate: bool = True):
        super().load(state, validate)
        self._scale = state.get("scale", self._scale)
        # `growth_tracker` / `hysteresis_tracker` are the key names of older checkpoints of this framework
        self._growth_tracker = state.get("growth", state.get("growth_tracker", 0))
        self._hysteresis_tracker = state.get("hysteresis", state.get("hysteresis_tracker", self._config.hysteresis))

    def check_overflow(self, grad_slices) -> bool:
        flag = torch.zeros(1, dtype=torch.float32, device=grad_slices[0].device if grad_slices else "cpu")
        for g in grad_slices:
            flag += (~torch.isfinite(g)).any().float()
        if self._distributed is not None:
            all_reduce(flag, group=self._distributed.world_group)
        return bool(flag.item() > 0)

    def update(self, found_overflow: bool) -> None:
        if found_overflow:
            self._growth_tracker = 0
            self._hysteresis_tracker -= 1
            if self._hysteresis_tracker <= 0:
                self._scale = max(self._scale / 2, self._config.minimum)
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= self._config.window:
                self._growth_tracker = 0
                self._hysteresis_tracker = self._config.hysteresis
                self._scale *= 2


def get_grad_scaler(config: GradientScalerConfig, compute_dtype: torch.dtype, distributed=None) -> GradScaler:
    if config.constant is not None and config.constant > 0:
        return ConstantGradScaler(config.constant, distributed)
    if compute_dtype == torch.float16:
        return DynamicGradScaler(config, distributed)
    return GradScaler(1.0, distributed)


class Optimizer:
    def __init__(self, config: OptimizerConfig, param_groups: list[dict], grad_norm_slices: list[torch.Tensor], distributed,
                 compute_dtype: torch.dtype = torch.float32, weight_arena=None, grad_norm_partials: torch.Tensor | None = None):
        config.validate()
        self._config = config
        self._param_groups = param_groups
        self._grad_norm_slices = grad_norm_slices
        self._distributed = distributed
        # weight buffers in NVLink symmetric memory: Adam pushes the new bf16 weights to every data-parallel peer
        self._weight_arena = weight_arena
        # per-block sums of squares of every reduced gradient shard, left by the fused reduction kernels
        self._grad_norm_partials = grad_norm_partials
        # stage index -> event recorded once every data rank's new weights of that stage have landed in the buffers
        self.stage_ready_events: dict[int, torch.cuda.Event] = {}
        self._lr_schedule = create_schedule_from_config(config.learning_rate)
        self._current_step = 0
        self._grad_scaler = get_grad_scaler(config.gradient_scaler, compute_dtype, distributed)
        device = distributed.device
        self._normsq = torch.zeros(1, dtype=torch.float32, device=device)
        self._coeff = torch.ones(1, dtype=torch.float32, device=device)
        self._norm = torch.zeros(1, dtype=torch.float32, device=device)

    @property
    def pushes_weights_to_peers(self) -> bool:
        return self._weight_arena is not None

    @property
    def grad_scale(self) -> float:
        return self._grad_scaler.grad_scale

    @property
    def current_step(self) -> int:
        return self._current_step

    @property
    def grad_norm(self) -> torch.Tensor:
        return self._norm

    def learning_rate(self, step: int | None = None) -> float:
        return self._lr_schedule(self._current_step if step is None else step)

    def _compute_clip_coefficient(self) -> None:
        first = True
        if self._grad_norm_partials is not None:
            sum_partials(self._grad_norm_partials, self._normsq)
            first = False
        else:
            for g in self._grad_norm_slices:
                if g.numel():
                    sumsq(g, self._normsq, accumulate=not first)
                    first = False
        if first:
            self._normsq.zero_()
        all_reduce(self._normsq, group=self._distributed.world_group)
        clip_coeff(self._normsq, self._config.gradient_norm_clipping, 1.0 / self._grad_scaler.grad_scale, self._coeff, self._norm)

    @torch.no_grad()
    def step(self, metrics: dict | None = None) -> bool:
        """Returns True if the weights were updated (False when an fp16 overflow skipped the step)."""
        overflow = self._grad_scaler.check_overflow([g["grads"] for g in self._param_groups])
        self._grad_scaler.update(overflow)
        if metrics is not None:
            metrics["loss_scale"] = self._grad_scaler.grad_scale
        if overflow:
            return False
        self._current_step += 1
        lr = self._lr_schedule(self._current_step)
        self._compute_clip_coefficient()
        c = self._config
        self.stage_ready_events.clear()
        for index, group in enumerate(self._param_groups):
            lr_scale = c.default_learning_rate_scale if group["lr_scale"] is None else group["lr_scale"]
            wd = c.weight_decay if group["weight_decay"] else 0.0
            if self._weight_arena is not None and group.get("buffer") is not None and group["params"].numel() % 4 == 0:
                from fast_llm_b200.parallel.symmetric import adam_push

                adam_push(self._weight_arena, group["params"], group["grads"], group["exp_avgs"], group["exp_avgs_sq"],
                          group["buffer"], lr * lr_scale, c.beta_1, c.beta_2, c.epsilon, wd, self._current_step, self._coeff)
            else:
                assert self._weight_arena is None, "parameter group not aligned for the fused update"
                adamw(group["params"], group["grads"], group["exp_avgs"], group["exp_avgs_sq"], group.get("buffer"),
                      lr * lr_scale, c.beta_1, c.beta_2, c.epsilon, wd, self._current_step, 1.0, self._coeff)
            stage = group.get("stage")
            last_of_stage = index + 1 == len(self._param_groups) or self._param_groups[index + 1].get("stage") != stage
            if self._weight_arena is not None and last_of_stage:
                # Every rank's pushes of this stage have landed once all ranks pass this barrier.  One barrier per stage (not
                # one at the end) lets the next step's first forwards start while the later stages are still being updated.
                self._weight_arena.barrier(1)
                if stage is not None:
                    event = torch.cuda.Event()
                    event.record()
                    self.stage_ready_events[stage] = event
        if metrics is not None:
            metrics["learning_rate"] = lr
            metrics["grad_norm"] = self._norm  # device tensor; converted when logged
        return True

    def save(self) -> dict:
        return {"current_step": self._current_step, "grad_scaler": self._grad_scaler.state_dict()}

    def load(self, state: dict, validate: bool = True) -> None:
        self._current_step = state.get("current_step", 0)
        self._grad_scaler.load(state.get("grad_scaler", {}), validate)

    def reset_state(self) -> None:
        self._current_step = 0
        for group in self._param_groups:
            group["exp_avgs"].zero_()
            group["exp_avgs_sq"].zero_()
