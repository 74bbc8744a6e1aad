"""Tensor logging for debugging and parity tests (parity: `fast_llm/logging.py:127-343`,
`fast_llm/engine/config_utils/logging.py:61-98`): a line per tensor with summary statistics, optionally stored so a run
can be compared tensor by tensor with another layout."""

import logging

import torch

logger = logging.getLogger(__name__)


class TensorLogs:
    enabled = False
    save = False
    show = True
    max_elements = 8
    full_tensors = False
    _logs: list[dict] = []

    @classmethod
    def reset(cls, save=False, show=True, max_elements=8, full_tensors=False):
        cls.enabled = True
        cls.save, cls.show, cls.max_elements, cls.full_tensors = save, show, max_elements, full_tensors
        cls._logs = []

    @classmethod
    def append(cls, stats: dict):
        cls._logs.append(stats)

    @classmethod
    def get(cls):
        return cls._logs

    @classmethod
    def clear(cls):
        cls._logs = []


def log_tensor(name: str, tensor: torch.Tensor, *, level: int = 2, scale: float = 1.0, log_fn=logger.info, storage: bool = True):
    if level < 1 or not torch.is_tensor(tensor):
        return None
    t = tensor.detach().float()
    if scale != 1.0:
        t = t * scale
    stats = {"name": name, "shape": list(tensor.shape), "dtype": str(tensor.dtype), "device": str(tensor.device)}
    if t.numel():
        stats.update(mu=t.mean().item(), std=t.std().item() if t.numel() > 1 else 0.0, min=t.min().item(), max=t.max().item(),
                     step=max(t.numel() // TensorLogs.max_elements, 1))
        if level >= 3:
            stats["samples"] = t.flatten()[:: stats["step"]][: TensorLogs.max_elements].tolist()
        if TensorLogs.full_tensors:
            stats["tensor"] = t.cpu()
    if TensorLogs.save and storage:
        TensorLogs.append(stats)
    if TensorLogs.show and log_fn is not None:
        text = f"{name:50s} shape={tuple(tensor.shape)} dtype={str(tensor.dtype):14s}"
        if t.numel():
            text += f" mu={stats['mu']:.6g} std={stats['std']:.6g} min={stats['min']:.6g} max={stats['max']:.6g}"
            if "samples" in stats:
                text += " samples=" + ",".join(f"{s:.5g}" for s in stats["samples"])
        log_fn(text)
    return stats


def log_grad(name: str, tensor: torch.Tensor, *, level: int = 2, scale: float = 1.0, log_fn=logger.info):
    if level < 1 or not tensor.requires_grad:
        return
    tensor.register_hook(lambda grad: log_tensor(name, grad, level=level, scale=scale, log_fn=log_fn) and None)


def log_distributed_tensor(name: str, tensor: torch.Tensor, *, level: int = 2, scale: float = 1.0, log_fn=logger.info, storage: bool = True,
                           shard_group=None, shard_dim: int = 0, duplicate_groups: tuple = (), global_: bool = True):
    """Log a tensor of which every rank of `shard_group` holds one slice along `shard_dim` (sequence-parallel activations, a
    tensor-parallel weight) and which is replicated over `duplicate_groups`.  With `global_` the slices are gathered and the
    whole tensor is logged once, by the first rank of all the groups, so the line (and the stored record) is the one a
    single-process run produces: logs of different parallel layouts can be compared record by record.  Otherwise every rank
    logs its own slice.  Every rank of the groups must make the call (the gather is a collective).
    Parity: `fast_llm/logging.py:247-277`."""
    if level < 1 or not torch.is_tensor(tensor):
        return None
    if not global_:
        return log_tensor(f"Local {name}", tensor, level=level, scale=scale, log_fn=log_fn, storage=storage)
    if shard_group is not None and shard_group.size() > 1:
        from fast_llm_b200.parallel.ops import gather_op

        tensor = gather_op(tensor.detach().contiguous(), shard_group, shard_dim)
    first = (shard_group is None or shard_group.rank() == 0) and all(g is None or g.rank() == 0 for g in duplicate_groups)
    if not first:
        return None
    return log_tensor(f"Global {name}", tensor, level=level, scale=scale, log_fn=log_fn, storage=storage)


def log_distributed_grad(name: str, tensor: torch.Tensor, *, level: int = 2, scale: float = 1.0, log_fn=logger.info, storage: bool = True,
                         shard_group=None, shard_dim: int = 0, duplicate_groups: tuple = (), global_: bool = True, grad_fn=None):
    """The same for the gradient that reaches `tensor` during backward (parity: `fast_llm/logging.py:280-307`)."""
    if level < 1 or not tensor.requires_grad:
        return
    tensor.register_hook(lambda grad: log_distributed_tensor(
        name, grad if grad_fn is None else grad_fn(grad), level=level, scale=scale, log_fn=log_fn, storage=storage, shard_group=shard_group,
        shard_dim=shard_dim, duplicate_groups=duplicate_groups, global_=global_) and None)


def log_generator(name: str, generator: "torch.Generator | torch.Tensor | None" = None, log_fn=logger.info):
    """The last words of a generator's state: equal on ranks (or runs) whose random streams are in step."""
    if generator is None:
        generator = torch.cuda.default_generators[torch.cuda.current_device()] if torch.cuda.is_available() else torch.random.default_generator
    state = generator.get_state() if isinstance(generator, torch.Generator) else generator
    return log_fn(f"{name} {state.view(torch.int64)[-8:].tolist() if state.numel() % 8 == 0 else int(state.long().sum())}")


def log_memory_usage(header: str, log_fn=logger.info):
    from fast_llm_b200.utils.misc import get_and_reset_memory_usage_mib

    report = get_and_reset_memory_usage_mib(reset_stats=False)
    return log_fn(f"{header}: " + ", ".join(f"{k} {v:,.0f} MiB" for k, v in report.items()))
