"""Thin collective wrappers that treat `group=None` as a single-rank group (no-op), plus scalar / object helpers.

Parity: `fast_llm/core/distributed.py:22-369`.
"""

import contextlib
import datetime
import io
import logging
import pickle

import torch
import torch.distributed as dist
from torch.distributed import ProcessGroup, ReduceOp

logger = logging.getLogger(__name__)


def group_size(group: ProcessGroup | None) -> int:
    return 1 if group is None else group.size()


def group_rank(group: ProcessGroup | None) -> int:
    return 0 if group is None else group.rank()


def _global_rank(group: ProcessGroup, group_rank_: int) -> int:
    return dist.get_global_rank(group, group_rank_)


@contextlib.contextmanager
def set_timeout(group: ProcessGroup | None, timeout: float | None = None):
    """Temporarily extend the timeout of a group's operations (slow ops such as checkpointing)."""
    if group is not None and timeout is not None and hasattr(group, "_set_default_timeout"):
        try:
            group._set_default_timeout(datetime.timedelta(seconds=timeout))
            yield
        finally:
            group._set_default_timeout(datetime.timedelta(seconds=dist.default_pg_timeout.total_seconds()))
    else:
        yield


def all_reduce(tensor: torch.Tensor, op=ReduceOp.SUM, group: ProcessGroup | None = None, async_op: bool = False):
    if group is None:
        return None
    if op == ReduceOp.AVG and dist.get_backend(group) == "gloo":
        work = dist.all_reduce(tensor, op=ReduceOp.SUM, group=group, async_op=False)
        tensor.div_(group.size())
        return None
    return dist.all_reduce(tensor, op=op, group=group, async_op=async_op)


def broadcast(tensor: torch.Tensor, src: int, group: ProcessGroup | None, async_op: bool = False):
    """`src` is a rank *within the group*."""
    if group is None:
        return None
    return dist.broadcast(tensor, src=_global_rank(group, src), group=group, async_op=async_op)


def all_gather_into_tensor(output: torch.Tensor, input_: torch.Tensor, group: ProcessGroup | None, async_op: bool = False):
    if group is None:
        output.copy_(input_.view_as(output))
        return None
    return dist.all_gather_into_tensor(output, input_, group=group, async_op=async_op)


def reduce_scatter_tensor(output: torch.Tensor, input_: torch.Tensor, op=ReduceOp.SUM, group: ProcessGroup | None = None,
                          async_op: bool = False):
    if group is None:
        output.copy_(input_.view_as(output))
        return None
    if dist.get_backend(group) == "gloo":
        # Gloo has no reduce-scatter: all-reduce a copy and keep this rank's slice.
        tmp = input_.clone()
        dist.all_reduce(tmp, op=ReduceOp.SUM, group=group)
        n = output.numel()
        output.copy_(tmp.view(-1)[group.rank() * n : (group.rank() + 1) * n].view_as(output))
        if op == ReduceOp.AVG:
            output.div_(group.size())
        return None
    return dist.reduce_scatter_tensor(output, input_, op=op, group=group, async_op=async_op)


def send(tensor: torch.Tensor, dst: int, group: ProcessGroup, async_op: bool = False, tag: int = 0):
    dst = _global_rank(group, dst)
    if async_op:
        return dist.isend(tensor, dst=dst, group=group, tag=tag)
    dist.send(tensor, dst=dst, group=group, tag=tag)
    return None


def recv(tensor: torch.Tensor, src: int, group: ProcessGroup, async_op: bool = False, tag: int = 0):
    src = _global_rank(group, src)
    if async_op:
        return dist.irecv(tensor, src=src, group=group, tag=tag)
    dist.recv(tensor, src=src, group=group, tag=tag)
    return None


def allreduce_scalar(value: float | int, dtype: torch.dtype = torch.float64, group: ProcessGroup | None = None,
                     op=ReduceOp.SUM, device=None):
    if group is None:
        return value
    dev = device or ("cuda" if dist.get_backend(group) == "nccl" else "cpu")
    t = torch.full([1], value, dtype=dtype, device=dev)
    dist.all_reduce(t, op=op, group=group)
    return t.item()


def all_gather_scalar(value: float | int, dtype: torch.dtype = torch.float64, group: ProcessGroup | None = None, device=None):
    if group is None:
        return [value]
    dev = device or ("cuda" if dist.get_backend(group) == "nccl" else "cpu")
    t = torch.full([1], value, dtype=dtype, device=dev)
    out = t.new_empty([group.size()])
    dist.all_gather_into_tensor(out, t, group=group)
    return out.tolist()


def broadcast_scalar(value: float | int, dtype: torch.dtype = torch.float64, group: ProcessGroup | None = None, src: int = 0, device=None):
    if group is None:
        return value
    dev = device or ("cuda" if dist.get_backend(group) == "nccl" else "cpu")
    t = torch.full([1], value if group.rank() == src else 0, dtype=dtype, device=dev)
    broadcast(t, src, group)
    return t.item()


def broadcast_object(obj, group: ProcessGroup | None, src: int = 0):
    if group is None:
        return obj
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    if group.rank() == src:
        payload = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8).to(dev)
        size = torch.tensor([payload.numel()], dtype=torch.int64, device=dev)
        broadcast(size, src, group)
        broadcast(payload, src, group)
        return obj
    size = torch.zeros(1, dtype=torch.int64, device=dev)
    broadcast(size, src, group)
    payload = torch.empty(int(size.item()), dtype=torch.uint8, device=dev)
    broadcast(payload, src, group)
    return pickle.load(io.BytesIO(payload.cpu().numpy().tobytes()))


def gather_object(obj, group: ProcessGroup | None, dst: int = 0):
    if group is None:
        return [obj]
    out = [None] * group.size() if group.rank() == dst else None
    dist.gather_object(obj, out, dst=_global_rank(group, dst), group=group)
    return out


def safe_barrier(group: ProcessGroup | None, value: int | str = 1, timeout: float | None = None, device=None) -> None:
    """Barrier that also detects desynchronised ranks: every rank must arrive with the same tag."""
    if group is None:
        return
    import zlib

    hashed = zlib.crc32(str(value).encode())  # stable across processes (str hashes are salted per process)
    with set_timeout(group, timeout):
        total = allreduce_scalar(hashed, dtype=torch.int64, group=group, device=device)
    if total != hashed * group.size():
        raise RuntimeError(f"Desync detected at barrier {value!r}: ranks arrived at different barriers")


def check_parallel_match(tensor: torch.Tensor, group: ProcessGroup | None, name: str) -> bool:
    """Debug helper: log when a tensor that should be replicated over `group` differs between its ranks."""
    if group is None:
        return True
    flat = tensor.contiguous().view(-1)
    gathered = flat.new_empty(group.size() * flat.numel())
    dist.all_gather_into_tensor(gathered, flat, group=group)
    mismatches = (gathered.view(group.size(), -1) != flat[None]).any(dim=0).sum().item()
    if mismatches:
        logger.error(f"MISMATCH {name}: {mismatches} of {tensor.numel()} entries differ between ranks")
    return mismatches == 0


@contextlib.contextmanager
def set_generator(generator: torch.Generator):
    """Make `generator` the default RNG of its device for the duration of the block."""
    default = torch.cuda.default_generators[generator.device.index] if generator.device.type == "cuda" else torch.default_generator
    if default is generator:
        yield
        return
    old = default.get_state()
    default.set_state(generator.get_state())
    try:
        yield
    finally:
        generator.set_state(default.get_state())
        default.set_state(old)
