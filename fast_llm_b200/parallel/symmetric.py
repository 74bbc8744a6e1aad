"""Symmetric memory over NVLink: buffers that exist at the same offset on every rank of a group and are mapped into
every process, so kernels address peers directly.

Allocation and the exchange of handles use `torch.distributed._symmetric_memory` (plumbing); everything that runs on
the data path - the barrier, the gradient reduction, the Adam update that pushes weights to peers - are this library's
own kernels (`csrc/zero_fused.cu`).  Device-side waits are bounded and report through an error word.
"""

import ctypes
import os
import logging

import torch

from fast_llm_b200.ops import _lib

logger = logging.getLogger(__name__)

_SIGNAL_SLOTS = 8
# One error word per device, shared by every arena of the process: a barrier of the gradient arena that gives up must
# also stop the Adam kernel that pushes through the weight arena.
_error_words: dict[int, torch.Tensor] = {}


def shared_error_word(device: torch.device) -> torch.Tensor:
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if index not in _error_words:
        from fast_llm_b200.utils.device_errors import register_error_source

        _error_words[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        register_error_source(f"symmetric_memory_cuda{index}", lambda: read_error_word(index))
    return _error_words[index]


def read_error_word(index: int) -> str | None:
    """Description of a device-side barrier that gave up since the last read (clears the word; synchronises)."""
    word = int(_error_words[index].item())
    if not word:
        return None
    _error_words[index].zero_()
    return f"a symmetric-memory barrier on cuda:{index} timed out waiting for rank {word - 100} of its group"


def set_barrier_limit_seconds(seconds: float, sm_clock_hz: float = 2.0e9) -> float:
    """Longest wait of later device-side barriers (default about 10 s); returns the previous limit in seconds.
    The kernel counts SM clock cycles, `sm_clock_hz` converts (the boost clock gives the shortest wait)."""
    old = _lib.get_lib().flb_symm_set_barrier_limit(max(int(seconds * sm_clock_hz), 1))
    return old / sm_clock_hz


class SymmetricArena:
    """One symmetric allocation of `nbytes` per rank plus a signal pad for barriers."""

    def __init__(self, nbytes: int, group, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world_size = group.size()
        self.rank = group.rank()
        self.device = device
        lib = _lib.get_lib()
        assert self.world_size <= lib.flb_symm_max_ranks()
        nbytes = (nbytes + 255) // 256 * 256
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self._handle = symm_mem.rendezvous(self.buffer, group)
        self.peer_ptrs = [int(p) for p in self._handle.buffer_ptrs]
        assert self.peer_ptrs[self.rank] == self.buffer.data_ptr()
        # one address for the same offset in every rank's allocation (NVLink multicast through NVSwitch); 0 where the fabric
        # or the driver has none
        self.multicast_ptr = int(getattr(self._handle, "multicast_ptr", 0) or 0)
        pad_bytes = lib.flb_symm_signal_pad_bytes(_SIGNAL_SLOTS)
        self._pad = symm_mem.empty(pad_bytes, dtype=torch.uint8, device=device)
        self._pad.zero_()
        self._pad_handle = symm_mem.rendezvous(self._pad, group)
        self._pad_ptrs = (ctypes.c_void_p * self.world_size)(*[int(p) for p in self._pad_handle.buffer_ptrs])
        self._epochs = [0] * _SIGNAL_SLOTS
        self.error_word = shared_error_word(device)
        torch.cuda.synchronize(device)
        torch.distributed.barrier(group)  # pads are zeroed everywhere before the first device-side barrier

    def peer_pointer_array(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.world_size)(*[p + byte_offset for p in self.peer_ptrs])

    def offset_of(self, tensor: torch.Tensor) -> int:
        off = tensor.data_ptr() - self.buffer.data_ptr()
        assert 0 <= off < self.buffer.numel(), "tensor is not inside this arena"
        return off

    def barrier(self, slot: int = 0) -> None:
        """Stream-ordered barrier of the group on the current stream (bounded wait)."""
        self._epochs[slot] += 1
        _lib.check(_lib.get_lib().flb_symm_barrier(self._pad_ptrs, self.rank, self.world_size, slot, self._epochs[slot],
                                                   self.error_word.data_ptr(), _lib.stream_ptr()), "flb_symm_barrier")
        _lib.count_launch()

    def check_errors(self) -> None:
        message = read_error_word(self.error_word.device.index)
        if message:
            raise RuntimeError(message)


def symmetric_memory_available(group, device) -> bool:
    if group is None or device.type != "cuda":
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401

        return torch.distributed.get_backend(group) == "nccl"
    except Exception:
        return False


def multimem_reduction_enabled() -> bool:
    """`FLB_ZERO_MULTIMEM=1`: gradient reduce-scatter through `multimem.ld_reduce` (in-switch sums).  Off by default: the order of
    the additions is the switch's, so results are not bit-identical to the rank-ordered kernel, and a rank that dies while its
    memory is bound to a multicast object disturbs its peers (runs that test failures keep this off)."""
    return os.environ.get("FLB_ZERO_MULTIMEM", "0") == "1"


def rs_reduce(arena: SymmetricArena, grad_buffer: torch.Tensor, grad_shard: torch.Tensor, shard_size: int, scale: float,
              accumulate: bool, sumsq_partial: torch.Tensor | None) -> None:
    """grad_shard (+)= scale * sum over ranks of their grad_buffer[rank*shard : (rank+1)*shard] (peer loads)."""
    if multimem_reduction_enabled() and arena.multicast_ptr and grad_buffer.dtype == torch.float32:
        # the sum is formed inside NVSwitch: this rank pulls its slice once instead of once per peer
        _lib.check(_lib.get_lib().flb_rs_reduce_multimem(arena.multicast_ptr + arena.offset_of(grad_buffer), arena.rank, arena.world_size, shard_size,
                                                         scale, grad_shard.data_ptr(), int(accumulate), _lib.ptr(sumsq_partial),
                                                         arena.error_word.data_ptr(), _lib.stream_ptr()), "flb_rs_reduce_multimem")
        _lib.count_launch()
        return
    ptrs = arena.peer_pointer_array(arena.offset_of(grad_buffer))
    dtype_code = 0 if grad_buffer.dtype == torch.float32 else 1
    _lib.check(_lib.get_lib().flb_rs_reduce(ptrs, dtype_code, arena.rank, arena.world_size, shard_size, scale,
                                            grad_shard.data_ptr(), int(accumulate), _lib.ptr(sumsq_partial), arena.error_word.data_ptr(),
                                            _lib.stream_ptr()), "flb_rs_reduce")
    _lib.count_launch()


def adam_push(arena: SymmetricArena, w, g, m, v, buffer_slice: torch.Tensor, lr, beta1, beta2, eps, wd, step, gscale_tensor) -> None:
    """AdamW on this rank's shard slice; the bf16 weights land in the same slice of every rank's weight buffer."""
    byte_offset = arena.offset_of(buffer_slice)
    assert byte_offset % 2 == 0
    ptrs = arena.peer_pointer_array(0)
    _lib.check(_lib.get_lib().flb_adam_push(w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), ptrs, arena.world_size,
                                            byte_offset // 2, w.numel(), lr, beta1, beta2, eps, wd, step, 1.0,
                                            _lib.ptr(gscale_tensor), arena.error_word.data_ptr(), _lib.stream_ptr()), "flb_adam_push")
    _lib.count_launch()
