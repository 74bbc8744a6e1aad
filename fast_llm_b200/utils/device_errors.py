"""Error words of bounded device-side waits, read where the host synchronises anyway.

Every kernel of this library that waits (a peer's barrier flag, an mbarrier of a TMA / tensor-core pipeline) gives up after
a limit, records a code in an error word and returns, so that a missing peer or a lost copy cannot hang the GPU.  The
price is that somebody has to read the words: the kernels that follow a failed barrier leave memory untouched, but the
step they belonged to is wrong.  Sources register here; the trainer calls `check_device_errors` at the logging interval,
before every checkpoint and export and at the end of training, and every rank raises if any rank saw a failure.
"""

import typing
import weakref

import torch


class DeviceWaitError(RuntimeError):
    """A bounded device-side wait ran out on this or another rank."""


# name -> callable returning a description of the failure, or None when the source is clean.  Reading may synchronise.
_sources: dict[str, typing.Callable[[], str | None]] = {}


def register_error_source(name: str, read: typing.Callable[[], str | None]) -> None:
    _sources[name] = read


def unregister_error_source(name: str) -> None:
    _sources.pop(name, None)


def register_object_source(name: str, obj, method: str) -> None:
    """Register `getattr(obj, method)` without keeping `obj` alive; the source disappears with the object."""
    ref = weakref.ref(obj)

    def read():
        target = ref()
        if target is None:
            _sources.pop(name, None)
            return None
        return getattr(target, method)()

    _sources[name] = read


def read_device_errors() -> dict[str, str]:
    """Failures recorded since the last read, by source (each source clears itself when read)."""
    found = {}
    for name, read in list(_sources.items()):
        message = read()
        if message:
            found[name] = message
    return found


def check_device_errors(group=None, device: torch.device | None = None) -> None:
    """Raise `DeviceWaitError` on EVERY rank of `group` if any rank recorded a failed wait."""
    found = read_device_errors()
    failed = bool(found)
    if group is not None and torch.distributed.is_initialized() and group.size() > 1:
        flag = torch.tensor([int(failed)], dtype=torch.int32, device=device if device is not None else "cpu")
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX, group=group)
        failed = bool(flag.item())
    if failed:
        detail = "; ".join(f"{k}: {v}" for k, v in found.items()) or "reported by another rank"
        raise DeviceWaitError(f"A bounded device-side wait ran out ({detail}); the results of the steps since the last check are invalid")


def _gemm_source() -> str | None:
    from fast_llm_b200.ops import _lib

    word = _lib.get_lib().flb_gemm_error_word()
    return f"tcgen05 GEMM gave up on a pipeline barrier (role code {word}; 15: rows of a tensor-parallel peer did not arrive)" if word > 0 else None


def _attention_source() -> str | None:
    from fast_llm_b200.ops import _lib

    lib = _lib.get_lib()
    fwd, bwd = lib.flb_attention_error_word(), lib.flb_attention_bwd_error_word()
    if fwd > 0 or bwd > 0:
        return f"attention kernel gave up on a pipeline barrier (forward code {fwd}, backward code {bwd})"
    return None


def _norm_source() -> str | None:
    from fast_llm_b200.ops import _lib

    if _lib.get_lib().flb_norm_error_word() > 0:
        return "a normalisation kernel gave up waiting for one of its row copies into shared memory"
    return None


def register_kernel_library_sources() -> None:
    """The error words that live inside the kernel library (GEMM, attention and normalisation pipelines); needs a GPU and the library."""
    register_error_source("gemm", _gemm_source)
    register_error_source("attention", _attention_source)
    register_error_source("normalisation", _norm_source)
