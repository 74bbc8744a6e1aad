"""Small host-side utilities (parity: `fast_llm/utils.py:220-492`)."""

import itertools
import logging
import signal
import typing

logger = logging.getLogger(__name__)


def div(x: int, y: int) -> int:
    """Exact integer division."""
    if x % y != 0:
        raise ValueError(f"{x} not divisible by {y}")
    return x // y


def get_unique(values: typing.Iterable):
    value = set(values)
    assert len(value) == 1, f"Expected a unique value, got {value}"
    return value.pop()


def padded_cumsum(x):
    import numpy as np

    y = np.hstack((0, np.asarray(x)))
    return y.cumsum(out=y)


def safe_merge_dicts(*dicts: dict) -> dict:
    out = {}
    for d in dicts:
        for k, v in d.items():
            if k in out and out[k] != v:
                raise ValueError(f"Conflicting values for key {k}: {out[k]} vs {v}")
            out[k] = v
    return out


class Registry:
    """Named collection of objects with helpful lookup errors."""

    def __init__(self, name: str, data: dict | None = None):
        self._name = name
        self._data = dict(data or {})

    def __getitem__(self, key):
        if key not in self._data:
            raise KeyError(f"Entry {key} not found in {self._name} registry (known: {sorted(map(str, self._data))})")
        return self._data[key]

    def __setitem__(self, key, value):
        if key in self._data:
            raise KeyError(f"Entry {key} already in {self._name} registry")
        self._data[key] = value

    def __contains__(self, key):
        return key in self._data

    def keys(self):
        return list(self._data)

    def items(self):
        return self._data.items()

    def get(self, key, default=None):
        return self._data.get(key, default)


def compare_nested(a, b, errors: list | None = None, prefix: tuple = ()) -> list:
    """Collect human-readable differences between two nested dict/list structures."""
    errors = [] if errors is None else errors
    if isinstance(a, dict) and isinstance(b, dict):
        for key in sorted(set(a) | set(b), key=str):
            if key not in a:
                errors.append(f"Missing on the left: {'.'.join(map(str, prefix + (key,)))}")
            elif key not in b:
                errors.append(f"Missing on the right: {'.'.join(map(str, prefix + (key,)))}")
            else:
                compare_nested(a[key], b[key], errors, prefix + (key,))
    elif isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        if len(a) != len(b):
            errors.append(f"Length mismatch at {'.'.join(map(str, prefix))}: {len(a)} != {len(b)}")
        for i, (x, y) in enumerate(zip(a, b)):
            compare_nested(x, y, errors, prefix + (i,))
    elif a != b:
        errors.append(f"Mismatch at {'.'.join(map(str, prefix))}: {a!r} != {b!r}")
    return errors


class Interrupter:
    """Turns SIGINT / SIGTERM into a flag so the training loop can checkpoint and leave cleanly."""

    def __init__(self, enabled: bool = True, signals=(signal.SIGINT, signal.SIGTERM)):
        self._enabled = enabled
        self._signals = signals
        self._active = False
        self._interrupted = False
        self._old = {}

    def __enter__(self):
        self._interrupted = False
        if self._enabled:
            self._active = True
            for sig in self._signals:
                try:
                    self._old[sig] = signal.signal(sig, self._handle)
                except ValueError:  # not in the main thread
                    self._active = False
        return self

    def __exit__(self, *exc):
        if self._active:
            for sig, old in self._old.items():
                signal.signal(sig, old)
        self._active = False
        self._old = {}

    def _handle(self, signum, frame):
        logger.warning(f"Interrupt signal {signal.Signals(signum).name} received; stopping at the next safe point.")
        self._interrupted = True

    @property
    def enabled(self) -> bool:
        return self._enabled

    @property
    def interrupted(self) -> bool:
        return self._interrupted


def set_global_variables(disable_torch_dynamo: bool = True) -> None:
    """Process-wide environment for reproducible, quiet runs."""
    import os

    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
    if disable_torch_dynamo:
        os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")


_memory_global_max = {"allocated": 0.0, "reserved": 0.0}


def get_and_reset_memory_usage_mib(relative_to: dict | None = None, reset_stats: bool = True, reset_global: bool = False) -> dict:
    import torch

    if not torch.cuda.is_available():
        return {}
    mib = 2**20
    report = {
        "allocated": torch.cuda.memory_allocated() / mib,
        "max_allocated": torch.cuda.max_memory_allocated() / mib,
        "reserved": torch.cuda.memory_reserved() / mib,
        "max_reserved": torch.cuda.max_memory_reserved() / mib,
    }
    _memory_global_max["allocated"] = max(_memory_global_max["allocated"], report["max_allocated"])
    _memory_global_max["reserved"] = max(_memory_global_max["reserved"], report["max_reserved"])
    report["global_max_reserved"] = _memory_global_max["reserved"]
    if relative_to:
        report = {k: v - relative_to.get(k, 0) for k, v in report.items()}
    if reset_stats:
        torch.cuda.reset_peak_memory_stats()
    if reset_global:
        _memory_global_max.update(allocated=0.0, reserved=0.0)
    return report


class InvalidObject:
    """Stand-in for an optional dependency that failed to import; raises on any use."""

    def __init__(self, error: Exception):
        self._error = error.__class__(*error.args)

    def __getattr__(self, item):
        raise self._error

    def __call__(self, *args, **kwargs):
        raise self._error


def try_decorate(get_decorator: typing.Callable, _return_decorator: bool = True):
    def wrapper(fn):
        try:
            return get_decorator()(fn)
        except Exception as e:
            return InvalidObject(e)

    return wrapper


def chunked(iterable, n):
    it = iter(iterable)
    while chunk := list(itertools.islice(it, n)):
        yield chunk
