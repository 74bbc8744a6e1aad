"""Assertion helpers with informative messages (parity: `fast_llm/utils.py:89-217` Assert namespace)."""

import typing


class Assert:
    @staticmethod
    def eq(x, *args, msg=None):
        for arg in args:
            assert x == arg, f"{x} != {arg}" + (f" ({msg})" if msg else "")

    @staticmethod
    def is_(x, y):
        assert x is y, f"{x} is not {y}"

    @staticmethod
    def geq(x, y):
        assert x >= y, f"{x} not >= {y}"

    @staticmethod
    def leq(x, y):
        assert x <= y, f"{x} not <= {y}"

    @staticmethod
    def gt(x, y):
        assert x > y, f"{x} not > {y}"

    @staticmethod
    def lt(x, y):
        assert x < y, f"{x} not < {y}"

    @staticmethod
    def in_range(x, low, high):
        assert low <= x < high, f"{x} not in range({low}, {high})"

    @staticmethod
    def in_range_incl(x, low, high):
        assert low <= x <= high, f"{x} not in range [{low}, {high}]"

    @staticmethod
    def none(x):
        assert x is None, f"Object of type {type(x)} is not None ({x})"

    @staticmethod
    def not_none(x):
        assert x is not None, "Unexpected None"

    @staticmethod
    def empty(x):
        assert len(x) == 0, f"Object of type {type(x)} is not empty ({x})"

    @staticmethod
    def incl(x, y):
        assert x in y, f"{x} not in {list(y)}"

    @staticmethod
    def not_incl(x, y):
        assert x not in y, f"{x} in {y}"

    @staticmethod
    def multiple(x, y):
        assert x % y == 0, f"{x} not a multiple of {y}"

    @staticmethod
    def rms_close(x, y, threshold):
        import torch

        rms = (x.float() - y.float()).pow(2).mean().sqrt().item()
        assert rms < threshold, f"Rms diff too big ({rms} > {threshold})"

    @staticmethod
    def rms_close_relative(x, y, threshold, min_threshold=0.0):
        scale = (x.float().pow(2).mean() + y.float().pow(2).mean()).sqrt().item() / 2**0.5
        Assert.rms_close(x, y, max(threshold * scale, min_threshold))

    @staticmethod
    def all_equal(x, *args):
        import torch

        for arg in args:
            a, b = torch.as_tensor(x), torch.as_tensor(arg)
            Assert.eq(a.shape, b.shape)
            assert bool((a == b).all()), f"Tensors differ: {(a != b).sum().item()} of {a.numel()} entries"

    @staticmethod
    def custom(fn: typing.Callable, *args, **kwargs):
        assert fn(*args, **kwargs), f"Assertion failed: fn({', '.join(map(str, args))})"

    @staticmethod
    def isinstance(x, cls):
        assert isinstance(x, cls), f"{x!r} is not an instance of {cls}"
