"""The allocation-free entry point `flb_sumsq_no_alloc`, called through its exported C symbol.

Some hosts of the kernel library may not allocate device memory when they need a gradient norm (an allocator frozen for
the duration of a job, or an application that gave the library a fixed memory budget up front), so they cannot provide
the scratch buffer `flb_sumsq` asks for.  The variant keeps that scratch inside the library image.  It must agree with
the regular entry point, also on a second call that finds the first call's leftovers in the shared scratch.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_sumsq_matches_regular_entry_point_twice():
    from fast_llm_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.KERNEL_LIB_PATH))  # plain C ABI, no Python-side wrapper involved
    fn = lib.flb_sumsq_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    regular = lib.flb_sumsq
    regular.restype = ctypes.c_int
    regular.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.flb_sumsq_scratch_floats.restype = ctypes.c_int

    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    scratch = torch.empty(lib.flb_sumsq_scratch_floats(), dtype=torch.float32, device="cuda")
    # two different inputs back to back: the second call sees the partial sums the first one left behind
    for n, scale in ((3_000_003, 1.0), (70_001, 7.0)):
        x = torch.randn(n, device="cuda") * scale
        expected = torch.zeros(1, device="cuda")
        got = torch.zeros(1, device="cuda")
        assert regular(x.data_ptr(), n, scratch.data_ptr(), expected.data_ptr(), 0, stream) == 0
        assert fn(x.data_ptr(), n, got.data_ptr(), 0, stream) == 0
        torch.cuda.synchronize()
        assert got.item() == expected.item()  # same kernels, same reduction order: bit-identical
        reference = x.double().pow(2).sum().item()
        assert abs(got.item() - reference) / reference < 1e-5
        # accumulate mode adds to what is there
        assert fn(x.data_ptr(), n, got.data_ptr(), 1, stream) == 0
        torch.cuda.synchronize()
        assert abs(got.item() - 2 * reference) / reference < 2e-5
    # sizes beyond the stated maximum are refused, nothing is launched
    assert fn(x.data_ptr(), (1 << 32) + 1, got.data_ptr(), 0, stream) == 4
    assert fn(x.data_ptr() + 4, 16, got.data_ptr(), 0, stream) == 1
