"""bf16 GEMMs on the tcgen05 tensor cores (`csrc/gemm_tcgen05.cu`) with a PyTorch path for CPU tensors.

Three contractions cover training (parity with the dense paths of the reference's `fast_llm/functional/linear.py:27-107`,
which calls cuBLAS through `torch.nn.functional.linear` / `addmm`):

    matmul_nt(x, w)            y  = x @ w.T          forward            (both operands K-major)
    matmul_nn(dy, w)           dx = dy @ w           input gradient     (B is MN-major in memory)
    matmul_tn(dy, x, out=...)  dw (+)= dy.T @ x      weight gradient    (both operands MN-major), accumulates in place
"""

import os

import torch

from fast_llm_b200.ops import _lib

_EPI_STORE_BF16, _EPI_STORE_F32, _EPI_ACC_F32, _EPI_ACC_BF16 = 0, 1, 2, 3


def _backend() -> str:
    return os.environ.get("FLB_GEMM", "tcgen05")


def _native_ok(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (
        a.is_cuda
        and a.dtype == torch.bfloat16
        and b.dtype == torch.bfloat16
        and _backend() == "tcgen05"
        and a.stride(-1) == 1
        and b.stride(-1) == 1
        and a.stride(0) % 8 == 0
        and b.stride(0) % 8 == 0
        and a.data_ptr() % 16 == 0
        and b.data_ptr() % 16 == 0
    )


library_fallbacks: dict[str, int] = {}  # reason -> number of CUDA GEMMs that went to torch.matmul (cuBLAS) instead


def _note_library_fallback(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """A CUDA GEMM that the tcgen05 kernels do not take is counted and announced once per reason: nothing falls back silently."""
    if not a.is_cuda:
        return
    if _backend() != "tcgen05":
        reason = f"FLB_GEMM={_backend()}"
    elif a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        reason = f"operand dtypes {a.dtype}, {b.dtype} (the tcgen05 kernels take bf16)"
    elif a.stride(-1) != 1 or b.stride(-1) != 1 or out.stride(-1) != 1:
        reason = "an operand whose last dimension is not contiguous"
    else:
        reason = "an operand that is not 16-byte aligned or whose row stride is not a multiple of 8 elements"
    count = library_fallbacks.get(reason, 0)
    library_fallbacks[reason] = count + 1
    if count == 0:
        import logging

        logging.getLogger(__name__).warning(f"GEMM runs on torch.matmul (cuBLAS), not on the tcgen05 kernels: {reason}; "
                                            f"shapes {tuple(a.shape)} x {tuple(b.shape)}.  Further ones of this kind are only counted "
                                            f"(`fast_llm_b200.ops.gemm.library_fallbacks`).")


def gemm_raw(a, b, out, m, n, k, a_mn, b_mn, epilogue, block_n=None, max_ctas=0, *, a_ptr=None, b_ptr=None, c_ptr=None,
             direct_store: bool = False):
    """block_n: None/0 = choose (CTA-pair kernel for large shapes), 128/256 = one-CTA kernel, 512 = CTA-pair kernel.

    `a_ptr` / `b_ptr` / `c_ptr` replace the address of the corresponding tensor (same layout, e.g. the same buffer in a
    tensor-parallel peer's symmetric memory); `direct_store` writes C with register stores instead of TMA."""
    lib = _lib.get_lib()
    if block_n is None:
        block_n = int(os.environ.get("FLB_GEMM_BLOCK_N", 0))
    _lib.check(
        lib.flb_gemm_bf16_ex(
            a.data_ptr() if a_ptr is None else a_ptr, b.data_ptr() if b_ptr is None else b_ptr,
            out.data_ptr() if c_ptr is None else c_ptr, m, n, k, a.stride(0), b.stride(0), out.stride(0),
            int(a_mn), int(b_mn), epilogue, block_n, max_ctas, int(direct_store), _lib.stream_ptr(),
        ),
        "flb_gemm_bf16",
    )
    _lib.count_launch()
    return out


def _epilogue(out: torch.Tensor, accumulate: bool) -> int:
    if out.dtype == torch.bfloat16:
        return _EPI_ACC_BF16 if accumulate else _EPI_STORE_BF16
    assert out.dtype == torch.float32, out.dtype
    return _EPI_ACC_F32 if accumulate else _EPI_STORE_F32


def matmul_nt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
              out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T -> [M, N]."""
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k, (x.shape, w.shape)
    if out is None:
        assert not accumulate
        out = torch.empty(m, n, dtype=out_dtype or x.dtype, device=x.device)
    if m == 0:
        return out
    if _native_ok(x, w) and out.stride(-1) == 1:
        return gemm_raw(x, w, out, m, n, k, False, False, _epilogue(out, accumulate))
    _note_library_fallback(x, w, out)
    res = torch.matmul(x, w.t())
    return out.add_(res) if accumulate else out.copy_(res)


def matmul_nn(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
              out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """dy [M, K] @ w[K, N] -> [M, N]."""
    m, k = dy.shape
    n = w.shape[1]
    assert w.shape[0] == k, (dy.shape, w.shape)
    if out is None:
        assert not accumulate
        out = torch.empty(m, n, dtype=out_dtype or dy.dtype, device=dy.device)
    if m == 0:
        return out
    if _native_ok(dy, w) and out.stride(-1) == 1:
        return gemm_raw(dy, w, out, m, n, k, False, True, _epilogue(out, accumulate))
    _note_library_fallback(dy, w, out)
    res = torch.matmul(dy, w)
    return out.add_(res) if accumulate else out.copy_(res)


def matmul_tn(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
              out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """dy[T, M]^T @ x[T, N] -> [M, N] (weight gradient); `out` may be the fp32 or bf16 gradient buffer."""
    t, m = dy.shape
    n = x.shape[1]
    assert x.shape[0] == t, (dy.shape, x.shape)
    if out is None:
        assert not accumulate
        out = torch.empty(m, n, dtype=out_dtype or dy.dtype, device=dy.device)
    if t == 0:
        return out if accumulate else out.zero_()
    if _native_ok(dy, x) and out.stride(-1) == 1:
        return gemm_raw(dy, x, out, m, n, t, True, True, _epilogue(out, accumulate))
    _note_library_fallback(dy, x, out)
    res = torch.matmul(dy.t(), x)
    return out.add_(res) if accumulate else out.copy_(res)


def gated_ok(x: torch.Tensor, w1: torch.Tensor) -> bool:
    """Whether `matmul_nt_gated` can run on these operands (otherwise: `matmul_nt` followed by the activation kernel)."""
    return _native_ok(x, w1) and x.dim() == 2 and w1.dim() == 2 and w1.shape[0] % 16 == 0 and x.shape[0] > 256


def matmul_nt_gated(x: torch.Tensor, w1: torch.Tensor, act_code: int) -> tuple[torch.Tensor, torch.Tensor]:
    """First layer of a gated MLP and its activation from one kernel: `h = x @ w1.T` with `w1 = [gate rows; up rows]` and
    `a = act(h[:, :F]) * h[:, F:]`, both bf16.  The activation is applied to the bf16-rounded `h`, so `a` equals what the
    standalone activation kernel computes from the stored `h`.  Replaces the Triton activation launch that follows the
    layer-1 GEMM in `fast_llm/functional/triton/mlp.py:207-290`."""
    m, k = x.shape
    f = w1.shape[0] // 2
    h = torch.empty(m, 2 * f, dtype=torch.bfloat16, device=x.device)
    a = torch.empty(m, f, dtype=torch.bfloat16, device=x.device)
    _lib.check(
        _lib.get_lib().flb_gemm_gated_bf16(x.data_ptr(), w1.data_ptr(), h.data_ptr(), a.data_ptr(), m, f, k, x.stride(0),
                                           w1.stride(0), h.stride(0), a.stride(0), act_code, _lib.stream_ptr()),
        "flb_gemm_gated_bf16",
    )
    _lib.count_launch()
    return h, a


def tensor_map_cache_stats() -> tuple[int, int]:
    """(hits, misses) of this thread's tensor-map table in the GEMM library."""
    import ctypes

    out = (ctypes.c_ulonglong * 2)()
    _lib.get_lib().flb_gemm_tmap_cache_stats(ctypes.cast(out, ctypes.c_void_p))
    return int(out[0]), int(out[1])


def check_device_errors() -> None:
    """Raise if a GEMM kernel gave up on a bounded wait since the last check (synchronises the device)."""
    word = _lib.get_lib().flb_gemm_error_word()
    if word:
        raise _lib.KernelLibraryError(f"tcgen05 GEMM aborted a bounded wait (role code {word})")
