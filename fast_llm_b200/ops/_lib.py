"""ctypes binding of the in-tree sm_100a kernel library (`csrc/libflb_kernels.so`).

The library exports a plain C ABI (raw device pointers, sizes, a CUDA stream), so it has no dependency on the PyTorch
C++ headers and compiles in seconds.  On a machine with a GPU the library is mandatory: `get_lib()` raises instead of
silently falling back, so a missing build cannot masquerade as a working CUDA path.
"""

import ctypes
import functools
import pathlib

import torch

_CSRC = pathlib.Path(__file__).resolve().parent.parent / "csrc"
KERNEL_LIB_PATH = _CSRC / "libflb_kernels.so"
HOST_LIB_PATH = _CSRC / "libflb_host.so"

_p, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

_SIGNATURES = {
    "flb_gemm_bf16": [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _i, _p],
    "flb_causal_conv1d_fwd": [_p, _p, _p, _p, _p, _ll, _i, _i, _i, _p],
    "flb_causal_conv1d_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _ll, _i, _i, _i, _i, _p],
    "flb_delta_state_scan": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "flb_selective_scan_chunks": [_ll],
    "flb_selective_scan_fwd": [_p] * 9 + [_ll, _i, _i, _i, _i, _p, _p, _p, _p],
    "flb_selective_scan_checkpoints": [_ll, _i],
    "flb_selective_scan_bwd": [_p] * 9 + [_ll, _i, _i, _i, _i] + [_p] * 14,
    "flb_moe_dispatch": [_p, _p, _p, _p, _i, _i, _i, _p],
    "flb_moe_combine": [_p, _p, _p, _p, _i, _i, _i, _p],
    "flb_moe_score_grad": [_p, _p, _p, _p, _i, _i, _i, _p],
    "flb_moe_route_blocks": [_i],
    "flb_moe_route": [_p, _i, _i, _i, _p, _p, _p, _p, _p],
    "flb_moe_route_bwd": [_p, _p, _p, _p, _p, _f, _i, _i, _i, _p, _p],
    "flb_moe_layout": [_p, _i, _i, _i, _p, _p, _p, _p],
    "flb_grouped_gemm_gated_bf16": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _p],
    "flb_grouped_gemm_bf16": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _p],
    "flb_gemm_bf16_ex": [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _p],
    "flb_gemm_gated_bf16": [_p, _p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _p],
    "flb_gemm_gathered_bf16": [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _p, ctypes.c_uint, _i, _i, _p],
    "flb_gemm_gathered_gated_bf16": [_p, _p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _p, ctypes.c_uint, _i, _i, _p],
    "flb_gemm_scatter_maps": [_p, _p, _i, _i, _i, _ll],
    "flb_gemm_scatter_bf16": [_p, _p, _p, _i, _i, _i, _ll, _ll, _i, _i, _i, _p],
    "flb_gemm_error_word": [],
    "flb_norm_error_word": [],
    "flb_gemm_tmap_cache_stats": [_p],
    "flb_norm_fwd": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _i, _i, _p],
    "flb_norm_bwd_parts": [_i, _i, _i],
    "flb_norm_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "flb_colsum": [_p, _p, _i, _i, _i, _i, _p],
    "flb_rope": [_p, _p, _p, _ll, _ll, _i, _i, _i, _i, _p],
    "flb_act_fwd": [_p, _p, _ll, _i, _i, _i, _p],
    "flb_act_bwd": [_p, _p, _p, _p, _ll, _i, _i, _i, _p],
    "flb_axpby": [_p, _i, _p, _i, _p, _i, _ll, _f, _f, _p],
    "flb_fill": [_p, _i, _ll, _f, _p],
    "flb_bias_residual": [_p, _p, _p, _p, _ll, _i, _f, _p],
    "flb_embedding_fwd": [_p, _p, _p, _ll, _i, _ll, _ll, _f, _p],
    "flb_embedding_bwd": [_p, _p, _p, _ll, _i, _ll, _ll, _f, _p],
    "flb_ce_stats": [_p, _i, _p, _p, _i, _i, _ll, _ll, _f, _p],
    "flb_ce_grad": [_p, _i, _p, _p, _p, _p, _p, _i, _i, _ll, _ll, _ll, _f, _f, _p, _f, _p],
    "flb_ce_stats_exchange": [_p, _i, _p, _p, _i, _i, _i, _i, _ll, _ll, _f, _p],
    "flb_ce_grad_slots": [_p, _i, _p, _p, _i, _p, _p, _p, _i, _i, _ll, _ll, _ll, _f, _f, _p, _f, _p],
    "flb_softmax_coeff_grad": [_p, _i, _p, _p, _i, _p, _p, _p, _i, _i, _ll, _ll, _ll, _f, _i, _p],
    "flb_dist_stats": [_p, _p, _i, _p, _i, _i, _ll, _ll, _f, _f, _p],
    "flb_dist_grad": [_p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _ll, _ll, _ll, _f, _f, _i, _p],
    "flb_sumsq_scratch_floats": [],
    "flb_sumsq": [_p, _ll, _p, _p, _i, _p],
    "flb_sum_partials": [_p, _i, _p, _i, _p],
    "flb_clip_coeff": [_p, _f, _f, _p, _p, _p],
    "flb_adamw": [_p, _p, _p, _p, _p, _ll, _f, _f, _f, _f, _f, _i, _f, _p, _p, _p],
    "flb_abi_version": [],
    "flb_attention_fwd": [_p, _ll, _i, _p, _ll, _i, _i, _p, _p, _i, _i, _ll, _ll, _i, _i, _i, _p, _p, _i, _i, _f, _p],
    "flb_attention_error_word": [],
    "flb_attention_set_forward_variant": [_i],
    "flb_attention_bwd": [_p, _ll, _i, _p, _ll, _i, _i, _p, _p, _p, _p, _p, _i, _i, _ll, _ll, _i, _i, _i, _p, _ll, _p, _ll, _p, _p,
                          _i, _i, _f, _p],
    "flb_attention_bwd_error_word": [],
    "flb_symm_max_ranks": [],
    "flb_symm_signal_pad_bytes": [_i],
    "flb_tp_wait": [_p, ctypes.c_uint, _i, _i, _p, _p],
    "flb_tp_push": [_p, _ll, _p, _ll, _ll, _ll, _i, _i, ctypes.c_uint, _p, _p, _i, _p],
    "flb_symm_barrier": [_p, _i, _i, _i, ctypes.c_uint, _p, _p],
    "flb_rs_reduce_blocks": [],
    "flb_rs_reduce_multimem": [_p, _i, _i, _ll, _f, _p, _i, _p, _p, _p],
    "flb_symm_set_barrier_limit": [_ll],
    "flb_rs_reduce": [_p, _i, _i, _i, _ll, _f, _p, _i, _p, _p, _p],
    "flb_slot_sum_bf16": [_p, _p, _i, _ll, _p, _p],
    "flb_peer_copy": [_p, _p, _ll, _i, _p],
    "flb_adam_push": [_p, _p, _p, _p, _p, _i, _ll, _ll, _f, _f, _f, _f, _f, _i, _f, _p, _p, _p],
}

_STATUS = {1: "unsupported shape or alignment", 2: "CUDA error", 3: "tensor map encoding failed", 4: "size exceeds the stated maximum"}


class KernelLibraryError(RuntimeError):
    pass


@functools.cache
def get_lib() -> ctypes.CDLL:
    if not KERNEL_LIB_PATH.exists():
        raise KernelLibraryError(
            f"{KERNEL_LIB_PATH} is missing: run `python -m fast_llm_b200.csrc.build` (or `__graft_entry__.build()`) first."
        )
    lib = ctypes.CDLL(str(KERNEL_LIB_PATH))
    for name, argtypes in _SIGNATURES.items():
        if not hasattr(lib, name):
            continue
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _i
    lib.flb_symm_set_barrier_limit.restype = _ll
    lib.flb_last_cuda_error.restype = ctypes.c_char_p
    lib.flb_last_cuda_error.argtypes = []
    return lib


def lib_available() -> bool:
    return KERNEL_LIB_PATH.exists()


def check(status: int, what: str) -> None:
    if status != 0:
        detail = _STATUS.get(status, f"status {status}")
        if status == 2:
            detail += ": " + get_lib().flb_last_cuda_error().decode()
        raise KernelLibraryError(f"{what}: {detail}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: "torch.Tensor | None") -> int | None:
    return None if t is None else t.data_ptr()


def use_cuda_kernels(*tensors: torch.Tensor) -> bool:
    """True when the operands live on a GPU; then the native kernels are the only path."""
    return any(t is not None and t.is_cuda for t in tensors)


# Counts launches of this library's kernels (bench.py reports it).
launch_count = 0


def count_launch(n: int = 1) -> None:
    global launch_count
    launch_count += n
