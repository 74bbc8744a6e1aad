"""In-tree build of the native libraries.

`build_all()` compiles every `.cu` file in this directory for sm_100a into `libflb_kernels.so` and the host-only
C++ sources into `libflb_host.so`, next to the sources.  Objects are rebuilt only when a source or header is newer.
nvcc cross-compiles without a GPU, so this also serves as the "does it build" check on CPU machines.
"""

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

CSRC = pathlib.Path(__file__).resolve().parent
BUILD = CSRC / "build"
KERNEL_LIB = CSRC / "libflb_kernels.so"
HOST_LIB = CSRC / "libflb_host.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


# Approximate division / sqrt / exp / log (`--use_fast_math`) only where the arithmetic tolerates it: the GEMM and
# attention pipelines (exp2 on scaled scores, checked against fp32 restatements), activations, norms and the SSM scans.
# The optimizer update, the loss kernels and the fused ZeRO kernels (AdamW's sqrt and divide, the cross-entropy's exp
# and log) compile with IEEE-accurate math, like the apex / Triton kernels they stand in for.
FAST_MATH_SOURCES = {"gemm_tcgen05.cu", "attention_fwd.cu", "attention_bwd.cu", "elementwise.cu", "norm.cu", "ssm.cu", "moe.cu"}


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    return nvcc


def _stale(target: pathlib.Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: pathlib.Path, headers, verbose: bool) -> pathlib.Path:
    obj = BUILD / (src.stem + ".o")
    if _stale(obj, [src, *headers]):
        cmd = [_nvcc(), *NVCC_FLAGS, *(["--use_fast_math"] if src.name in FAST_MATH_SOURCES else []), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
    return obj


def build_kernels(verbose: bool = False, force: bool = False) -> pathlib.Path:
    BUILD.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted([*CSRC.glob("*.cuh"), *CSRC.glob("*.h"), pathlib.Path(__file__)])
    if force:
        for o in BUILD.glob("*.o"):
            o.unlink()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, headers, verbose), sources))
    if force or _stale(KERNEL_LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", str(KERNEL_LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return KERNEL_LIB


def build_host(force: bool = False) -> pathlib.Path:
    sources = sorted(CSRC.glob("*.cpp"))
    if not sources:
        return HOST_LIB
    if force or _stale(HOST_LIB, sources):
        cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-o", str(HOST_LIB), *map(str, sources)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{res.stdout}\n{res.stderr}")
    return HOST_LIB


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_host(force=force)
    build_kernels(verbose=verbose, force=force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(KERNEL_LIB, HOST_LIB)
