"""Builds libggq_b200.so (the C-ABI library of include/ggq.h) in-tree with nvcc for sm_100a.

Usage: ``python -m gguf_jax_b200.build [--force] [--verbose]``.
The compiled library sits beside this file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libggq_b200.so")

SOURCES = ["capi.cu", "dequant.cu", "gemv.cu", "gemv_generic.cu", "gemv_stream.cu", "gemv_q4k.cu", "gemv_q5k.cu", "gemv_q6k.cu", "gemm_tcgen05.cu", "gemv_mma.cu", "gemv_tile.cu", "gemv_wide.cu", "gemm_codes.cu", "gemm_bf16w.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++20",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    # decode must match numpy float32 bit for bit: no fast-math, no flush-to-zero
    "-ftz=false", "-prec-div=true", "-prec-sqrt=true",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "ggq.h"))
    env = dict(os.environ)
    # nvcc's host compiler: prefer the system g++ over whatever CC/CXX point to.
    ccbin = ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        path = os.path.join(CSRC, src)
        if force or _stale(obj, [path] + headers):
            cmd = [_nvcc(), *ccbin, *NVCC_FLAGS, "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            r = subprocess.run(cmd, capture_output=True, text=True, env=env)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), *ccbin, "-shared", "--cudart", "shared", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def build_xla_ffi(verbose: bool = False) -> str | None:
    """Compile csrc/xla_ffi.cc (the jax.ffi handlers over the C ABI) into libggq_xla_ffi.so when the
    XLA FFI headers are available, i.e. when ``import jax.ffi`` works; returns None otherwise."""
    try:
        import jax.ffi as jffi
    except Exception:  # noqa: BLE001 -- no jaxlib on this machine: nothing to build against
        return None
    build()
    out = os.path.join(HERE, "libggq_xla_ffi.so")
    src = os.path.join(CSRC, "xla_ffi.cc")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", f"-I{jffi.include_dir()}", f"-I{os.path.join(HERE, '..', 'include')}",
           "-I/usr/local/cuda/include", src, f"-L{HERE}", "-lggq_b200", f"-Wl,-rpath,{HERE}", "-o", out]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"xla_ffi.cc failed to compile:\n{r.stdout}\n{r.stderr}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print("XLA FFI adapter:", build_xla_ffi(verbose="--verbose" in sys.argv) or "skipped (jax.ffi is not importable here)")
