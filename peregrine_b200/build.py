"""Builds libperegrine_b200.so (the CUDA kernels and the C ABI) with nvcc for sm_100a.

The library is built in-tree, next to this file, so that it travels with the package.
`python -m peregrine_b200.build` rebuilds it; `ensure_built()` rebuilds only when a source is
newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "lib", "obj")
LIB = os.path.join(HERE, "lib", "libperegrine_b200.so")

SOURCES = [
    "pg_api.cu",
    "pg_quantize.cu",
    "pg_gemm_naive.cu",
    "pg_gemv_w8a8.cu", "pg_gemv_wstream.cu",
    "pg_gemm_tcgen05.cu",
    "pg_gemm_tcgen05_2cta.cu",
    "pg_gguf.cu",
    "pg_gguf_stream.cu",
    "pg_noalloc.cu",
    "pg_w8a32.cu",
    "pg_peer.cu",
    "pg_llama.cu", "pg_llama_attn.cu",
    "pg_huffman.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    # bit-exactness: IEEE division/sqrt, denormals kept; FMA contraction is avoided in the
    # kernels themselves through the *_rn intrinsics
    "--ftz=false", "--prec-div=true", "--prec-sqrt=true",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libperegrine_b200.so cannot be built")


def _sources():
    deps = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cuh")]
    deps += [os.path.join(ROOT, "include", f) for f in ("peregrine_b200.h", "peregrine_b200_tune.h")] + [os.path.abspath(__file__)]
    return [os.path.join(CSRC, s) for s in SOURCES], deps


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    srcs, deps = _sources()
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in srcs + deps)


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    srcs, _ = _sources()
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-o", LIB + ".tmp", *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(LIB + ".tmp", LIB)
    return LIB


def ensure_built() -> str:
    if is_stale():
        build()
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, ptxas_info="--ptxas" in sys.argv))
