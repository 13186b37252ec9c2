"""Builds see_ai_b200/libsee_cuda.so in-tree: CUDA kernels for sm_100a with nvcc,
C++23 host code with g++, linked against the static CUDA runtime so the library
carries its own runtime and needs nothing but the driver at load time.

    python -m see_ai_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libsee_cuda.so")
PROBE = os.path.join(HERE, "see-cuda-plan-probe")   # the seeml-plan-probe-compatible executable over the C ABI
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

# Kernels whose arithmetic must round like the reference's x86 build are compiled
# without fused multiply-add contraction; the tensor-core kernel does not care.
CU_SOURCES = {
    "k_elementwise.cu": ["-fmad=false"],
    "k_norm.cu": ["-fmad=false"],
    "k_loss.cu": ["-fmad=false"],
    "k_optim.cu": ["-fmad=false"],
    "k_attention.cu": ["-fmad=false"],
    "k_gemm_exact.cu": ["-fmad=false"],
    "k_gemm_skinny.cu": ["-fmad=false"],
    "k_gemm_umma.cu": ["-fmad=false"],
    "k_eval.cu": [],
    "k_attn_umma.cu": [],
    "k_no_alloc.cu": ["-fmad=false"],
    "k_lora.cu": [],
    "k_gemm_skinny_fast.cu": [],
    "k_lora_mma.cu": [],
    "k_lora_umma.cu": [],
}
CC_SOURCES = ["extents.cc", "cuda_backend.cc", "c_api.cc", "umma_gemm.cc", "engine.cc", "exchange.cc"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "--expt-extended-lambda", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xptxas", "-v"]
CXX_FLAGS = ["-std=c++23", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter",
             f"-I{CUDA_HOME}/include"]


def _stale(obj: str, deps) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "see_cuda.h"))
    jobs = []
    objs = []
    for src, extra in CU_SOURCES.items():
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ, src + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            jobs.append([NVCC] + NVCC_FLAGS + extra + ["-c", path, "-o", obj])
    for src in CC_SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ, src + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            jobs.append(["g++"] + CXX_FLAGS + ["-c", path, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stderr[-4000:]}")
        return r

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(run, jobs))
    if jobs or force or not os.path.exists(LIB):
        run(["g++", "-shared", "-o", LIB] + objs +
            [f"-L{CUDA_HOME}/lib64", "-lcudart_static", "-lrt", "-ldl", "-lpthread",
             "-Wl,--no-undefined"])
    probe_src = os.path.join(CSRC, "probe_main.cc")
    if os.path.exists(probe_src) and (jobs or force or _stale(PROBE, [probe_src, LIB] + headers)):
        run(["g++"] + CXX_FLAGS + [probe_src, os.path.join(OBJ, "extents.cc.o"), "-o", PROBE, f"-L{HERE}",
                                   "-lsee_cuda", "-Wl,-rpath,$ORIGIN"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
