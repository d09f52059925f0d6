"""Builds libkai_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python deep-learning-framework_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically and
takes the one driver entry point it needs (cuTensorMapEncodeTiled) at run time, so it
loads on machines without libcuda; computing there fails with a CUDA error.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBDIR = HERE / "lib"
LIB = LIBDIR / "libkai_b200.so"
SOURCES = ["kai_api.cu", "kai_gemm_tc.cu", "kai_gemm_simt.cu", "kai_gemm_skinny.cu", "kai_elementwise.cu", "kai_attention.cu",
           "kai_attention_mma.cu", "kai_attention_tc.cu", "kai_attention_fused.cu", "kai_conv.cu", "kai_conv_igemm.cu", "kai_conv_igemm_tma.cu"]
HEADERS = ["kai_common.cuh", "kai_act.cuh", "kai_tcgen05.cuh", "../../include/kai_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # The reference is built without FMA contraction (engine/CMakeLists.txt:189-208); the
    # kernels here ask for fused multiply-add explicitly (fmaf) where they want it.
    "-fmad=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
    "-Xptxas", "-v",
]


def nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = Path(home) / "bin" / "nvcc"
    return str(exe) if exe.exists() else "nvcc"


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    srcs = [s for s in SOURCES if (CSRC / s).exists()]
    hdrs = [CSRC / h for h in HEADERS]
    objs = []
    jobs = []
    for s in srcs:
        obj = LIBDIR / (Path(s).stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [CSRC / s, *hdrs, Path(__file__)]):
            jobs.append((s, obj))

    def compile_one(job):
        s, obj = job
        cmd = [nvcc(), *NVCC_FLAGS, "-c", str(CSRC / s), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (LIBDIR / (Path(s).stem + ".ptxas.log")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return s

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or force or _stale(LIB, objs):
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
