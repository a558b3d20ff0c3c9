"""Builds ``libcaten_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m caten_b200.build [--force] [--verbose] [--timing]

``--timing`` builds a second library, ``libcaten_b200_timing.so``, whose single-kernel decode step
records per-phase timestamps of CTA 0 (``-DDS_TIMING``; read by ``microbench.py decode_step``).
It is a development aid: load it with ``CATEN_B200_LIB=caten_b200/libcaten_b200_timing.so``.

``-fmad=false``: multiply-add contraction is off so that element-wise formulas round exactly as
written (they restate the reference's op-by-op definitions); hot loops call fmaf() explicitly.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libcaten_b200.so")
SOURCES = ["capi.cu", "decode_small.cu", "kernels_misc.cu", "gemv.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_dense.cu", "attention.cu", "attention_tc.cu", "gguf.cu", "expr.cu", "dequant_extra.cu", "sample.cu", "dist.cu", "llama_ops.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-fmad=false", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _deps():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out.append(os.path.join(INCLUDE, "caten_b200.h"))
    out.append(os.path.abspath(__file__))
    return out


def build(force: bool = False, verbose: bool = False, timing: bool = False) -> str:
    lib = LIB.replace(".so", "_timing.so") if timing else LIB
    obj_dir = OBJ_DIR + ("_timing" if timing else "")
    flags = NVCC_FLAGS + (["-DDS_TIMING", "-DDS_TIMING_CTA=0"] if timing else [])
    newest = max(os.path.getmtime(p) for p in _deps())
    if not force and os.path.exists(lib) and os.path.getmtime(lib) >= newest:
        return lib
    nvcc = _nvcc()
    os.makedirs(obj_dir, exist_ok=True)
    env = dict(os.environ)
    # use the system host compiler even when CC/CXX point elsewhere
    host = shutil.which("g++") or "g++"

    def compile_one(src):
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, "-ccbin", host, *flags, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        return src, obj, r

    objs = []
    with cf.ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 2)) as ex:
        for src, obj, r in ex.map(compile_one, SOURCES):
            if verbose or r.returncode:
                sys.stderr.write(f"--- {src}\n{r.stdout}{r.stderr}\n")
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(obj)
            with open(os.path.join(obj_dir, src + ".ptxas.log"), "w") as f:
                f.write(r.stderr)
    link = [nvcc, "-ccbin", host, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib, *objs, "-ldl"]
    r = subprocess.run(link, capture_output=True, text=True, env=env)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, timing="--timing" in sys.argv))
