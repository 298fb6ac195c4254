"""Build ``libtfb200.so`` in-tree with nvcc for sm_100a.

    python -m tilefoundry_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB = CSRC / "libtfb200.so"
SOURCES = ("api.cu", "api_minicpm3.cu", "gemv.cu", "gemv_stream.cu", "attn_gqa.cu", "attn_mla.cu", "attn_mla_latent.cu", "mamba2.cu", "moe.cu", "api_granite.cu", "misc.cu",
           "gemv_persist.cu", "gemv_async.cu", "chain.cu", "gemm_tc.cu", "collective.cu", "gemv_f32.cu", "gdn.cu", "attn_gated.cu", "api_qwen35.cu",
           "batch.cu", "api_batch.cu", "step_fused.cu", "moe_grouped.cu")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Xcudafe", "--diag_suppress=177"]
# Approximate exp / division / rsqrt only where every output is a bf16-rounded activation.  The files that decide
# integers (expert selection, its softmax) or carry f32 recurrent state across tokens keep IEEE arithmetic.
PRECISE = frozenset({"moe.cu", "moe_grouped.cu", "gemv_f32.cu", "mamba2.cu", "gdn.cu", "collective.cu"})


def flags_for(src: str) -> list:
    return list(FLAGS) if src in PRECISE else [*FLAGS, "--use_fast_math"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the kernel library can only be built with the CUDA toolkit")
    return found


def stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in CSRC.iterdir() if p.suffix in (".cu", ".cuh", ".h"))
    newest = max(newest, (CSRC.parents[1] / "include" / "tfb200.h").stat().st_mtime)
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in SOURCES:
        obj = CSRC / (src + ".o")
        cmd = [nvcc, *flags_for(src), "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            print(f"--- {src} ---\n{out}", file=sys.stderr)
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the log above")
    subprocess.run([nvcc, "-shared", "-o", str(LIB), *objs], check=True)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
