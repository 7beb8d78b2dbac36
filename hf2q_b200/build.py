"""Builds libhf2q_cuda.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python -m hf2q_b200.build``.  nvcc cross-compiles without a GPU, so this also serves as
the "does it build" check.  The library lands next to this file so it travels with the tree.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libhf2q_cuda.so"
SOURCES = ["api.cu", "k0_dequant.cu", "k1_gemv.cu", "k1_gemv_mma.cu", "k2_gemm_tc.cu", "k4_moe_prep.cu", "moe_router.cu", "ffn_elementwise.cu", "decoder_ops.cu", "comm_nccl.cu", "ffn_builders.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps.append(PKG.parent / "include" / "hf2q_cuda.h")
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return OUT
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    env = dict(os.environ)
    env.pop("CXX", None)
    env.pop("CC", None)
    objs, procs = [], []
    for src in SOURCES:
        obj = objdir / (src + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, *shlex.split(os.environ.get("HF2Q_NVCC_EXTRA", "")), "-ccbin", "g++", "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append(f"== {src}\n{out}")
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    (objdir / "ptxas.log").write_text("\n".join(log))
    cmd = [_nvcc(), "-shared", "-ccbin", "g++", "-o", str(OUT), *objs, "-ldl"]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    if verbose:
        print("\n".join(log))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
