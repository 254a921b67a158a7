"""Builds the shared libraries in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Two targets, so that a model family compiles only what it runs on: "llama" = libgten_b200.so (the TinyLlama hot path,
include/gten_b200.h) and "seq" = libgten_b200_seq.so (layer-list sequence models, include/gten_b200_seq.h; it carries its own
copy of the context / memory layer, gtb_api.cu).

-fmad=false is part of the numeric contract (gtb_dev.cuh): nvcc must never contract a*b+c, the
reference's AVX build has no FMA.  Explicit fmaf()/fma() calls stay fused.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libgten_b200.so"
SOURCES = ["gtb_api.cu", "gtb_ops.cu", "gtb_engine.cu", "gtb_prefill.cu", "gtb_xrows.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O2", "--expt-relaxed-constexpr",
]
SEQ_LIB = HERE / "libgten_b200_seq.so"
SEQ_SOURCES = ["gtb_api.cu", "gtb_seq.cu", "gtb_seq_gemm.cu"]
# the sequence models have no bit-exact contract with a CPU program: fused multiply-adds are welcome (gtb_api.cu keeps the flag)
SEQ_FLAGS = [f for f in NVCC_FLAGS if f != "-fmad=false"]
TARGETS = {
    "llama": (LIB, SOURCES, {}),
    "seq": (SEQ_LIB, SEQ_SOURCES, {"gtb_seq.cu": SEQ_FLAGS, "gtb_seq_gemm.cu": SEQ_FLAGS}),
}


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.sep not in c or os.path.exists(c)):
            return c
    return "nvcc"


def needs_build(target: str = "llama") -> bool:
    lib = TARGETS[target][0]
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [HERE.parent / "include" / "gten_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra: list[str] | None = None, target: str = "llama") -> Path:
    LIB, SOURCES, flag_sets = TARGETS[target]
    if not force and not needs_build(target):
        return LIB
    ccbin = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    objs = []
    procs = []
    bdir = HERE / "build" / target
    bdir.mkdir(parents=True, exist_ok=True)
    for s in SOURCES:
        o = bdir / (s + ".o")
        cmd = [_nvcc(), "-ccbin", ccbin, *flag_sets.get(s, NVCC_FLAGS), *(extra or []), "-c", str(CSRC / s), "-o", str(o)]
        if verbose:
            print(" ".join(cmd))
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(o))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [_nvcc(), "-ccbin", ccbin, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIB), *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print(r.stdout, r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    extra = (["-Xptxas", "-v"] if "--ptxas" in sys.argv else []) + (["-DGTB_FD_TRACE"] if "--trace" in sys.argv else [])
    for tgt in TARGETS:
        if "--target" in sys.argv and sys.argv[sys.argv.index("--target") + 1] != tgt:
            continue
        print("built", build(force="--force" in sys.argv or "--trace" in sys.argv, verbose=True, extra=extra or None, target=tgt))
