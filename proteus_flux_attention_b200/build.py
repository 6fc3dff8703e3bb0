"""Build recipe for libaspa_b200.so: nvcc, sm_100a only, in-tree output.

    python -m proteus_flux_attention_b200.build

The library has no Python or torch dependency; it exports the C ABI declared in
include/aspa_b200.h and is loaded with ctypes by ``_native.py``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libaspa_b200.so"
SOURCES = ["router.cu", "router_tc.cu", "select.cu", "rope_quant.cu", "plan.cu", "attention.cu", "attention_tc.cu", "attention_picks.cu", "ema_chunk.cu",
           "memory_bank.cu", "quantile.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "aspa_b200.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    flags = [f for f in FLAGS if not f.startswith("--use_fast_math")]
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for s in SOURCES:
        obj = CSRC / (Path(s).stem + ".o")
        objs.append(str(obj))
        procs.append((s, subprocess.Popen([_nvcc(), *flags, "-c", str(CSRC / s), "-o", str(obj)],
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {s}\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIB), *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
