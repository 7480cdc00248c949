"""Builds libmoonmath_attention_sm100.so with nvcc for sm_100a, in-tree.

Takes the place of the reference's setup.py / Makefile (setup.py:56-93,
Makefile:29-33), which build three per-rounding-mode copies with hipcc.  One
library is built here; the rounding mode is a run-time argument.

    python amd-kernels_b200/build.py [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
PKG = HERE / "moonmath_attention"
LIB = PKG / "libmoonmath_attention_sm100.so"
OBJ_DIR = HERE / "build"

SOURCES = ["ma_abi.cu", "attn_simple.cu", "attn_pipelined.cu", "attn_lite.cu", "attn_merge.cu", "mla_decode.cu", "selftest.cu"]
HEADERS = ["sm100_ptx.cuh", "attn_common.cuh", "attn_launch.h", "tail_plan.h", "lite_list.h"]

# `-arch=sm_100a` also emits a plain compute_100 PTX pass that rejects tcgen05;
# the explicit -gencode pair compiles arch-specific code only.
NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return cand


def _fingerprint() -> str:
    h = hashlib.sha256()
    for name in SOURCES + HEADERS:
        h.update((CSRC / name).read_bytes())
    h.update((HERE.parent / "include" / "moonmath_attention.h").read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library if the sources changed; returns its path."""
    stamp = OBJ_DIR / "fingerprint"
    fp = _fingerprint()
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == fp:
        return LIB
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> tuple[str, str]:
        obj = OBJ_DIR / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return src, r.stderr

    with ThreadPoolExecutor(max_workers=4) as pool:
        logs = list(pool.map(compile_one, SOURCES))
    (OBJ_DIR / "ptxas.log").write_text("\n".join(f"==== {s}\n{log}" for s, log in logs))
    if verbose:
        for s, log in logs:
            print(f"==== {s}\n{log}")
    objs = [str(OBJ_DIR / (s + ".o")) for s in SOURCES]
    cmd = [nvcc, "-shared", "-o", str(LIB), *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(fp)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    sys.exit(0)
