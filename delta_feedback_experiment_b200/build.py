"""Builds ``libpkda_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m delta_feedback_experiment_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is rebuilt only when a source
file is newer than the existing ``.so`` (or ``--force`` is given).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_PATH = os.path.join(HERE, "libpkda_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

SOURCES = ["pkda_abi.cu", "pkda_recurrent.cu", "pkda_chunk_fwd.cu", "pkda_chunk_bwd.cu",
           "pkda_static_scratch.cu", "pkda_intra_fwd_tc.cu", "pkda_intra_bwd_tc.cu", "pkda_out_tc.cu", "pkda_scan_tc.cu", "pkda_scan_bwd_tc.cu",
           "pkda_recurrent_bwd.cu", "pkda_qkv_conv.cu", "pkda_norm_gate.cu", "pkda_decode_step.cu", "pkda_controls.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-ftz=true",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libpkda_b200.so")
    return exe


def _deps() -> list[str]:
    out = [os.path.join(INCLUDE, "pkda_b200.h"), os.path.abspath(__file__)]  # the flags live in this file
    for name in os.listdir(CSRC):
        out.append(os.path.join(CSRC, name))
    return out


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    stamp = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > stamp for d in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> tuple[str, str]:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    cmd = [nvcc, "-shared", "-o", LIB_PATH, *[o for o, _ in results], "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
