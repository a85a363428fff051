"""Build libffa_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m ffa_speedtest_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libffa_b200.so"
SOURCES = ["ffa_lib.cu", "ffa_decode.cu", "ffa_decode_tma.cu", "ffa_decode_ws.cu", "ffa_decode_ws_fp8.cu",
           "ffa_decode_ws_q2.cu", "ffa_decode_ws_fp4.cu", "ffa_decode_ws_nf4.cu", "ffa_decode_ws_nvfp4.cu",
           "ffa_quantize.cu", "ffa_kproj.cu", "ffa_static.cu", "ffa_peer.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math=false",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def up_to_date() -> bool:
    if not OUT.exists():
        return False
    t = OUT.stat().st_mtime
    deps = (list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
            + [PKG.parent / "include" / "ffa_b200.h"])
    return all(d.stat().st_mtime <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and up_to_date():
        return OUT
    objs = []
    procs = []
    bdir = PKG / "build"
    bdir.mkdir(exist_ok=True)
    for src in sources():
        obj = bdir / (src.stem + ".o")
        cmd = [_nvcc(), *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], *os.environ.get("FFA_NVCC_EXTRA", "").split(),
               "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode:
            sys.stdout.write(out)
        if pr.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
    link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(OUT), *map(str, objs)]
    subprocess.run(link, check=True)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
