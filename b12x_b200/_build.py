"""In-tree build of the sm_100a extension (``b12x_b200/csrc/libb200moe.so``).

The library is plain CUDA behind a C ABI (``include/b200moe.h``); it is compiled with nvcc
directly so that the result lives next to the sources and travels with the tree.
"""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_PATH = CSRC / "libb200moe.so"
SOURCES = (
    "api.cu",
    "route_sort.cu",
    "gate_route.cu",
    "quant_combine.cu",
    "grouped_gemm_bs.cu",
    "grouped_gemm_small.cu",
    "grouped_gemm_pair.cu",
    "grouped_gemm_other.cu",
    "ep_peer.cu",
)
NVCC_FLAGS = (
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    # products and sums must round separately, as the torch oracle does
    "--fmad=false",
    "-Xcompiler",
    "-fPIC",
)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [CSRC / "common.cuh", CSRC / "gemm_shared.cuh", CSRC / "route_shared.cuh", CSRC / "quant_shared.cuh", CSRC / "cluster_pair.cuh", CSRC.parents[1] / "include" / "b200moe.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``.cu`` source for sm_100a and link the shared library."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in SOURCES:
        obj = CSRC / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = []
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode != 0:
            failed.append(f"{src}:\n{out}")
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
