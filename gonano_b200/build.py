"""Builds the CUDA library in-tree: gonano_b200/libgonano_cuda.so (sm_100a only).

Run as ``python -m gonano_b200.build``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "_obj"
LIB = HERE / "libgonano_cuda.so"

NVCC = os.environ.get("GN_NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "-ccbin", "g++",
    "--expt-relaxed-constexpr",
]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(src: Path, obj: Path) -> bool:
    if not obj.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + [src, HERE.parent / "include" / "gonano_cuda.h"])
    return newest > obj.stat().st_mtime


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = sources()
    defines = []
    if (CSRC / "gemm_tcgen05.cu").exists():
        defines.append("-DGN_HAVE_TCGEN05")
    defines += os.environ.get("GN_EXTRA_NVCC_FLAGS", "").split()   # e.g. -DGN_TC_TRACE for the pipeline timeline

    def compile_one(src: Path):
        obj = OBJ / (src.stem + ".o")
        if not force and not _stale(src, obj):
            return src.name, 0, ""
        cmd = [NVCC, *FLAGS, *defines, "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return src.name, proc.returncode, proc.stdout + proc.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(compile_one, srcs))
    failed = [r for r in results if r[1] != 0]
    for name, code, out in results:
        if out.strip() and (verbose or code != 0):
            print(f"--- {name}\n{out}", file=sys.stderr)
    if failed:
        raise RuntimeError("nvcc failed for: " + ", ".join(r[0] for r in failed))
    objs = [str(OBJ / (s.stem + ".o")) for s in srcs]
    if force or not LIB.exists() or any(Path(o).stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [NVCC, "-shared", "-o", str(LIB), *objs, "-lcudart", "-ldl"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("link failed:\n" + proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
