"""Build ``libsq_b200.so`` in-tree with nvcc for sm_100a.

    python fastwamjoint-quantization_b200/build.py [--force] [--verbose]

The library has a C ABI only (``include/sq_b200.h``); it links the CUDA runtime
statically and needs neither PyTorch nor libcuda at link time (the one driver
call it makes, ``cuTensorMapEncodeTiled``, is looked up at run time).
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "lib" / "libsq_b200.so"
SOURCES = ("sq_prepass.cu", "sq_gemm_tc.cu", "sq_gemm_ts.cu", "sq_api.cu")
HEADERS = ("sq_internal.h", "sq_ptx.cuh", "../../include/sq_b200.h")
NVCC_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden")


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; libsq_b200.so cannot be built.")
    return found


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    obj_dir = HERE / "build"
    obj_dir.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    compiler = nvcc()

    def compile_one(source: str) -> Path:
        obj = obj_dir / (source + ".o")
        cmd = [compiler, *NVCC_FLAGS, "-c", str(CSRC / source), "-o", str(obj)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
            print(" ".join(cmd), flush=True)
        done = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or done.returncode:
            sys.stderr.write(done.stdout + done.stderr)
        if done.returncode:
            raise RuntimeError(f"nvcc failed on {source}")
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, SOURCES))
    tmp = LIB.with_suffix(".so.tmp")
    link = [compiler, "-shared", "-o", str(tmp), *map(str, objects), "-cudart", "static",
            "-gencode", "arch=compute_100a,code=sm_100a"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode:
        sys.stderr.write(done.stdout + done.stderr)
        raise RuntimeError("linking libsq_b200.so failed")
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))
