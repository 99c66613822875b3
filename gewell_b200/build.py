"""Build the CUDA library in-tree: every csrc/*.cu -> one shared library
gewell_b200/_C/libgewell_b200.so, compiled for sm_100a only.

    python -m gewell_b200.build            # incremental
    python -m gewell_b200.build --force
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
OUT_DIR = PACKAGE / "_C"
OBJ_DIR = PACKAGE.parent / "build" / "obj"
LIBRARY = OUT_DIR / "libgewell_b200.so"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(s.stat().st_mtime > stamp for s in sources)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((PACKAGE.parent / "include").glob("*.h"))
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    compiler = nvcc()

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [compiler, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                print(" ".join(cmd), flush=True)
            done = subprocess.run(cmd, capture_output=True, text=True)
            if done.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{done.stdout}\n{done.stderr}")
            if verbose and done.stderr.strip():
                print(done.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objects = list(pool.map(compile_one, sources))
    if force or _stale(LIBRARY, objects):
        cmd = [compiler, "-shared", "-o", str(LIBRARY), *map(str, objects), "-lcudart"]
        if verbose:
            print(" ".join(cmd), flush=True)
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIBRARY


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("-v", "--verbose", action="store_true")
    args = parser.parse_args()
    print(build(args.force, args.verbose))
