"""Builds libzck_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python zig-cu-kernels_b200/build.py [--force] [--verbose]

The library lands next to the Python package (`zig_cu_kernels/libzck_b200.so`) so that it travels with the tree.
A source-hash stamp skips the build when nothing changed.
"""

import hashlib
import os
import pathlib
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = pathlib.Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
INCLUDE = ROOT.parent / "include"
OUT = ROOT / "zig_cu_kernels" / "libzck_b200.so"
OBJ = ROOT / "build"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def nvcc():
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; libzck_b200 has no prebuilt or CPU fallback")
    return found


def sources():
    return sorted(CSRC.glob("*.cu"))


def digest():
    h = hashlib.sha256()
    for path in [*sources(), *sorted(CSRC.glob("*.h")), *sorted(CSRC.glob("*.cuh")), *sorted(INCLUDE.glob("*.h")),
                 pathlib.Path(__file__)]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def compile_one(source, verbose):
    obj = OBJ / (source.stem + ".o")
    command = [nvcc(), *ARCH, *FLAGS, "-I", str(INCLUDE), "-c", str(source), "-o", str(obj)]
    result = subprocess.run(command, capture_output=True, text=True)
    (OBJ / (source.stem + ".ptxas.txt")).write_text(result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(result.stderr)
    return obj


def build(force=False, verbose=False):
    stamp = OBJ / "stamp"
    current = digest()
    if not force and OUT.exists() and stamp.exists() and stamp.read_text() == current:
        return OUT
    OBJ.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, len(sources()))) as pool:
        objects = list(pool.map(lambda source: compile_one(source, verbose), sources()))
    command = [nvcc(), *ARCH, "-shared", "-o", str(OUT), *map(str, objects)]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    stamp.write_text(current)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
