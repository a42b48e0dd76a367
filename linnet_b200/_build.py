"""Builds `libb200q.so` (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python -m linnet_b200._build            # build if sources are newer than the library
    python -m linnet_b200._build --force

nvcc cross-compiles for sm_100a without a GPU.  The library links the CUDA runtime
statically, so it carries no dependency on a particular libcudart next to PyTorch's.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
INCLUDE = PACKAGE.parent / "include"
LIBRARY = PACKAGE / "libb200q.so"
OBJECTS = PACKAGE / "build"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", str(INCLUDE)]
# The quantizer must round exactly as IEEE binary32 does (no contraction into
# fused multiply-adds, true division, denormals kept).
PER_FILE = {"quantize.cu": ["-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false"]}


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the b200q kernels cannot be built")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > built for p in deps)


def _compile(source: Path, verbose: bool) -> Path:
    obj = OBJECTS / (source.stem + ".o")
    cmd = [nvcc(), *ARCH, *COMMON, *PER_FILE.get(source.name, []), "-c", str(source), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{done.stdout}{done.stderr}")
    if verbose:
        (OBJECTS / (source.stem + ".ptxas.log")).write_text(done.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every `csrc/*.cu` for sm_100a and links `libb200q.so`."""
    if not force and not stale():
        return LIBRARY
    OBJECTS.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(lambda s: _compile(s, verbose), sources()))
    link = [nvcc(), *ARCH, "-shared", "-o", str(LIBRARY), *map(str, objects), "-cudart", "static"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"linking libb200q.so failed:\n{done.stdout}{done.stderr}")
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
