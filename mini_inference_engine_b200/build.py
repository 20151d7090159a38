"""Build ``libmie_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

The library is plain CUDA C++ with ``extern "C"`` entry points: it does not
link against PyTorch, so the build is a handful of ``nvcc`` invocations and
the result can be loaded from any host language.  ``python -m
mini_inference_engine_b200.build`` rebuilds when a source changed.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
INCLUDE_DIR = PACKAGE_DIR.parent / "include"
LIB_PATH = PACKAGE_DIR / "libmie_b200.so"
STAMP_PATH = PACKAGE_DIR / "libmie_b200.stamp"
OBJ_DIR = PACKAGE_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; the CUDA extension cannot be built")


def _sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def source_digest() -> str:
    digest = hashlib.sha256()
    for path in [*_sources(), *sorted(CSRC_DIR.glob("*.cuh")), *sorted(INCLUDE_DIR.glob("*.h"))]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == source_digest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link the shared library; returns its path."""

    if not force and is_current():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    log_dir = OBJ_DIR

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        (log_dir / (src.stem + ".ptxas.log")).write_text(done.stdout + done.stderr)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{done.stdout}\n{done.stderr}")
        if verbose:
            print(done.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, _sources()))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects)]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    STAMP_PATH.write_text(source_digest())
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
