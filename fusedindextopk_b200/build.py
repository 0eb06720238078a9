"""Build ``libitk_b200.so`` in-tree with nvcc for sm_100a.

``python -m fusedindextopk_b200.build`` compiles ``csrc/itk_api.cu`` (which
includes the kernel headers) into ``fusedindextopk_b200/libitk_b200.so``.  The
build is ahead-of-time: nvcc cross-compiles without a GPU, and the resulting
library needs only the CUDA runtime and driver on the target machine.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIBRARY = PACKAGE_DIR / "libitk_b200.so"
STAMP = PACKAGE_DIR / "libitk_b200.so.srchash"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def source_hash() -> str:
    digest = hashlib.sha256()
    for path in _sources():
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_current() -> bool:
    return LIBRARY.exists() and STAMP.exists() and STAMP.read_text().strip() == source_hash()


def build(*, force: bool = False, verbose: bool = False) -> Path:
    """Compile the library unless an up-to-date one is already in the tree."""

    if not force and is_current():
        return LIBRARY
    command = [find_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(LIBRARY), str(CSRC / "itk_api.cu")]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    (PACKAGE_DIR / "libitk_b200.ptxas.log").write_text(result.stdout + result.stderr)
    STAMP.write_text(source_hash() + "\n")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
