"""Build the sm_100a kernel library in-tree with nvcc.

``python -m aotolith_b200.csrc.build`` compiles every ``.cu`` file of this
directory into ``aotolith_b200/_lib/libaoto_sm100.so``. The compile is a plain
cross-compile: it needs nvcc, not a GPU.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
REPO = PACKAGE.parent
LIB_DIR = PACKAGE / "_lib"
LIB_PATH = LIB_DIR / "libaoto_sm100.so"
STAMP = LIB_DIR / "libaoto_sm100.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or add the CUDA toolkit to PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    digest = hashlib.sha256()
    for path in [*sources(), *sorted(CSRC.glob("*.cuh")), REPO / "include" / "aoto_sm100.h"]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if its sources changed; return its path."""

    digest = _digest()
    if not force and LIB_PATH.exists() and STAMP.exists() and STAMP.read_text() == digest:
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    objects = []
    nvcc = _nvcc()
    build_dir = LIB_DIR / "obj"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for source in sources():
        obj = build_dir / (source.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(REPO / "include"), "-I", str(CSRC), "-c", str(source), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(obj)
    failed = False
    for source, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            print(f"--- {source.name}\n{out}", file=sys.stderr)
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the log above")
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects), "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(link, check=True)
    STAMP.write_text(digest)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
