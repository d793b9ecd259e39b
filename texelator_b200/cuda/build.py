"""Build libtexelator_b200.so in-tree with nvcc for sm_100a.

    python -m texelator_b200.cuda.build [--force] [--verbose]

The library is a plain C-ABI shared object (see include/texelator_b200.h); it links only the CUDA
runtime.  Reference counterpart: setup.py:9-36 / texelator/runtime.py:43-62, which build a torch
extension with no -gencode at all.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCES = ["tx_api.cu", "tx_pack.cu", "tx_gemv.cu", "tx_prefill.cu", "tx_aux.cu", "tx_encode.cu"]
LIBRARY = HERE / "libtexelator_b200.so"
STAMP = HERE / ".build_stamp"


def source_digest() -> str:
    digest = hashlib.sha256()
    for path in sorted(HERE.glob("*.cu")) + sorted(HERE.glob("*.cuh")) + [HERE.parent.parent / "include" / "texelator_b200.h"]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc was not found; the CUDA library cannot be built")
    return found


def build(force: bool = False, verbose: bool = False) -> Path:
    digest = source_digest()
    if not force and LIBRARY.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
        return LIBRARY
    sources = [str(HERE / name) for name in SOURCES if (HERE / name).exists()]
    command = [
        nvcc_path(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-Xptxas", "-v", "--shared", "-Xcompiler", "-fPIC", "--threads", "4",
        "-o", str(LIBRARY), *sources,
    ]
    result = subprocess.run(command, capture_output=True, text=True)
    (HERE / "build.log").write_text(" ".join(command) + "\n" + result.stdout + result.stderr)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}; see {HERE / 'build.log'}")
    STAMP.write_text(digest + "\n")
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path, os.path.getsize(path), "bytes")
