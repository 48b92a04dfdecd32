"""Build the sm_100a shared library in-tree with nvcc.

``python -m nvfp4moe_b200.build`` compiles every ``csrc/*.cu`` file into
``nvfp4moe_b200/liblightmoe_b200.so``.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import hashlib
import pathlib
import subprocess
import sys

PACKAGE_DIR = pathlib.Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIBRARY = PACKAGE_DIR / "liblightmoe_b200.so"
STAMP = PACKAGE_DIR / "liblightmoe_b200.so.stamp"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math=false",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]


def _sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    digest = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) +
                       [PACKAGE_DIR.parent / "include" / "lightmoe_b200.h"]):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    fingerprint = _fingerprint()
    if not force and LIBRARY.exists() and STAMP.exists() and STAMP.read_text() == fingerprint:
        return LIBRARY
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    cmd = ["nvcc", *flags]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIBRARY), *map(str, _sources())]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(result.stderr)
    STAMP.write_text(fingerprint)
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
