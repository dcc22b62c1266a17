"""Builds the oracle's shared objects.  Test infrastructure: see oracle/__init__.py.

oracle/_build/librestate.so   from oracle/restate.c (gcc)

The reference's own sources for this path are SYCL (icpx -fsycl, Level-Zero, a PyTorch source
tree): they cannot be compiled with the gcc/g++/nvcc toolchain here, so no oracle/_ref is built.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_build"
RESTATE_SO = OUT_DIR / "librestate.so"


def build_restate(force: bool = False) -> Path:
    src = HERE / "restate.c"
    OUT_DIR.mkdir(exist_ok=True)
    import hashlib
    stamp = OUT_DIR / "librestate.stamp"
    digest = hashlib.sha256(src.read_bytes()).hexdigest()
    if force or not RESTATE_SO.exists() or not stamp.exists() or stamp.read_text().strip() != digest:
        cmd = ["gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-std=c11", str(src), "-o", str(RESTATE_SO), "-lm"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + proc.stdout + proc.stderr)
        stamp.write_text(digest)
    return RESTATE_SO


if __name__ == "__main__":
    print(build_restate(force=True))
