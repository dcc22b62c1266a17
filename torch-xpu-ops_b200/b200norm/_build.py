"""In-tree build of the two shared objects.

libb200norm.so      CUDA kernels + C ABI (include/b200norm.h); nvcc, sm_100a only, no torch.
_b200norm_aten.so   ATen dispatcher registration (csrc/aten_register.cpp); g++ against the torch
                    headers, linked to libb200norm.so through an $ORIGIN rpath.

Both land next to this file so a snapshot of the tree carries them.  Objects are cached under
torch-xpu-ops_b200/build/ and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent            # torch-xpu-ops_b200/
CSRC = ROOT / "csrc"
INCLUDE = ROOT.parent / "include"
BUILD = ROOT / "build"
LIB = PKG_DIR / "libb200norm.so"
ATEN_LIB = PKG_DIR / "_b200norm_aten.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--threads", "2",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _digest(paths, extra: str = "") -> str:
    """Content hash of the given files: the up-to-date test that survives a copy of the tree (mtimes do not)."""
    import hashlib
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _stamp_ok(stamp: Path, digest: str, product: Path) -> bool:
    return product.exists() and stamp.exists() and stamp.read_text().strip() == digest


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def _run(cmd) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(map(str, cmd)) + "\n" + proc.stdout + proc.stderr)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    hdr_time = _newest(headers)
    sources = sorted(CSRC.glob("*.cu"))
    stamp = PKG_DIR / ".libb200norm.stamp"
    digest = _digest(headers + sources, " ".join(NVCC_FLAGS))
    if not force and _stamp_ok(stamp, digest, LIB):
        return LIB
    nvcc = _nvcc()
    jobs = []
    objects = []
    for src in sources:
        obj = BUILD / (src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            jobs.append([nvcc, *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)])
    if jobs:
        if verbose:
            print(f"[b200norm] compiling {len(jobs)} CUDA source(s) for sm_100a", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=max(1, (os.cpu_count() or 2) // 2)) as pool:
            list(pool.map(_run, jobs))
    if jobs or force or not LIB.exists() or LIB.stat().st_mtime < _newest(objects):
        _run([nvcc, "-shared", "-o", str(LIB), *map(str, objects), "-cudart", "shared"])
    stamp.write_text(digest)
    return LIB


def build_aten(force: bool = False, verbose: bool = False) -> Path:
    from torch.utils import cpp_extension as ce
    import torch

    src = CSRC / "aten_register.cpp"
    deps = [src, INCLUDE / "b200norm.h"]
    stamp = PKG_DIR / "._b200norm_aten.stamp"
    digest = _digest(deps, torch.__version__)
    if not force and _stamp_ok(stamp, digest, ATEN_LIB):
        return ATEN_LIB
    if verbose:
        print("[b200norm] compiling the ATen registration", file=sys.stderr)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{INCLUDE}"]
    torch_lib = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, str(src), "-o", str(ATEN_LIB),
        f"-L{PKG_DIR}", "-lb200norm", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}", "-Wl,--no-as-needed",
    ]
    _run(cmd)
    stamp.write_text(digest)
    return ATEN_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_aten(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print(LIB)
    print(ATEN_LIB)
