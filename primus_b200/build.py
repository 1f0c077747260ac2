"""Builds the native library (``primus_b200/lib/libprimus_b200.so``) from ``primus_b200/csrc``.

All device code targets sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); nvcc
cross-compiles it on hosts without a GPU.  The library exposes plain ``extern "C"`` launchers
(raw pointers + a CUDA stream) that :mod:`primus_b200.ops._lib` binds with ctypes, so no torch
headers are needed and a full rebuild takes seconds.

Run ``python -m primus_b200.build`` (add ``--force`` to rebuild everything, ``--verbose`` to see
ptxas resource usage).
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libprimus_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))


def _needs_build(src: Path, obj: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or any(h.stat().st_mtime > t for h in headers)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> tuple[Path, int, str]:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd = [nvcc, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    elif verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    return src, p.returncode, p.stdout + p.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile out-of-date sources and link the shared library. Returns the library path."""
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    jobs = []
    objs = []
    for src in _sources():
        obj = OBJ_DIR / (src.name + ".o")
        objs.append(obj)
        if force or _needs_build(src, obj, headers):
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            results = list(ex.map(lambda so: _compile_one(nvcc, so[0], so[1], verbose), jobs))
        failed = [(s, out) for s, rc, out in results if rc != 0]
        if verbose:
            for s, rc, out in results:
                print(f"--- {s.name}\n{out}")
        if failed:
            msg = "\n".join(f"{s}:\n{out}" for s, out in failed)
            raise RuntimeError(f"nvcc failed:\n{msg}")
    if jobs or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart", "-ldl"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stdout}{p.stderr}")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    path = build(force=a.force, verbose=a.verbose)
    print(path)


if __name__ == "__main__":
    sys.exit(main())
