"""Builds ``libturbo_gnn_b200.so`` in-tree with nvcc for sm_100a.

Usage: ``python -m turbo_gnn_b200.build [--force] [--jobs N]``.

The library has no dependency on torch or Python: every translation unit under
``csrc/`` is compiled straight to an object file and the objects are linked
into one shared library next to this package.  Objects are rebuilt only when
their source, a header or the flag set changed.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
OBJ_DIR = CSRC / "_obj"
LIB_PATH = PKG_DIR / "libturbo_gnn_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libturbo_gnn_b200.so")
    return found


def _fingerprint(paths: list[Path]) -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")


def build(force: bool = False, jobs: int | None = None, verbose: bool = False) -> Path:
    """Compile what is stale and link the shared library; returns its path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    header_print = _fingerprint(headers)
    stale: list[tuple[Path, Path, Path, str]] = []
    objects: list[Path] = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        stamp = OBJ_DIR / (src.stem + ".stamp")
        want = hashlib.sha256((header_print + _fingerprint([src])).encode()).hexdigest()
        objects.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != want:
            stale.append((src, obj, stamp, want))
    if stale:
        workers = jobs or min(len(stale), os.cpu_count() or 4)
        with ThreadPoolExecutor(max_workers=workers) as pool:
            futures = [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o, _, _ in stale]
            for f in futures:
                f.result()
        for _, _, stamp, want in stale:
            stamp.write_text(want)
    if stale or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true", help="rebuild every object")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args(argv)
    print(build(force=ns.force, jobs=ns.jobs, verbose=ns.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
