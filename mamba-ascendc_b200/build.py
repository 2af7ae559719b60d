"""Build libssd_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: ``python mamba-ascendc_b200/build.py [--force] [--verbose]``.  The shared
object is written next to the Python package so that ``ascend_kernel`` finds it
without any install step.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ_DIR = ROOT / "build"
LIB_PATH = ROOT / "ascend_kernel" / "libssd_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libssd_b200.so cannot be built")
    return exe


# Sources that exist for the test suite only (tile-level checks of the tensor-core path and of the give-up
# path of the bounded waits, behind the ssd_selftest_* entry points).  They are linked into the library by
# default so that one shared object serves the product and its tests; ``--product-only`` leaves them out.
TEST_HOOK_SOURCES = {"ssd_selftest.cu"}


def _sources(product_only: bool = False) -> list[Path]:
    return sorted(p for p in CSRC.glob("*.cu") if not (product_only and p.name in TEST_HOOK_SOURCES))


def _deps_mtime() -> float:
    deps = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [ROOT.parent / "include" / "ssd_b200.h"]
    return max(p.stat().st_mtime for p in deps)


def build(force: bool = False, verbose: bool = False, product_only: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` to an object and link the shared library (without the test hooks if
    ``product_only``; the Python binding then simply has no ``ssd_selftest_*`` functions)."""
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdr_mtime = _deps_mtime()
    jobs = []
    objs = []
    for src in _sources(product_only):
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_mtime)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, res

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, res in pool.map(run, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    flavour = OBJ_DIR / ".flavour"
    want_flavour = "product-only" if product_only else "with-test-hooks"
    relink = not flavour.exists() or flavour.read_text() != want_flavour
    need_link = bool(jobs) or not LIB_PATH.exists() or relink
    if need_link:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("linking libssd_b200.so failed")
        flavour.write_text(want_flavour)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/shared-memory usage")
    ap.add_argument("--product-only", action="store_true", help="leave the test-only ssd_selftest_* entry points out")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose, product_only=args.product_only))
