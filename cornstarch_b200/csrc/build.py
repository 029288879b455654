"""In-tree build of the native sm_100a library.

Every ``*.cu`` file in this directory is compiled with nvcc for ``sm_100a`` only and linked into
``cornstarch_b200/lib/libcornstarch_b200.so``.  The library exposes a plain C ABI (see the
``CSB_API`` functions) that :mod:`cornstarch_b200.ops._native` loads with ``ctypes``; no torch
headers are involved, so a full rebuild takes well under a minute and works on a machine without a
GPU (nvcc cross-compiles).

Run ``python -m cornstarch_b200.csrc.build`` (add ``--force`` to rebuild everything, ``-v`` for the
ptxas resource report, ``--bounds-check`` for the debug library with index checks).
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_DIR = PKG / "lib"
OBJ_DIR = CSRC / "build"
LIB_PATH = LIB_DIR / "libcornstarch_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")
    return cand


def _headers() -> list[Path]:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def _needs_build(src: Path, obj: Path) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    if src.stat().st_mtime > t:
        return True
    return any(h.stat().st_mtime > t for h in _headers())


def _compile(src: Path, obj: Path, verbose: bool, defines: tuple = ()) -> str:
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, *[f"-D{d}" for d in defines], "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return res.stderr


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


DEBUG_LIB_PATH = LIB_DIR / "libcornstarch_b200_dbg.so"
# Only the translation units that index memory by DATA carry bounds checks; the debug library reuses the release objects
# of the others.
BOUNDS_CHECKED_UNITS = ("elementwise", "moe_dispatch", "symm")


def build(force: bool = False, verbose: bool = False, bounds_check: bool = False) -> Path:
    """Compile what is stale and (re)link the shared library.  Returns its path.

    ``bounds_check=True`` builds ``lib/libcornstarch_b200_dbg.so`` instead: the same library with ``-DCSB_BOUNDS_CHECK``
    (indices that kernels take from data are checked against the extents passed in; a violation is recorded and the
    access skipped).  Load it with ``CORNSTARCH_B200_LIB=<path>``; ``ops._native.bounds_status()`` reads the record."""
    if bounds_check:
        build(force, verbose)  # the release objects of the unchecked units
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    srcs = sources()
    objs = [OBJ_DIR / (s.stem + ".o") for s in srcs]
    lib_path, defines = LIB_PATH, ()
    if bounds_check:
        objs = [OBJ_DIR / (s.stem + ("_dbg.o" if s.stem in BOUNDS_CHECKED_UNITS else ".o")) for s in srcs]
        lib_path, defines = DEBUG_LIB_PATH, ("CSB_BOUNDS_CHECK",)
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _needs_build(s, o)]
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            futs = {ex.submit(_compile, s, o, verbose, defines if o.name.endswith("_dbg.o") else ()): s for s, o in todo}
            for f in cf.as_completed(futs):
                log = f.result()
                if verbose and log:
                    print(f"--- {futs[f].name}\n{log}", file=sys.stderr)
    stale = (not lib_path.exists()) or any(o.stat().st_mtime > lib_path.stat().st_mtime for o in objs)
    if todo or stale:
        cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(lib_path), *map(str, objs), "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv, bounds_check="--bounds-check" in sys.argv)
    print(p)
