"""Builds ``libkeepvq.so`` (CUDA, sm_100a only) next to this file.

    python -m keep_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects land in ``keep_b200/build/``; the library is rebuilt
only when a source or header is newer than it.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIBRARY = PACKAGE_DIR / "libkeepvq.so"
OBJ_DIR = PACKAGE_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(d.stat().st_mtime > stamp for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link the shared library.  Returns its path."""
    nvcc = find_nvcc()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    srcs = sources()
    OBJ_DIR.mkdir(exist_ok=True)
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or ptxas_info or _stale(obj, [src] + headers):
            cmd = [nvcc, *flags, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
            done = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or ptxas_info or done.returncode:
                sys.stderr.write(f"$ {' '.join(cmd)}\n{done.stdout}{done.stderr}")
            if done.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    if force or _stale(LIBRARY, objs):
        cmd = [nvcc, "-shared", "-o", str(LIBRARY), *map(str, objs)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or done.returncode:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{done.stdout}{done.stderr}")
        if done.returncode:
            raise RuntimeError("linking libkeepvq.so failed")
    return LIBRARY


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    ns = ap.parse_args()
    print(build(force=ns.force, verbose=ns.verbose, ptxas_info=ns.ptxas_info))


if __name__ == "__main__":
    main()
