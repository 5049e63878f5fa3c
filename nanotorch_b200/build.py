"""Build step of the package: compiles csrc/*.cu for sm_100a and links lib/libnt_b200.so.

Run as ``python nanotorch_b200/build.py`` (add ``--force`` to rebuild everything); it is run by
path because importing the package needs the library this script produces.  Objects are
rebuilt only when their source or a header is newer.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "_obj"
LIB = PKG / "lib" / "libnt_b200.so"
INCLUDE = PKG.parent / "include"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

# --fmad=false: no implicit a*b+c contraction anywhere, so every kernel rounds exactly where its
# source says; the GEMM kernels call fmaf() explicitly.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++20", "--fmad=false",
    "-Xcompiler", "-fPIC,-fvisibility=default",
    "-Xptxas", "-v",
]


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(INCLUDE.glob("*.h"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, force: bool) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    if not force and not _stale(obj, [src] + _headers()):
        return obj, ""
    cmd = [NVCC, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    (OBJ / (src.stem + ".log")).write_text(log)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{log[-4000:]}")
    return obj, log


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library; returns its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile(s, force), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or _stale(LIB, objs):
        cmd = [
            NVCC, "-shared", "-o", str(LIB), *map(str, objs),
            "-lcudart", "-ldl", "-Xlinker", f"-rpath={CUDA_HOME / 'lib64'}",
        ]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("link failed:\n" + proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
