"""Builds ``libneuronspark_b200.so`` in-tree with nvcc for sm_100a.

    python -m neuronspark_b200.build [--force]

The library has no dependency on PyTorch or Python: it is a plain C-ABI shared
object (see ``include/neuronspark_b200.h``) with the CUDA runtime linked
statically. nvcc cross-compiles without a GPU, so this also runs on a CPU-only
build box.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libneuronspark_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-diag-suppress", "549",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _deps_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "neuronspark_b200.h"]
    return max(p.stat().st_mtime for p in hdrs)


def _extra_flags() -> list[str]:
    """Extra nvcc flags for experiments, e.g. NSB_NVCC_FLAGS="-DNSB_X2=0"."""
    return os.environ.get("NSB_NVCC_FLAGS", "").split()


def _compile_one(nvcc: str, src: Path, force: bool, hdr_mtime: float) -> Path:
    obj = OBJ / (src.stem + ".o")
    if (not force and obj.exists() and obj.stat().st_mtime >= src.stat().st_mtime
            and obj.stat().st_mtime >= hdr_mtime):
        return obj
    cmd = [nvcc, *NVCC_FLAGS, *_extra_flags(), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    srcs = sources()
    hdr_mtime = _deps_mtime()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile_one(nvcc, s, force, hdr_mtime), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(f"built {LIB} from {len(srcs)} sources")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
