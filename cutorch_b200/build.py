"""Builds libthcb200.so (sm_100a) from cutorch_b200/csrc with nvcc.

Run as ``python -m cutorch_b200.build`` or call :func:`build`.  Objects are rebuilt only
when a source or header is newer; translation units compile in parallel.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libthcb200.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",            # mul+add chains of the op table must not contract to FMAs
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-cudart", "shared",
    "-I", str(INCLUDE),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _newest_header() -> float:
    hs = (list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.rglob("*.h")) + list(INCLUDE.rglob("*.cuh")) +
          list(CSRC.glob("*.inc")))
    return max(h.stat().st_mtime for h in hs)


def build(verbose: bool = False, jobs: int | None = None) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    hdr = _newest_header()
    todo = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            todo.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return src.name, r.stderr

    if todo:
        with ThreadPoolExecutor(max_workers=jobs or min(len(todo), os.cpu_count() or 4)) as ex:
            for name, log in ex.map(compile_one, todo):
                if verbose:
                    print(f"--- {name}\n{log}", file=sys.stderr)
    if todo or not LIB.exists():
        cmd = [nvcc, "-shared", "-cudart", "shared", "-o", str(LIB), *map(str, objs),
               "-ldl",   # NCCL is bound with dlopen when a communicator is first asked for
               "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


USERTEST_SRC = PKG.parent / "tests" / "csrc" / "user_apply_test.cu"
USERTEST_LIB = PKG / "lib" / "libthcb200_usertest.so"


def build_user_test() -> Path:
    """Compiles tests/csrc/user_apply_test.cu (user functors through include/THC/THCApply.cuh) against
    the library, the way a downstream CUDA project would."""
    if not USERTEST_SRC.exists():
        return USERTEST_LIB
    newest = max(USERTEST_SRC.stat().st_mtime, _newest_header(), LIB.stat().st_mtime if LIB.exists() else 0)
    if USERTEST_LIB.exists() and USERTEST_LIB.stat().st_mtime >= newest:
        return USERTEST_LIB
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
           "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "shared", "-shared", "-I", str(INCLUDE),
           str(USERTEST_SRC), "-o", str(USERTEST_LIB), "-L", str(LIB.parent), "-lthcb200", "-Xlinker", "-rpath,$ORIGIN",
           "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the user-functor test library failed:\n{r.stdout}\n{r.stderr}")
    return USERTEST_LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
    print(build_user_test())
