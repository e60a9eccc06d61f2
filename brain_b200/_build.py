"""In-tree native build: every ``csrc/**/*.cu`` is compiled by nvcc for sm_100a into one shared
library (``brain_b200/_lib/libbrain_b200.so``, C ABI, loaded with ctypes) and the host runtime
(``csrc/**/*.cpp``) into ``brain_b200/_lib/libbrain_host.so``.

Nothing here needs a GPU: nvcc cross-compiles.  Objects are rebuilt only when their source (or a
header) is newer, so repeated calls are cheap.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "_lib"
OBJDIR = ROOT / "build" / "obj"

CUDA_LIB = LIBDIR / "libbrain_b200.so"
HOST_LIB = LIBDIR / "libbrain_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
#: translation units whose arithmetic feeds the optimiser state or the loss: compiled without
#: --use_fast_math (IEEE division and square root in the AdamW update, exact exp/log in the CE)
EXACT_MATH = {"adamw.cu", "rs_adamw.cu", "ce.cu"}
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-march=x86-64-v3"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _stale(src: Path, obj: Path, hdr_mtime: float) -> bool:
    if not obj.exists():
        return True
    m = obj.stat().st_mtime
    return src.stat().st_mtime > m or hdr_mtime > m


def _run(cmd: list[str], log: Path | None = None) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(p.stdout)
    if p.returncode != 0:
        sys.stderr.write(p.stdout)
        raise RuntimeError("build failed: " + " ".join(cmd))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted(CSRC.rglob("*.cu"))
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJDIR / (str(s.relative_to(CSRC)).replace("/", "__") + ".o")
        objs.append(o)
        if force or _stale(s, o, hdr):
            jobs.append((s, o))

    def compile_one(so):
        s, o = so
        extra = ["-DBB_TIMELINE"] if os.environ.get("BB_TIMELINE") == "1" else []
        flags = NVCC_FLAGS
        if s.name in EXACT_MATH:
            flags = [f for f in NVCC_FLAGS if f != "--use_fast_math"]
        _run([nvcc, *flags, *extra, "-I", str(CSRC), "-c", str(s), "-o", str(o)],
             log=o.with_suffix(".log"))
        if verbose:
            print(f"[build] {s.relative_to(ROOT)}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not CUDA_LIB.exists():
        _run([nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-lcudart"])
    return CUDA_LIB


def build_host(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted(CSRC.rglob("*.cpp"))
    if not srcs:
        return HOST_LIB
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    cxx = os.environ.get("CXX", "g++")
    jobs, objs = [], []
    for s in srcs:
        o = OBJDIR / (str(s.relative_to(CSRC)).replace("/", "__") + ".o")
        objs.append(o)
        if force or _stale(s, o, hdr):
            jobs.append((s, o))

    def compile_one(so):
        s, o = so
        _run([cxx, *CXX_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)])
        if verbose:
            print(f"[build] {s.relative_to(ROOT)}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not HOST_LIB.exists():
        _run([cxx, "-shared", "-o", str(HOST_LIB), *map(str, objs), "-pthread"])
    return HOST_LIB


#: translation units of the bounds-checking library (kernels whose addresses depend on data) and
#: what they need at link time
BOUNDS_TUS = ["kernels/elementwise.cu", "kernels/ce.cu", "kernels/moe.cu", "common/host.cu"]
BOUNDS_LIB = LIBDIR / "libbrain_b200_bounds.so"


def build_bounds(force: bool = False, verbose: bool = False) -> Path:
    """A second, small library of the index-driven kernels compiled with -DBB_DEBUG_BOUNDS: every
    data-dependent index is checked against its extent, a violation writes an error code and skips
    the access.  Loaded by tests only: production code never links it."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    nvcc = _nvcc()
    objs, jobs = [], []
    for rel in BOUNDS_TUS:
        s = CSRC / rel
        o = OBJDIR / ("bounds__" + rel.replace("/", "__") + ".o")
        objs.append(o)
        if force or _stale(s, o, hdr):
            jobs.append((s, o))
    for s, o in jobs:
        flags = [f for f in NVCC_FLAGS if f != "--use_fast_math"] if s.name in EXACT_MATH else NVCC_FLAGS
        _run([nvcc, *flags, "-DBB_DEBUG_BOUNDS", "-I", str(CSRC), "-c", str(s), "-o", str(o)],
             log=o.with_suffix(".log"))
        if verbose:
            print(f"[build] bounds {s.relative_to(ROOT)}")
    if jobs or not BOUNDS_LIB.exists():
        _run([nvcc, "-shared", "-o", str(BOUNDS_LIB), *map(str, objs), "-lcudart"])
    return BOUNDS_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force, verbose)
    build_cuda(force, verbose)
    build_bounds(force, verbose)


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last build (registers, spills, smem per kernel)."""
    out = []
    for log in sorted(OBJDIR.glob("*.log")):
        out.append(f"== {log.name}\n{log.read_text()}")
    return "\n".join(out)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    if "--report" in sys.argv:
        print(ptxas_report())
