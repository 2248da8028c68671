"""Builds the native libraries in-tree with nvcc / g++ (no JIT cache outside the repository).

``libxbow_cuda.so`` - every sm_100a kernel + the device program / learner executor (nvcc, -gencode arch=compute_100a).
``libxbow_rt.so``   - host-only C++ runtime: queues, replica pool, scheduler, result ring, auto-tuner, checkpoint
                      and data-set pipeline (g++; loads on machines without a GPU driver).
Objects are rebuilt only when a source or header is newer than the library.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "_lib"
OBJDIR = LIBDIR / "obj"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--use_fast_math", "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def cuda_sources():
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "runtime").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))


def rt_sources():
    return sorted((CSRC / "runtime").glob("*.cpp")) + sorted((CSRC / "data").glob("*.cpp"))


def _headers():
    return list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp"))


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd, log: Path):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.write_text(" ".join(map(str, cmd)) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}\n{r.stdout[-4000:]}")
    return r.stdout


def build_cuda(force=False, verbose=False) -> Path:
    lib = LIBDIR / "libxbow_cuda.so"
    srcs, hdrs = cuda_sources(), _headers()
    if not force and not _stale(lib, srcs + hdrs):
        return lib
    OBJDIR.mkdir(parents=True, exist_ok=True)
    jobs = []
    for s in srcs:
        o = OBJDIR / (s.stem + ".o")
        if force or _stale(o, [s] + hdrs):
            jobs.append(([_nvcc(), *NVCC_FLAGS, "-c", str(s), "-o", str(o)], OBJDIR / (s.stem + ".log")))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for out in ex.map(lambda j: _run(*j), jobs):
            if verbose:
                print(out)
    objs = [str(OBJDIR / (s.stem + ".o")) for s in srcs]
    _run([_nvcc(), "-shared", "-o", str(lib), *objs, "-lcudart", "-lcuda", "-ldl"], OBJDIR / "link_cuda.log")
    return lib


def build_rt_selftest(sanitize: str = "thread") -> Path:
    """Stand-alone self-test of the host runtime (csrc/selftest/rt_selftest.cpp) built with -fsanitize=<thread|address>."""
    exe = LIBDIR / f"rt_selftest_{sanitize}"
    srcs = rt_sources() + [CSRC / "selftest" / "rt_selftest.cpp", CSRC / "selftest" / "fake_exec.cpp"]
    if _stale(exe, srcs + _headers()):
        LIBDIR.mkdir(parents=True, exist_ok=True)
        OBJDIR.mkdir(parents=True, exist_ok=True)
        _run(["g++", "-O1", "-g", "-std=c++17", "-pthread", f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-o", str(exe),
              *map(str, srcs), "-lpthread", "-ldl"], OBJDIR / f"rt_selftest_{sanitize}.log")
    return exe


def build_rt_fake() -> Path:
    """Test-only library with the fake executor (csrc/selftest/fake_exec.cpp); it is not part of libxbow_rt.so."""
    lib = LIBDIR / "libxbow_rt_fake.so"
    src = CSRC / "selftest" / "fake_exec.cpp"
    if _stale(lib, [src]):
        OBJDIR.mkdir(parents=True, exist_ok=True)
        _run(["g++", *CXX_FLAGS, "-shared", "-o", str(lib), str(src), "-lpthread"], OBJDIR / "link_rt_fake.log")
    return lib


def build_rt(force=False) -> Path:
    lib = LIBDIR / "libxbow_rt.so"
    srcs, hdrs = rt_sources(), _headers()
    if not srcs:
        return lib
    if not force and not _stale(lib, srcs + hdrs):
        return lib
    OBJDIR.mkdir(parents=True, exist_ok=True)
    _run(["g++", *CXX_FLAGS, "-shared", "-o", str(lib), *map(str, srcs), "-lpthread"], OBJDIR / "link_rt.log")
    return lib


def build_all(force=False, verbose=False):
    return build_cuda(force, verbose), build_rt(force)


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("\n".join(str(l) for l in libs))
