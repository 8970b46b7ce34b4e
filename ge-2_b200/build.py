"""Builds the native pieces in-tree: libge2_b200.so (CUDA kernels + C ABI, sm_100a only) and, on request, the
libtorch host layer.  `python ge-2_b200/build.py [--force] [--host]`."""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libge2_b200.so"
HOST_LIB = PKG / "ge2_host.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + [ROOT / "include" / "ge2_b200.h"]
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append([NVCC, *NVCC_FLAGS, *( ["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)])
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out:
                print(out)
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(LIB, objs):
        _run([NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC"])  # static cudart; libcuda is not linked (driver entry points are looked up at run time)
    return LIB


def build_host(force: bool = False) -> Path:
    """The libtorch host layer (C++ mirror of the reference's trainer/model/storage interface) + its Python binding."""
    import sysconfig

    import torch

    tdir = Path(torch.__file__).parent
    srcs = sorted((PKG / "host").glob("*.cpp"))
    hdrs = list((PKG / "host").glob("*.h")) + [ROOT / "include" / "ge2_b200.h"]
    if not srcs:
        raise RuntimeError("no host sources")
    OBJ.mkdir(exist_ok=True)
    flags = ["-std=c++17", "-O2", "-fPIC", "-w", f"-I{ROOT / 'include'}", f"-I{tdir / 'include'}",
             f"-I{tdir / 'include/torch/csrc/api/include'}", f"-I{sysconfig.get_paths()['include']}", "-I/usr/local/cuda/include",
             "-DTORCH_EXTENSION_NAME=ge2_host", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / ("host_" + s.stem + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(["g++", *flags, "-c", str(s), "-o", str(o)])
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    if force or jobs or _stale(HOST_LIB, objs + [LIB]):
        _run(["g++", "-shared", "-o", str(HOST_LIB), *map(str, objs), f"-L{PKG}", "-lge2_b200", f"-L{tdir / 'lib'}",
              "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
              f"-Wl,-rpath,{tdir / 'lib'}", "-Wl,-rpath,$ORIGIN"])
    return HOST_LIB


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_kernels(force=force, verbose="-v" in sys.argv))
    if "--host" in sys.argv:
        print(build_host(force=force))
