"""Builds the two native libraries of the package, in-tree.

``libopsgnn_b200.so``  hand-written sm_100a kernels behind a plain C ABI (nvcc, no torch headers);
``_pybind.so``         the torch extension with the C++ launch planners, linked against the first.

Both land in ``ops_gnn/sm100/``.  nvcc cross-compiles without a GPU, so the build runs anywhere the
CUDA toolkit and torch headers are installed.  Usage: ``python build.py [--force] [--jobs N]``.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
CUDA_SRC = ROOT / "csrc" / "cuda"
HOST_SRC = ROOT / "csrc" / "host"
OBJ_DIR = ROOT / "build"
OUT_DIR = ROOT / "ops_gnn" / "sm100"
CUDA_LIB = OUT_DIR / "libopsgnn_b200.so"
PYBIND_LIB = OUT_DIR / "_pybind.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc_flags():
    # OPSGNN_CHECKED=1 builds the self-checking diagnostic variant of the CSR reduce kernels.
    extra = ["-DOPSGNN_CHECKED"] if os.environ.get("OPSGNN_CHECKED") == "1" else []
    return NVCC_FLAGS + extra


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return str(Path(home) / "bin" / "nvcc")


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _run(cmd) -> None:
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + result.stdout + result.stderr)


def _compile_many(jobs, workers: int) -> None:
    if not jobs:
        return
    with ThreadPoolExecutor(max_workers=workers) as pool:
        list(pool.map(_run, jobs))


def build_cuda(force: bool = False, workers: int = 8) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    headers = list(CUDA_SRC.glob("*.cuh")) + list(CUDA_SRC.glob("*.h")) + [REPO / "include" / "opsgnn_b200.h"]
    header_time = _newest(headers)
    sources = sorted(CUDA_SRC.glob("*.cu"))
    jobs, objects = [], []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            jobs.append([_nvcc(), *_nvcc_flags(), "-I", str(REPO / "include"), "-c", str(src), "-o", str(obj)])
    _compile_many(jobs, workers)
    if jobs or not CUDA_LIB.exists():
        _run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(CUDA_LIB),
              *map(str, objects), "-Xlinker", "-soname,libopsgnn_b200.so"])
    return CUDA_LIB


def build_pybind(force: bool = False, workers: int = 8) -> Path:
    import torch
    from torch.utils import cpp_extension

    OBJ_DIR.mkdir(exist_ok=True)
    sources = sorted(HOST_SRC.glob("*.cpp"))
    headers = list(HOST_SRC.glob("*.h")) + [REPO / "include" / "opsgnn_b200.h"]
    header_time = _newest(headers)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], str(REPO / "include"),
                str(Path(cuda_home) / "include")]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=_pybind",
             "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "-Wno-attributes"]
    jobs, objects = [], []
    for src in sources:
        obj = OBJ_DIR / ("host_" + src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            cmd = ["g++", *flags]
            for inc in includes:
                cmd += ["-isystem", inc]
            cmd += ["-c", str(src), "-o", str(obj)]
            jobs.append(cmd)
    _compile_many(jobs, workers)
    stale = not PYBIND_LIB.exists() or PYBIND_LIB.stat().st_mtime < CUDA_LIB.stat().st_mtime
    if jobs or stale:
        lib_dirs = cpp_extension.library_paths()
        cmd = ["g++", "-shared", "-o", str(PYBIND_LIB), *map(str, objects), f"-L{OUT_DIR}", "-lopsgnn_b200",
               "-Wl,-rpath,$ORIGIN"]
        for d in lib_dirs:
            cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
        cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
        _run(cmd)
    return PYBIND_LIB


def build_all(force: bool = False, workers: int = 8) -> None:
    build_cuda(force, workers)
    build_pybind(force, workers)


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    parser.add_argument("--cuda-only", action="store_true")
    args = parser.parse_args()
    if args.cuda_only:
        print(build_cuda(args.force, args.jobs))
    else:
        build_all(args.force, args.jobs)
        print(CUDA_LIB, PYBIND_LIB, sep="\n")
    sys.exit(0)
