"""In-tree build of the native code: the sm_100a kernel library and the C++ executor module.

``python -m nanoflow_b200.ops.build`` compiles every ``csrc/kernels/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into ``nanoflow_b200/ops/libnanoflow_kernels.so``
and ``csrc/executor/*.cpp`` into ``nanoflow_b200/runtime/_executor*.so``. Objects are cached under
``build/`` and rebuilt only when a source or header is newer. nvcc cross-compiles without a GPU.

The reference builds with CMake for sm_80 (pipeline/CMakeLists.txt:5-8, gemv/CMakeLists.txt:8);
this is the equivalent for a single architecture and no third-party submodules.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
ROOT = PKG.parent
KERNEL_DIR = PKG / "csrc" / "kernels"
EXEC_DIR = PKG / "csrc" / "executor"
BUILD_DIR = ROOT / "build"
KERNEL_LIB = PKG / "ops" / "libnanoflow_kernels.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr"]


def executor_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / "runtime" / f"_executor{suffix}"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr, flush=True)
    return res


def build_kernels(verbose: bool = False, ptxas_info: bool = False) -> Path:
    BUILD_DIR.mkdir(exist_ok=True)
    headers = list(KERNEL_DIR.glob("*.cuh")) + list(KERNEL_DIR.glob("*.h"))
    sources = sorted(KERNEL_DIR.glob("*.cu"))
    objs = []
    jobs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        objs.append(obj)
        if _newer(obj, [src] + headers) or ptxas_info:
            cmd = [NVCC, *ARCH_FLAGS, *NVCC_FLAGS, "-I", KERNEL_DIR, "-c", src, "-o", obj]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    if jobs or _newer(KERNEL_LIB, objs):
        _run([NVCC, *ARCH_FLAGS, "-shared", "-o", KERNEL_LIB, *objs], verbose)  # static cudart
    return KERNEL_LIB


def build_executor(verbose: bool = False) -> Path:
    import pybind11

    out = executor_lib_path()
    sources = sorted(EXEC_DIR.glob("*.cpp"))
    if not sources:
        return out
    headers = list(EXEC_DIR.glob("*.h")) + list(KERNEL_DIR.glob("*.h"))
    if _newer(out, sources + headers + [KERNEL_LIB]):
        inc = sysconfig.get_paths()["include"]
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
               "-I", pybind11.get_include(), "-I", inc, "-I", "/usr/local/cuda/include",
               "-I", KERNEL_DIR, *sources, "-o", out,
               "-L", KERNEL_LIB.parent, "-l:libnanoflow_kernels.so",
               "-L", "/usr/local/cuda/lib64", "-lcudart_static", "-ldl", "-lrt", "-lpthread",
               "-Wl,-rpath,$ORIGIN/../ops"]
        _run(cmd, verbose)
    return out


def executor_host_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / "runtime" / f"_executor_host{suffix}"


def build_executor_host(verbose: bool = False, sanitize: str = "") -> Path:
    """The executor compiled against ``csrc/executor/host_cuda.h`` instead of the CUDA runtime: the
    same worker thread, symbol patching, event wiring and graph-mode logic, with every runtime call
    logged instead of made. Links nothing from CUDA, so it loads and runs on a machine without a GPU.
    ``sanitize="thread"`` (or ``"address"``) builds an instrumented copy under ``build/<sanitize>/``
    for a run with the sanitizer's runtime preloaded."""
    import pybind11

    out = executor_host_lib_path()
    if sanitize:
        out = BUILD_DIR / sanitize / out.name
        out.parent.mkdir(parents=True, exist_ok=True)
    sources = sorted(EXEC_DIR.glob("*.cpp"))
    if not sources:
        return out
    if _newer(out, sources + list(EXEC_DIR.glob("*.h"))):
        inc = sysconfig.get_paths()["include"]
        cmd = ["g++", "-O1", "-g", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
               "-DNF_HOST_CUDA", "-DNF_EXECUTOR_MODULE=_executor_host",
               "-I", pybind11.get_include(), "-I", inc, "-I", EXEC_DIR, *sources, "-o", out, "-lpthread"]
        if sanitize:
            cmd.insert(1, f"-fsanitize={sanitize}")
        _run(cmd, verbose)
    return out


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_executor(verbose)
    build_executor_host(verbose)


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--ptxas" in sys.argv:
        build_kernels(True, ptxas_info=True)
    else:
        build_all(v)
    print("built", KERNEL_LIB, executor_lib_path())
