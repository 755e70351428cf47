"""In-tree build of the native extensions.

Two shared objects are produced next to this file:

* ``_core``  – host-only C++ (codec, tree join, TCP edges, CPU replica node); built with g++.
* ``_cuda``  – sm_100a kernels, the peer-memory transport and the GPU engine; built with nvcc for
  ``compute_100a/sm_100a`` only, CUDA runtime linked statically so the module also imports on a
  machine without a GPU or driver.

``python -m sharedtensor_b200._build`` builds both; ``ensure_built()`` rebuilds what is stale.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"

CORE_SOURCES = ["core/codec.cpp", "core/codec_fast.cpp", "core/tree.cpp", "core/node.cpp", "core/bindings.cpp"]
CUDA_SOURCES_CU = ["cuda/elementwise.cu", "cuda/round.cu", "cuda/noalloc.cu"]
CUDA_SOURCES_CPP = ["core/codec.cpp", "core/codec_fast.cpp", "core/tree.cpp", "cuda/vmm.cpp", "cuda/engine.cpp", "cuda/gpu_node.cpp",
                    "cuda/bindings_cuda.cpp"]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def _includes() -> list[str]:
    import pybind11

    return [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}", "-I/usr/local/cuda/include"]


def target_path(name: str) -> Path:
    return HERE / f"{name}{_ext_suffix()}"


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    deps = list(sources) + list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))
    return any(p.exists() and p.stat().st_mtime > t for p in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed ({res.returncode}):\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout.strip() or res.stderr.strip()):
        print(res.stdout + res.stderr, flush=True)


def _compile_cpp(src: Path, obj: Path, verbose: bool, extra: list[str] | None = None) -> None:
    cmd = [CXX, "-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-ffp-contract=off", "-fvisibility=hidden", "-pthread",
           *_includes(), *(extra or []), "-c", str(src), "-o", str(obj)]
    _run(cmd, verbose)


def _compile_cu(src: Path, obj: Path, verbose: bool, ptxas_v: bool) -> None:
    cmd = [NVCC, "-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "--fmad=false" if src.name in ("round.cu",) else "--fmad=true",
           *os.environ.get("ST_NVCC_FLAGS", "").split(), *_includes(), "-c", str(src), "-o", str(obj)]
    if ptxas_v:
        cmd.insert(1, "-Xptxas=-v")
    _run(cmd, verbose or ptxas_v)


def build_core(force: bool = False, verbose: bool = False) -> Path:
    target = target_path("_core")
    srcs = [CSRC / s for s in CORE_SOURCES]
    if not force and not _stale(target, srcs):
        return target
    OBJ.mkdir(exist_ok=True)
    objs = [OBJ / (s.replace("/", "_") + ".core.o") for s in CORE_SOURCES]
    with ThreadPoolExecutor(4) as ex:
        list(ex.map(lambda so: _compile_cpp(so[0], so[1], verbose), zip(srcs, objs)))
    _run([CXX, "-shared", "-pthread", "-o", str(target), *map(str, objs)], verbose)
    return target


def build_cuda(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    target = target_path("_cuda")
    cu = [CSRC / s for s in CUDA_SOURCES_CU if (CSRC / s).exists()]
    cpp = [CSRC / s for s in CUDA_SOURCES_CPP if (CSRC / s).exists()]
    if not force and not _stale(target, cu + cpp):
        return target
    OBJ.mkdir(exist_ok=True)
    cu_objs = [OBJ / (s.name + ".o") for s in cu]
    cpp_objs = [OBJ / (s.parent.name + "_" + s.name + ".cuda.o") for s in cpp]
    with ThreadPoolExecutor(6) as ex:
        futs = [ex.submit(_compile_cu, s, o, verbose, ptxas_v) for s, o in zip(cu, cu_objs)]
        futs += [ex.submit(_compile_cpp, s, o, verbose, ["-DST_WITH_CUDA"]) for s, o in zip(cpp, cpp_objs)]
        for f in futs:
            f.result()
    _run([NVCC, "-shared", *ARCH_FLAGS, "-cudart", "static", "-Xcompiler", "-pthread", "-o", str(target),
          *map(str, cu_objs + cpp_objs), "-ldl", "-lrt"], verbose)
    return target


def ensure_built(verbose: bool = False) -> None:
    build_core(verbose=verbose)
    build_cuda(verbose=verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    build_core(force=force, verbose=True)
    build_cuda(force=force, verbose=True, ptxas_v="--ptxas-v" in sys.argv)
    print("built:", target_path("_core").name, target_path("_cuda").name)
