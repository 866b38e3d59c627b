"""Ahead-of-time build of the two in-tree shared objects (no JIT, nothing is built on import).

  consumer_int8/libci8.so   the sm_100a kernels behind the C ABI of include/ci8.h (nvcc)
  consumer_int8/_C.so       torch stable-ABI operators over that C ABI (g++)

Run ``python build.py`` from this directory, or call :func:`build`. Compiles for
``-gencode arch=compute_100a,code=sm_100a`` only; a GPU is not needed to build. Follows the
reference's setup.py:9-26 flags (stable ABI defines, -O3, -lineinfo, no fast-math).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
PKG = HERE / "consumer_int8"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-shared",
]
STABLE_DEFINES = [
    "-DTORCH_STABLE_ONLY", "-DUSE_CUDA", "-DPy_LIMITED_API=0x030A0000",
    "-DTORCH_TARGET_VERSION=0x020A000000000000",
]


def _host_cxx() -> str:
    """The distribution's g++ (dynamic libstdc++). A toolchain wrapper that links libstdc++
    statically would put a second, uninitialised copy of the iostream/locale state inside
    _C.so, and the first formatted error message would crash; CI8_CXX overrides the choice."""
    override = os.environ.get("CI8_CXX")
    if override:
        return override
    return "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    stamp = target.stat().st_mtime
    return all(src.stat().st_mtime <= stamp for src in sources)


def _run(cmd: list[str]) -> None:
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def build_kernels(force: bool = False, verbose_ptxas: bool = False) -> Path:
    target = PKG / "libci8.so"
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "ci8.h"]
    if not force and _newer(target, sources):
        return target
    nvcc = shutil.which("nvcc") or str(CUDA_HOME / "bin" / "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", target, CSRC / "c_api.cu"]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    _run(cmd)
    return target


def build_bindings(force: bool = False) -> Path:
    import torch  # only for the header and library locations

    target = PKG / "_C.so"
    sources = [CSRC / "bindings.cpp", HERE.parent / "include" / "ci8.h"]
    if not force and _newer(target, sources):
        return target
    torch_root = Path(torch.__file__).resolve().parent
    includes = [
        torch_root / "include",
        torch_root / "include" / "torch" / "csrc" / "api" / "include",
        CUDA_HOME / "include",
        Path(sysconfig.get_paths()["include"]),
    ]
    cmd = [
        _host_cxx(), "-O3", "-std=c++17", "-fPIC", "-shared", *STABLE_DEFINES,
        *[f"-I{p}" for p in includes],
        "-o", target, CSRC / "bindings.cpp",
        f"-L{PKG}", "-lci8", "-Wl,-rpath,$ORIGIN",
        f"-L{torch_root / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10",
        f"-Wl,-rpath,{torch_root / 'lib'}",
    ]
    _run(cmd)
    return target


def build(force: bool = False) -> None:
    build_kernels(force)
    build_bindings(force)


if __name__ == "__main__":
    build(force="--force" in sys.argv)
