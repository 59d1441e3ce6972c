"""In-tree build of the CUDA library (libb200_int4_gemms.so) for sm_100a.

Stands where the reference's ``native/CMakeLists.txt`` (assemble every AMDGCN ``.s`` into a
code object, then build the dispatcher) stood: here the kernels are CUDA sources compiled
straight into the one shared library that exports the C ABI of ``include/b200_int4_gemms.h``.

Usage: ``python build.py [--force] [--verbose]`` from this directory, or
``build_native()`` from Python.  nvcc cross-compiles; no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "lib"
LIB_NAME = "libb200_int4_gemms.so"
SOURCES = ("b200_int4_gemms.cu",)
HEADERS = ("ptx.cuh", "gemm_kernel.cuh", "simt_kernel.cuh")
GENCODE = "arch=compute_100a,code=sm_100a"


def library_path() -> Path:
    return LIB_DIR / LIB_NAME


def _nvcc() -> str:
    found = shutil.which("nvcc")
    if found:
        return found
    candidate = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    raise RuntimeError("nvcc was not found; set CUDA_HOME or put nvcc on PATH")


def _is_stale(target: Path) -> bool:
    if not target.exists():
        return True
    built = target.stat().st_mtime
    deps = [CSRC_DIR / name for name in (*SOURCES, *HEADERS)]
    deps.append(PACKAGE_DIR.parent / "include" / "b200_int4_gemms.h")
    return any(dep.stat().st_mtime > built for dep in deps if dep.exists())


def build_native(*, force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (), output: Path | None = None) -> Path:
    """Compile the library if it is missing or older than its sources; return its path.

    ``defines`` (e.g. ``("B200_UNPACK_WARPS=4",)``) and ``output`` build a tuning variant beside
    the default library; the B200_NVCC_DEFINES environment variable (comma separated) adds more.
    """
    target = Path(output) if output is not None else library_path()
    env_defines = tuple(d for d in os.environ.get("B200_NVCC_DEFINES", "").split(",") if d)
    defines = tuple(defines) + env_defines
    if not force and not _is_stale(target):
        return target
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cmd = [
        _nvcc(),
        "-gencode",
        GENCODE,
        "-lineinfo",
        "-O3",
        "-std=c++17",
        "-shared",
        "-Xcompiler",
        "-fPIC",
        "-diag-suppress",
        "128",
    ]
    cmd += [f"-D{item}" for item in defines]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(target)]
    cmd += [str(CSRC_DIR / name) for name in SOURCES]
    result = subprocess.run(cmd, cwd=str(CSRC_DIR), capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout)
        sys.stderr.write(result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}: {' '.join(cmd)}")
    return target


if __name__ == "__main__":
    path = build_native(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
