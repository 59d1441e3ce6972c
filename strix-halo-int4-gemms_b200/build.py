"""In-tree build of the CUDA library (libb200_int4_gemms.so) for sm_100a.

Stands where the reference's ``native/CMakeLists.txt`` (assemble every AMDGCN ``.s`` into a
code object, then build the dispatcher) stood: here the kernels are CUDA sources compiled
straight into the one shared library that exports the C ABI of ``include/b200_int4_gemms.h``.

The tensor-core kernel instantiations are spread over ``TC_PARTS`` translation units
(``tc_kernels.cu`` compiled once per part) which, with the host code, are compiled in parallel
and linked into one library.

Usage: ``python build.py [--force] [--verbose]`` from this directory, or
``build_native()`` from Python.  nvcc cross-compiles; no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "lib"
LIB_NAME = "libb200_int4_gemms.so"
HOST_SOURCE = "b200_int4_gemms.cu"
KERNEL_SOURCE = "tc_kernels.cu"
TC_PARTS = 8  # kTcParts of csrc/tc_table.h
SOURCES = (HOST_SOURCE, KERNEL_SOURCE)
HEADERS = ("ptx.cuh", "gemm_kernel.cuh", "simt_kernel.cuh", "prep_kernels.cuh", "tc_table.h")
GENCODE = "arch=compute_100a,code=sm_100a"
# the build of the bounded-wait test: a short wait limit and an MMA warp that never signals "accumulator full"
# (see csrc/ptx.cuh); tests/test_gpu_wait_timeout.py loads it from TEST_LIB_NAME, nothing else does
TEST_LIB_NAME = "libb200_int4_gemms_wait_test.so"
TEST_DEFINES = ("B200_TEST_WAIT_LIMIT_NS=5000000ull", "B200_TEST_DROP_ACC_FULL_SIGNAL=1")


def library_path() -> Path:
    return LIB_DIR / LIB_NAME


def test_library_path() -> Path:
    return LIB_DIR / TEST_LIB_NAME


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
    deps.append(Path(__file__).resolve())
    return any(dep.stat().st_mtime > built for dep in deps if dep.exists())


def _run(cmd: list[str], verbose: bool) -> str:
    result = subprocess.run(cmd, cwd=str(CSRC_DIR), capture_output=True, text=True)
    if result.returncode != 0:
        sys.stderr.write(result.stdout)
        sys.stderr.write(result.stderr)
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}: {' '.join(cmd)}")
    return result.stdout + result.stderr


def build_native(*, force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (),
                 output: Path | None = None, jobs: int | None = None) -> Path:
    """Compile the library if it is missing or older than its sources; return its path.

    ``defines`` and ``output`` build a variant beside the default library (the bounded-wait test build
    uses them, see ``build_wait_test_library``).
    """
    target = Path(output) if output is not None else library_path()
    if not force and not _is_stale(target):
        return target
    target.parent.mkdir(parents=True, exist_ok=True)
    common = [_nvcc(), "-gencode", GENCODE, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-diag-suppress", "128"]
    common += [f"-D{item}" for item in defines]
    if verbose:
        common += ["-Xptxas", "-v"]
    with tempfile.TemporaryDirectory(prefix="b200_build_") as tmp:
        units = [(HOST_SOURCE, [], Path(tmp) / "host.o")]
        units += [(KERNEL_SOURCE, [f"-DB200_TC_PART={part}"], Path(tmp) / f"tc_part_{part}.o") for part in range(TC_PARTS)]

        def compile_unit(unit):
            source, extra, obj = unit
            return _run(common + extra + ["-c", str(CSRC_DIR / source), "-o", str(obj)], verbose)

        workers = jobs or min(len(units), os.cpu_count() or 1)
        with ThreadPoolExecutor(max_workers=workers) as pool:
            logs = list(pool.map(compile_unit, units))
        if verbose:
            sys.stderr.write("".join(logs))
        _run([_nvcc(), "-gencode", GENCODE, "-shared", "-o", str(target)] + [str(obj) for _, _, obj in units], verbose)
    return target


def build_wait_test_library(*, force: bool = False) -> Path:
    """The test-only build whose per-channel kernels give up on a wait after 5 ms (see TEST_DEFINES)."""
    return build_native(force=force, defines=TEST_DEFINES, output=test_library_path())


if __name__ == "__main__":
    path = build_native(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
