"""Kernel choice from measured records (reference: heuristics.py:9-62)."""
from __future__ import annotations

from .benchmarking import BenchmarkDatabase, BenchmarkShape
from .metadata import Epilogue, GemmLayout, KernelMetadata, KernelSchedule, OperandDType, ScaleSpec
from .registry import KernelRegistry, default_registry
from .template_config import LaunchShape, is_tile_multiple_shape


def kernel_supports_shape(kernel: KernelMetadata, *, m: int, n: int, k: int) -> bool:
    """Even-K entry whose multiples divide the shape; activations only without split-K."""
    if kernel.epilogue is not Epilogue.NONE and kernel.tile.split_k != 1:
        return False
    return kernel.tile.even_k and is_tile_multiple_shape(kernel, LaunchShape(m, n, k))


def estimate_kernel_score(
    kernel: KernelMetadata, *, m: int, n: int, k: int, benchmark_db: BenchmarkDatabase | None = None
) -> float:
    """Measured TOPS for this exact shape when the database has it, else a prior.

    The prior favours large registered multiples (fewer masked rows and columns) and charges
    split-K variants for their float32 output.
    """
    if not kernel_supports_shape(kernel, m=m, n=n, k=k):
        return float("-inf")
    if benchmark_db is not None:
        best = benchmark_db.best_record(kernel, BenchmarkShape(m, n, k))
        if best is not None:
            return best.tops
    prior = kernel.measured_tops or 1.0
    prior /= kernel.tile.split_k
    prior *= 1.0 + (kernel.tile.block_m * kernel.tile.block_n) / (128.0 * 256.0)
    return prior


def choose_kernel(
    *,
    m: int,
    n: int,
    k: int,
    dtype: OperandDType,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec,
    epilogue: Epilogue,
    schedule: KernelSchedule = KernelSchedule.STANDARD,
    registry: KernelRegistry = default_registry,
    benchmark_db: BenchmarkDatabase | None = None,
) -> KernelMetadata:
    pool = [
        kernel
        for kernel in registry.all()
        if kernel.a_dtype is dtype
        and kernel.b_dtype is dtype
        and kernel.layout is layout
        and kernel.scale == scale
        and kernel.epilogue is epilogue
        and kernel.schedule is schedule
        and kernel_supports_shape(kernel, m=m, n=n, k=k)
    ]
    if not pool:
        raise LookupError("no kernels match logical dtype/layout/scale/epilogue request and shape")
    return max(pool, key=lambda kernel: estimate_kernel_score(kernel, m=m, n=n, k=k, benchmark_db=benchmark_db))
