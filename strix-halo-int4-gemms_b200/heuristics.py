"""Choosing a launch form without running anything.

The reference ranks pre-generated code objects by a benchmark database and a tile-area prior
(heuristics.py:9-62).  What this library can choose between is different: one CTA or a CTA pair
per output tile, how many K slices, and how wide the raster is.  Of these the first two decide
almost everything, and both follow from counting: how many waves of tiles the SMs (or SM pairs)
need, and how long a tile's K loop is.  ``choose_kernel`` keeps the reference's name and
arguments; measured records still win over the model when the database has them.
"""
from __future__ import annotations

import math

from .benchmarking import BenchmarkDatabase, BenchmarkShape
from .metadata import Epilogue, GemmLayout, KernelMetadata, KernelSchedule, OperandDType, ScaleSpec
from .registry import KernelRegistry, default_registry
from .template_config import LaunchShape, is_tile_multiple_shape

NUM_SMS = 148                 # B200
PAIR_TILE_TIME = 0.87         # a pair's 256 x 256 K block in units of a single CTA's 128 x 256 one
TILE_OVERHEAD_K = 512.0       # prologue + epilogue of a tile, expressed in K values of mainloop time
REDUCE_COST_PER_SLICE = 0.15  # second pass of a split: extra time per slice, relative to one tile's overhead


def kernel_supports_shape(kernel: KernelMetadata, *, m: int, n: int, k: int) -> bool:
    """Even-K entry whose multiples divide the shape; activations only without split-K."""
    if kernel.epilogue is not Epilogue.NONE and kernel.tile.split_k != 1:
        return False
    return kernel.tile.even_k and is_tile_multiple_shape(kernel, LaunchShape(m, n, k))


def _tiles(m: int, n: int, rows: int, cols: int) -> int:
    return math.ceil(m / rows) * math.ceil(n / cols)


def modelled_time(kernel: KernelMetadata, *, m: int, n: int, k: int, num_sms: int = NUM_SMS) -> float:
    """Relative run time of an entry's launch on a shape: waves x (K loop + per-tile overhead) per wave, in
    units of one K value of a single-CTA tile.  Not a prediction of microseconds; only the order matters."""
    cols = 128 if kernel.epilogue is Epilogue.SWIGLU else 256
    split = kernel.tile.split_k
    k_slice = math.ceil(k / split)
    single = math.ceil(_tiles(m, n, 128, cols) * split / num_sms) * (k_slice + TILE_OVERHEAD_K)
    pairs = math.ceil(_tiles(m, n, 256, cols) * split / (num_sms // 2)) * (PAIR_TILE_TIME * k_slice + TILE_OVERHEAD_K)
    if kernel.schedule is KernelSchedule.PERSISTENT_2CTA:
        cost = pairs
    elif kernel.schedule is KernelSchedule.STANDARD:
        cost = min(single, pairs) if m > 128 else single  # the library's own rule picks the cheaper form
    elif kernel.schedule is KernelSchedule.TILE_PER_CTA:
        cost = single * 1.15  # no overlap of one tile's epilogue with the next tile's mainloop
    else:
        cost = single
    if split > 1:
        cost += split * REDUCE_COST_PER_SLICE * TILE_OVERHEAD_K
    return cost


def estimate_kernel_score(
    kernel: KernelMetadata, *, m: int, n: int, k: int, benchmark_db: BenchmarkDatabase | None = None
) -> float:
    """Higher is better: measured TOPS for this exact shape when the database has them, else the inverse of
    the modelled time scaled below any measured figure (so that one measured entry outranks every modelled one
    only when it was really measured on this shape)."""
    if not kernel_supports_shape(kernel, m=m, n=n, k=k):
        return float("-inf")
    if benchmark_db is not None:
        best = benchmark_db.best_record(kernel, BenchmarkShape(m, n, k))
        if best is not None:
            return best.tops
    if kernel.measured_tops:
        return float(kernel.measured_tops)
    return 1.0e-3 * (k / modelled_time(kernel, m=m, n=n, k=k))


def choose_kernel(
    *,
    m: int,
    n: int,
    k: int,
    dtype: OperandDType,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec,
    epilogue: Epilogue,
    schedule: KernelSchedule | None = KernelSchedule.STANDARD,
    registry: KernelRegistry = default_registry,
    benchmark_db: BenchmarkDatabase | None = None,
) -> KernelMetadata:
    """Best entry of the cell for the shape; ``schedule=None`` compares every launch form, split-K included
    (split entries return float32, so callers that need bf16 keep the default)."""
    pool = [
        kernel
        for kernel in registry.all()
        if kernel.a_dtype is dtype
        and kernel.b_dtype is dtype
        and kernel.layout is layout
        and kernel.scale == scale
        and kernel.epilogue is epilogue
        and (schedule is None or kernel.schedule is schedule)
        and kernel_supports_shape(kernel, m=m, n=n, k=k)
    ]
    if not pool:
        raise LookupError("no kernels match logical dtype/layout/scale/epilogue request and shape")
    return max(pool, key=lambda kernel: (estimate_kernel_score(kernel, m=m, n=n, k=k, benchmark_db=benchmark_db),
                                         kernel.tile.block_m * kernel.tile.block_n))
