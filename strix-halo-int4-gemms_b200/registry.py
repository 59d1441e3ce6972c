"""Registry of sm_100a GEMM variants and the selection rule of the dense API.

Same surface as the reference's ``registry.py`` (``KernelRegistry.register/get/all/select/
select_reference/with_status`` :254-349, ``default_registry`` :352, ``seed_tile_configs`` :112,
``iter_supported_kernel_metadata`` :202) with the variant matrix re-keyed to what this library can
launch differently.  An entry names, besides its cell (operand type, scale spec, epilogue, layout):

* the launch form (``KernelSchedule``): ``STANDARD`` = the library's own choice for the shape,
  ``PERSISTENT`` = one CTA per 128-row tile, ``PERSISTENT_2CTA`` = a CTA pair per 256-row tile
  (only for the cells that have a paired kernel), ``TILE_PER_CTA`` = one CTA per tile without the
  persistent grid;
* the raster width ``group_size_m`` handed to the launch (0 = the library's default for the form);
* the split-K factor (plain epilogue only, and only where the library has the partial-sum kernel);
* the shape multiples it accepts (``block_m``, ``block_n``, ``block_k``).

``STANDARD`` entries also come with smaller row multiples (64 / 32 / 16 rows, 128 columns): the same
launch, accepted for shapes that leave the last tile partly empty.  Selection keeps the reference's
rule: among even-K entries of the requested schedule whose multiples divide the shape, take the one
with the best measured TOPS, ties broken by the largest ``block_m * block_n``.  Masked-K entries
(``even_k=False``: any K) are listed for ``explicit_mm`` as in the reference.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Iterable, Iterator

from .metadata import (
    ACC_DTYPE,
    ARCH,
    SCALE_DTYPE_BF16,
    SUPPORTED_GEMM_LAYOUTS,
    SUPPORTED_SPLIT_K,
    Epilogue,
    GemmLayout,
    KernelMetadata,
    KernelSchedule,
    KernelStatus,
    OperandDType,
    ScaleMode,
    ScaleSpec,
    TileConfig,
    make_kernel_id,
    output_dtype_for_split_k,
    supported_scale_specs,
)
from .template_config import LaunchShape, is_tile_multiple_shape

ROW_MULTIPLES = (128, 64, 32, 16)   # STANDARD entries: the 128-row tile and the row multiples it masks down to
COLUMN_MULTIPLES = (256, 128)
SWIGLU_COLUMN_MULTIPLES = (128,)    # one tile = 128 up columns + the matching 128 gate columns
K_STEP = 32                         # one tcgen05.mma kind::i8 instruction reduces 32 K values
PAIR_ROWS = 256                     # output rows of a CTA pair's tile
# raster widths (row tiles walked before the next column tile) registered per forced form; the first one is
# what the library itself uses for the form
RASTER_WIDTHS = {KernelSchedule.PERSISTENT: (8, 32), KernelSchedule.PERSISTENT_2CTA: (16, 8), KernelSchedule.TILE_PER_CTA: (8,)}
DEVICE_KERNEL = "b200::gemm_i8_tcgen05_kernel"
SCHEDULES = (KernelSchedule.STANDARD, KernelSchedule.PERSISTENT, KernelSchedule.PERSISTENT_2CTA, KernelSchedule.TILE_PER_CTA)


def has_pair_kernel(dtype: OperandDType, scale: ScaleSpec, epilogue: Epilogue, layout: GemmLayout) -> bool:
    """Whether the library holds a CTA-pair instantiation for the cell (bf16 output; csrc/tc_table.h)."""
    sub = scale.mode is ScaleMode.SUBCHANNEL
    if sub and (scale.subchannel_size or 0) < 128:
        return False  # paired kernels hand the accumulator over per 128-deep K block
    if layout is GemmLayout.NN:
        return True
    if sub or epilogue is Epilogue.SWIGLU:
        return False
    if layout is GemmLayout.NT:
        return epilogue is Epilogue.NONE or dtype is OperandDType.INT8
    if layout is GemmLayout.TN:
        return dtype is OperandDType.INT4 and epilogue is Epilogue.NONE
    return False


def has_split_k_kernel(dtype: OperandDType, scale: ScaleSpec, layout: GemmLayout, *, pair: bool = False) -> bool:
    """Whether the library holds the partial-sum kernel a split-K launch of the cell needs: raw s32
    accumulators for per-channel scales (layouts NN and NT), fp32 partial sums for int4 subchannel scales."""
    if scale.mode is ScaleMode.PER_CHANNEL:
        return layout is GemmLayout.NN or (layout is GemmLayout.NT and not pair)
    if dtype is not OperandDType.INT4:
        return False
    if pair:
        return layout is GemmLayout.NN and (scale.subchannel_size or 0) >= 128
    return layout in (GemmLayout.NN, GemmLayout.NT)


def cta_warps(dtype: OperandDType, scale: ScaleSpec) -> int:
    """Warps of the kernel's CTA.  Per-channel: TMA + MMA warps, 4 epilogue warps, 8 unpack warps for int4.
    Subchannel: a warpgroup of 4 for TMA / MMA (two of them idle), 8 epilogue warps, 4 unpack warps for int4."""
    if scale.mode is ScaleMode.SUBCHANNEL:
        return 4 + 8 + (4 if dtype is OperandDType.INT4 else 0)
    return 2 + 4 + (8 if dtype is OperandDType.INT4 else 0)


def pipeline_stages(dtype: OperandDType, schedule: KernelSchedule = KernelSchedule.STANDARD) -> int:
    """Depth of the int8 operand pipeline in shared memory: a CTA of a pair holds one block of B, so more fit."""
    if schedule is KernelSchedule.PERSISTENT_2CTA:
        return 4 if dtype is OperandDType.INT4 else 6
    return 3 if dtype is OperandDType.INT4 else 4


def seed_tile_configs(
    dtype: OperandDType = OperandDType.INT4,
    *,
    epilogue: Epilogue | None = None,
    scale: ScaleSpec | None = None,
    schedule: KernelSchedule = KernelSchedule.STANDARD,
    layout: GemmLayout = GemmLayout.NN,
) -> tuple[TileConfig, ...]:
    """Tile records registered for one (dtype, scale, epilogue, layout) cell and launch form."""
    if dtype not in (OperandDType.INT4, OperandDType.INT8):
        raise ValueError(f"unsupported dtype: {dtype}")
    scale = scale if scale is not None else ScaleSpec(ScaleMode.PER_CHANNEL)
    epilogue = epilogue if epilogue is not None else Epilogue.NONE
    pair = schedule is KernelSchedule.PERSISTENT_2CTA
    if pair and not has_pair_kernel(dtype, scale, epilogue, layout):
        return ()
    swiglu = epilogue is Epilogue.SWIGLU
    splits = tuple(
        split for split in (SUPPORTED_SPLIT_K if epilogue is Epilogue.NONE else (1,))
        if split == 1 or (schedule is not KernelSchedule.TILE_PER_CTA and has_split_k_kernel(dtype, scale, layout, pair=pair))
    )
    if schedule is KernelSchedule.STANDARD:
        shapes = [(rows, cols, 0) for cols in (SWIGLU_COLUMN_MULTIPLES if swiglu else COLUMN_MULTIPLES) for rows in ROW_MULTIPLES]
    else:
        rows = PAIR_ROWS if pair else 128
        shapes = [(rows, 128 if swiglu else 256, width) for width in RASTER_WIDTHS[schedule]]
    warps = cta_warps(dtype, scale)
    stages = pipeline_stages(dtype, schedule)
    return tuple(
        TileConfig(
            block_m=rows,
            block_n=cols,
            block_k=K_STEP,
            group_size_m=width,
            num_warps=warps,
            num_stages=stages,
            waves_per_eu=0,
            even_k=even_k,
            split_k=split_k,
        )
        for split_k in splits
        for even_k in (True, False)
        for rows, cols, width in shapes
    )


def _describe(
    dtype: OperandDType,
    scale: ScaleSpec,
    epilogue: Epilogue,
    tile: TileConfig,
    layout: GemmLayout,
    schedule: KernelSchedule,
) -> KernelMetadata:
    return KernelMetadata(
        kernel_id=make_kernel_id(dtype, scale, epilogue, tile, layout=layout, schedule=schedule),
        arch=ARCH,
        a_dtype=dtype,
        b_dtype=dtype,
        acc_dtype=ACC_DTYPE,
        output_dtype=output_dtype_for_split_k(tile.split_k),
        scale_dtype=SCALE_DTYPE_BF16,
        scale=scale,
        epilogue=epilogue,
        tile=tile,
        device_kernel=DEVICE_KERNEL,
        layout=layout,
        schedule=schedule,
        status=KernelStatus.COMPILED,
    )


def iter_supported_kernel_metadata(
    *, tiles: Iterable[TileConfig] | None = None
) -> Iterator[KernelMetadata]:
    """Every registered variant; ``tiles`` replaces the seed tile list of every cell."""
    forced = None if tiles is None else tuple(tiles)
    for schedule in SCHEDULES:
        for dtype in (OperandDType.INT4, OperandDType.INT8):
            for scale in supported_scale_specs():
                for epilogue in (Epilogue.NONE, Epilogue.RELU2, Epilogue.SWIGLU):
                    for layout in SUPPORTED_GEMM_LAYOUTS:
                        cell = forced if forced is not None else seed_tile_configs(
                            dtype, epilogue=epilogue, scale=scale, schedule=schedule, layout=layout)
                        for tile in cell:
                            yield _describe(dtype, scale, epilogue, tile, layout, schedule)


def launch_signature(kernel: KernelMetadata) -> tuple:
    """What distinguishes one entry's launch from another's within a cell: entries with equal signatures run
    the same kernel with the same parameters (they differ only in the shapes they accept)."""
    return (kernel.schedule, kernel.tile.group_size_m, kernel.tile.split_k)


_CellKey = tuple[OperandDType, ScaleSpec, Epilogue, GemmLayout, KernelSchedule]


def _cell_of(kernel: KernelMetadata) -> _CellKey:
    return (kernel.a_dtype, kernel.scale, kernel.epilogue, kernel.layout, kernel.schedule)


def _preference(kernel: KernelMetadata) -> tuple[float, int]:
    return (kernel.measured_tops or 0.0, kernel.tile.block_m * kernel.tile.block_n)


class KernelRegistry:
    """Kernel metadata by id, with an index per (dtype, scale, epilogue, layout, schedule) cell."""

    def __init__(self, kernels: Iterable[KernelMetadata] = ()) -> None:
        self._kernels: dict[str, KernelMetadata] = {}
        self._cells: dict[_CellKey, list[str]] = {}
        for kernel in kernels:
            self.register(kernel)

    def register(self, kernel: KernelMetadata) -> None:
        if kernel.kernel_id in self._kernels:
            raise ValueError(f"duplicate kernel id: {kernel.kernel_id}")
        if kernel.a_dtype is not kernel.b_dtype:
            raise ValueError("mixed operand types are not supported")
        self._kernels[kernel.kernel_id] = kernel
        self._cells.setdefault(_cell_of(kernel), []).append(kernel.kernel_id)

    def get(self, kernel_id: str) -> KernelMetadata:
        return self._kernels[kernel_id]

    def all(self) -> tuple[KernelMetadata, ...]:
        return tuple(self._kernels.values())

    def __len__(self) -> int:
        return len(self._kernels)

    def _eligible(
        self,
        dtype: OperandDType,
        scale: ScaleSpec,
        epilogue: Epilogue,
        layout: GemmLayout,
        schedule: KernelSchedule,
        split_k: int | None,
    ) -> list[KernelMetadata]:
        found = []
        for kernel_id in self._cells.get((dtype, scale, epilogue, layout, schedule), ()):
            kernel = self._kernels[kernel_id]
            if not kernel.tile.even_k:
                continue
            if epilogue is not Epilogue.NONE and kernel.tile.split_k != 1:
                continue
            if split_k is not None and kernel.tile.split_k != split_k:
                continue
            found.append(kernel)
        return found

    def select(
        self,
        *,
        dtype: OperandDType,
        scale: ScaleSpec,
        epilogue: Epilogue,
        m: int,
        n: int,
        k: int,
        layout: GemmLayout = GemmLayout.NN,
        split_k: int | None = None,
        schedule: KernelSchedule = KernelSchedule.STANDARD,
        require_compiled: bool = False,
    ) -> KernelMetadata:
        shape = LaunchShape(m, n, k)
        fits = [
            kernel
            for kernel in self._eligible(dtype, scale, epilogue, layout, schedule, split_k)
            if is_tile_multiple_shape(kernel, shape)
        ]
        if require_compiled:
            ready = (KernelStatus.COMPILED, KernelStatus.BENCHMARKED)
            fits = [kernel for kernel in fits if kernel.status in ready]
        if not fits:
            raise LookupError(
                f"no kernel for dtype={dtype.value}, scale={scale.label}, epilogue={epilogue.value}, "
                f"layout={layout.value}, schedule={schedule.value}, "
                f"shape=({m}, {n}, {k})"
            )
        return max(fits, key=_preference)

    def select_reference(
        self,
        *,
        dtype: OperandDType,
        scale: ScaleSpec,
        epilogue: Epilogue,
        layout: GemmLayout = GemmLayout.NN,
        split_k: int | None = 1,
        schedule: KernelSchedule = KernelSchedule.STANDARD,
    ) -> KernelMetadata:
        """Metadata for the CPU reference math: any shape, so no tile-multiple filter."""
        fits = self._eligible(dtype, scale, epilogue, layout, schedule, split_k)
        if not fits:
            raise LookupError(
                f"no reference kernel metadata for dtype={dtype.value}, scale={scale.label}, "
                f"epilogue={epilogue.value}, layout={layout.value}, schedule={schedule.value}"
            )
        return max(fits, key=_preference)

    def with_status(self, kernel_id: str, status: KernelStatus, **updates: object) -> "KernelRegistry":
        """A copy of the registry in which one entry has a new status (and other fields)."""
        changed = replace(self._kernels[kernel_id], status=status, **updates)
        return KernelRegistry(changed if k.kernel_id == kernel_id else k for k in self._kernels.values())


default_registry = KernelRegistry(iter_supported_kernel_metadata())
