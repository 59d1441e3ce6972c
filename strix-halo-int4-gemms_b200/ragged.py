"""Grouped ("ragged") int4 GEMMs: the forward M-ragged dot and the backward K-ragged dot.

Surface of the reference's ``ragged.py``: ``RaggedDotConfig`` (:11-36), ``RaggedBwdDotConfig``
(:39-59), ``RaggedGroupInfo`` (:62-72), ``calculate_group_info`` (:201-323),
``ragged_dot_int4`` (:1008-1229), ``ragged_dot_int4_bwd`` (:1232-1402), the even-K predicates
(:326-366) and the shape / scale validators (:834-1005).

What is different underneath: the reference had three Triton kernels (JIT or pre-compiled) and
a Triton task builder; here both operations run on the persistent tcgen05 kernel of the CUDA
library, whose scheduler walks (row-block task x column tile) pairs for the forward pass and
(group x row tile x column tile) triples for the backward pass.  There is no JIT path:
``use_native=False`` raises, and ``allow_triton`` is accepted and ignored.

Tile defaults are the kernel's real ones (128-row tasks, 256 columns, 128-deep K stages).  The
kernel masks rows outside ``[actual_start, actual_end)`` of a task itself, so any task height
up to 256 that is a multiple of ``align_tile`` works.  Tasks of more than 128 rows run on pairs
of SMs (one 256 x 256 tile per pair); ``RaggedDotConfig.pair_tasks`` says when the default
128-row tasks are widened to 256 rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any

from .metadata import GemmLayout, ScaleMode, ScaleSpec

MAX_TASK_ROWS = 256
PAIR_TASK_ROWS = 256          # task height of the CTA-pair kernel
PAIR_MIN_MEAN_GROUP_ROWS = 256  # widen tasks automatically when groups average at least this many rows

RAGGED_FAMILY = "ragged_dot_int4"
RAGGED_FWD = "fwd"
RAGGED_BWD = "bwd"
RAGGED_EVEN_K = "evenk"
RAGGED_MASK_K = "maskk"


@dataclass(frozen=True, slots=True)
class RaggedDotConfig:
    """Launch configuration of the forward grouped dot."""

    block_m: int = 128
    block_n: int = 256
    block_k: int = 128
    align_tile: int = 8
    group_size_tasks: int = 1
    enable_even_k_fast_path: bool = True
    num_warps: int = 14   # TMA + MMA + 4 epilogue + 8 unpack warps of the per-channel kernel
    num_stages: int = 3
    # None: 128-row tasks are widened to 256 rows (CTA pairs) when the groups are large enough and
    # the kernel supports it for the call; False: never; True: whenever the kernel supports it.
    # Only looked at when ``block_m`` is 128 and no prebuilt ``group_info`` is passed.
    pair_tasks: bool | None = None

    def __post_init__(self) -> None:
        if min(self.block_m, self.block_n, self.block_k) <= 0:
            raise ValueError("block_m, block_n, and block_k must be positive")
        if self.block_k % 2:
            raise ValueError("block_k must be even for packed int4 operands")
        if self.align_tile <= 0:
            raise ValueError("align_tile must be positive")
        if self.block_m % self.align_tile:
            raise ValueError("block_m must be a multiple of align_tile")
        if self.group_size_tasks <= 0:
            raise ValueError("group_size_tasks must be positive")
        if self.num_warps <= 0 or self.num_stages <= 0:
            raise ValueError("num_warps and num_stages must be positive")


@dataclass(frozen=True, slots=True)
class RaggedBwdDotConfig:
    """Launch configuration of the backward (K-ragged) grouped dot.

    ``split_k`` is accepted for compatibility.  Every output tile is reduced by a single CTA
    in a fixed order, so results are deterministic and identical for every ``split_k``.
    ``pair_tiles``: None lets the library run 256-row tiles on CTA pairs when M is a multiple of 256
    and a paired kernel exists, False keeps one CTA per 128-row tile, True asks for pairs (one CTA
    per tile where no paired kernel applies).  Results are bit-identical either way.
    """

    block_m: int = 128
    block_n: int = 256
    block_k: int = 128
    split_k: int = 1
    num_warps: int = 20   # TMA / MMA warpgroup + 8 epilogue + 8 unpack warps of the K-masked kernel
    num_stages: int = 2
    enable_even_k_fast_path: bool = True
    pair_tiles: bool | None = None

    def __post_init__(self) -> None:
        if min(self.block_m, self.block_n, self.block_k) <= 0:
            raise ValueError("block_m, block_n, and block_k must be positive")
        if self.block_k % 2:
            raise ValueError("block_k must be even for packed int4 operands")
        if self.split_k <= 0:
            raise ValueError("split_k must be positive")
        if self.num_warps <= 0 or self.num_stages <= 0:
            raise ValueError("num_warps and num_stages must be positive")


@dataclass(frozen=True, slots=True)
class RaggedGroupInfo:
    """Row-block tasks of a grouped forward dot, one entry per task (int64 tensors)."""

    group_id: Any
    block_start: Any
    actual_start: Any
    actual_end: Any
    start_within_block: Any
    actual_size: Any
    num_tasks: int
    # set by calculate_group_info_on_device: the task count as a one-element int32 device tensor
    # (``num_tasks`` is then the capacity of the arrays) and a flag that is 1 when the capacity was too small
    device_num_tasks: Any | None = None
    device_overflow: Any | None = None
    # the block height and alignment the tasks were cut with (None for records built by older callers);
    # ragged_dot_int4 launches prebuilt tasks with this height, whatever its config says
    tile: int | None = None
    align_tile: int | None = None


def _torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError("torch is required for ragged_dot_int4") from exc
    return torch


def _cdiv(x: int, y: int) -> int:
    return -(-x // y)


def _is_integer_dtype(torch: Any, dtype: Any) -> bool:
    return dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


def _check_layout(layout: GemmLayout) -> GemmLayout:
    if type(layout) is not GemmLayout:
        raise TypeError(f"layout must be a GemmLayout, got {type(layout).__name__}")
    return layout


def ragged_config_label(config: Any) -> str:
    head = f"BM{config.block_m}_BN{config.block_n}_BK{config.block_k}"
    if hasattr(config, "group_size_tasks"):
        return f"{head}_GST{config.group_size_tasks}_W{config.num_warps}_S{config.num_stages}"
    return f"{head}_W{config.num_warps}_S{config.num_stages}_SK{config.split_k}"


def ragged_kernel_id(
    *,
    mode: str,
    layout: GemmLayout,
    scale: ScaleSpec,
    config: Any,
    variant: str,
    output_dtype: str | None = None,
    arch: str = "sm_100a",
) -> str:
    """Name of a grouped-dot variant, same grammar as the reference's ragged_artifacts.py:25-47."""
    if mode not in (RAGGED_FWD, RAGGED_BWD):
        raise ValueError(f"ragged mode must be one of {(RAGGED_FWD, RAGGED_BWD)}; got {mode!r}")
    if variant not in (RAGGED_EVEN_K, RAGGED_MASK_K):
        raise ValueError(f"ragged variant must be one of {(RAGGED_EVEN_K, RAGGED_MASK_K)}; got {variant!r}")
    stored = output_dtype or ("bfloat16" if mode == RAGGED_FWD else "float32")
    return (
        f"{arch}_ragged_int4_{mode}_{layout.value}_{scale.label.lower()}_"
        f"{variant}_{stored}_{ragged_config_label(config).lower()}"
    )


def calculate_group_info(
    group_sizes: Any,
    tile: int,
    *,
    tid_size: int | None = None,
    align_tile: int = 8,
    allow_triton: bool = True,
) -> RaggedGroupInfo:
    """Cut each group's contiguous row range into blocks of ``tile`` rows.

    Group ``g`` owns rows ``[start_g, end_g)`` with ``start_g = sum(group_sizes[:g])``.  Its
    blocks begin at ``floor(start_g / align_tile) * align_tile`` and step by ``tile``; a block
    may therefore begin before ``start_g`` and end after ``end_g``, and the consumer masks
    rows outside ``[actual_start, actual_end)``.  Empty groups produce no task.  Tasks are
    numbered group by group.  With ``tid_size`` the arrays have that length and the unused
    tail is zero (``actual_size == 0``).

    ``allow_triton`` is ignored (there is no Triton builder); results are the reference's.
    """
    del allow_triton
    torch = _torch()
    if not torch.is_tensor(group_sizes):
        raise TypeError("group_sizes must be a torch.Tensor")
    if group_sizes.ndim != 1:
        raise ValueError(f"group_sizes must be 1D; got shape {tuple(group_sizes.shape)}")
    if not _is_integer_dtype(torch, group_sizes.dtype):
        raise ValueError(f"group_sizes must have integer dtype; got {group_sizes.dtype}")
    if tile <= 0:
        raise ValueError("tile must be positive")
    if align_tile <= 0:
        raise ValueError("align_tile must be positive")
    if tile % align_tile:
        raise ValueError("tile must be a multiple of align_tile")
    if tid_size is not None and tid_size < 0:
        raise ValueError("tid_size must be non-negative")

    device = group_sizes.device
    i64 = dict(device=device, dtype=torch.int64)
    sizes = group_sizes.to(torch.int64).clamp_min(0)
    groups = int(sizes.numel())

    def blank(length: int, num_tasks: int, *, zero: bool) -> RaggedGroupInfo:
        make = torch.zeros if zero else torch.empty
        fields = [make((length,), **i64) for _ in range(6)]
        return RaggedGroupInfo(*fields, num_tasks=num_tasks, tile=int(tile), align_tile=int(align_tile))

    if groups == 0:
        return blank(tid_size or 0, 0, zero=True)

    ends = torch.cumsum(sizes, dim=0)
    starts = ends - sizes
    first_block = torch.div(starts, align_tile, rounding_mode="floor") * align_tile
    blocks = torch.div(ends - first_block + (tile - 1), tile, rounding_mode="floor")
    blocks = torch.where(sizes == 0, torch.zeros_like(blocks), blocks)
    task_ends = torch.cumsum(blocks, dim=0)       # first task index after each group
    num_tasks = int(task_ends[-1].item())         # the one host sync of the builder
    length = num_tasks if tid_size is None else tid_size
    if length < num_tasks:
        raise ValueError(f"tid_size must be at least {num_tasks}; got {length}")
    if length == 0:
        return blank(0, num_tasks, zero=False)

    task = torch.arange(length, **i64)
    live = task < num_tasks
    owner = torch.searchsorted(task_ends, task, right=True).clamp_max(groups - 1)
    index_in_group = task - (task_ends[owner] - blocks[owner])
    block_start = first_block[owner] + index_in_group * tile
    actual_start = torch.maximum(block_start, starts[owner])
    actual_end = torch.minimum(block_start + tile, ends[owner])
    zero = torch.zeros_like(task)

    def keep(values: Any) -> Any:
        return torch.where(live, values, zero)

    return RaggedGroupInfo(
        group_id=keep(owner),
        block_start=keep(block_start),
        actual_start=keep(actual_start),
        actual_end=keep(actual_end),
        start_within_block=keep(actual_start - block_start),
        actual_size=keep((actual_end - actual_start).clamp_min(0)),
        num_tasks=num_tasks,
        tile=int(tile),
        align_tile=int(align_tile),
    )


def _can_use_even_k_fast_path(*, logical_k: int, scale: ScaleSpec, config: RaggedDotConfig) -> bool:
    """Whether K needs no tail handling: selects the ``evenk`` / ``maskk`` variant name only."""
    if not config.enable_even_k_fast_path or logical_k % config.block_k:
        return False
    if scale.mode is ScaleMode.SUBCHANNEL:
        sub = scale.subchannel_size or 0
        if logical_k % sub:
            return False
        if sub % config.block_k and config.block_k % sub:
            return False
    return True


def _can_use_bwd_even_k_fast_path(torch: Any, *, group_sizes: Any, scale: ScaleSpec, config: RaggedBwdDotConfig) -> bool:
    if not config.enable_even_k_fast_path:
        return False
    sizes = group_sizes.detach().cpu()
    used = sizes[sizes > 0]
    if used.numel() == 0:
        return True
    if bool((used % config.block_k != 0).any()):
        return False
    if scale.mode is ScaleMode.SUBCHANNEL:
        sub = scale.subchannel_size or 0
        if sub <= 0 or bool((used % sub != 0).any()):
            return False
        if sub % config.block_k and config.block_k % sub:
            return False
    return True


def _require_cuda_tensor(torch: Any, name: str, tensor: Any) -> None:
    if not torch.is_tensor(tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")


def _require_bfloat16_scale(torch: Any, name: str, tensor: Any | None) -> None:
    if tensor is not None and tensor.dtype != torch.bfloat16:
        raise ValueError(f"{name} must have dtype torch.bfloat16; got {tensor.dtype}")


def _check_group_sizes_tensor(torch: Any, group_sizes: Any, groups: int, what: str) -> Any:
    if not torch.is_tensor(group_sizes):
        raise TypeError("group_sizes must be a torch.Tensor")
    if group_sizes.ndim != 1:
        raise ValueError(f"group_sizes must be 1D; got shape {tuple(group_sizes.shape)}")
    if int(group_sizes.shape[0]) != groups:
        raise ValueError(f"group_sizes length must match {what} groups {groups}; got {int(group_sizes.shape[0])}")
    if not _is_integer_dtype(torch, group_sizes.dtype):
        raise ValueError(f"group_sizes must have integer dtype; got {group_sizes.dtype}")
    host = group_sizes.detach().cpu()
    if bool((host < 0).any()):
        raise ValueError("group_sizes must be non-negative")
    return host


def _validate_group_sizes(torch: Any, group_sizes: Any, *, groups: int, rows: int) -> None:
    host = _check_group_sizes_tensor(torch, group_sizes, groups, "rhs")
    total = int(host.sum().item())
    if total != rows:
        raise ValueError(f"sum(group_sizes) must equal lhs rows {rows}; got {total}")


def _validate_k_group_sizes(torch: Any, group_sizes: Any, *, groups: int, max_k: int) -> Any:
    host = _check_group_sizes_tensor(torch, group_sizes, groups, "operand")
    largest = int(host.max().item()) if groups else 0
    if largest > max_k:
        raise ValueError(f"group_sizes entries must be <= logical padded K {max_k}; got {largest}")
    return host


def _validate_scale_shapes(
    *, a_scale: Any | None, b_scale: Any | None, scale: ScaleSpec, groups: int, rows: int, cols: int, scale_cols: int
) -> None:
    if scale.mode is ScaleMode.PER_CHANNEL:
        if a_scale is not None and tuple(a_scale.shape) != (rows,):
            raise ValueError(f"a_scale must have shape ({rows},); got {tuple(a_scale.shape)}")
        if b_scale is not None and tuple(b_scale.shape) != (groups, cols):
            raise ValueError(f"b_scale must have shape ({groups}, {cols}); got {tuple(b_scale.shape)}")
        return
    if a_scale is not None and tuple(a_scale.shape) != (rows, scale_cols):
        raise ValueError(f"a_scale must have shape ({rows}, {scale_cols}); got {tuple(a_scale.shape)}")
    if b_scale is not None and tuple(b_scale.shape) != (groups, scale_cols, cols):
        raise ValueError(
            "subchannel b_scale must use weight-matched layout "
            f"({groups}, {scale_cols}, {cols}) == (groups, scale_cols, N); got {tuple(b_scale.shape)}. "
            "If you have logical layout "
            f"({groups}, {cols}, {scale_cols}) == (groups, N, scale_cols), "
            "call pack_ragged_rhs_subchannel_scales(...) first."
        )


def _validate_bwd_scale_shapes(
    *, a_scale: Any | None, b_scale: Any | None, scale: ScaleSpec, groups: int, rows: int, cols: int, scale_cols: int
) -> None:
    if scale.mode is ScaleMode.PER_CHANNEL:
        if a_scale is not None and tuple(a_scale.shape) != (groups, rows):
            raise ValueError(f"a_scale must have shape ({groups}, {rows}); got {tuple(a_scale.shape)}")
        if b_scale is not None and tuple(b_scale.shape) != (groups, cols):
            raise ValueError(f"b_scale must have shape ({groups}, {cols}); got {tuple(b_scale.shape)}")
        return
    if a_scale is not None and tuple(a_scale.shape) != (groups, rows, scale_cols):
        raise ValueError(f"a_scale must have shape ({groups}, {rows}, {scale_cols}); got {tuple(a_scale.shape)}")
    if b_scale is not None and tuple(b_scale.shape) != (groups, scale_cols, cols):
        raise ValueError(
            "subchannel b_scale must use weight-matched layout "
            f"({groups}, {scale_cols}, {cols}) == (groups, scale_cols, N); got {tuple(b_scale.shape)}"
        )


def _forward_logical_shape(lhs: Any, rhs: Any, layout: GemmLayout) -> tuple[int, int, int, int]:
    """(rows, cols, k_packed, groups) of ``lhs [M, Kb]`` / ``[Kb, M]`` and ``rhs [G, Kb, N]`` / ``[G, N, Kb]``."""
    if layout not in (GemmLayout.NN, GemmLayout.NT, GemmLayout.TN, GemmLayout.TT):
        raise ValueError(f"unsupported GEMM layout {layout.value}")
    lhs_t = layout in (GemmLayout.TN, GemmLayout.TT)
    rhs_t = layout in (GemmLayout.NT, GemmLayout.TT)
    k_packed, rows = (int(lhs.shape[0]), int(lhs.shape[1])) if lhs_t else (int(lhs.shape[1]), int(lhs.shape[0]))
    groups = int(rhs.shape[0])
    cols, rhs_k = (int(rhs.shape[1]), int(rhs.shape[2])) if rhs_t else (int(rhs.shape[2]), int(rhs.shape[1]))
    if rhs_k != k_packed:
        raise ValueError(f"lhs and rhs packed K mismatch for layout={layout.value}: {k_packed} vs {rhs_k}")
    return rows, cols, k_packed, groups


def _bwd_logical_shape(lhs: Any, rhs: Any, layout: GemmLayout) -> tuple[int, int, int, int]:
    """(rows, cols, k_packed, groups) of ``lhs [G, M, Kb]`` / ``[G, Kb, M]`` and ``rhs [G, Kb, N]`` / ``[G, N, Kb]``."""
    if layout not in (GemmLayout.NN, GemmLayout.NT, GemmLayout.TN, GemmLayout.TT):
        raise ValueError(f"unsupported GEMM layout {layout.value}")
    lhs_t = layout in (GemmLayout.TN, GemmLayout.TT)
    rhs_t = layout in (GemmLayout.NT, GemmLayout.TT)
    groups = int(lhs.shape[0])
    k_packed, rows = (int(lhs.shape[1]), int(lhs.shape[2])) if lhs_t else (int(lhs.shape[2]), int(lhs.shape[1]))
    cols, rhs_k = (int(rhs.shape[1]), int(rhs.shape[2])) if rhs_t else (int(rhs.shape[2]), int(rhs.shape[1]))
    if int(rhs.shape[0]) != groups:
        raise ValueError(f"lhs and rhs group mismatch for layout={layout.value}: {groups} vs {int(rhs.shape[0])}")
    if rhs_k != k_packed:
        raise ValueError(f"lhs and rhs packed K mismatch for layout={layout.value}: {k_packed} vs {rhs_k}")
    return rows, cols, k_packed, groups


def _unit_scale(torch: Any, shape: tuple[int, ...], device: Any) -> Any:
    return torch.ones(shape, device=device, dtype=torch.bfloat16)


def ragged_dot_int4(
    lhs: Any,
    rhs: Any,
    group_sizes: Any,
    *,
    a_scale: Any | None = None,
    b_scale: Any | None = None,
    scale: ScaleSpec = ScaleSpec(ScaleMode.PER_CHANNEL),
    config: RaggedDotConfig = RaggedDotConfig(),
    layout: GemmLayout = GemmLayout.NN,
    out: Any | None = None,
    output_dtype: Any | None = None,
    use_native: bool | None = None,
    native_root: str | None = None,
    native_library_path: str | None = None,
    group_info: RaggedGroupInfo | None = None,
) -> Any:
    """Forward grouped int4 dot: rows of group ``g`` are multiplied by ``rhs[g]``.

    ``NN``: ``lhs [M, K/2]`` (uint8, nibbles packed along K), ``rhs [G, K/2, N]``; ``NT``, ``TN``
    and ``TT`` move the packed-K axis as in the dense API.  ``group_sizes [G]`` partitions the
    ``M`` rows into contiguous groups and must sum to ``M``.  Scales: per-channel ``a_scale [M]``,
    ``b_scale [G, N]``; subchannel ``S``: ``a_scale [M, ceil(K/S)]``, ``b_scale [G, ceil(K/S), N]``.
    A missing scale is treated as all ones unless ``use_native=True``.  Output ``[M, N]``, bf16
    by default (float32 on request).  No autograd.

    ``group_info`` (not in the reference) lets a caller who reuses the same ``group_sizes`` pass
    the prebuilt task arrays and skip the two host synchronisations of validation and task
    building.  The tasks run with the block height they were built with (``group_info.tile``).  For
    tasks built on the device nothing about them is read on the host: the kernel clamps task bounds to
    the operand, and a task list that overflowed its arrays is reported after the fact through
    ``native.device_status()`` (code 3) and ``group_info.device_overflow`` - rows of the tasks that did
    not fit stay unwritten, so size ``max_tasks`` by the documented bound.
    """
    layout = _check_layout(layout)
    torch = _torch()
    _require_cuda_tensor(torch, "lhs", lhs)
    _require_cuda_tensor(torch, "rhs", rhs)
    if lhs.dtype != torch.uint8:
        raise ValueError(f"lhs must be packed int4 torch.uint8; got {lhs.dtype}")
    if rhs.dtype != torch.uint8:
        raise ValueError(f"rhs must be packed int4 torch.uint8; got {rhs.dtype}")
    if lhs.ndim != 2:
        raise ValueError(f"lhs must have shape (M, K/2); got {tuple(lhs.shape)}")
    if rhs.ndim != 3:
        raise ValueError(f"rhs must have shape (G, K/2, N); got {tuple(rhs.shape)}")
    if not lhs.is_contiguous():
        raise ValueError("lhs must be contiguous")
    if not rhs.is_contiguous():
        raise ValueError("rhs must be contiguous")
    if use_native is False:
        raise ValueError("use_native=False asks for the JIT path, which this library does not have")
    if config.block_m > MAX_TASK_ROWS:
        raise ValueError(f"config.block_m must be at most {MAX_TASK_ROWS}; got {config.block_m}")

    rows, cols, k_packed, groups = _forward_logical_shape(lhs, rhs, layout)
    pair_capable = layout is GemmLayout.NN and (
        scale.mode is ScaleMode.PER_CHANNEL or (scale.subchannel_size or 0) >= 128)
    if config.block_m > 128 and not pair_capable:
        raise ValueError("tasks of more than 128 rows need layout NN and per-channel scales or K-groups of at least 128")
    if group_info is not None and group_info.tile is not None and group_info.tile != config.block_m:
        # prebuilt tasks carry their own height: a launch with another one would skip rows of every block
        if config.block_m != RaggedDotConfig().block_m:
            raise ValueError(
                f"group_info was built with tile={group_info.tile} but config.block_m={config.block_m}; "
                "build the tasks with the block height of the config (or leave block_m at its default)")
        if group_info.tile > 128 and not pair_capable:
            raise ValueError("tasks of more than 128 rows need layout NN and per-channel scales or K-groups of at least 128")
        config = replace(config, block_m=int(group_info.tile))
    if group_info is None and config.block_m == 128 and pair_capable and config.pair_tasks is not False:
        if config.pair_tasks is True or rows >= PAIR_MIN_MEAN_GROUP_ROWS * groups:
            if PAIR_TASK_ROWS % config.align_tile == 0:
                config = replace(config, block_m=PAIR_TASK_ROWS)
    if group_info is None and layout in (GemmLayout.TN, GemmLayout.TT) and config.align_tile % 16 and config.block_m % 16 == 0:
        # a transposed lhs reaches the tensor cores only with tasks that start on multiples of 16 rows; where the
        # tasks start changes nothing in the result (rows outside a group are masked), so cut them that way
        config = replace(config, align_tile=math.lcm(config.align_tile, 16))
    if group_info is None:
        _validate_group_sizes(torch, group_sizes, groups=groups, rows=rows)
        if group_sizes.device != lhs.device:
            group_sizes = group_sizes.to(device=lhs.device)
        group_info = calculate_group_info(group_sizes, config.block_m, align_tile=config.align_tile)

    _require_bfloat16_scale(torch, "a_scale", a_scale)
    _require_bfloat16_scale(torch, "b_scale", b_scale)
    if a_scale is not None:
        _require_cuda_tensor(torch, "a_scale", a_scale)
    if b_scale is not None:
        _require_cuda_tensor(torch, "b_scale", b_scale)

    logical_k = 2 * k_packed
    scale_cols = 1
    if scale.mode is ScaleMode.SUBCHANNEL:
        sub = scale.subchannel_size or 0
        if sub % 2:
            raise ValueError("subchannel_size must be even for packed int4 operands")
        scale_cols = _cdiv(logical_k, sub)
    _validate_scale_shapes(
        a_scale=a_scale, b_scale=b_scale, scale=scale, groups=groups, rows=rows, cols=cols, scale_cols=scale_cols
    )
    if a_scale is not None and not a_scale.is_contiguous():
        raise ValueError("a_scale must be contiguous")
    if b_scale is not None and not b_scale.is_contiguous():
        raise ValueError("b_scale must be contiguous")

    if output_dtype is None:
        output_dtype = torch.bfloat16
    if output_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"output_dtype must be torch.bfloat16 or torch.float32; got {output_dtype}")
    if out is None:
        out = torch.empty((rows, cols), device=lhs.device, dtype=output_dtype)
    else:
        _require_cuda_tensor(torch, "out", out)
        if tuple(out.shape) != (rows, cols):
            raise ValueError(f"out must have shape ({rows}, {cols}); got {tuple(out.shape)}")
        if out.dtype != output_dtype:
            raise ValueError(f"out dtype {out.dtype} does not match output_dtype {output_dtype}")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
    if group_info.num_tasks == 0:
        return out

    if a_scale is None or b_scale is None:
        if use_native is True:
            raise ValueError("native ragged forward dispatch requires a_scale and b_scale")
        pc = scale.mode is ScaleMode.PER_CHANNEL
        if a_scale is None:
            a_scale = _unit_scale(torch, (rows,) if pc else (rows, scale_cols), lhs.device)
        if b_scale is None:
            b_scale = _unit_scale(torch, (groups, cols) if pc else (groups, scale_cols, cols), lhs.device)

    even_k = _can_use_even_k_fast_path(logical_k=logical_k, scale=scale, config=config)
    from .native import launch_ragged_fwd_kernel

    return launch_ragged_fwd_kernel(
        lhs,
        rhs,
        group_info=group_info,
        a_scale=a_scale,
        b_scale=b_scale,
        out=out,
        scale=scale,
        config=config,
        layout=layout,
        variant=RAGGED_EVEN_K if even_k else RAGGED_MASK_K,
        rows=rows,
        cols=cols,
        k_packed=k_packed,
        scale_cols=scale_cols,
        root=native_root,
        library_path=native_library_path,
    )


def ragged_dot_int4_bwd(
    lhs: Any,
    rhs: Any,
    group_sizes: Any,
    *,
    a_scale: Any | None = None,
    b_scale: Any | None = None,
    scale: ScaleSpec = ScaleSpec(ScaleMode.PER_CHANNEL),
    config: RaggedBwdDotConfig = RaggedBwdDotConfig(),
    layout: GemmLayout = GemmLayout.NN,
    out: Any | None = None,
    use_native: bool | None = None,
    native_root: str | None = None,
    native_library_path: str | None = None,
    validate_group_sizes: bool = True,
) -> Any:
    """Backward-style grouped dot: ``out[g] = op(lhs[g]) @ op(rhs[g])`` over the first ``group_sizes[g]`` K values.

    Operands are padded to one packed-K capacity: ``NN`` ``lhs [G, M, K/2]``, ``rhs [G, K/2, N]``;
    ``NT`` ``rhs [G, N, K/2]``; ``TN`` ``lhs [G, K/2, M]``; ``TT`` both.  Whatever lies beyond
    ``group_sizes[g]`` (padding, or the unused high nibble of an odd length) is ignored; an empty
    group yields zeros.  Scales: ``a_scale [G, M]`` / ``[G, M, S]``, ``b_scale [G, N]`` /
    ``[G, S, N]``.  Output float32 ``[G, M, N]``, bit-identical from run to run.

    ``validate_group_sizes=False`` (not in the reference) skips the host-side range check of
    ``group_sizes`` and with it the host synchronisation.
    """
    layout = _check_layout(layout)
    torch = _torch()
    _require_cuda_tensor(torch, "lhs", lhs)
    _require_cuda_tensor(torch, "rhs", rhs)
    if lhs.dtype != torch.uint8:
        raise ValueError(f"lhs must be packed int4 torch.uint8; got {lhs.dtype}")
    if rhs.dtype != torch.uint8:
        raise ValueError(f"rhs must be packed int4 torch.uint8; got {rhs.dtype}")
    if lhs.ndim != 3:
        raise ValueError(f"lhs must be a grouped packed tensor; got shape {tuple(lhs.shape)}")
    if rhs.ndim != 3:
        raise ValueError(f"rhs must be a grouped packed tensor; got shape {tuple(rhs.shape)}")
    if not lhs.is_contiguous():
        raise ValueError("lhs must be contiguous")
    if not rhs.is_contiguous():
        raise ValueError("rhs must be contiguous")
    if use_native is False:
        raise ValueError("use_native=False asks for the JIT path, which this library does not have")

    rows, cols, k_packed, groups = _bwd_logical_shape(lhs, rhs, layout)
    capacity = 2 * k_packed
    if validate_group_sizes:
        _validate_k_group_sizes(torch, group_sizes, groups=groups, max_k=capacity)
    if group_sizes.device != lhs.device:
        group_sizes = group_sizes.to(device=lhs.device)

    _require_bfloat16_scale(torch, "a_scale", a_scale)
    _require_bfloat16_scale(torch, "b_scale", b_scale)
    if a_scale is not None:
        _require_cuda_tensor(torch, "a_scale", a_scale)
    if b_scale is not None:
        _require_cuda_tensor(torch, "b_scale", b_scale)
    scale_cols = 1
    if scale.mode is ScaleMode.SUBCHANNEL:
        sub = scale.subchannel_size or 0
        if sub % 2:
            raise ValueError("subchannel_size must be even for packed int4 operands")
        scale_cols = _cdiv(capacity, sub)
    _validate_bwd_scale_shapes(
        a_scale=a_scale, b_scale=b_scale, scale=scale, groups=groups, rows=rows, cols=cols, scale_cols=scale_cols
    )
    if a_scale is not None and not a_scale.is_contiguous():
        raise ValueError("a_scale must be contiguous")
    if b_scale is not None and not b_scale.is_contiguous():
        raise ValueError("b_scale must be contiguous")

    if out is None:
        out = torch.empty((groups, rows, cols), device=lhs.device, dtype=torch.float32)
    else:
        _require_cuda_tensor(torch, "out", out)
        if tuple(out.shape) != (groups, rows, cols):
            raise ValueError(f"out must have shape ({groups}, {rows}, {cols}); got {tuple(out.shape)}")
        if out.dtype != torch.float32:
            raise ValueError(f"out dtype must be torch.float32; got {out.dtype}")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
    if groups * rows * cols == 0:
        return out

    if a_scale is None or b_scale is None:
        if use_native is True:
            raise ValueError("native ragged backward dispatch requires a_scale and b_scale")
        pc = scale.mode is ScaleMode.PER_CHANNEL
        if a_scale is None:
            a_scale = _unit_scale(torch, (groups, rows) if pc else (groups, rows, scale_cols), lhs.device)
        if b_scale is None:
            b_scale = _unit_scale(torch, (groups, cols) if pc else (groups, scale_cols, cols), lhs.device)

    from .native import launch_ragged_bwd_kernel

    return launch_ragged_bwd_kernel(
        lhs,
        rhs,
        group_sizes,
        a_scale=a_scale,
        b_scale=b_scale,
        out=out,
        scale=scale,
        config=config,
        layout=layout,
        variant=RAGGED_MASK_K,
        rows=rows,
        cols=cols,
        k_packed=k_packed,
        scale_cols=scale_cols,
        root=native_root,
        library_path=native_library_path,
    )


def calculate_group_info_on_device(
    group_sizes: Any,
    tile: int,
    *,
    total_rows: int,
    align_tile: int = 8,
    max_tasks: int | None = None,
) -> RaggedGroupInfo:
    """``calculate_group_info`` without a host round trip (CUDA kernel of the native library).

    The reference reads the task count back to the host to size its launch (ragged.py:275); here the
    arrays are sized by an upper bound (``total_rows // tile + 2 * groups`` tasks always fit) and the
    count stays on the GPU in ``device_num_tasks``; the forward kernel reads it there.  Entries past
    the count are empty tasks.  ``total_rows`` must be the sum of ``group_sizes`` (it only sizes the
    arrays; nothing checks it).  Same task arrays, element for element, as ``calculate_group_info``.
    """
    torch = _torch()
    if tile <= 0:
        raise ValueError("tile must be positive")
    if align_tile <= 0:
        raise ValueError("align_tile must be positive")
    if tile % align_tile:
        raise ValueError("tile must be a multiple of align_tile")
    if group_sizes.ndim != 1:
        raise ValueError("group_sizes must be a 1-D tensor")
    groups = int(group_sizes.numel())
    if groups == 0:
        raise ValueError("group_sizes must not be empty")
    capacity = int(max_tasks) if max_tasks is not None else int(total_rows) // tile + 2 * groups
    from .native import group_info_on_device

    gid, bstart, astart, aend, count, overflow = group_info_on_device(
        group_sizes, tile, align_tile=align_tile, max_tasks=max(capacity, 1))
    return RaggedGroupInfo(
        group_id=gid, block_start=bstart, actual_start=astart, actual_end=aend,
        start_within_block=astart - bstart, actual_size=aend - astart, num_tasks=max(capacity, 1),
        device_num_tasks=count, device_overflow=overflow, tile=int(tile), align_tile=int(align_tile),
    )


def ragged_dot_int4_bwd_flat(
    lhs: Any,
    rhs: Any,
    group_sizes: Any,
    *,
    a_scale: Any,
    b_scale: Any,
    out: Any | None = None,
    native_library_path: str | None = None,
    static_scratch: bool = False,
) -> Any:
    """Backward grouped int4 dot over flat token-packed operands (not in the reference).

    ``out[g] = (lhs[tokens of g]^T @ rhs[tokens of g]) * a_scale[g][:, None] * b_scale[g][None, :]``.
    ``lhs [ceil(T/2), M]`` and ``rhs [ceil(T/2), N]`` hold the ``T`` tokens back to back, two per byte along
    the token axis (``repack_int4_tokens`` builds this form from the forward operand format), so
    there is no per-group padding to a common capacity as ``ragged_dot_int4_bwd`` needs.  Groups may
    start on odd tokens.  Per-channel scales ``a_scale [G, M]``, ``b_scale [G, N]`` (bf16); output
    ``[G, M, N]`` float32.  ``group_sizes`` must sum to the number of real tokens (``2 * lhs.shape[0]``, or one less when the
    last byte row holds a single token); it is not read on the host.

    ``static_scratch=True`` uses the library's built-in scratch instead of a workspace tensor (at most
    4096 groups, one call at a time per device); with ``out`` given and ``group_sizes`` already an int64
    CUDA tensor, such a call allocates nothing at all.
    """
    torch = _torch()
    _require_cuda_tensor(torch, "lhs", lhs)
    _require_cuda_tensor(torch, "rhs", rhs)
    if lhs.dtype != torch.uint8 or rhs.dtype != torch.uint8:
        raise ValueError("lhs and rhs must be packed int4 torch.uint8")
    if lhs.ndim != 2 or rhs.ndim != 2 or lhs.shape[0] != rhs.shape[0]:
        raise ValueError(f"lhs and rhs must have shapes (T/2, M) and (T/2, N); got {tuple(lhs.shape)} and {tuple(rhs.shape)}")
    if not lhs.is_contiguous() or not rhs.is_contiguous():
        raise ValueError("lhs and rhs must be contiguous")
    if group_sizes.ndim != 1 or group_sizes.numel() == 0:
        raise ValueError("group_sizes must be a non-empty 1-D tensor")
    _require_cuda_tensor(torch, "a_scale", a_scale)
    _require_cuda_tensor(torch, "b_scale", b_scale)
    groups, m, n = int(group_sizes.numel()), int(lhs.shape[1]), int(rhs.shape[1])
    if tuple(a_scale.shape) != (groups, m) or tuple(b_scale.shape) != (groups, n):
        raise ValueError(f"a_scale must have shape ({groups}, {m}) and b_scale ({groups}, {n})")
    if group_sizes.device != lhs.device:
        if static_scratch:
            raise ValueError("static_scratch=True requires group_sizes on the operands' device")
        group_sizes = group_sizes.to(device=lhs.device)
    if out is None:
        out = torch.empty((groups, m, n), device=lhs.device, dtype=torch.float32)
    elif tuple(out.shape) != (groups, m, n) or out.dtype != torch.float32 or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous float32 tensor of shape ({groups}, {m}, {n})")
    from .native import launch_ragged_bwd_flat_kernel

    return launch_ragged_bwd_flat_kernel(lhs, rhs, group_sizes, a_scale=a_scale, b_scale=b_scale, out=out,
                                         tokens=2 * int(lhs.shape[0]), library_path=native_library_path,
                                         static_scratch=static_scratch)
