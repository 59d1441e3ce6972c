"""Partitioning of the GEMMs over the GPUs of one box: one process per GPU, no collective on the hot path.

The reference is single-device (its dispatcher only forwards a device index, dispatch.cpp:246), so
everything here is new surface:

* dense GEMMs are column-parallel along N: rank ``r`` owns a contiguous block of output columns,
  keeps its own contiguous copy of those columns of B (and of ``b_scale``), A is replicated;
  for the fused SwiGLU rank ``r`` owns columns ``r`` of *both* halves, re-concatenated locally
  as ``[up_r | gate_r]``;
* grouped GEMMs are expert-parallel: whole groups are assigned to ranks, greedy largest-first
  so that the rows per rank stay balanced under skewed group sizes;
* outputs stay local.  ``all_gather_columns`` / ``all_gather_rows`` build the full result with one
  NCCL all-gather when a caller asks for it; they are separate calls so that their cost is
  measured separately.

All functions are device-agnostic tensor code, so the same logic runs under ``gloo`` on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Sequence

from .metadata import GemmLayout


def column_block(n: int, world_size: int, rank: int, *, multiple: int = 16) -> tuple[int, int]:
    """[start, stop) of rank ``rank``'s output columns: as even as possible in units of ``multiple``.

    ``multiple`` keeps every shard's pitch a multiple of 16 bytes (the TMA rule); the last rank
    takes what is left when ``n`` is not a multiple.
    """
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    if n <= 0 or multiple <= 0:
        raise ValueError("n and multiple must be positive")
    units = -(-n // multiple)
    share, extra = divmod(units, world_size)
    first = rank * share + min(rank, extra)
    count = share + (1 if rank < extra else 0)
    return min(first * multiple, n), min((first + count) * multiple, n)


def shard_dense_rhs(
    b: Any,
    b_scale: Any,
    *,
    layout: GemmLayout,
    world_size: int,
    rank: int,
    swiglu: bool = False,
    multiple: int = 16,
) -> tuple[Any, Any, tuple[int, int]]:
    """This rank's contiguous copy of B and ``b_scale`` and its output column range.

    ``b`` is stored ``[Kb, cols]`` (NN, TN) or ``[cols, Kb]`` (NT); ``b_scale`` is ``[cols]`` or
    ``[K-groups, cols]``.  With ``swiglu`` the stored columns are ``[up | gate]`` and the column
    range refers to the ``D = cols / 2`` output columns.
    """
    import torch

    n_axis = 0 if layout in (GemmLayout.NT, GemmLayout.TT) else b.ndim - 1
    cols = int(b.shape[n_axis])
    if swiglu:
        if cols % 2:
            raise ValueError("fused SwiGLU needs an even number of stored B columns")
        d = cols // 2
        lo, hi = column_block(d, world_size, rank, multiple=multiple)
        index = torch.cat((torch.arange(lo, hi), torch.arange(d + lo, d + hi))).to(b.device)
    else:
        lo, hi = column_block(cols, world_size, rank, multiple=multiple)
        index = torch.arange(lo, hi, device=b.device)
    b_local = b.index_select(n_axis, index).contiguous()
    scale_local = b_scale.index_select(b_scale.ndim - 1, index.to(b_scale.device)).contiguous()
    return b_local, scale_local, (lo, hi)


def assign_groups(group_sizes: Sequence[int], world_size: int, *, per_group_cost: int = 0) -> list[list[int]]:
    """Greedy largest-first (LPT) assignment of groups to ranks by row count.

    ``per_group_cost`` is a fixed cost per group in units of rows.  The forward dot costs rows only (0); the
    backward dot writes one ``[M, N]`` fp32 slab per group whatever its size, empty groups included, so its cost per
    group is mostly that slab: pass the number of rows whose arithmetic takes as long as one slab's write.

    Returns, per rank, its group indices in ascending order.  Deterministic: ties go to the lower
    group index first and to the lower rank.
    """
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    if per_group_cost < 0:
        raise ValueError("per_group_cost must not be negative")
    order = sorted(range(len(group_sizes)), key=lambda g: (-int(group_sizes[g]), g))
    load = [0] * world_size
    owned: list[list[int]] = [[] for _ in range(world_size)]
    for g in order:
        r = min(range(world_size), key=lambda i: (load[i], i))
        owned[r].append(g)
        load[r] += int(group_sizes[g]) + per_group_cost
    return [sorted(groups) for groups in owned]


def load_imbalance(group_sizes: Sequence[int], assignment: Sequence[Sequence[int]]) -> float:
    """max over ranks of assigned rows divided by the mean (1.0 = perfectly balanced)."""
    loads = [sum(int(group_sizes[g]) for g in groups) for groups in assignment]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean > 0 else 1.0


@dataclass(frozen=True)
class RaggedShard:
    """One rank's share of a grouped forward dot."""

    groups: tuple[int, ...]     # global group ids, ascending
    row_index: Any              # int64 [local rows]: global row of each local row
    lhs: Any
    rhs: Any
    a_scale: Any
    b_scale: Any
    group_sizes: Any            # int64 [len(groups)]


def shard_ragged_fwd(
    lhs: Any, rhs: Any, a_scale: Any, b_scale: Any, group_sizes: Any, groups: Sequence[int], *, layout: GemmLayout = GemmLayout.NN
) -> RaggedShard:
    """Rows, weights and scales of the groups in ``groups`` (kept in ascending group order)."""
    import torch

    sizes = group_sizes.detach().cpu().to(torch.int64)
    ends = torch.cumsum(sizes, 0)
    starts = ends - sizes
    pieces = [torch.arange(int(starts[g]), int(ends[g])) for g in groups]
    rows = torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.int64)
    gsel = torch.tensor(list(groups), dtype=torch.int64)
    row_axis = 1 if layout in (GemmLayout.TN, GemmLayout.TT) else 0
    return RaggedShard(
        groups=tuple(int(g) for g in groups),
        row_index=rows,
        lhs=lhs.index_select(row_axis, rows.to(lhs.device)).contiguous(),
        rhs=rhs.index_select(0, gsel.to(rhs.device)).contiguous(),
        a_scale=a_scale.index_select(0, rows.to(a_scale.device)).contiguous(),
        b_scale=b_scale.index_select(0, gsel.to(b_scale.device)).contiguous(),
        group_sizes=sizes.index_select(0, gsel).to(group_sizes.device),
    )


def shard_ragged_bwd(lhs: Any, rhs: Any, a_scale: Any, b_scale: Any, group_sizes: Any, groups: Sequence[int]) -> tuple[Any, ...]:
    """Backward operands are already grouped on axis 0: take this rank's groups."""
    import torch

    gsel = torch.tensor(list(groups), dtype=torch.int64)

    def take(t: Any) -> Any:
        return t.index_select(0, gsel.to(t.device)).contiguous()

    return take(lhs), take(rhs), take(a_scale), take(b_scale), take(group_sizes)


def all_gather_columns(local_out: Any, column_ranges: Sequence[tuple[int, int]], *, group: Any = None) -> Any:
    """Full ``[M, N]`` result from every rank's ``[M, N_r]`` block (ranges may differ in width)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    widest = max(hi - lo for lo, hi in column_ranges)
    m = int(local_out.shape[0])
    padded = local_out.new_zeros((m, widest))
    padded[:, : local_out.shape[1]] = local_out
    flat = local_out.new_empty((world * m, widest))  # concatenation along dim 0 suits every backend
    dist.all_gather_into_tensor(flat, padded, group=group)
    gathered = flat.view(world, m, widest)
    total = max(hi for _lo, hi in column_ranges)
    full = local_out.new_empty((m, total))
    for r, (lo, hi) in enumerate(column_ranges):
        full[:, lo:hi] = gathered[r, :, : hi - lo]
    return full


def all_gather_rows(local_out: Any, row_indices: Sequence[Any], total_rows: int, *, group: Any = None) -> Any:
    """Full ``[rows, N]`` result of a grouped forward dot from every rank's rows (uneven counts)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    most = max(int(idx.numel()) for idx in row_indices)
    n = int(local_out.shape[1])
    padded = local_out.new_zeros((most, n))
    padded[: local_out.shape[0]] = local_out
    flat = local_out.new_empty((world * most, n))
    dist.all_gather_into_tensor(flat, padded, group=group)
    gathered = flat.view(world, most, n)
    full = local_out.new_zeros((total_rows, n))
    for r, idx in enumerate(row_indices):
        full[idx.to(full.device)] = gathered[r, : idx.numel()]
    return full
