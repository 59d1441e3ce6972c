"""Launch-shape contract of a registry entry (reference: template_config.py:8-80).

A variant is registered for multiples of its ``block_m`` / ``block_n`` / ``block_k * split_k``
(and of the subchannel length).  The sm_100a kernels themselves mask partial tiles, but the
dense API stays as strict as the reference's: asking an entry to run a shape outside its
multiples raises ``ValueError`` with the same message prefix.
"""
from __future__ import annotations

from dataclasses import dataclass

from .metadata import Epilogue, KernelMetadata, OperandDType, ScaleMode


def tile_multiple_rejection_reasons(kernel: KernelMetadata, shape: "LaunchShape") -> tuple[str, ...]:
    m, n, k = shape.m, shape.n, shape.k
    if min(m, n, k) <= 0:
        return (f"M, N, and K must be positive; got ({m}, {n}, {k})",)
    tile = kernel.tile
    found: list[str] = []
    if m % tile.block_m:
        found.append(f"M={m} is not divisible by BLOCK_M={tile.block_m}")
    if n % tile.block_n:
        found.append(f"N={n} is not divisible by BLOCK_N={tile.block_n}")
    k_step = tile.block_k * tile.split_k
    if k % k_step:
        found.append(f"K={k} is not divisible by BLOCK_K*SPLIT_K={k_step}")
    sub = kernel.scale.subchannel_size if kernel.scale.mode is ScaleMode.SUBCHANNEL else None
    if sub is not None and k % sub:
        found.append(f"K={k} is not divisible by SUBCHANNEL={sub}")
    return tuple(found)


@dataclass(frozen=True, slots=True)
class LaunchShape:
    m: int
    n: int
    k: int

    def validate_for(self, kernel: KernelMetadata) -> None:
        problems = tile_multiple_rejection_reasons(kernel, self)
        if problems:
            raise ValueError(f"{kernel.kernel_id} requires tile-multiple shape: " + "; ".join(problems))


def is_tile_multiple_shape(kernel: KernelMetadata, shape: LaunchShape) -> bool:
    return len(tile_multiple_rejection_reasons(kernel, shape)) == 0


@dataclass(frozen=True, slots=True)
class TemplatePlan:
    """What a (kernel, shape) pair asks of the device code; used by tooling and tests."""

    kernel: KernelMetadata
    shape: LaunchShape
    needs_packed_int4: bool
    needs_subchannel_loop: bool
    needs_per_channel_epilogue_scale: bool
    needs_relu2_activation: bool
    needs_fused_swiglu_up_gate: bool
    even_k: bool
    split_k: int


def plan_template(kernel: KernelMetadata, shape: LaunchShape) -> TemplatePlan:
    shape.validate_for(kernel)
    subchannel = kernel.scale.mode is ScaleMode.SUBCHANNEL
    return TemplatePlan(
        kernel=kernel,
        shape=shape,
        needs_packed_int4=kernel.a_dtype is OperandDType.INT4,
        needs_subchannel_loop=subchannel,
        needs_per_channel_epilogue_scale=not subchannel,
        needs_relu2_activation=kernel.epilogue is Epilogue.RELU2,
        needs_fused_swiglu_up_gate=kernel.epilogue is Epilogue.SWIGLU,
        even_k=kernel.tile.even_k,
        split_k=kernel.tile.split_k,
    )


def representative_generation_shape(kernel: KernelMetadata) -> LaunchShape:
    """Smallest shape the entry accepts: one tile, K a common multiple of its K constraints."""
    step = kernel.tile.block_k * kernel.tile.split_k
    k = step
    if kernel.scale.mode is ScaleMode.SUBCHANNEL:
        sub = kernel.scale.subchannel_size or step
        while k % sub:
            k += step
    return LaunchShape(kernel.tile.block_m, kernel.tile.block_n, k)
