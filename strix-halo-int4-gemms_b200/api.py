"""Dense GEMM entry points: ``mm``, ``fused_swiglu_up_gate``, ``explicit_mm``, ``reference_mm``.

Same signatures, validation and error types as the reference's ``api.py`` (``mm`` :119,
``fused_swiglu_up_gate`` :167, ``explicit_mm`` :217, ``reference_mm`` :257,
``_scaled_reference_mm`` :299, shape/scale checks :36-116).  Dispatch goes to the sm_100a CUDA
library through :mod:`native`; it is strict and never falls back: a shape no registry entry
accepts raises ``LookupError``, a missing library or a non-CUDA tensor raises.

``use_reference=True`` is the reference API's numerical-check switch: it evaluates the same
metadata with plain PyTorch ops on whatever device the tensors live on.  It is only ever
reached when the caller asks for it.
"""
from __future__ import annotations

from typing import Any

from .exceptions import KernelNotAvailableError
from .metadata import (
    SUPPORTED_GEMM_LAYOUTS,
    Epilogue,
    GemmLayout,
    KernelMetadata,
    KernelSchedule,
    KernelStatus,
    OperandDType,
    ScaleMode,
    ScaleSpec,
)
from .native import launch_generated_kernel
from .quant import unpack_int4_k_major
from .registry import KernelRegistry, default_registry


def _torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError("torch is required for GEMM APIs") from exc
    return torch


def _require_supported_layout(layout: GemmLayout) -> None:
    if layout in SUPPORTED_GEMM_LAYOUTS:
        return
    names = ", ".join(item.value for item in SUPPORTED_GEMM_LAYOUTS)
    raise ValueError(f"unsupported GEMM layout {layout.value}; generated layouts are {names}")


def _holds_packed_int4(dtype: OperandDType, tensor: Any) -> bool:
    return dtype is OperandDType.INT4 and str(getattr(tensor, "dtype", "")) in ("torch.uint8", "uint8")


def _logical_problem_shape(
    a: Any, b: Any, *, dtype: OperandDType, layout: GemmLayout, swiglu: bool
) -> tuple[int, int, int]:
    """(M, N, K) of the logical GEMM.  A packed uint8 operand counts two K values per byte."""
    _require_supported_layout(layout)
    a_k_axis, a_m_axis = (-2, -1) if layout is GemmLayout.TN else (-1, -2)
    b_k_axis, b_n_axis = (-1, -2) if layout is GemmLayout.NT else (-2, -1)
    m = int(a.shape[a_m_axis])
    n = int(b.shape[b_n_axis])
    k_a = int(a.shape[a_k_axis]) * (2 if _holds_packed_int4(dtype, a) else 1)
    k_b = int(b.shape[b_k_axis]) * (2 if _holds_packed_int4(dtype, b) else 1)
    if k_a != k_b:
        raise ValueError(f"logical K mismatch for layout={layout.value}: A has {k_a}, B has {k_b}")
    if swiglu:
        if n % 2:
            raise ValueError("fused_swiglu_up_gate requires the logical B output dimension to be even")
        n //= 2
    return m, n, k_a


def _scale_cols(k: int, scale: ScaleSpec) -> int:
    if scale.subchannel_size is None:
        raise ValueError("subchannel scale mode requires subchannel_size")
    return -(-k // scale.subchannel_size)


def _validate_scale_shapes(
    *, kernel: KernelMetadata, m: int, n: int, k: int, a_scale: Any | None, b_scale: Any | None
) -> None:
    out_cols = 2 * n if kernel.epilogue is Epilogue.SWIGLU else n
    if kernel.scale.mode is ScaleMode.PER_CHANNEL:
        if a_scale is not None and tuple(a_scale.shape) != (m,):
            raise ValueError(f"a_scale must have shape ({m},); got {tuple(a_scale.shape)}")
        if b_scale is not None and tuple(b_scale.shape) != (out_cols,):
            raise ValueError(f"b_scale must have shape ({out_cols},); got {tuple(b_scale.shape)}")
        return
    groups = _scale_cols(k, kernel.scale)
    if a_scale is not None and tuple(a_scale.shape) != (m, groups):
        raise ValueError(f"a_scale must have shape ({m}, {groups}); got {tuple(a_scale.shape)}")
    if b_scale is not None and tuple(b_scale.shape) != (groups, out_cols):
        raise ValueError(
            "subchannel b_scale must use weight-matched layout "
            f"{(groups, out_cols)} == (scale_cols, output_cols); got {tuple(b_scale.shape)}. "
            f"If you have logical layout {(out_cols, groups)} == (output_cols, scale_cols), "
            "call pack_rhs_subchannel_scales(...) first."
        )


def mm(
    a: Any,
    b: Any,
    *,
    a_scale: Any | None = None,
    b_scale: Any | None = None,
    gate: Any | None = None,
    dtype: OperandDType = OperandDType.INT4,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec = ScaleSpec(ScaleMode.PER_CHANNEL),
    epilogue: Epilogue = Epilogue.NONE,
    schedule: KernelSchedule = KernelSchedule.STANDARD,
    registry: KernelRegistry = default_registry,
    use_reference: bool = False,
) -> Any:
    """Pick a registry entry for the operands' shape and run it on the GPU.

    ``C = epilogue((A_q @ B_q) * a_scale[:, None] * b_scale[None, :])`` with exact int32
    accumulation, bf16 output.  Strict: no entry for the shape -> ``LookupError``.
    """
    if epilogue is Epilogue.SWIGLU:
        raise ValueError("SwiGLU is exposed through fused_swiglu_up_gate(...), not mm(...)")
    _require_supported_layout(layout)
    m, n, k = _logical_problem_shape(a, b, dtype=dtype, layout=layout, swiglu=False)
    common = dict(dtype=dtype, layout=layout, scale=scale, epilogue=epilogue, schedule=schedule)
    if use_reference:
        kernel = registry.select_reference(**common)
    else:
        kernel = registry.select(m=m, n=n, k=k, **common)
    return explicit_mm(
        a, b, kernel=kernel, a_scale=a_scale, b_scale=b_scale, gate=gate, use_reference=use_reference
    )


def fused_swiglu_up_gate(
    a: Any,
    b_up_gate: Any,
    *,
    a_scale: Any | None = None,
    b_scale: Any | None = None,
    dtype: OperandDType = OperandDType.INT4,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec = ScaleSpec(ScaleMode.PER_CHANNEL),
    registry: KernelRegistry = default_registry,
    use_reference: bool = False,
) -> Any:
    """``up * silu(gate)`` of one GEMM against ``[up | gate]`` weights.

    ``b_up_gate`` holds ``2*D`` output columns, the up projection first; the result is
    ``(M, D)``.  One CTA owns output column ``j`` and its gate column ``D + j``, so the
    full ``(M, 2D)`` product is never written.
    """
    _require_supported_layout(layout)
    m, n, k = _logical_problem_shape(a, b_up_gate, dtype=dtype, layout=layout, swiglu=True)
    common = dict(dtype=dtype, layout=layout, scale=scale, epilogue=Epilogue.SWIGLU, split_k=1)
    if use_reference:
        kernel = registry.select_reference(**common)
    else:
        kernel = registry.select(m=m, n=n, k=k, **common)
    return explicit_mm(a, b_up_gate, kernel=kernel, a_scale=a_scale, b_scale=b_scale, use_reference=use_reference)


def explicit_mm(
    a: Any,
    b: Any,
    *,
    kernel: KernelMetadata,
    a_scale: Any | None = None,
    b_scale: Any | None = None,
    gate: Any | None = None,
    use_reference: bool = False,
) -> Any:
    """Run the registry entry the caller chose (or its PyTorch reference math)."""
    _require_supported_layout(kernel.layout)
    swiglu = kernel.epilogue is Epilogue.SWIGLU
    if swiglu and gate is not None:
        raise ValueError("SwiGLU kernels use fused up/gate columns; pass gate through b_up_gate")
    m, n, k = _logical_problem_shape(a, b, dtype=kernel.a_dtype, layout=kernel.layout, swiglu=swiglu)
    _validate_scale_shapes(kernel=kernel, m=m, n=n, k=k, a_scale=a_scale, b_scale=b_scale)
    if use_reference:
        return reference_mm(a, b, kernel=kernel, a_scale=a_scale, b_scale=b_scale, gate=gate)
    launch = dict(kernel=kernel, a_scale=a_scale, b_scale=b_scale, gate=gate)
    if kernel.status in (KernelStatus.COMPILED, KernelStatus.BENCHMARKED):
        return launch_generated_kernel(a, b, **launch)
    try:
        return launch_generated_kernel(a, b, **launch)
    except Exception as exc:
        raise KernelNotAvailableError(
            f"{kernel.kernel_id} is {kernel.status.value}; native generated dispatch is unavailable: {exc}"
        ) from exc


def _logical_operands(a: Any, b: Any, kernel: KernelMetadata) -> tuple[Any, Any]:
    """Operands as logical ``A[M, K]`` and ``B[K, N]`` integer tensors (packed int4 expanded)."""
    torch = _torch()
    a_stored_t = kernel.layout in (GemmLayout.TN, GemmLayout.TT)  # A stored [Kb, M]
    b_stored_t = kernel.layout in (GemmLayout.NT, GemmLayout.TT)  # B stored [N, Kb]
    if kernel.a_dtype is OperandDType.INT4:
        # nibbles are packed along K, which is the last axis only in the K-major forms
        if a.dtype is torch.uint8:
            a = unpack_int4_k_major(a.transpose(-2, -1)).transpose(-2, -1) if a_stored_t else unpack_int4_k_major(a)
        if b.dtype is torch.uint8:
            b = unpack_int4_k_major(b) if b_stored_t else unpack_int4_k_major(b.transpose(-2, -1)).transpose(-2, -1)
    if a_stored_t:
        a = a.transpose(-2, -1)
    if b_stored_t:
        b = b.transpose(-2, -1)
    return a, b


def reference_mm(
    a: Any,
    b: Any,
    *,
    kernel: KernelMetadata,
    a_scale: Any | None,
    b_scale: Any | None,
    gate: Any | None = None,
) -> Any:
    """PyTorch statement of what ``kernel`` computes: unpack, int32 matmul, fp32 scale, epilogue, cast."""
    torch = _torch()
    a, b = _logical_operands(a, b, kernel)
    out = _scaled_reference_mm(a, b, kernel=kernel, a_scale=a_scale, b_scale=b_scale)
    if kernel.epilogue is Epilogue.SWIGLU:
        if gate is not None:
            raise ValueError("SwiGLU reference uses fused up/gate columns; external gate is not supported")
        if out.shape[-1] % 2:
            raise ValueError("fused SwiGLU reference requires an even output dimension")
        up, gate_values = out.split(out.shape[-1] // 2, dim=-1)
        out = up * (gate_values / (1.0 + torch.exp(-gate_values)))
    elif kernel.epilogue is Epilogue.RELU2:
        out = torch.relu(out).square()
    if kernel.output_dtype == "bfloat16":
        return out.to(torch.bfloat16)
    if kernel.output_dtype == "float32":
        return out
    raise ValueError(f"unsupported kernel output dtype: {kernel.output_dtype}")


def _scaled_reference_mm(a: Any, b: Any, *, kernel: KernelMetadata, a_scale: Any | None, b_scale: Any | None) -> Any:
    """fp32 result before the epilogue.  Per-channel: ``(acc * sa) * sb``.  Subchannel: K-groups in
    ascending order, each ``(acc_g * sa_g) * sb_g`` added to a zero-initialised fp32 sum."""
    torch = _torch()
    a_int = a.to(torch.int32)
    b_int = b.to(torch.int32)
    sa = None if a_scale is None else a_scale.to(torch.float32)
    sb = None if b_scale is None else b_scale.to(torch.float32)
    if kernel.scale.mode is ScaleMode.PER_CHANNEL:
        out = torch.matmul(a_int, b_int).to(torch.float32)
        if sa is not None:
            out = out * sa[..., :, None]
        if sb is not None:
            out = out * sb[..., None, :]
        return out
    group = kernel.scale.subchannel_size
    if group is None:
        raise ValueError("subchannel scale mode requires subchannel_size")
    k = int(a_int.shape[-1])
    out = torch.zeros((*a_int.shape[:-1], b_int.shape[-1]), device=a_int.device, dtype=torch.float32)
    for index, start in enumerate(range(0, k, group)):
        stop = min(start + group, k)
        part = torch.matmul(a_int[..., start:stop], b_int[..., start:stop, :]).to(torch.float32)
        if sa is not None:
            part = part * sa[..., :, index, None]
        if sb is not None:
            part = part * sb[..., index, :][..., None, :]
        out += part
    return out
