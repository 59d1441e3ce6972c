"""``torch.library`` custom op around the dense launcher (reference: torch_ops.py:24-87).

``torch.ops.b200_int4_gemms.gemm(a, b, a_scale, b_scale, gate, kernel_id, has_gate)`` with a
fake (meta) implementation, so the GEMM can sit inside traced or compiled graphs.  No autograd.
"""
from __future__ import annotations

from typing import Any

from .metadata import KernelMetadata
from .native import launch_generated_kernel
from .registry import default_registry

TORCH_OP_NAMESPACE = "b200_int4_gemms"
TORCH_GEMM_OP = f"{TORCH_OP_NAMESPACE}::gemm"
_SCHEMA = "(Tensor a, Tensor b, Tensor a_scale, Tensor b_scale, Tensor gate, str kernel_id, bool has_gate) -> Tensor"

_registered = False


def _torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError("torch is required to register b200_int4_gemms custom ops") from exc
    return torch


def register_torch_ops() -> None:
    """Define the op once per process; later calls are no-ops."""
    global _registered
    if _registered:
        return
    torch = _torch()

    @torch.library.custom_op(TORCH_GEMM_OP, mutates_args=(), device_types="cuda", schema=_SCHEMA)
    def gemm(a, b, a_scale, b_scale, gate, kernel_id, has_gate):
        entry = default_registry.get(kernel_id)
        return launch_generated_kernel(
            a, b, kernel=entry, a_scale=a_scale, b_scale=b_scale, gate=gate if has_gate else None
        )

    @gemm.register_fake
    def _(a, b, a_scale, b_scale, gate, kernel_id, has_gate):
        entry = default_registry.get(kernel_id)
        from .native import _logical_problem_shape

        m, n, _k = _logical_problem_shape(entry, a, b)
        out_dtype = torch.bfloat16 if entry.output_dtype == "bfloat16" else torch.float32
        return a.new_empty((m, n), dtype=out_dtype)

    _registered = True


def torch_gemm(
    a: Any,
    b: Any,
    *,
    kernel: KernelMetadata,
    a_scale: Any,
    b_scale: Any,
    gate: Any | None = None,
) -> Any:
    torch = _torch()
    register_torch_ops()
    placeholder = gate if gate is not None else torch.empty((0,), device=a.device, dtype=torch.float32)
    op = getattr(torch.ops, TORCH_OP_NAMESPACE).gemm
    return op(a, b, a_scale, b_scale, placeholder, kernel.kernel_id, gate is not None)
