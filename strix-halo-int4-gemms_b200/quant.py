"""Operand format helpers: int4/int8 fake quantisation, K-major nibble packing, scale re-layout.

Bit-exact with the reference's ``quant.py`` (``fake_quant_int`` :14-29, ``pack_int4_k_major``
:32-38, ``unpack_int4_k_major`` :41-51, ``pack_rhs_subchannel_scales`` :54-65,
``pack_ragged_rhs_subchannel_scales`` :68-73, ``apply_scales`` :76-81).

Packed format: one ``uint8`` holds two signed 4-bit codes that are neighbours along the last
(K) axis; the even index sits in bits 0..3, the odd index in bits 4..7; an odd-length axis is
padded with one zero code.
"""
from __future__ import annotations

from typing import Any


def _torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover - torch is a hard dependency in practice
        raise RuntimeError("torch is required for quantization helpers") from exc
    return torch


def fake_quant_int(x: Any, *, bits: int, scale: float) -> Any:
    """Quantise ``x`` to signed ``bits``-bit codes (int8 storage): clamp(round(x / scale)).

    Rounding is round-half-to-even on the float32 quotient, as ``torch.round`` does.
    """
    torch = _torch()
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if isinstance(scale, bool) or not isinstance(scale, (int, float)):
        raise TypeError("scale must be a positive Python int or float scalar")
    if scale <= 0:
        raise ValueError("scale must be positive")
    top = (1 << (bits - 1)) - 1
    codes = torch.round(x.float() / scale)
    return torch.clamp(codes, -top - 1, top).to(torch.int8)


def pack_int4_k_major(x: Any) -> Any:
    """int8 codes ``[..., K]`` -> uint8 ``[..., ceil(K/2)]``."""
    torch = _torch()
    if x.shape[-1] & 1:
        x = torch.nn.functional.pad(x, (0, 1))
    wide = x.to(torch.int16)
    low = wide[..., 0::2] & 0xF
    high = wide[..., 1::2] & 0xF
    return (low | (high << 4)).to(torch.uint8).contiguous()


def unpack_int4_k_major(x_packed: Any) -> Any:
    """uint8 ``[..., Kb]`` -> int8 codes ``[..., 2*Kb]`` (two's-complement nibbles, -8..7)."""
    torch = _torch()
    nibbles = torch.stack(((x_packed & 0xF), ((x_packed >> 4) & 0xF)), dim=-1).to(torch.int8)
    signed = torch.where(nibbles >= 8, nibbles - 16, nibbles)
    return signed.reshape(*x_packed.shape[:-1], x_packed.shape[-1] * 2).contiguous()


def pack_rhs_subchannel_scales(b_scale: Any) -> Any:
    """``(..., N, K-groups)`` -> ``(..., K-groups, N)`` contiguous, the layout the kernels read."""
    if b_scale.ndim < 2:
        raise ValueError("b_scale must have at least 2 dimensions to pack RHS subchannel scales")
    return b_scale.transpose(-2, -1).contiguous()


def pack_ragged_rhs_subchannel_scales(b_scale: Any) -> Any:
    """Grouped form of :func:`pack_rhs_subchannel_scales`: ``(G, N, S)`` -> ``(G, S, N)``."""
    if b_scale.ndim != 3:
        raise ValueError("ragged b_scale must have shape (G, N, scale_cols)")
    return pack_rhs_subchannel_scales(b_scale)


def apply_scales(result: Any, a_scale: Any | None, b_scale: Any | None) -> Any:
    """``result * a_scale[:, None] * b_scale[None, :]``, skipping scales that are None."""
    if a_scale is not None:
        result = result * a_scale[..., :, None]
    if b_scale is not None:
        result = result * b_scale[..., None, :]
    return result


def quantize_int_cuda(x: Any, *, bits: int, scale: float) -> Any:
    """``fake_quant_int`` (+ ``pack_int4_k_major`` for ``bits=4``) as one CUDA kernel of the native library.

    ``x``: CUDA bfloat16 ``[..., K]``.  Returns packed uint8 ``[..., ceil(K/2)]`` for ``bits=4`` and int8
    codes ``[..., K]`` for ``bits=8``, bit-identical to the host helpers above.
    """
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if isinstance(scale, bool) or not isinstance(scale, (int, float)):
        raise TypeError("scale must be a positive Python int or float scalar")
    if scale <= 0:
        raise ValueError("scale must be positive")
    from .native import quantize_on_device

    return quantize_on_device(x, bits=bits, scale=float(scale))


def repack_int4_tokens(x_packed: Any) -> Any:
    """Packed int4 ``[T, F/2]`` (pairs of features per byte) -> ``[ceil(T/2), F]`` (pairs of tokens per byte).

    The operand format of ``ragged_dot_int4_bwd_flat``; CUDA tensors go through the native kernel,
    host tensors through the equivalent torch expression.
    """
    torch = _torch()
    if getattr(x_packed, "is_cuda", False):
        from .native import repack_tokens_on_device

        return repack_tokens_on_device(x_packed)
    codes = unpack_int4_k_major(x_packed)          # [T, F]
    return pack_int4_k_major(codes.t().contiguous()).t().contiguous()  # pack along tokens, back to [T/2, F]
