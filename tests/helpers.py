"""Helpers shared by the test modules: bf16 bit views and oracle adapters for torch tensors."""
from __future__ import annotations

import numpy as np
import torch

from oracle import reference_math as oracle

LAYOUT_NAMES = {"nn": "NN", "nt": "NT", "tn": "TN", "tt": "TT"}


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def as_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().to(torch.float32).numpy()


def random_scales(shape, generator) -> torch.Tensor:
    return ((torch.rand(shape, generator=generator) + 0.5) * 0.05).to(torch.bfloat16)


def store_operand(codes: torch.Tensor, *, int4: bool, k_last: bool, pack) -> torch.Tensor:
    stored = pack(codes) if int4 else codes
    return stored.contiguous() if k_last else stored.transpose(-2, -1).contiguous()


def dense_case(pkg, *, m, n, k, dtype="int4", layout="nn", sub=0, epilogue="none", seed=0):
    """Seeded dense operands in storage layout plus the oracle's expected output (float32 array)."""
    g = torch.Generator().manual_seed(seed)
    int4 = dtype == "int4"
    lo, hi = (-8, 8) if int4 else (-127, 128)
    cols = 2 * n if epilogue == "swiglu" else n
    a_codes = torch.randint(lo, hi, (m, k), generator=g, dtype=torch.int8)
    b_codes_t = torch.randint(lo, hi, (cols, k), generator=g, dtype=torch.int8)
    a = store_operand(a_codes, int4=int4, k_last=layout in ("nn", "nt"), pack=pkg.pack_int4_k_major)
    b = store_operand(b_codes_t, int4=int4, k_last=layout in ("nt", "tt"), pack=pkg.pack_int4_k_major)
    if sub == 0:
        sa, sb = random_scales((m,), g), random_scales((cols,), g)
    else:
        groups = -(-k // sub)
        sa, sb = random_scales((m, groups), g), random_scales((groups, cols), g)
    return {"a": a, "b": b, "a_scale": sa, "b_scale": sb, "a_codes": a_codes, "b_codes": b_codes_t.t().contiguous()}


def oracle_dense(case, *, dtype="int4", layout="nn", sub=0, epilogue="none", out_bf16=True) -> np.ndarray:
    return oracle.reference_mm(
        case["a"].numpy(), case["b"].numpy(), int4=dtype == "int4", layout=layout,
        a_scale_bits=bf16_bits(case["a_scale"]), b_scale_bits=bf16_bits(case["b_scale"]),
        subchannel=sub, epilogue=epilogue, out_bf16=out_bf16,
    )


def scale_spec(pkg, sub):
    return pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, sub) if sub else pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)


def assert_close_rms(got: np.ndarray, want: np.ndarray, *, rtol=1e-2, atol_rms=1e-2, what=""):
    """|got - want| <= atol_rms * RMS(want) + rtol * |want| elementwise (the bf16 output bar)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    bound = atol_rms * rms + rtol * np.abs(want)
    bad = np.abs(got - want) > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} elements outside tolerance; worst {np.abs(got - want).max()}"
