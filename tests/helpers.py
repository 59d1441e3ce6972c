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


# ----------------------------------------------------------------------------------------------
# GPU side: calls through the C ABI (ctypes) with arbitrary shapes
# ----------------------------------------------------------------------------------------------
def abi_dense(pkg, case, *, m, n, k, dtype="int4", layout="nn", sub=0, epilogue="none", out="bf16", path=0, schedule="persistent", cta_group=0,
              order="reference", a_operand=0, tail=None, wide=None):
    """One dense launch through ``b200_int4_gemms_launch_dense``; returns the CUDA output tensor.  ``order``: the
    subchannel accumulation order, "reference" (every rounding of the reference math: what the bit-equality checks
    use) or "fused" (the library's default)."""
    from strix_halo_int4_gemms_b200 import native

    out_dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "s32": torch.int32}[out]
    code = {"bf16": native.OUT_BF16, "f32": native.OUT_F32, "s32": native.OUT_S32}[out]
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    c = torch.empty((m, n), device="cuda", dtype=out_dtype)
    c.fill_(-77 if out == "s32" else float("nan"))
    variant = native.make_variant(
        dtype=pkg.OperandDType(dtype), layout=getattr(pkg.GemmLayout, layout.upper()), scale=scale_spec(pkg, sub),
        epilogue=pkg.Epilogue(epilogue), out_dtype=code, path=path,
        # "persistent": the library's persistent grid with the CTA form given by cta_group (0 = its own choice);
        # "tile_per_cta": one CTA per output tile
        schedule=pkg.KernelSchedule.TILE_PER_CTA if schedule == "tile_per_cta" else pkg.KernelSchedule.STANDARD,
        cta_group=cta_group,
        accumulate_order=native.ACCUMULATE_REFERENCE if order == "reference" else native.ACCUMULATE_FUSED,
        a_operand=a_operand,
        tail_balance=native.TAIL_OFF if tail is False else (native.TAIL_ALWAYS if tail is True else native.TAIL_AUTO),
        wide_tiles=native.WIDE_OFF if wide is False else (native.WIDE_ON if wide is True else native.WIDE_AUTO),
    )
    stream = torch.cuda.current_stream().cuda_stream
    # tail=True / False: hand the launch the workspace the balanced tail needs and ask for it wherever it applies
    # (False switches it off in the variant);
    # None: no workspace, as a caller that does not know about it would launch
    workspace = native.dense_workspace(variant, m=m, n=n, k=k, device=c.device, stream_handle=stream) if tail is not None else (0, 0)
    native.launch_dense(
        variant, device_index=0, stream_handle=stream,
        a_ptr=dev["a"].data_ptr(), b_ptr=dev["b"].data_ptr(), a_scale_ptr=dev["a_scale"].data_ptr(),
        b_scale_ptr=dev["b_scale"].data_ptr(), c_ptr=c.data_ptr(), m=m, n=n, k=k,
        workspace_ptr=workspace[0], workspace_bytes=workspace[1],
    )
    torch.cuda.synchronize()
    status, detail = native.device_status(0)
    assert status == 0, f"device status {status} {detail}"
    return c


def check_dense(pkg, *, m, n, k, dtype="int4", layout="nn", sub=0, epilogue="none", out="bf16", path=0, seed=0, exact=None, schedule="persistent", cta_group=0,
                order="reference"):
    """Run one dense case on the GPU and compare with the oracle.  ``exact`` defaults to bit
    equality for everything except SwiGLU (whose exp() is implementation-defined to an ulp) and
    the fused subchannel accumulation order (one rounding fewer per K-group than the reference)."""
    case = dense_case(pkg, m=m, n=n, k=k, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, seed=seed)
    got = abi_dense(pkg, case, m=m, n=n, k=k, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, out=out, path=path, schedule=schedule,
                    cta_group=cta_group, order=order)
    if exact is None and order == "fused" and sub:
        exact = False
    if out == "s32":
        want = oracle.int32_accumulators(case["a"].numpy(), case["b"].numpy(), int4=dtype == "int4", layout=layout)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        return
    want = oracle_dense(case, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, out_bf16=out == "bf16")
    got = as_f32(got)
    assert not np.isnan(got).any()
    assert_close_rms(got, want, what=f"{dtype} {layout} sub={sub} {epilogue} {m}x{n}x{k}")
    if exact is None:
        exact = epilogue != "swiglu"
    if exact:
        np.testing.assert_array_equal(got, want)
