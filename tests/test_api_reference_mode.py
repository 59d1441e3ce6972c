"""Dense API on CPU: shape derivation, scale validation, error types, and ``use_reference=True``
against the oracle and the reference fixtures.  Modelled on the reference's tests/test_api_shapes.py
and tests/test_quant.py:136-158."""
import numpy as np
import pytest
import torch

from helpers import as_f32, bits_to_bf16, dense_case, oracle_dense, scale_spec

LAYOUTS = ("nn", "nt", "tn")


def _layout(pkg, name):
    return getattr(pkg.GemmLayout, name.upper())


@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("sub", [0, 32, 256])
@pytest.mark.parametrize("epilogue", ["none", "relu2", "swiglu"])
def test_reference_mode_matches_oracle_on_non_tile_shapes(pkg, dtype, layout, sub, epilogue):
    m, n, k = 17, 24, 66
    case = dense_case(pkg, m=m, n=n, k=k, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, seed=11)
    kwargs = dict(
        a_scale=case["a_scale"], b_scale=case["b_scale"], dtype=pkg.OperandDType(dtype),
        layout=_layout(pkg, layout), scale=scale_spec(pkg, sub), use_reference=True,
    )
    if epilogue == "swiglu":
        out = pkg.fused_swiglu_up_gate(case["a"], case["b"], **kwargs)
    else:
        out = pkg.mm(case["a"], case["b"], epilogue=pkg.Epilogue(epilogue), **kwargs)
    assert out.dtype is torch.bfloat16 and tuple(out.shape) == (m, n)
    want = oracle_dense(case, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue)
    if epilogue == "swiglu":
        np.testing.assert_allclose(as_f32(out), want, rtol=2.0 ** -7, atol=0)
    else:
        np.testing.assert_array_equal(as_f32(out), want)


def test_reference_mode_matches_reference_fixtures(pkg, golden):
    for key in (str(n) for n in golden["dense/names"]):
        dtype, layout, scale, epilogue = key.split("/")[1].split("_")
        sub = 0 if scale == "pc" else int(scale[2:])
        kernel = pkg.default_registry.select_reference(
            dtype=pkg.OperandDType(dtype), layout=_layout(pkg, layout), scale=scale_spec(pkg, sub), epilogue=pkg.Epilogue(epilogue)
        )
        out = pkg.explicit_mm(
            torch.from_numpy(golden[f"{key}/a"]), torch.from_numpy(golden[f"{key}/b"]), kernel=kernel,
            a_scale=bits_to_bf16(golden[f"{key}/a_scale_bits"]), b_scale=bits_to_bf16(golden[f"{key}/b_scale_bits"]),
            use_reference=True,
        )
        assert torch.equal(out, bits_to_bf16(golden[f"{key}/out_bits"])), key


def test_integer_matmul_known_answer(pkg):
    a = torch.tensor([[1, -2, 3, -4], [5, 6, -7, 0]], dtype=torch.int8)
    b = torch.tensor([[1, 2], [-3, 4], [5, -6], [7, 0]], dtype=torch.int8)
    ap = pkg.pack_int4_k_major(a)
    bp = pkg.pack_int4_k_major(b.t()).t().contiguous()
    out = pkg.mm(ap, bp, use_reference=True)
    assert out.tolist() == [[-6.0, -24.0], [-48.0, 76.0]]


def test_swiglu_goes_through_its_own_entry_point(pkg):
    a = torch.zeros((16, 16), dtype=torch.uint8)
    b = torch.zeros((16, 64), dtype=torch.uint8)
    with pytest.raises(ValueError, match="fused_swiglu_up_gate"):
        pkg.mm(a, b, epilogue=pkg.Epilogue.SWIGLU, use_reference=True)
    with pytest.raises(ValueError, match="to be even"):
        pkg.fused_swiglu_up_gate(a, torch.zeros((16, 63), dtype=torch.uint8), use_reference=True)
    kernel = pkg.default_registry.select_reference(
        dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.SWIGLU
    )
    with pytest.raises(ValueError, match="pass gate through b_up_gate"):
        pkg.explicit_mm(a, b, kernel=kernel, gate=torch.zeros(1), use_reference=True)


def test_k_mismatch_and_layout_rejection(pkg):
    a = torch.zeros((16, 16), dtype=torch.uint8)
    with pytest.raises(ValueError, match="logical K mismatch for layout=nn: A has 32, B has 24"):
        pkg.mm(a, torch.zeros((12, 64), dtype=torch.uint8), use_reference=True)
    with pytest.raises(ValueError, match="unsupported GEMM layout tt"):
        pkg.mm(a, torch.zeros((64, 16), dtype=torch.uint8), layout=pkg.GemmLayout.TT, use_reference=True)


def test_scale_shape_validation(pkg):
    a = torch.zeros((16, 32), dtype=torch.uint8)  # K = 64
    b = torch.zeros((32, 48), dtype=torch.uint8)
    ones = lambda *s: torch.ones(s, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match=r"a_scale must have shape \(16,\)"):
        pkg.mm(a, b, a_scale=ones(15), b_scale=ones(48), use_reference=True)
    with pytest.raises(ValueError, match=r"b_scale must have shape \(48,\)"):
        pkg.mm(a, b, a_scale=ones(16), b_scale=ones(47), use_reference=True)
    sc = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 32)
    with pytest.raises(ValueError, match=r"a_scale must have shape \(16, 2\)"):
        pkg.mm(a, b, a_scale=ones(16), b_scale=ones(2, 48), scale=sc, use_reference=True)
    with pytest.raises(ValueError, match="weight-matched layout"):
        pkg.mm(a, b, a_scale=ones(16, 2), b_scale=ones(48, 2), scale=sc, use_reference=True)
    out = pkg.mm(a, b, a_scale=ones(16, 2), b_scale=pkg.pack_rhs_subchannel_scales(ones(48, 2)), scale=sc, use_reference=True)
    assert tuple(out.shape) == (16, 48)


def test_native_dispatch_is_strict_without_a_gpu(pkg, native_lib):
    """No silent fallback: CPU tensors, or a shape no entry accepts, raise."""
    a = torch.zeros((128, 32), dtype=torch.uint8)
    b = torch.zeros((32, 256), dtype=torch.uint8)
    ones = lambda *s: torch.ones(s, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        pkg.mm(a, b, a_scale=ones(128), b_scale=ones(256))
    with pytest.raises(LookupError, match=r"no kernel for dtype=int4, scale=pc, epilogue=none, layout=nn, schedule=standard, shape=\(17, 256, 64\)"):
        pkg.mm(torch.zeros((17, 32), dtype=torch.uint8), b, a_scale=ones(17), b_scale=ones(256))


def test_split_k_reference_output_is_float32(pkg):
    case = dense_case(pkg, m=16, n=128, k=256, seed=2)
    kernel = pkg.default_registry.select(
        dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.NONE,
        m=16, n=128, k=256, split_k=4,
    )
    assert kernel.output_dtype == "float32" and kernel.tile.split_k == 4
    out = pkg.explicit_mm(case["a"], case["b"], kernel=kernel, a_scale=case["a_scale"], b_scale=case["b_scale"], use_reference=True)
    assert out.dtype is torch.float32
    np.testing.assert_array_equal(out.numpy(), oracle_dense(case, out_bf16=False))
