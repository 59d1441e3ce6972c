"""Dense GEMM parity on a B200: CUDA path (through the C ABI) against the oracle on the same seeded inputs.

Bar: int32 accumulators and packing bit-exact; bf16 / fp32 outputs within rtol 1e-2 and
atol 1e-2 x RMS of the reference output (and in fact bit-equal wherever the arithmetic is
fully specified: everything except the SwiGLU's exp)."""
import numpy as np
import pytest
import torch

from helpers import abi_dense, as_f32, assert_close_rms, bits_to_bf16, check_dense, dense_case, oracle_dense, scale_spec
from oracle import reference_math as oracle

pytestmark = pytest.mark.gpu
TCGEN05, SIMT = 1, 2


@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 512, 512), (384, 768, 1024), (128, 1024, 64)])
def test_accumulators_bit_exact(pkg, dtype, shape):
    m, n, k = shape
    check_dense(pkg, m=m, n=n, k=k, dtype=dtype, out="s32", path=TCGEN05)


def test_accumulator_headroom_extreme_values(pkg):
    """All operands at -8 (int4) / -127..127 extremes: the 16x nibble encoding must not overflow."""
    m, n, k = 128, 256, 8192
    a = torch.full((m, k), -8, dtype=torch.int8)
    b = torch.full((k, n), -8, dtype=torch.int8)
    b[:, ::2] = 7
    case = {"a": pkg.pack_int4_k_major(a), "b": pkg.pack_int4_k_major(b.t()).t().contiguous(),
            "a_scale": torch.ones(m, dtype=torch.bfloat16), "b_scale": torch.ones(n, dtype=torch.bfloat16)}
    got = abi_dense(pkg, case, m=m, n=n, k=k, out="s32", path=TCGEN05).cpu()
    assert got[:, 1::2].unique().tolist() == [64 * k] and got[:, ::2].unique().tolist() == [-56 * k]


@pytest.mark.parametrize("cta_group", [0, 1])   # the library's choice (CTA pairs where they exist), and single CTAs
@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("epilogue", ["none", "relu2", "swiglu"])
@pytest.mark.parametrize("sub", [0, 32, 64, 128, 256])
def test_scale_modes_and_epilogues(pkg, dtype, epilogue, sub, cta_group):
    check_dense(pkg, m=256, n=384, k=512, dtype=dtype, sub=sub, epilogue=epilogue, path=TCGEN05, seed=sub + 1,
                cta_group=cta_group)


@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
@pytest.mark.parametrize("dtype", ["int4", "int8"])
def test_layouts(pkg, layout, dtype):
    for cta_group in (0, 1):
        check_dense(pkg, m=256, n=512, k=512, dtype=dtype, layout=layout, seed=3, cta_group=cta_group)
        check_dense(pkg, m=256, n=512, k=512, dtype=dtype, layout=layout, sub=128, epilogue="relu2", seed=4, cta_group=cta_group)


@pytest.mark.parametrize("shape", [(1, 16, 32), (200, 272, 160), (129, 48, 96), (17, 1040, 4128), (513, 2064, 32)])
def test_partial_tiles_on_the_tensor_core_path(pkg, shape):
    m, n, k = shape
    check_dense(pkg, m=m, n=n, k=k, path=TCGEN05)
    check_dense(pkg, m=m, n=n, k=k, path=TCGEN05, cta_group=1)
    check_dense(pkg, m=m, n=n, k=k, out="f32", path=TCGEN05)
    check_dense(pkg, m=m, n=n, k=k, out="f32", path=TCGEN05, cta_group=1)
    check_dense(pkg, m=m, n=n, k=k, sub=32, epilogue="swiglu" if n % 32 == 0 else "relu2", path=TCGEN05)


@pytest.mark.parametrize("shape", [(17, 129, 65), (3, 7, 5), (64, 40, 33)])
def test_unaligned_shapes_take_the_cuda_core_kernel(pkg, shape):
    """Pitches that are not multiples of 16 bytes cannot be described to TMA; AUTO falls to the plain kernel."""
    m, n, k = shape
    for dtype in ("int4", "int8"):
        check_dense(pkg, m=m, n=n, k=k, dtype=dtype)
        check_dense(pkg, m=m, n=n, k=k, dtype=dtype, sub=32, epilogue="relu2")
        check_dense(pkg, m=m, n=n, k=k, dtype=dtype, out="s32")
    from strix_halo_int4_gemms_b200 import native

    case = dense_case(pkg, m=17, n=129, k=65)
    with pytest.raises(RuntimeError, match="tcgen05 kernel needs"):
        abi_dense(pkg, case, m=17, n=129, k=65, path=native.PATH_TCGEN05)


def test_both_kernels_agree_bit_for_bit(pkg):
    for sub, epilogue in ((0, "none"), (64, "relu2")):
        case = dense_case(pkg, m=192, n=320, k=384, sub=sub, epilogue=epilogue, seed=8)
        tc = abi_dense(pkg, case, m=192, n=320, k=384, sub=sub, epilogue=epilogue, path=TCGEN05)
        simt = abi_dense(pkg, case, m=192, n=320, k=384, sub=sub, epilogue=epilogue, path=SIMT)
        assert torch.equal(tc, simt)


def test_standard_and_persistent_schedules_agree(pkg):
    case = dense_case(pkg, m=2048, n=2048, k=256, seed=9)
    a = abi_dense(pkg, case, m=2048, n=2048, k=256, schedule="standard")
    b = abi_dense(pkg, case, m=2048, n=2048, k=256, schedule="persistent")
    assert torch.equal(a, b)


SINGLE, PAIR = 1, 2  # b200_gemm_variant.cta_group


@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("shape", [(256, 256, 128), (512, 768, 1024), (390, 528, 416)])
def test_cta_pair_accumulators_bit_exact(pkg, dtype, shape):
    """256-row tiles over two SMs (tcgen05 cta_group::2), incl. an M whose last pair is half empty."""
    m, n, k = shape
    check_dense(pkg, m=m, n=n, k=k, dtype=dtype, out="s32", path=TCGEN05, cta_group=PAIR)


@pytest.mark.parametrize("dtype,layout,sub,epilogue,out", [
    ("int4", "nn", 0, "none", "bf16"), ("int4", "nn", 0, "relu2", "bf16"), ("int4", "nn", 0, "swiglu", "bf16"),
    ("int4", "nn", 0, "none", "f32"), ("int4", "nn", 256, "none", "bf16"), ("int4", "nn", 128, "swiglu", "bf16"),
    ("int4", "nt", 0, "none", "bf16"), ("int8", "nn", 0, "none", "bf16"), ("int8", "nn", 0, "relu2", "bf16"),
    ("int8", "nn", 0, "swiglu", "bf16"), ("int8", "nn", 256, "none", "bf16"), ("int8", "nn", 128, "relu2", "bf16"),
    ("int8", "nn", 256, "swiglu", "bf16"), ("int8", "nt", 0, "none", "bf16"), ("int8", "nt", 0, "relu2", "bf16"),
    ("int4", "nn", 256, "relu2", "bf16"), ("int4", "tn", 0, "none", "bf16"),
])
def test_cta_pair_kernels_match_the_oracle(pkg, dtype, layout, sub, epilogue, out):
    check_dense(pkg, m=640, n=384, k=1024, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, out=out,
                path=TCGEN05, cta_group=PAIR, seed=21)
    edge_m = 208 if layout == "tn" else 200   # A [K/2, M]: TMA needs the pitch M to be a multiple of 16 bytes
    check_dense(pkg, m=edge_m, n=272, k=160, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, out=out,
                path=TCGEN05, cta_group=PAIR, seed=22)


def test_cta_pair_and_single_agree_bit_for_bit(pkg):
    """Many tiles per cluster (persistent loop, both accumulator buffers, all pipeline phases)."""
    for dtype, sub, epilogue in (("int4", 0, "none"), ("int8", 0, "relu2"), ("int4", 256, "swiglu")):
        case = dense_case(pkg, m=2048, n=4608, k=1280, dtype=dtype, sub=sub, epilogue=epilogue, seed=23)
        kw = dict(m=2048, n=4608, k=1280, dtype=dtype, sub=sub, epilogue=epilogue, path=TCGEN05)
        one = abi_dense(pkg, case, cta_group=SINGLE, **kw)
        two = abi_dense(pkg, case, cta_group=PAIR, **kw)
        assert torch.equal(one, two)


@pytest.mark.parametrize("dtype", ["int4", "int8"])
def test_layout_tt_on_the_tensor_core_kernel(pkg, dtype):
    """A [Kb, M] with B [N, Kb]: both operands in the layout the other one usually has."""
    check_dense(pkg, m=384, n=512, k=1024, dtype=dtype, layout="tt", path=TCGEN05, seed=31)
    check_dense(pkg, m=208, n=272, k=160, dtype=dtype, layout="tt", path=TCGEN05, seed=32)
    if dtype == "int4":
        check_dense(pkg, m=256, n=256, k=512, dtype=dtype, layout="tt", sub=128, path=TCGEN05, seed=33)
        check_dense(pkg, m=256, n=256, k=512, dtype=dtype, layout="tt", out="f32", path=TCGEN05, seed=34)


@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("epilogue", ["none", "relu2", "swiglu"])
@pytest.mark.parametrize("sub", [0, 128, 256])
def test_layout_tn_with_every_scale_mode_and_epilogue_on_the_tensor_core_kernel(pkg, dtype, epilogue, sub):
    """A stored [Kb, M]: the registry's TN cells (both dtypes, per-channel and subchannel, all three epilogues) have
    tensor-core kernels; path = TCGEN05 makes a missing one an error instead of a detour over the CUDA cores."""
    check_dense(pkg, m=256, n=384, k=512, dtype=dtype, layout="tn", sub=sub, epilogue=epilogue, path=TCGEN05, seed=61 + sub)
    check_dense(pkg, m=144, n=208, k=384, dtype=dtype, layout="tn", sub=sub, epilogue=epilogue, path=TCGEN05, seed=62 + sub)
    if sub:   # and in the library's default (fused) accumulation order
        check_dense(pkg, m=256, n=384, k=512, dtype=dtype, layout="tn", sub=sub, epilogue=epilogue, path=TCGEN05, seed=63 + sub, order="fused")


def test_cta_pair_falls_back_when_no_paired_kernel_exists(pkg):
    check_dense(pkg, m=256, n=256, k=256, sub=32, path=TCGEN05, cta_group=PAIR)      # K-groups of 32: single-CTA kernel
    check_dense(pkg, m=256, n=256, k=256, layout="tn", path=TCGEN05, cta_group=PAIR)


def test_reference_fixtures_on_the_gpu(pkg, golden):
    """The 54 dense cells the reference package produced on CPU, recomputed by the CUDA path."""
    for key in (str(n) for n in golden["dense/names"]):
        dtype, layout, scale, epilogue = key.split("/")[1].split("_")
        sub = 0 if scale == "pc" else int(scale[2:])
        case = {"a": torch.from_numpy(golden[f"{key}/a"]), "b": torch.from_numpy(golden[f"{key}/b"]),
                "a_scale": bits_to_bf16(golden[f"{key}/a_scale_bits"]), "b_scale": bits_to_bf16(golden[f"{key}/b_scale_bits"])}
        got = abi_dense(pkg, case, m=24, n=32, k=96, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue)
        want = bits_to_bf16(golden[f"{key}/out_bits"])
        if epilogue == "swiglu":
            assert_close_rms(as_f32(got), as_f32(want), what=key)
        else:
            assert torch.equal(got.cpu(), want), key


def test_quickstart_configuration(pkg, golden):
    """BASELINE configuration 1 through the public API: mm() on packed operands with unit scales."""
    a = torch.from_numpy(golden["quickstart/a"]).cuda()
    b = torch.from_numpy(golden["quickstart/b"]).cuda()
    out = pkg.mm(a, b, a_scale=torch.ones(128, dtype=torch.bfloat16, device="cuda"), b_scale=torch.ones(1024, dtype=torch.bfloat16, device="cuda"))
    assert out.dtype is torch.bfloat16 and tuple(out.shape) == (128, 1024)
    assert torch.equal(out.cpu(), bits_to_bf16(golden["quickstart/out_bits"]))


def test_public_api_dispatch(pkg):
    """mm / fused_swiglu_up_gate / explicit_mm / torch_gemm on CUDA tensors against reference mode."""
    case = dense_case(pkg, m=256, n=512, k=256, sub=256, epilogue="swiglu", seed=12)
    dev = {k: v.cuda() for k, v in case.items() if k in ("a", "b", "a_scale", "b_scale")}
    sc = scale_spec(pkg, 256)
    got = pkg.fused_swiglu_up_gate(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], scale=sc)
    want = pkg.fused_swiglu_up_gate(case["a"], case["b"], a_scale=case["a_scale"], b_scale=case["b_scale"], scale=sc, use_reference=True)
    assert_close_rms(as_f32(got), as_f32(want), what="swiglu api")
    case = dense_case(pkg, m=128, n=256, k=512, dtype="int8", epilogue="relu2", seed=13)
    dev = {k: v.cuda() for k, v in case.items() if k in ("a", "b", "a_scale", "b_scale")}
    for schedule in (pkg.KernelSchedule.STANDARD, pkg.KernelSchedule.PERSISTENT):
        got = pkg.mm(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], dtype=pkg.OperandDType.INT8,
                     epilogue=pkg.Epilogue.RELU2, schedule=schedule)
        want = pkg.mm(case["a"], case["b"], a_scale=case["a_scale"], b_scale=case["b_scale"], dtype=pkg.OperandDType.INT8,
                      epilogue=pkg.Epilogue.RELU2, use_reference=True)
        assert torch.equal(got.cpu(), want)
    kernel = pkg.default_registry.select(dtype=pkg.OperandDType.INT8, scale=scale_spec(pkg, 0), epilogue=pkg.Epilogue.NONE, m=128, n=256, k=512, split_k=4)
    got = pkg.explicit_mm(dev["a"], dev["b"], kernel=kernel, a_scale=dev["a_scale"], b_scale=dev["b_scale"])
    assert got.dtype is torch.float32
    np.testing.assert_array_equal(got.cpu().numpy(), oracle_dense(case, dtype="int8", out_bf16=False))
    op_out = pkg.torch_gemm(dev["a"], dev["b"], kernel=kernel, a_scale=dev["a_scale"], b_scale=dev["b_scale"])
    assert torch.equal(op_out, got)
    with pytest.raises(ValueError, match="requires tile-multiple shape"):
        pkg.explicit_mm(dev["a"][:100].contiguous(), dev["b"], kernel=kernel, a_scale=dev["a_scale"][:100].contiguous(), b_scale=dev["b_scale"])
    with pytest.raises(ValueError, match="must have dtype torch.bfloat16"):
        pkg.launch_generated_kernel(dev["a"], dev["b"], kernel=kernel, a_scale=dev["a_scale"].float(), b_scale=dev["b_scale"])
    with pytest.raises(ValueError, match="must be contiguous"):
        pkg.launch_generated_kernel(dev["a"].t(), dev["b"], kernel=kernel, a_scale=dev["a_scale"], b_scale=dev["b_scale"])


@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("epilogue", ["none", "relu2", "swiglu"])
@pytest.mark.parametrize("sub", [32, 64, 128, 256])
@pytest.mark.parametrize("cta_group", [1, 2])
def test_fused_subchannel_order_is_within_the_output_tolerance(pkg, dtype, epilogue, sub, cta_group):
    """The default order of subchannel launches (one fma per K-group for the scaled add) against the oracle: inside
    the bf16 bar, and in fact within a few units in the last place of the fp32 sum."""
    m, n, k = 384, 512, 1280   # five K-groups of 256; a partial pair tile in M
    check_dense(pkg, m=m, n=n, k=k, dtype=dtype, sub=sub, epilogue=epilogue, cta_group=cta_group, order="fused", seed=sub + cta_group)
    if epilogue == "none" and dtype == "int4":
        case = dense_case(pkg, m=m, n=n, k=k, sub=sub, seed=7)
        fused = abi_dense(pkg, case, m=m, n=n, k=k, sub=sub, out="f32", cta_group=cta_group, order="fused").cpu().numpy()
        exact = abi_dense(pkg, case, m=m, n=n, k=k, sub=sub, out="f32", cta_group=cta_group, order="reference").cpu().numpy()
        np.testing.assert_array_equal(exact, oracle_dense(case, sub=sub, out_bf16=False))
        scale = np.abs(exact).max()
        assert np.abs(fused - exact).max() <= 4e-6 * scale          # a handful of fp32 ulps of the largest sum
        np.testing.assert_array_equal(fused, abi_dense(pkg, case, m=m, n=n, k=k, sub=sub, out="f32", cta_group=cta_group, order="fused").cpu().numpy())


def test_fused_order_other_layouts(pkg):
    for layout in ("nt", "tn", "tt"):
        check_dense(pkg, m=256, n=512, k=1024, layout=layout, sub=128, order="fused", seed=3)
    check_dense(pkg, m=256, n=512, k=1024, dtype="int8", layout="nt", sub=256, epilogue="relu2", order="fused", seed=4)


@pytest.mark.parametrize("layout", ["nn", "nt"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 768, 1024), (384, 520 // 8 * 8 + 8, 2176), (1024, 2048, 4096), (4096, 512, 96)])
def test_a_operand_through_tmem_equals_shared_memory_and_the_oracle(pkg, layout, m, n, k):
    """Per-channel int4 CTA pairs can keep the unpacked A operand in TMEM (the library's choice for long reductions);
    b200_gemm_variant.a_operand pins either.  Same integers either way: raw accumulators and scaled outputs must be bit-identical, over more
    K blocks than the seven TMEM stages, partial tiles in M and N, and a K that ends inside a K block."""
    from strix_halo_int4_gemms_b200 import native

    case = dense_case(pkg, m=m, n=n, k=k, layout=layout, seed=m + n + k)
    outs = ("s32", "bf16") if layout == "nn" else ("bf16",)
    for out in outs:
        tmem = abi_dense(pkg, case, m=m, n=n, k=k, layout=layout, out=out, path=TCGEN05, cta_group=PAIR, a_operand=native.A_OPERAND_TMEM)
        smem = abi_dense(pkg, case, m=m, n=n, k=k, layout=layout, out=out, path=TCGEN05, cta_group=PAIR, a_operand=native.A_OPERAND_SMEM)
        assert torch.equal(tmem, smem), out
        if out == "s32":
            np.testing.assert_array_equal(tmem.cpu().numpy(), oracle.int32_accumulators(case["a"].numpy(), case["b"].numpy(), int4=True, layout=layout))
        else:
            np.testing.assert_array_equal(as_f32(tmem), oracle_dense(case, layout=layout))
    if layout == "nn":
        for epilogue in ("relu2", "swiglu"):
            nn = n // 32 * 16 if epilogue == "swiglu" else n      # D a multiple of 16: the gate block starts on a TMA boundary
            ecase = dense_case(pkg, m=m, n=nn, k=k, epilogue=epilogue, seed=k)
            a = abi_dense(pkg, ecase, m=m, n=nn, k=k, epilogue=epilogue, path=TCGEN05, cta_group=PAIR, a_operand=native.A_OPERAND_TMEM)
            b = abi_dense(pkg, ecase, m=m, n=nn, k=k, epilogue=epilogue, path=TCGEN05, cta_group=PAIR, a_operand=native.A_OPERAND_SMEM)
            assert torch.equal(a, b), epilogue


def test_swiglu_with_an_unaligned_gate_offset_leaves_the_tensor_core_path(pkg):
    """D = 264: the gate half of B [Kb, 2D] starts at byte column 264, which no TMA load can start at.  The library
    must notice on the host (a launch would raise an illegal-instruction fault): AUTO takes the CUDA-core kernel,
    forcing the tensor-core path is refused."""
    from strix_halo_int4_gemms_b200 import native

    m, d, k = 128, 264, 256
    case = dense_case(pkg, m=m, n=d, k=k, epilogue="swiglu", seed=2)
    got = abi_dense(pkg, case, m=m, n=d, k=k, epilogue="swiglu")
    assert native.last_launch_path() == native.LAUNCHED_SIMT
    assert_close_rms(as_f32(got), oracle_dense(case, epilogue="swiglu"), what="swiglu D=264")
    with pytest.raises(RuntimeError, match="n a multiple of 16"):
        abi_dense(pkg, case, m=m, n=d, k=k, epilogue="swiglu", path=TCGEN05)


def test_runs_are_deterministic(pkg):
    case = dense_case(pkg, m=512, n=768, k=1024, sub=256, seed=21)
    first = abi_dense(pkg, case, m=512, n=768, k=1024, sub=256, out="f32")
    for _ in range(3):
        assert torch.equal(first, abi_dense(pkg, case, m=512, n=768, k=1024, sub=256, out="f32"))


def test_unpack_kernel_matches_oracle(pkg):
    g = torch.Generator().manual_seed(4)
    for shape in ((64, 2048), (3, 41), (1, 16)):
        packed = torch.randint(0, 256, shape, generator=g, dtype=torch.uint8)
        got = pkg.unpack_int4_on_device(packed.cuda())
        np.testing.assert_array_equal(got.cpu().numpy(), oracle.unpack_int4_k_major(packed.numpy()))


def test_pre_expanded_int8_path_equals_fused_int4_path(pkg):
    """A/B partner of the fused unpack: expand int4 -> int8 once, then the int8 GEMM; same bits out."""
    case = dense_case(pkg, m=256, n=512, k=1024, seed=30)
    fused = abi_dense(pkg, case, m=256, n=512, k=1024)
    a8 = pkg.unpack_int4_on_device(case["a"].cuda())
    b8 = pkg.unpack_int4_on_device(case["b"].t().contiguous().cuda()).t().contiguous()
    expanded = abi_dense(pkg, {"a": a8.cpu(), "b": b8.cpu(), "a_scale": case["a_scale"], "b_scale": case["b_scale"]}, m=256, n=512, k=1024, dtype="int8")
    assert torch.equal(fused, expanded)


def test_autotune_on_device_with_validation(pkg):
    result = pkg.autotune(m=256, n=256, k=256, dtype=pkg.OperandDType.INT4, scale=scale_spec(pkg, 0), epilogue=pkg.Epilogue.RELU2,
                          warmup_ms=1, rep_ms=3, validate=True)
    # the library's choice, one CTA per tile x 2 raster widths, CTA pairs x 2 raster widths, one tile per CTA
    assert len(result.records) == 6 and all(r.success and r.tops > 0 for r in result.records)
    assert {k.schedule for k in result.candidates} == set(pkg.KernelSchedule)
    assert result.best_record.metadata["timing_backend"] == "cuda_events" and result.best_record.metadata["validated"] is True
