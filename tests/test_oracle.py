"""The oracle against (1) the reference tests' known-answer vectors and (2) fixtures produced by
running the reference package.  No GPU, no product code: this pins the checker itself."""
import numpy as np
import pytest

from oracle import reference_math as oracle


def test_pack_unpack_known_vector():
    # reference tests/test_quant.py:34-38
    x = np.array([[-8, -1, 0, 7], [3, -4, 5, -6]], dtype=np.int8)
    packed = oracle.pack_int4_k_major(x)
    assert packed.dtype == np.uint8
    assert packed.tolist() == [[0xF8, 0x70], [0xC3, 0xA5]]
    np.testing.assert_array_equal(oracle.unpack_int4_k_major(packed), x)


def test_pack_pads_odd_k_with_zero():
    # reference tests/test_quant.py:41-45
    packed = oracle.pack_int4_k_major(np.array([[1, -2, 3]], dtype=np.int8))
    np.testing.assert_array_equal(oracle.unpack_int4_k_major(packed), np.array([[1, -2, 3, 0]], dtype=np.int8))


def test_integer_matmul_known_answer():
    # reference tests/test_quant.py:56-76
    a = np.array([[1, -2, 3, -4], [5, 6, -7, 0]], dtype=np.int8)
    b = np.array([[1, 2], [-3, 4], [5, -6], [7, 0]], dtype=np.int8)
    ap = oracle.pack_int4_k_major(a)
    bp = np.ascontiguousarray(oracle.pack_int4_k_major(b.T).T)
    out = oracle.reference_mm(ap, bp, int4=True)
    np.testing.assert_array_equal(out, np.array([[-6, -24], [-48, 76]], dtype=np.float32))
    np.testing.assert_array_equal(oracle.int32_accumulators(ap, bp, int4=True), a.astype(np.int32) @ b.astype(np.int32))


def test_group_info_known_vectors():
    # reference tests/test_ragged_dot.py:120-147
    info = oracle.calculate_group_info([17, 31, 24], 32, align_tile=8)
    assert info["num_tasks"] == 3
    assert info["block_start"].tolist() == [0, 16, 48]
    assert info["actual_start"].tolist() == [0, 17, 48]
    assert info["actual_end"].tolist() == [17, 48, 72]
    assert info["start_within_block"].tolist() == [0, 1, 0]
    assert info["actual_size"].tolist() == [17, 31, 24]
    info = oracle.calculate_group_info([2, 0, 7], 16, tid_size=4, align_tile=8)
    assert info["num_tasks"] == 2
    assert info["group_id"].tolist() == [0, 2, 0, 0]
    assert info["actual_end"].tolist() == [2, 9, 0, 0]
    with pytest.raises(ValueError, match="tid_size must be at least 3"):
        oracle.calculate_group_info([17, 31, 24], 32, tid_size=2, align_tile=8)


def test_tops_known_answer(golden):
    # reference tests/test_benchmarking.py:50-52
    assert oracle.tops_for_runtime(1024, 1024, 1024, 1.0) == pytest.approx(2.147483648)
    assert float(golden["metric/tops_1024_1ms"]) == pytest.approx(2.147483648)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 0.0], dtype=np.float32)
    import torch

    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    np.testing.assert_array_equal(oracle.round_to_bf16(x), want)


@pytest.mark.parametrize("name", ["even", "odd", "batched"])
def test_pack_against_reference_fixture(golden, name):
    x = golden[f"pack/{name}/x"]
    np.testing.assert_array_equal(oracle.pack_int4_k_major(x), golden[f"pack/{name}/packed"])
    np.testing.assert_array_equal(oracle.unpack_int4_k_major(golden[f"pack/{name}/packed"]), golden[f"pack/{name}/unpacked"])


def test_fake_quant_against_reference_fixture(golden):
    x = oracle.bf16_bits_to_f32(golden["fake_quant/x_bits"])
    np.testing.assert_array_equal(oracle.fake_quant_int(x, bits=4, scale=0.1), golden["fake_quant/q4_scale0p1"])
    np.testing.assert_array_equal(oracle.fake_quant_int(x, bits=8, scale=0.01), golden["fake_quant/q8_scale0p01"])


def test_scale_pack_against_reference_fixture(golden):
    np.testing.assert_array_equal(oracle.pack_rhs_subchannel_scales(golden["scale_pack/in_bits"]), golden["scale_pack/out_bits"])


def _dense_names(golden):
    return [str(n) for n in golden["dense/names"]]


def test_dense_against_reference_fixtures(golden):
    """All 54 (dtype, layout, scale, epilogue) cells: bit-equal, except SwiGLU where exp() may differ by an ulp."""
    checked = 0
    for key in _dense_names(golden):
        _, ident = key.split("/")
        dtype, layout, scale, epilogue = ident.split("_")
        sub = 0 if scale == "pc" else int(scale[2:])
        out = oracle.reference_mm(
            golden[f"{key}/a"], golden[f"{key}/b"], int4=dtype == "int4", layout=layout,
            a_scale_bits=golden[f"{key}/a_scale_bits"], b_scale_bits=golden[f"{key}/b_scale_bits"],
            subchannel=sub, epilogue=epilogue,
        )
        want = oracle.bf16_bits_to_f32(golden[f"{key}/out_bits"])
        if epilogue == "swiglu":
            # one bf16 ulp at most, and only where exp() rounds differently
            np.testing.assert_allclose(out, want, rtol=2.0 ** -7, atol=0)
            assert np.mean(out == want) > 0.99
        else:
            np.testing.assert_array_equal(out, want, err_msg=key)
        checked += 1
    assert checked == 54


def test_dense_float32_and_accumulators_against_reference_fixture(golden):
    out = oracle.reference_mm(
        golden["dense_f32/a"], golden["dense_f32/b"], int4=True,
        a_scale_bits=golden["dense_f32/a_scale_bits"], b_scale_bits=golden["dense_f32/b_scale_bits"], out_bf16=False,
    )
    np.testing.assert_array_equal(out, golden["dense_f32/out"])
    np.testing.assert_array_equal(oracle.int32_accumulators(golden["dense_f32/a"], golden["dense_f32/b"], int4=True), golden["dense_f32/acc"])


def test_quickstart_against_reference_fixture(golden):
    """BASELINE configuration 1: M=128, N=1024, K=64, unit scales, through the reference's mm(use_reference=True)."""
    ones = lambda n: np.full((n,), 0x3F80, dtype=np.uint16)
    out = oracle.reference_mm(golden["quickstart/a"], golden["quickstart/b"], int4=True, a_scale_bits=ones(128), b_scale_bits=ones(1024))
    np.testing.assert_array_equal(oracle.f32_to_bf16_bits(out), golden["quickstart/out_bits"])


def test_engines_agree():
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (33, 257), dtype=np.int8)
    b = rng.integers(-127, 128, (257, 19), dtype=np.int8)
    np.testing.assert_array_equal(oracle.exact_int_matmul(a, b), oracle.exact_int_matmul(a, b, engine="torch_int32"))


def test_group_info_against_reference_fixtures(golden):
    for i in range(int(golden["group_info/count"])):
        tile, align, tid, num_tasks = (int(v) for v in golden[f"group_info/{i}/params"])
        info = oracle.calculate_group_info(golden[f"group_info/{i}/sizes"], tile, tid_size=None if tid < 0 else tid, align_tile=align)
        assert info["num_tasks"] == num_tasks
        for field in ("group_id", "block_start", "actual_start", "actual_end", "start_within_block", "actual_size"):
            np.testing.assert_array_equal(info[field], golden[f"group_info/{i}/{field}"], err_msg=f"case {i} {field}")


@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("scale", ["pc", "sc32"])
def test_ragged_fwd_against_reference_fixtures(golden, layout, scale):
    key = f"ragged_fwd/{layout}_{scale}"
    out = oracle.ragged_dot_fwd(
        golden[f"{key}/lhs"], golden[f"{key}/rhs"], golden[f"{key}/group_sizes"],
        golden[f"{key}/a_scale_bits"], golden[f"{key}/b_scale_bits"], layout=layout,
        subchannel=0 if scale == "pc" else 32, out_bf16=False,
    )
    np.testing.assert_array_equal(out, golden[f"{key}/out_f32"])


@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("scale", ["pc", "sc32"])
def test_ragged_bwd_against_reference_fixtures(golden, layout, scale):
    key = f"ragged_bwd/{layout}_{scale}"
    out = oracle.ragged_dot_bwd(
        golden[f"{key}/lhs"], golden[f"{key}/rhs"], golden[f"{key}/group_sizes"],
        golden[f"{key}/a_scale_bits"], golden[f"{key}/b_scale_bits"], layout=layout, subchannel=0 if scale == "pc" else 32,
    )
    np.testing.assert_array_equal(out, golden[f"{key}/out_f32"])
