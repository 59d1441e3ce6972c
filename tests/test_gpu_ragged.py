"""Grouped int4 dots on a B200 against the oracle: forward (M-ragged) and backward (K-ragged).
Cases follow the reference's tests/test_ragged_dot.py:260-586: empty groups, odd K, groups that start
inside an aligned block, every layout, per-channel and subchannel scales."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from helpers import as_f32, assert_close_rms, bf16_bits, bits_to_bf16, scale_spec
from oracle import reference_math as oracle
from strix_halo_int4_gemms_b200.autotune import make_ragged_bwd_inputs, make_ragged_fwd_inputs

pytestmark = pytest.mark.gpu


def _layout(pkg, name):
    return getattr(pkg.GemmLayout, name.upper())


def _status_clean():
    from strix_halo_int4_gemms_b200 import native

    torch.cuda.synchronize()
    status, detail = native.device_status(0)
    assert status == 0, (status, detail)


def _fwd(pkg, sizes, k, n, *, layout="nn", sub=0, seed=0, config=None, out_dtype=None, **kw):
    data = make_ragged_fwd_inputs(m=sum(sizes), n=n, k=k, group_sizes=sizes, layout=_layout(pkg, layout), scale=scale_spec(pkg, sub), seed=seed)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    out = pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                              scale=scale_spec(pkg, sub), layout=_layout(pkg, layout), config=config or pkg.RaggedDotConfig(),
                              output_dtype=out_dtype, **kw)
    _status_clean()
    want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]),
                                 layout=layout, subchannel=sub, out_bf16=out_dtype is not torch.float32)
    return out, want


@pytest.mark.parametrize("sub", [0, 32, 128])
@pytest.mark.parametrize("sizes", [[17, 0, 31, 24, 300, 5], [128, 128, 128], [1], [0, 0, 513, 0]])
def test_forward_matches_oracle(pkg, sizes, sub):
    out, want = _fwd(pkg, sizes, 256, 512, sub=sub, seed=len(sizes))
    assert out.dtype is torch.bfloat16
    np.testing.assert_array_equal(as_f32(out), want)


def test_forward_column_edge_and_float32_output(pkg):
    out, want = _fwd(pkg, [100, 0, 260, 128, 7], 512, 1408, seed=2)
    np.testing.assert_array_equal(as_f32(out), want)
    out, want = _fwd(pkg, [100, 0, 260, 128, 7], 512, 1408, seed=2, out_dtype=torch.float32)
    assert out.dtype is torch.float32
    np.testing.assert_array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("block_m,align", [(64, 8), (32, 32), (128, 128), (16, 16)])
def test_forward_task_heights(pkg, block_m, align):
    cfg = pkg.RaggedDotConfig(block_m=block_m, align_tile=align)
    out, want = _fwd(pkg, [100, 0, 260, 128, 7, 33], 256, 256, config=cfg, seed=5)
    np.testing.assert_array_equal(as_f32(out), want)


@pytest.mark.parametrize("sub,out_dtype", [(0, None), (0, torch.float32), (128, None), (256, torch.float32)])
def test_forward_256_row_tasks_on_cta_pairs(pkg, sub, out_dtype):
    """Tasks of 256 rows: one 256 x 256 tile per pair of SMs, rank 1 takes rows 128..255 of the block."""
    cfg = pkg.RaggedDotConfig(block_m=256)
    sizes = [300, 0, 256, 7, 129, 512, 1, 255]
    out, want = _fwd(pkg, sizes, 512, 1408, sub=sub, config=cfg, out_dtype=out_dtype, seed=11)
    np.testing.assert_array_equal(as_f32(out), want)


@pytest.mark.parametrize("sub", [0, 128])
def test_forward_nt_layout_on_the_tensor_core_kernel(pkg, sub):
    """rhs stored [G, N, K/2] (K-major B): groups stacked along N, column edge inside the last tile."""
    out, want = _fwd(pkg, [100, 0, 260, 128, 7], 512, 1408, layout="nt", sub=sub, seed=13)
    np.testing.assert_array_equal(as_f32(out), want)
    out, want = _fwd(pkg, [300, 40], 256, 200, layout="nt", sub=sub, seed=14, out_dtype=torch.float32)
    np.testing.assert_array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("layout", ["tn", "tt"])
@pytest.mark.parametrize("sub", [0, 128])
def test_forward_transposed_lhs_on_the_tensor_core_kernel(pkg, layout, sub):
    """lhs stored [K/2, M]: the task's first row is a TMA x coordinate, so the tensor cores take it when the tasks
    were built with an ``align_tile`` that is a multiple of 16; with the default of 8 the CUDA-core kernel runs
    (and says so).  Both must equal the oracle bit for bit."""
    import warnings
    from strix_halo_int4_gemms_b200 import native

    sizes = [100, 0, 260, 128, 7, 33]           # 528 rows: a multiple of 16, as the packed pitch of [K/2, M] needs
    aligned = pkg.RaggedDotConfig(block_m=128, align_tile=16, pair_tasks=False)
    out, want = _fwd(pkg, sizes, 512, 1408, layout=layout, sub=sub, config=aligned, seed=21)
    assert native.last_launch_path() == native.LAUNCHED_TCGEN05
    np.testing.assert_array_equal(as_f32(out), want)
    out32, want32 = _fwd(pkg, sizes, 512, 208, layout=layout, sub=sub, config=pkg.RaggedDotConfig(block_m=64, align_tile=32, pair_tasks=False),
                         seed=22, out_dtype=torch.float32)
    if sub == 0:    # an fp32 result exists on the tensor cores for per-channel scales; subchannel fp32 goes to the CUDA cores
        assert native.last_launch_path() == native.LAUNCHED_TCGEN05
    np.testing.assert_array_equal(out32.cpu().numpy(), want32)
    default, _ = _fwd(pkg, sizes, 512, 1408, layout=layout, sub=sub, seed=21)      # the default config is cut to suit
    assert native.last_launch_path() == native.LAUNCHED_TCGEN05
    assert torch.equal(default, out)
    info8 = pkg.calculate_group_info(torch.tensor(sizes).cuda(), 128, align_tile=8)   # prebuilt tasks that start anywhere
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        loose, _ = _fwd(pkg, sizes, 512, 1408, layout=layout, sub=sub, seed=21, group_info=info8)
    assert native.last_launch_path() == native.LAUNCHED_SIMT
    assert torch.equal(loose, out)


def test_forward_transposed_lhs_with_a_broken_alignment_promise_is_reported_not_run(pkg):
    """Tasks built with align_tile = 8 but declared as 16: the kernel skips the tasks whose first row is not a
    multiple of 16 and reports them; nothing faults, and the context stays usable."""
    from strix_halo_int4_gemms_b200 import native

    sizes = [104, 24]                            # group 1 starts on row 104: a multiple of 8, not of 16
    data = make_ragged_fwd_inputs(m=128, n=256, k=256, group_sizes=sizes, layout=pkg.GemmLayout.TN, scale=scale_spec(pkg, 0), seed=3)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    info = pkg.calculate_group_info(dev["group_sizes"], 128, align_tile=8)
    lying = replace(info, align_tile=16)
    out = torch.full((128, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    native.launch_ragged_fwd_kernel(dev["lhs"], dev["rhs"], group_info=lying, a_scale=dev["a_scale"], b_scale=dev["b_scale"], out=out,
                                    scale=scale_spec(pkg, 0), config=pkg.RaggedDotConfig(), layout=pkg.GemmLayout.TN, rows=128, cols=256,
                                    k_packed=128, scale_cols=1, path=native.PATH_TCGEN05)
    torch.cuda.synchronize()
    status, detail = native.device_status(0)
    assert status == 4 and detail[0] == 1, (status, detail)       # task 1 (group 1, block start 104)
    native.reset_device_status(0)
    want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]), layout="tn")
    np.testing.assert_array_equal(as_f32(out[:104]), want[:104])  # the well-formed task ran
    assert bool((out[104:] == 7.0).all())                         # the other one wrote nothing
    again, want2 = _fwd(pkg, sizes, 256, 256, layout="tn", seed=3)
    np.testing.assert_array_equal(as_f32(again), want2)


def test_forward_widens_tasks_for_large_groups(pkg):
    """Default config: groups averaging >= 256 rows are cut into 256-row tasks; the result is the same
    as with 128-row tasks pinned."""
    sizes = [512, 300, 700, 256]
    auto, want = _fwd(pkg, sizes, 1024, 768, seed=12)
    pinned, _ = _fwd(pkg, sizes, 1024, 768, seed=12, config=pkg.RaggedDotConfig(pair_tasks=False))
    np.testing.assert_array_equal(as_f32(auto), want)
    assert torch.equal(auto, pinned)
    with pytest.raises(ValueError, match="more than 128 rows"):
        _fwd(pkg, sizes, 1024, 768, sub=32, config=pkg.RaggedDotConfig(block_m=256), seed=12)


@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("sub", [0, 32])
def test_forward_layouts_and_odd_k(pkg, layout, sub):
    """K = 78 (39 packed bytes): not describable to TMA, so this goes through the CUDA-core kernel."""
    out, want = _fwd(pkg, [17, 0, 31, 24], 78, 48, layout=layout, sub=sub, seed=6)
    np.testing.assert_array_equal(as_f32(out), want)
    out, want = _fwd(pkg, [17, 0, 31, 24], 256, 64, layout=layout, sub=sub, seed=7)
    np.testing.assert_array_equal(as_f32(out), want)


def test_forward_reference_fixtures(pkg, golden):
    for layout in ("nn", "nt", "tn", "tt"):
        for scale, sub in (("pc", 0), ("sc32", 32)):
            key = f"ragged_fwd/{layout}_{scale}"
            out = pkg.ragged_dot_int4(
                torch.from_numpy(golden[f"{key}/lhs"]).cuda(), torch.from_numpy(golden[f"{key}/rhs"]).cuda(),
                torch.from_numpy(golden[f"{key}/group_sizes"]).cuda(), a_scale=bits_to_bf16(golden[f"{key}/a_scale_bits"]).cuda(),
                b_scale=bits_to_bf16(golden[f"{key}/b_scale_bits"]).cuda(), scale=scale_spec(pkg, sub), layout=_layout(pkg, layout),
                output_dtype=torch.float32,
            )
            np.testing.assert_array_equal(out.cpu().numpy(), golden[f"{key}/out_f32"], err_msg=key)


def test_forward_untouched_rows_prebuilt_tasks_and_missing_scales(pkg):
    sizes = [40, 0, 24]
    data = make_ragged_fwd_inputs(m=64, n=256, k=128, group_sizes=sizes, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0), seed=8)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    info = pkg.calculate_group_info(dev["group_sizes"], 128)
    out = torch.full((64, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    got = pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], out=out, group_info=info)
    assert got is out
    want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]))
    np.testing.assert_array_equal(as_f32(out), want)
    unscaled = pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], output_dtype=torch.float32)
    ones_a = bf16_bits(torch.ones(64, dtype=torch.bfloat16))
    ones_b = bf16_bits(torch.ones((3, 256), dtype=torch.bfloat16))
    np.testing.assert_array_equal(unscaled.cpu().numpy(), oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, ones_a, ones_b, out_bf16=False))
    with pytest.raises(ValueError, match="requires a_scale and b_scale"):
        pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], use_native=True)
    with pytest.raises(ValueError, match="JIT path"):
        pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], use_native=False)
    with pytest.raises(ValueError, match=r"sum\(group_sizes\) must equal lhs rows 64; got 63"):
        pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], torch.tensor([40, 0, 23]).cuda(), a_scale=dev["a_scale"], b_scale=dev["b_scale"])
    empty = pkg.ragged_dot_int4(dev["lhs"][:0], dev["rhs"], torch.zeros(3, dtype=torch.int64).cuda(), a_scale=dev["a_scale"][:0], b_scale=dev["b_scale"])
    assert tuple(empty.shape) == (0, 256)


def _bwd(pkg, sizes, m, n, *, layout="tn", sub=0, seed=0, k_capacity=None, config=None):
    cap = max(max(sizes), 2) if k_capacity is None else k_capacity
    data = make_ragged_bwd_inputs(m=m, n=n, k_capacity=cap, group_sizes=sizes, layout=_layout(pkg, layout), scale=scale_spec(pkg, sub), seed=seed)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    out = pkg.ragged_dot_int4_bwd(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                                  scale=scale_spec(pkg, sub), layout=_layout(pkg, layout), config=config or pkg.RaggedBwdDotConfig())
    _status_clean()
    want = oracle.ragged_dot_bwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]),
                                 layout=layout, subchannel=sub)
    return out, want


@pytest.mark.parametrize("layout", ["tn", "nn", "nt", "tt"])
def test_backward_on_cta_pairs_and_on_single_ctas(pkg, layout):
    """M = 512 is two 256-row pair tiles per group; the per-channel backward kernels exist in both forms and
    RaggedBwdDotConfig.pair_tiles pins either: both must reproduce the oracle."""
    from strix_halo_int4_gemms_b200 import native

    sizes = [17, 0, 300, 128, 255, 512, 1]
    for forced, path in ((True, native.LAUNCHED_TCGEN05_PAIR), (False, native.LAUNCHED_TCGEN05), (None, native.LAUNCHED_TCGEN05_PAIR)):
        out, want = _bwd(pkg, sizes, 512, 1408, layout=layout, k_capacity=512, seed=41, config=pkg.RaggedBwdDotConfig(pair_tiles=forced))
        assert native.last_launch_path() == path
        np.testing.assert_array_equal(out.cpu().numpy(), want, err_msg=f"pair_tiles {forced}")


@pytest.mark.parametrize("layout", ["tn", "nn", "nt", "tt"])
@pytest.mark.parametrize("sub", [0, 32, 128])
def test_backward_matches_oracle(pkg, layout, sub):
    # capacity 512 keeps every operand pitch a multiple of 16 bytes: tensor-core path for nn / tn
    out, want = _bwd(pkg, [17, 0, 300, 128, 255, 512], 256, 512, layout=layout, sub=sub, k_capacity=512, seed=3)
    assert out.dtype is torch.float32 and tuple(out.shape) == (6, 256, 512)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    assert float(out[1].abs().max()) == 0.0  # the empty group


@pytest.mark.parametrize("layout", ["nt", "tt"])
def test_backward_with_a_k_major_rhs_masks_bytes_past_the_group(pkg, layout):
    """rhs stored [G, N, K/2]: the tensor-core kernel zeroes the bytes of a 16-byte piece that lie past the group's
    length.  Lengths on every residue of 32 around a piece's end, odd lengths, a group of one token, N with a column
    edge; the tail of the capacity holds random data that must not leak in."""
    from strix_halo_int4_gemms_b200 import native

    sizes = [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 0, 256]
    for sub in (0, 32, 128):
        out, want = _bwd(pkg, sizes, 256, 200, layout=layout, sub=sub, k_capacity=256, seed=51 + sub)
        assert native.last_launch_path() in (native.LAUNCHED_TCGEN05, native.LAUNCHED_TCGEN05_PAIR), sub
        np.testing.assert_array_equal(out.cpu().numpy(), want, err_msg=f"K-groups of {sub}")


def test_backward_odd_lengths_and_column_edge(pkg):
    out, want = _bwd(pkg, [37, 0, 64, 5], 24, 40, layout="nn", seed=4, k_capacity=64)   # CUDA-core kernel
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    out, want = _bwd(pkg, [64, 0, 513, 1], 2048, 1408, layout="tn", seed=5, k_capacity=544)
    np.testing.assert_array_equal(out.cpu().numpy(), want)


def test_backward_reference_fixtures(pkg, golden):
    for layout in ("nn", "nt", "tn", "tt"):
        for scale, sub in (("pc", 0), ("sc32", 32)):
            key = f"ragged_bwd/{layout}_{scale}"
            out = pkg.ragged_dot_int4_bwd(
                torch.from_numpy(golden[f"{key}/lhs"]).cuda(), torch.from_numpy(golden[f"{key}/rhs"]).cuda(),
                torch.from_numpy(golden[f"{key}/group_sizes"]).cuda(), a_scale=bits_to_bf16(golden[f"{key}/a_scale_bits"]).cuda(),
                b_scale=bits_to_bf16(golden[f"{key}/b_scale_bits"]).cuda(), scale=scale_spec(pkg, sub), layout=_layout(pkg, layout),
            )
            np.testing.assert_array_equal(out.cpu().numpy(), golden[f"{key}/out_f32"], err_msg=key)


def test_backward_is_deterministic_and_split_k_is_a_no_op(pkg):
    first, want = _bwd(pkg, [256, 100, 0, 384], 256, 256, k_capacity=384, seed=6)
    for split in (1, 2, 4):
        again, _ = _bwd(pkg, [256, 100, 0, 384], 256, 256, k_capacity=384, seed=6, config=pkg.RaggedBwdDotConfig(split_k=split))
        assert torch.equal(first, again)
    with pytest.raises(ValueError, match="group_sizes entries must be <= logical padded K 64; got 65"):
        lhs = torch.zeros((2, 16, 32), dtype=torch.uint8, device="cuda")   # [G, M, K/2], K capacity 64
        rhs = torch.zeros((2, 32, 48), dtype=torch.uint8, device="cuda")   # [G, K/2, N]
        pkg.ragged_dot_int4_bwd(lhs, rhs, torch.tensor([65, 1]).cuda())


def test_ragged_autotune_on_device(pkg):
    from strix_halo_int4_gemms_b200.autotune import RaggedDotMode

    res = pkg.autotune_ragged_dot(mode=RaggedDotMode.FWD, m=1024, n=256, k=256, groups=4, warmup_ms=1, rep_ms=3, continue_on_error=False)
    assert all(r.success for r in res.records) and res.best_record.tops > 0
    res = pkg.autotune_ragged_dot(mode=RaggedDotMode.BWD, m=256, n=256, k=1024, groups=4, layout=pkg.GemmLayout.TN, warmup_ms=1, rep_ms=3, continue_on_error=False)
    assert all(r.success for r in res.records) and res.shape.k == 1024


def test_forward_pair_tasks_with_the_lhs_through_tmem(pkg):
    """256-row tasks on CTA pairs with the unpacked lhs kept in TMEM (the library's own choice only for long K):
    same bits as with the lhs in shared memory, and as the oracle."""
    from strix_halo_int4_gemms_b200 import native

    sizes = [300, 0, 256, 7, 129, 512, 1, 255]
    data = make_ragged_fwd_inputs(m=sum(sizes), n=768, k=1024, group_sizes=sizes, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0), seed=9)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    cfg = pkg.RaggedDotConfig(block_m=256)
    info = pkg.calculate_group_info(dev["group_sizes"], 256, align_tile=cfg.align_tile)
    outs = []
    for a_operand in (native.A_OPERAND_TMEM, native.A_OPERAND_SMEM):
        out = torch.full((sum(sizes), 768), float("nan"), device="cuda", dtype=torch.bfloat16)
        native.launch_ragged_fwd_kernel(dev["lhs"], dev["rhs"], group_info=info, a_scale=dev["a_scale"], b_scale=dev["b_scale"], out=out,
                                        scale=scale_spec(pkg, 0), config=cfg, layout=pkg.GemmLayout.NN, rows=sum(sizes), cols=768,
                                        k_packed=512, scale_cols=1, path=native.PATH_TCGEN05, a_operand=a_operand)
        assert native.last_launch_path() == native.LAUNCHED_TCGEN05_PAIR
        outs.append(out)
    _status_clean()
    assert torch.equal(outs[0], outs[1])
    want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]), layout="nn")
    np.testing.assert_array_equal(as_f32(outs[0]), want)
