"""Host side of the grouped dots (CPU): task builder against the oracle and the reference fixtures,
even-K predicates, configuration validation.  Modelled on the reference's tests/test_ragged_dot.py:120-237."""
import numpy as np
import pytest
import torch

from oracle import reference_math as oracle
from strix_halo_int4_gemms_b200.ragged import _can_use_bwd_even_k_fast_path, _can_use_even_k_fast_path, ragged_kernel_id

FIELDS = ("group_id", "block_start", "actual_start", "actual_end", "start_within_block", "actual_size")


def test_group_info_known_vectors(pkg):
    info = pkg.calculate_group_info(torch.tensor([17, 31, 24], dtype=torch.int32), tile=32, align_tile=8)
    assert info.num_tasks == 3
    assert info.group_id.tolist() == [0, 1, 2]
    assert info.block_start.tolist() == [0, 16, 48]
    assert info.actual_start.tolist() == [0, 17, 48]
    assert info.actual_end.tolist() == [17, 48, 72]
    assert info.start_within_block.tolist() == [0, 1, 0]
    assert info.actual_size.tolist() == [17, 31, 24]
    info = pkg.calculate_group_info(torch.tensor([2, 0, 7]), tile=16, tid_size=4, align_tile=8)
    assert info.num_tasks == 2
    assert info.group_id.tolist() == [0, 2, 0, 0]
    assert info.actual_start.tolist() == [0, 2, 0, 0]
    assert info.actual_end.tolist() == [2, 9, 0, 0]
    assert info.actual_size.tolist() == [2, 7, 0, 0]
    with pytest.raises(ValueError, match="tid_size must be at least 3"):
        pkg.calculate_group_info(torch.tensor([17, 31, 24]), tile=32, tid_size=2, align_tile=8)


def test_group_info_matches_reference_fixtures(pkg, golden):
    for i in range(int(golden["group_info/count"])):
        tile, align, tid, num_tasks = (int(v) for v in golden[f"group_info/{i}/params"])
        info = pkg.calculate_group_info(torch.from_numpy(golden[f"group_info/{i}/sizes"]), tile, tid_size=None if tid < 0 else tid, align_tile=align)
        assert info.num_tasks == num_tasks
        for field in FIELDS:
            np.testing.assert_array_equal(getattr(info, field).numpy(), golden[f"group_info/{i}/{field}"], err_msg=f"case {i} {field}")


def test_group_info_random_against_oracle(pkg):
    g = torch.Generator().manual_seed(9)
    for _ in range(40):
        groups = int(torch.randint(1, 12, (1,), generator=g))
        sizes = torch.randint(0, 300, (groups,), generator=g)
        sizes[torch.rand(groups, generator=g) < 0.3] = 0
        align = int(torch.tensor([1, 8, 16, 32])[torch.randint(0, 4, (1,), generator=g)])
        tile = align * int(torch.randint(1, 6, (1,), generator=g))
        info = pkg.calculate_group_info(sizes, tile, align_tile=align)
        want = oracle.calculate_group_info(sizes.tolist(), tile, align_tile=align)
        assert info.num_tasks == want["num_tasks"]
        for field in FIELDS:
            np.testing.assert_array_equal(getattr(info, field).numpy(), want[field])
        # every row is covered exactly once by the [actual_start, actual_end) ranges
        covered = np.zeros(int(sizes.sum()), dtype=np.int32)
        for lo, hi in zip(info.actual_start.tolist(), info.actual_end.tolist()):
            covered[lo:hi] += 1
        assert (covered == 1).all()


def test_group_info_edge_cases(pkg):
    empty = pkg.calculate_group_info(torch.zeros(0, dtype=torch.int64), 64)
    assert empty.num_tasks == 0 and empty.group_id.numel() == 0
    padded = pkg.calculate_group_info(torch.zeros(0, dtype=torch.int64), 64, tid_size=3)
    assert padded.actual_size.tolist() == [0, 0, 0]
    none = pkg.calculate_group_info(torch.tensor([0, 0]), 64)
    assert none.num_tasks == 0 and none.block_start.numel() == 0
    negative = pkg.calculate_group_info(torch.tensor([-5, 9]), 8)
    assert negative.actual_size.tolist() == [8, 1]  # negative sizes are clamped to zero
    with pytest.raises(TypeError, match="must be a torch.Tensor"):
        pkg.calculate_group_info([1, 2], 8)
    with pytest.raises(ValueError, match="must be 1D"):
        pkg.calculate_group_info(torch.ones((2, 2), dtype=torch.int64), 8)
    with pytest.raises(ValueError, match="integer dtype"):
        pkg.calculate_group_info(torch.ones(2), 8)
    with pytest.raises(ValueError, match="multiple of align_tile"):
        pkg.calculate_group_info(torch.tensor([1]), 12, align_tile=8)


def test_even_k_predicates(pkg):
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    cfg = pkg.RaggedDotConfig(block_k=64)
    assert _can_use_even_k_fast_path(logical_k=128, scale=pc, config=cfg)
    assert not _can_use_even_k_fast_path(logical_k=96, scale=pc, config=cfg)
    assert not _can_use_even_k_fast_path(logical_k=128, scale=pc, config=pkg.RaggedDotConfig(block_k=64, enable_even_k_fast_path=False))
    sc32 = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 32)
    assert _can_use_even_k_fast_path(logical_k=128, scale=sc32, config=cfg)
    assert not _can_use_even_k_fast_path(logical_k=192, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 128), config=cfg)
    bwd = pkg.RaggedBwdDotConfig(block_k=64)
    assert _can_use_bwd_even_k_fast_path(torch, group_sizes=torch.tensor([64, 0, 128]), scale=pc, config=bwd)
    assert not _can_use_bwd_even_k_fast_path(torch, group_sizes=torch.tensor([64, 37]), scale=pc, config=bwd)
    assert _can_use_bwd_even_k_fast_path(torch, group_sizes=torch.tensor([0, 0]), scale=pc, config=bwd)
    assert not _can_use_bwd_even_k_fast_path(torch, group_sizes=torch.tensor([64, 192]), scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 128), config=bwd)


def test_config_validation_and_ids(pkg):
    with pytest.raises(ValueError, match="block_k must be even"):
        pkg.RaggedDotConfig(block_k=33)
    with pytest.raises(ValueError, match="multiple of align_tile"):
        pkg.RaggedDotConfig(block_m=100, align_tile=8)
    with pytest.raises(ValueError, match="split_k must be positive"):
        pkg.RaggedBwdDotConfig(split_k=0)
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    assert ragged_kernel_id(mode="fwd", layout=pkg.GemmLayout.NN, scale=pc, config=pkg.RaggedDotConfig(), variant="evenk") == (
        "sm_100a_ragged_int4_fwd_nn_pc_evenk_bfloat16_bm128_bn256_bk128_gst1_w14_s3"
    )
    assert ragged_kernel_id(mode="bwd", layout=pkg.GemmLayout.TN, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 32),
                            config=pkg.RaggedBwdDotConfig(), variant="maskk") == (
        "sm_100a_ragged_int4_bwd_tn_sc32_maskk_float32_bm128_bn256_bk128_w20_s2_sk1"
    )
    with pytest.raises(ValueError, match="ragged mode"):
        ragged_kernel_id(mode="x", layout=pkg.GemmLayout.NN, scale=pc, config=pkg.RaggedDotConfig(), variant="evenk")


def test_ragged_api_rejects_cpu_tensors_and_bad_layout(pkg):
    lhs = torch.zeros((8, 16), dtype=torch.uint8)
    rhs = torch.zeros((2, 16, 32), dtype=torch.uint8)
    gs = torch.tensor([4, 4])
    with pytest.raises(TypeError, match="layout must be a GemmLayout"):
        pkg.ragged_dot_int4(lhs, rhs, gs, layout="nn")
    if not torch.cuda.is_available():
        with pytest.raises(ValueError, match="lhs must be a CUDA tensor"):
            pkg.ragged_dot_int4(lhs, rhs, gs)
        with pytest.raises(ValueError, match="lhs must be a CUDA tensor"):
            pkg.ragged_dot_int4_bwd(rhs, rhs, gs)


def test_group_info_records_its_tile_and_a_mismatched_config_is_refused(pkg):
    """Prebuilt tasks run with the height they were cut with; a config that names another height is an error
    (launching 256-row tasks as 128-row ones would leave half of every block unwritten)."""
    import torch

    from strix_halo_int4_gemms_b200.ragged import RaggedGroupInfo

    info = pkg.calculate_group_info(torch.tensor([300, 0, 200]), 256, align_tile=8)
    assert (info.tile, info.align_tile) == (256, 8)
    assert pkg.calculate_group_info(torch.tensor([], dtype=torch.int64), 64).tile == 64
    legacy = RaggedGroupInfo(*(torch.zeros(0, dtype=torch.int64) for _ in range(6)), num_tasks=0)
    assert legacy.tile is None
    if torch.cuda.is_available():
        lhs = torch.zeros((500, 64), dtype=torch.uint8, device="cuda")
        rhs = torch.zeros((3, 64, 256), dtype=torch.uint8, device="cuda")
        sizes = torch.tensor([300, 0, 200], device="cuda")
        with pytest.raises(ValueError, match="group_info was built with tile=256 but config.block_m=64"):
            pkg.ragged_dot_int4(lhs, rhs, sizes, config=pkg.RaggedDotConfig(block_m=64), group_info=info)
