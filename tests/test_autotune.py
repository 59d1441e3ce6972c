"""Tuner bookkeeping with injected runners (CPU).  Reference: tests/test_autotune.py:151-375."""
import pytest
import torch

from oracle import reference_math as oracle
from strix_halo_int4_gemms_b200.autotune import (
    RaggedAutotuneCandidate,
    RaggedDotMode,
    _validation_tolerances,
    make_dense_inputs,
    make_ragged_bwd_inputs,
    make_ragged_fwd_inputs,
)
from strix_halo_int4_gemms_b200.benchmarking import BenchmarkDatabase, BenchmarkRecord, BenchmarkShape, tops_for_runtime
from helpers import as_f32, bf16_bits


def _pc(pkg):
    return pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)


def test_candidates_are_launches_that_differ(pkg):
    from strix_halo_int4_gemms_b200.registry import launch_signature

    found = pkg.find_autotune_candidates(m=256, n=512, k=256, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.NONE)
    # library's choice x split 1/2/4/8; one CTA per tile x raster 8/32 x split; CTA pairs x raster 16/8 x split; tile per CTA
    assert len(found) == 4 + 2 * 4 + 2 * 4 + 1 == 21
    assert len({launch_signature(k) for k in found}) == len(found)      # no two candidates run the same launch
    assert all(k.tile.even_k for k in found)
    assert {k.schedule for k in found} == set(pkg.KernelSchedule)
    standard = pkg.find_autotune_candidates(m=256, n=512, k=256, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.NONE,
                                            schedule=pkg.KernelSchedule.STANDARD)
    assert [k.tile.split_k for k in standard] == [1, 2, 4, 8]
    assert all((k.tile.block_m, k.tile.block_n) == (128, 256) for k in standard)   # largest multiples that divide the shape
    # M = 128: nothing for CTA pairs (256-row tiles)
    skinny = pkg.find_autotune_candidates(m=128, n=1024, k=64, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.NONE)
    assert pkg.KernelSchedule.PERSISTENT_2CTA not in {k.schedule for k in skinny}
    odd = pkg.find_autotune_candidates(m=48, n=128, k=96, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.RELU2)
    assert {(k.tile.block_m, k.tile.block_n, k.schedule) for k in odd} == {(16, 128, pkg.KernelSchedule.STANDARD)}
    assert pkg.generated_shape_for_kernel(found[0]) is None


def test_autotune_picks_best_successful_record_and_appends_to_db(pkg, tmp_path):
    shape = BenchmarkShape(256, 512, 256)
    seen = []

    def runner(kernel, tuned):
        seen.append(kernel.kernel_id)
        assert tuned == shape
        ms = 1.0 + 0.01 * len(seen)
        if kernel.schedule is pkg.KernelSchedule.PERSISTENT_2CTA and kernel.tile.group_size_m == 8 and kernel.tile.split_k == 1:
            ms = 0.25
        ok = not (kernel.schedule is pkg.KernelSchedule.PERSISTENT and kernel.tile.split_k == 8)
        return BenchmarkRecord(kernel.kernel_id, tuned, ms, tops_for_runtime(tuned, ms) if ok else 1e9, 7, 25, success=ok)

    path = tmp_path / "db.json"
    old = BenchmarkRecord("older", shape, 3.0, 0.1, 1, 1)
    BenchmarkDatabase([old]).save(path)
    result = pkg.autotune(m=256, n=512, k=256, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.NONE,
                          benchmark_db_path=path, benchmark_runner=runner)
    assert len(result.records) == len(result.candidates) == 21 == len(seen)
    assert result.best_kernel.schedule is pkg.KernelSchedule.PERSISTENT_2CTA and result.best_kernel.tile.group_size_m == 8
    assert result.best_record.runtime_ms == 0.25 and result.shape == shape
    stored = BenchmarkDatabase.load(path).records()
    assert stored[0] == old and len(stored) == 22


def test_autotune_errors(pkg):
    with pytest.raises(LookupError, match=r"no pregenerated kernels match dtype=int4, layout=nn, scale=pc, epilogue=none, schedule=any, shape=\(17, 512, 256\)"):
        pkg.autotune(m=17, n=512, k=256, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.NONE, benchmark_runner=lambda k, s: None)
    failing = lambda kernel, shape: BenchmarkRecord(kernel.kernel_id, shape, 1.0, 1.0, 1, 1, success=False)
    with pytest.raises(RuntimeError, match="no successful benchmark records"):
        pkg.autotune(m=128, n=256, k=64, dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.SWIGLU, benchmark_runner=failing)


def test_validation_tolerances(pkg):
    bf16 = pkg.default_registry.select(dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.RELU2, m=128, n=256, k=64)
    assert _validation_tolerances(bf16) == (8.0e-3, 1.0e-2)
    f32 = pkg.default_registry.select(dtype=pkg.OperandDType.INT4, scale=_pc(pkg), epilogue=pkg.Epilogue.NONE, m=128, n=256, k=64, split_k=2)
    assert _validation_tolerances(f32) == (1.0e-4, 1.0e-3)


def test_default_ragged_candidates(pkg):
    fwd = pkg.default_ragged_dot_candidates(RaggedDotMode.FWD)
    assert all(isinstance(c.config, pkg.RaggedDotConfig) and c.config.pair_tasks is False for c in fwd)
    assert [c.config.block_m for c in fwd] == [256, 128, 64, 32]        # CTA-pair tasks first, then single-CTA heights
    assert fwd[1].kernel_id == "ragged_dot_int4_fwd_nn_pc_bm128_bn256_bk128_gst1_w14_s3"
    tn = pkg.default_ragged_dot_candidates(RaggedDotMode.FWD, layout=pkg.GemmLayout.TN)
    assert max(c.config.block_m for c in tn) == 128                      # no paired kernel for a transposed lhs
    bwd = pkg.default_ragged_dot_candidates(RaggedDotMode.BWD, layout=pkg.GemmLayout.TN, split_ks=(1, 4))
    assert [c.config.split_k for c in bwd] == [1, 4]
    assert bwd[1].kernel_id == "ragged_dot_int4_bwd_tn_pc_bm128_bn256_bk128_w20_s2_sk4"
    with pytest.raises(TypeError, match="mode must be a RaggedDotMode"):
        pkg.default_ragged_dot_candidates("fwd")


def test_ragged_autotune_bookkeeping(pkg, tmp_path):
    calls = []

    def runner(candidate, shape):
        calls.append(candidate.kernel_id)
        if candidate.config.block_m == 32:
            raise RuntimeError("boom")
        ms = 2.0 if candidate.config.block_m == 128 else 1.0
        return BenchmarkRecord(candidate.kernel_id, shape, ms, tops_for_runtime(shape, ms), 5, 25)

    result = pkg.autotune_ragged_dot(mode=RaggedDotMode.FWD, m=1000, n=256, k=128, groups=3, benchmark_runner=runner,
                                     benchmark_db_path=tmp_path / "r.json")
    assert result.group_sizes == (334, 333, 333)
    assert len(result.records) == len(result.candidates) == len(calls)
    failed = [r for r in result.records if not r.success]
    assert len(failed) == 1 and "boom" in failed[0].metadata["error"] and failed[0].tops == 0.0
    assert result.best_record.runtime_ms == 1.0 and result.best_candidate.kernel_id == result.best_record.kernel_id
    with pytest.raises(RuntimeError, match="boom"):
        pkg.autotune_ragged_dot(mode=RaggedDotMode.FWD, m=1000, n=256, k=128, groups=3, benchmark_runner=runner, continue_on_error=False)


def test_ragged_autotune_argument_checks(pkg):
    ok = lambda c, s: BenchmarkRecord(c.kernel_id, s, 1.0, 1.0, 1, 1)
    with pytest.raises(ValueError, match="forward group_sizes must sum to M=10; got 9"):
        pkg.autotune_ragged_dot(mode=RaggedDotMode.FWD, m=10, n=8, k=8, group_sizes=[4, 5], benchmark_runner=ok)
    with pytest.raises(ValueError, match="backward group_sizes must sum to K=64; got 60"):
        pkg.autotune_ragged_dot(mode=RaggedDotMode.BWD, m=8, n=8, k=64, group_sizes=torch.tensor([20, 40]), benchmark_runner=ok)
    with pytest.raises(ValueError, match="k_capacity is only configurable for backward"):
        pkg.autotune_ragged_dot(mode=RaggedDotMode.FWD, m=8, n=8, k=8, k_capacity=16, benchmark_runner=ok)
    with pytest.raises(ValueError, match=r"k_capacity must be >= max\(group_sizes\)=40"):
        pkg.autotune_ragged_dot(mode=RaggedDotMode.BWD, m=8, n=8, k=64, group_sizes=[24, 40], k_capacity=32, benchmark_runner=ok)
    with pytest.raises(TypeError, match="forward ragged-dot candidates must use RaggedDotConfig"):
        bad = RaggedAutotuneCandidate(RaggedDotMode.FWD, pkg.GemmLayout.NN, _pc(pkg), pkg.RaggedBwdDotConfig())
        pkg.autotune_ragged_dot(mode=RaggedDotMode.FWD, m=8, n=8, k=8, candidates=[bad], benchmark_runner=ok)
    res = pkg.autotune_ragged_dot(mode=RaggedDotMode.BWD, m=8, n=8, k=64, group_sizes=[24, 40], candidates=[pkg.RaggedBwdDotConfig(split_k=2)], benchmark_runner=ok)
    assert res.candidates[0].config.split_k == 2 and res.shape == BenchmarkShape(8, 8, 64)


def test_synthetic_inputs_are_seeded_and_well_formed(pkg):
    kernel = pkg.default_registry.select(dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 64),
                                         epilogue=pkg.Epilogue.SWIGLU, m=32, n=128, k=128, layout=pkg.GemmLayout.NT)
    a, b, sa, sb = make_dense_inputs(kernel, BenchmarkShape(32, 128, 128))
    a2, b2, _, _ = make_dense_inputs(kernel, BenchmarkShape(32, 128, 128))
    assert torch.equal(a, a2) and torch.equal(b, b2)
    assert tuple(a.shape) == (32, 64) and tuple(b.shape) == (256, 64) and a.dtype is torch.uint8
    assert tuple(sa.shape) == (32, 2) and tuple(sb.shape) == (2, 256) and sa.dtype is torch.bfloat16
    out = pkg.explicit_mm(a, b, kernel=kernel, a_scale=sa, b_scale=sb, use_reference=True)
    assert tuple(out.shape) == (32, 128)
    fwd = make_ragged_fwd_inputs(m=20, n=16, k=64, group_sizes=[5, 0, 15], layout=pkg.GemmLayout.TN, scale=_pc(pkg))
    assert tuple(fwd["lhs"].shape) == (32, 20) and tuple(fwd["rhs"].shape) == (3, 32, 16)
    want = oracle.ragged_dot_fwd(fwd["lhs"].numpy(), fwd["rhs"].numpy(), [5, 0, 15], bf16_bits(fwd["a_scale"]), bf16_bits(fwd["b_scale"]), layout="tn", out_bf16=False)
    direct = oracle.scaled_matmul(fwd["x"].numpy()[5:], fwd["w"][2].numpy(), as_f32(fwd["a_scale"])[5:], as_f32(fwd["b_scale"])[2])
    assert (want[5:] == direct).all()
    bwd = make_ragged_bwd_inputs(m=8, n=16, k_capacity=37, group_sizes=[37, 3], layout=pkg.GemmLayout.NT, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 32))
    assert tuple(bwd["lhs"].shape) == (2, 8, 19) and tuple(bwd["rhs"].shape) == (2, 16, 19) and tuple(bwd["a_scale"].shape) == (2, 8, 2)
