"""Registry matrix, ids and the selection rule (CPU).  Modelled on the reference's tests/test_registry.py."""
import pytest


def test_matrix_and_unique_ids(pkg):
    from collections import Counter

    kernels = pkg.default_registry.all()
    per_form = Counter(k.schedule for k in kernels)
    assert set(per_form) == set(pkg.KernelSchedule)
    # the library's own choice comes with every shape multiple; forced forms with their raster widths only
    assert per_form[pkg.KernelSchedule.STANDARD] > per_form[pkg.KernelSchedule.PERSISTENT] > per_form[pkg.KernelSchedule.PERSISTENT_2CTA]
    assert len({k.kernel_id for k in kernels}) == len(kernels)
    assert all(k.arch == "sm_100a" and k.acc_dtype == "int32" and k.scale_dtype == "bfloat16" for k in kernels)
    assert {k.layout for k in kernels} == set(pkg.SUPPORTED_GEMM_LAYOUTS)
    assert pkg.GemmLayout.TT not in {k.layout for k in kernels}
    for k in kernels:
        if k.schedule is pkg.KernelSchedule.PERSISTENT_2CTA:
            assert k.tile.block_m == 256 and k.tile.group_size_m in (16, 8)
            assert not (k.scale.mode is pkg.ScaleMode.SUBCHANNEL and k.scale.subchannel_size < 128)
        elif k.schedule is pkg.KernelSchedule.STANDARD:
            assert k.tile.group_size_m == 0          # raster width left to the library
        else:
            assert k.tile.block_m == 128 and k.tile.group_size_m > 0


def test_forced_forms_exist_only_where_the_library_has_the_kernel(pkg):
    from strix_halo_int4_gemms_b200.registry import has_pair_kernel, has_split_k_kernel

    pc, sc256, sc64 = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 256), pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 64)
    i4, i8 = pkg.OperandDType.INT4, pkg.OperandDType.INT8
    nn, nt, tn = pkg.GemmLayout.NN, pkg.GemmLayout.NT, pkg.GemmLayout.TN
    assert has_pair_kernel(i4, sc256, pkg.Epilogue.SWIGLU, nn) and has_pair_kernel(i8, pc, pkg.Epilogue.RELU2, nt)
    assert not has_pair_kernel(i4, sc64, pkg.Epilogue.NONE, nn) and not has_pair_kernel(i8, pc, pkg.Epilogue.NONE, tn)
    assert has_split_k_kernel(i4, pc, nn, pair=True) and has_split_k_kernel(i8, pc, nt) and has_split_k_kernel(i4, sc64, nt)
    assert not has_split_k_kernel(i4, pc, tn) and not has_split_k_kernel(i8, sc256, nn) and not has_split_k_kernel(i4, pc, nt, pair=True)
    splits = {k.tile.split_k for k in pkg.default_registry.all() if k.layout is tn}
    assert splits == {1}


def test_activations_have_no_split_k_and_split_k_means_float32(pkg):
    for k in pkg.default_registry.all():
        if k.epilogue is not pkg.Epilogue.NONE:
            assert k.tile.split_k == 1
        assert k.output_dtype == ("bfloat16" if k.tile.split_k == 1 else "float32")
        if k.epilogue is pkg.Epilogue.SWIGLU:
            assert k.tile.block_n == 128


def test_kernel_id_grammar(pkg):
    tile = pkg.TileConfig(128, 256, 32, 8, 10, 3, 0, even_k=True)
    from strix_halo_int4_gemms_b200.metadata import make_kernel_id

    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    assert make_kernel_id(pkg.OperandDType.INT4, pc, pkg.Epilogue.NONE, tile) == (
        "sm_100a_int4xint4_nn_pc_none_bm128_bn256_bk32_gm8_w10_s3_weu0_sk1_evenk"
    )
    sc = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 256)
    masked = pkg.TileConfig(16, 128, 32, 8, 10, 4, 0, even_k=False, split_k=2)
    assert make_kernel_id(
        pkg.OperandDType.INT8, sc, pkg.Epilogue.RELU2, masked, layout=pkg.GemmLayout.TN, schedule=pkg.KernelSchedule.PERSISTENT
    ) == "sm_100a_int8xint8_tn_sc256_relu2_persistent_bm16_bn128_bk32_gm8_w10_s4_weu0_sk2_maskk"


def test_scale_spec_and_tile_validation(pkg):
    with pytest.raises(ValueError, match="subchannel_size must be one of"):
        pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 48)
    with pytest.raises(ValueError, match="must not set subchannel_size"):
        pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL, 32)
    with pytest.raises(ValueError, match="split_k must be one of"):
        pkg.TileConfig(128, 256, 32, 8, 10, 3, 0, even_k=True, split_k=3)
    assert pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 64).label == "sc64"


def _select(pkg, **kw):
    base = dict(dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.NONE)
    base.update(kw)
    return pkg.default_registry.select(**base)


def test_selection_prefers_largest_registered_multiples(pkg):
    k = _select(pkg, m=4096, n=4096, k=4096)
    assert (k.tile.block_m, k.tile.block_n, k.tile.split_k, k.tile.even_k) == (128, 256, 1, True)
    assert k.kernel_id == "sm_100a_int4xint4_nn_pc_none_bm128_bn256_bk32_gm0_w14_s3_weu0_sk1_evenk"
    assert k.schedule is pkg.KernelSchedule.STANDARD      # the default form: the library pairs CTAs itself when that pays
    pair = _select(pkg, m=4096, n=4096, k=4096, schedule=pkg.KernelSchedule.PERSISTENT_2CTA)
    assert (pair.tile.block_m, pair.tile.group_size_m, pair.tile.num_stages) == (256, 16, 4) and "_persistent_2cta_" in pair.kernel_id
    with pytest.raises(LookupError):
        _select(pkg, m=128, n=1024, k=64, schedule=pkg.KernelSchedule.PERSISTENT_2CTA)   # a pair's tile has 256 rows
    assert _select(pkg, m=128, n=1024, k=64).tile.block_m == 128          # the quick-start shape
    small = _select(pkg, m=48, n=384, k=96)
    assert (small.tile.block_m, small.tile.block_n) == (16, 128)
    swiglu = _select(pkg, m=4096, n=14336, k=4096, epilogue=pkg.Epilogue.SWIGLU, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 256))
    assert (swiglu.tile.block_m, swiglu.tile.block_n) == (128, 128)
    int8 = _select(pkg, m=8192, n=8192, k=8192, dtype=pkg.OperandDType.INT8, epilogue=pkg.Epilogue.RELU2)
    assert int8.tile.num_warps == 6 and int8.tile.num_stages == 4


def test_selection_honours_split_k_schedule_layout(pkg):
    k = _select(pkg, m=128, n=256, k=1024, split_k=8, schedule=pkg.KernelSchedule.PERSISTENT, layout=pkg.GemmLayout.NT)
    assert k.tile.split_k == 8 and k.schedule is pkg.KernelSchedule.PERSISTENT and k.layout is pkg.GemmLayout.NT
    assert "_persistent_" in k.kernel_id and k.output_dtype == "float32"
    with pytest.raises(LookupError, match="no kernel for dtype=int4"):
        _select(pkg, m=128, n=256, k=128, split_k=8)  # K must be a multiple of 32 * 8
    with pytest.raises(LookupError):
        _select(pkg, m=128, n=256, k=96, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 64))  # K % S != 0
    with pytest.raises(LookupError):
        _select(pkg, m=128, n=256, k=128, layout=pkg.GemmLayout.TT)


def test_measured_tops_override_size_preference(pkg):
    small = _select(pkg, m=16, n=128, k=32)
    tuned = pkg.default_registry.with_status(small.kernel_id, pkg.KernelStatus.BENCHMARKED, measured_tops=123.0)
    assert tuned.select(
        dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.NONE, m=4096, n=4096, k=4096
    ).kernel_id == small.kernel_id
    assert pkg.default_registry.get(small.kernel_id).measured_tops is None  # the original is untouched


def test_select_reference_ignores_shape(pkg):
    k = pkg.default_registry.select_reference(
        dtype=pkg.OperandDType.INT8, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 128), epilogue=pkg.Epilogue.SWIGLU
    )
    assert k.tile.even_k and k.tile.split_k == 1 and k.epilogue is pkg.Epilogue.SWIGLU


def test_register_rejects_duplicates(pkg):
    reg = pkg.KernelRegistry()
    k = pkg.default_registry.all()[0]
    reg.register(k)
    with pytest.raises(ValueError, match="duplicate kernel id"):
        reg.register(k)
    assert reg.get(k.kernel_id) is k and len(reg) == 1


def test_metadata_to_dict(pkg):
    k = _select(pkg, m=128, n=256, k=256, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 256))
    d = k.to_dict()
    assert d["a_dtype"] == "int4" and d["layout"] == "nn" and d["schedule"] == "standard" and d["status"] == "compiled"
    assert d["scale"] == {"mode": "subchannel", "subchannel_size": 256}
    assert d["rhs_subchannel_scale_layout"] == "kgroup_output"
    assert d["tile"]["block_m"] == 128
