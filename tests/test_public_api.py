"""Public surface (CPU).  Reference: tests/test_public_api.py:31-87 and __init__.py:55-107."""
import inspect

import pytest

# names of the reference's ``__all__`` that describe the operation rather than AMD artefacts
CARRIED_OVER = [
    "ACC_DTYPE", "ARCH", "AutotuneResult", "BenchmarkDatabase", "BenchmarkRecord", "BenchmarkShape",
    "RHS_SUBCHANNEL_SCALE_LAYOUT", "SCALE_DTYPE_BF16", "SUPPORTED_GEMM_LAYOUTS", "SUPPORTED_SUBCHANNELS",
    "Epilogue", "GemmLayout", "KernelMetadata", "KernelRegistry", "KernelSchedule", "KernelStatus",
    "NativeRuntimeStatus", "OperandDType", "RaggedAutotuneCandidate", "RaggedAutotuneResult", "RaggedBwdDotConfig",
    "RaggedDotMode", "RaggedDotConfig", "RaggedGroupInfo", "ScaleMode", "ScaleSpec", "TileConfig", "TORCH_GEMM_OP",
    "TORCH_OP_NAMESPACE", "autotune", "autotune_ragged_dot", "calculate_group_info", "default_registry",
    "default_ragged_dot_candidates", "dispatch_runtime_status", "explicit_mm", "find_autotune_candidates",
    "fused_swiglu_up_gate", "generated_shape_for_kernel", "launch_generated_kernel", "mm", "native_library_path",
    "ragged_dot_int4_bwd", "ragged_dot_int4", "register_torch_ops", "torch_gemm",
]
# AMD-artefact names with no meaning here: hsaco_dir, hsaco_path_for_kernel_id, amdgcn_metadata_dir,
# amdgcn_metadata_path_for_kernel_id, launch_hsaco (replaced by launch_dense)


def test_reference_names_are_exported(pkg):
    missing = [name for name in CARRIED_OVER if not hasattr(pkg, name) or name not in pkg.__all__]
    assert not missing
    assert pkg.ARCH == "sm_100a" and pkg.ACC_DTYPE == "int32" and pkg.SUPPORTED_SUBCHANNELS == (32, 64, 128, 256)
    assert pkg.TORCH_GEMM_OP == "b200_int4_gemms::gemm"
    assert [e.value for e in pkg.Epilogue] == ["none", "relu2", "swiglu"]
    assert [e.value for e in pkg.GemmLayout] == ["nn", "nt", "tn", "tt"]
    assert [e.value for e in pkg.KernelSchedule][:2] == ["standard", "persistent"]   # the reference's two, then this library's forms
    assert [e.value for e in pkg.OperandDType] == ["int4", "int8"]


def _kwonly(fn):
    return [p.name for p in inspect.signature(fn).parameters.values() if p.kind is p.KEYWORD_ONLY]


def test_keyword_signatures_match_the_reference(pkg):
    assert _kwonly(pkg.mm) == ["a_scale", "b_scale", "gate", "dtype", "layout", "scale", "epilogue", "schedule", "registry", "use_reference"]
    assert _kwonly(pkg.fused_swiglu_up_gate) == ["a_scale", "b_scale", "dtype", "layout", "scale", "registry", "use_reference"]
    assert _kwonly(pkg.explicit_mm) == ["kernel", "a_scale", "b_scale", "gate", "use_reference"]
    assert _kwonly(pkg.ragged_dot_int4)[:11] == [
        "a_scale", "b_scale", "scale", "config", "layout", "out", "output_dtype", "use_native", "native_root", "native_library_path", "group_info"
    ]
    assert _kwonly(pkg.ragged_dot_int4_bwd)[:9] == [
        "a_scale", "b_scale", "scale", "config", "layout", "out", "use_native", "native_root", "native_library_path"
    ]
    assert _kwonly(pkg.calculate_group_info) == ["tid_size", "align_tile", "allow_triton"]
    assert _kwonly(pkg.autotune) == [
        "m", "n", "k", "dtype", "layout", "scale", "epilogue", "schedule", "registry", "benchmark_db", "benchmark_db_path",
        "root", "library_path", "warmup_ms", "rep_ms", "validate", "benchmark_runner",
    ]
    assert _kwonly(pkg.torch_gemm) == ["kernel", "a_scale", "b_scale", "gate"]
    defaults = inspect.signature(pkg.autotune).parameters
    assert defaults["warmup_ms"].default == 25 and defaults["rep_ms"].default == 100


def test_type_errors_for_non_enum_arguments(pkg):
    import torch

    with pytest.raises(TypeError, match="layout must be a GemmLayout"):
        pkg.ragged_dot_int4_bwd(torch.zeros(1), torch.zeros(1), torch.zeros(1), layout="tn")
    with pytest.raises(TypeError, match="mode must be a RaggedDotMode"):
        pkg.autotune_ragged_dot(mode="fwd", m=8, n=8, k=8)


def test_choose_kernel_uses_database(pkg):
    from strix_halo_int4_gemms_b200.benchmarking import BenchmarkDatabase, BenchmarkRecord, BenchmarkShape

    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    default = pkg.choose_kernel(m=256, n=256, k=256, dtype=pkg.OperandDType.INT4, scale=pc, epilogue=pkg.Epilogue.NONE)
    assert (default.tile.block_m, default.tile.block_n, default.tile.split_k) == (128, 256, 1)
    pick = pkg.default_registry.select(dtype=pkg.OperandDType.INT4, scale=pc, epilogue=pkg.Epilogue.NONE, m=32, n=128, k=64, split_k=2)
    db = BenchmarkDatabase([BenchmarkRecord(pick.kernel_id, BenchmarkShape(256, 256, 256), 0.01, 999.0, 3, 3)])
    assert pkg.choose_kernel(m=256, n=256, k=256, dtype=pkg.OperandDType.INT4, scale=pc, epilogue=pkg.Epilogue.NONE, benchmark_db=db).kernel_id == pick.kernel_id
    with pytest.raises(LookupError):
        pkg.choose_kernel(m=7, n=256, k=256, dtype=pkg.OperandDType.INT4, scale=pc, epilogue=pkg.Epilogue.NONE)
