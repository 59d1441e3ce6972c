"""B200 (sm_100a) quantized GEMMs: W4A4 / W8A8 dense, fused SwiGLU, grouped (ragged) int4 dots.

Drop-in for the public surface of the reference package ``amd_strix_halo_kernels``
(``__init__.py:55-107``): same function names, keyword signatures, operand format and error
types, backed by hand-written tcgen05 / TMA kernels in ``lib/libb200_int4_gemms.so`` instead of
pre-generated AMDGCN code objects.  Names that only made sense for the AMD artefacts
(``hsaco_dir``, ``amdgcn_metadata_dir`` ...) are not carried over; ``launch_dense`` takes the
place of ``launch_hsaco``.
"""
from .api import explicit_mm, fused_swiglu_up_gate, mm, reference_mm
from .autotune import (
    AutotuneResult,
    RaggedAutotuneCandidate,
    RaggedAutotuneResult,
    RaggedDotMode,
    autotune,
    autotune_ragged_dot,
    default_ragged_dot_candidates,
    find_autotune_candidates,
    generated_shape_for_kernel,
)
from .benchmarking import BenchmarkDatabase, BenchmarkRecord, BenchmarkShape, tops_for_runtime
from .exceptions import KernelError, KernelNotAvailableError
from .heuristics import choose_kernel
from .metadata import (
    ACC_DTYPE,
    ARCH,
    RHS_SUBCHANNEL_SCALE_LAYOUT,
    SCALE_DTYPE_BF16,
    SUPPORTED_GEMM_LAYOUTS,
    SUPPORTED_SUBCHANNELS,
    Epilogue,
    GemmLayout,
    KernelMetadata,
    KernelSchedule,
    KernelStatus,
    OperandDType,
    ScaleMode,
    ScaleSpec,
    TileConfig,
)
from .native import (
    NativeRuntimeStatus,
    accumulation_order,
    device_status,
    dispatch_runtime_status,
    launch_accumulators,
    launch_dense,
    launch_generated_kernel,
    native_library_path,
    unpack_int4_on_device,
)
from .quant import (
    fake_quant_int,
    pack_int4_k_major,
    pack_ragged_rhs_subchannel_scales,
    pack_rhs_subchannel_scales,
    quantize_int_cuda,
    repack_int4_tokens,
    unpack_int4_k_major,
)
from .ragged import (
    RaggedBwdDotConfig,
    RaggedDotConfig,
    RaggedGroupInfo,
    calculate_group_info,
    calculate_group_info_on_device,
    ragged_dot_int4,
    ragged_dot_int4_bwd,
    ragged_dot_int4_bwd_flat,
)
from .registry import KernelRegistry, default_registry
from .torch_ops import TORCH_GEMM_OP, TORCH_OP_NAMESPACE, register_torch_ops, torch_gemm

__all__ = [
    "calculate_group_info_on_device",
    "quantize_int_cuda",
    "ragged_dot_int4_bwd_flat",
    "repack_int4_tokens",
    "ACC_DTYPE",
    "ARCH",
    "AutotuneResult",
    "BenchmarkDatabase",
    "BenchmarkRecord",
    "BenchmarkShape",
    "Epilogue",
    "GemmLayout",
    "KernelError",
    "KernelMetadata",
    "KernelNotAvailableError",
    "KernelRegistry",
    "KernelSchedule",
    "KernelStatus",
    "NativeRuntimeStatus",
    "accumulation_order",
    "OperandDType",
    "RHS_SUBCHANNEL_SCALE_LAYOUT",
    "RaggedAutotuneCandidate",
    "RaggedAutotuneResult",
    "RaggedBwdDotConfig",
    "RaggedDotConfig",
    "RaggedDotMode",
    "RaggedGroupInfo",
    "SCALE_DTYPE_BF16",
    "SUPPORTED_GEMM_LAYOUTS",
    "SUPPORTED_SUBCHANNELS",
    "ScaleMode",
    "ScaleSpec",
    "TORCH_GEMM_OP",
    "TORCH_OP_NAMESPACE",
    "TileConfig",
    "autotune",
    "autotune_ragged_dot",
    "calculate_group_info",
    "choose_kernel",
    "default_ragged_dot_candidates",
    "default_registry",
    "device_status",
    "dispatch_runtime_status",
    "explicit_mm",
    "fake_quant_int",
    "find_autotune_candidates",
    "fused_swiglu_up_gate",
    "generated_shape_for_kernel",
    "launch_accumulators",
    "launch_dense",
    "launch_generated_kernel",
    "mm",
    "native_library_path",
    "pack_int4_k_major",
    "pack_ragged_rhs_subchannel_scales",
    "pack_rhs_subchannel_scales",
    "ragged_dot_int4",
    "ragged_dot_int4_bwd",
    "reference_mm",
    "register_torch_ops",
    "tops_for_runtime",
    "torch_gemm",
    "unpack_int4_k_major",
    "unpack_int4_on_device",
]
