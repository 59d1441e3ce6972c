"""ctypes binding of libb200_int4_gemms.so and the tensor-level launchers built on it.

Stands where the reference's ``native.py`` stood (ctypes prototypes :54-143, status :146-155,
``launch_generated_kernel`` :690-767, ragged launch wrappers :533-667).  The reference read a
JSON record per kernel to learn its grid, block and shared-memory size and passed them across
the C boundary; here the library decides those itself and the binding passes a plain variant
record, the caller's stream, pointers and sizes.

There is no CPU or JIT fallback: when the shared library is missing, or the tensors are not on
a CUDA device, the launchers raise.
"""
from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .metadata import Epilogue, GemmLayout, KernelMetadata, KernelSchedule, OperandDType, ScaleMode, ScaleSpec
from .template_config import LaunchShape

NATIVE_LIBRARY_NAME = "libb200_int4_gemms.so"
THREADS_PER_WARP = 32

DTYPE_CODES = {OperandDType.INT4: 0, OperandDType.INT8: 1}
LAYOUT_CODES = {GemmLayout.NN: 0, GemmLayout.NT: 1, GemmLayout.TN: 2, GemmLayout.TT: 3}
EPILOGUE_CODES = {Epilogue.NONE: 0, Epilogue.RELU2: 1, Epilogue.SWIGLU: 2}
OUT_BF16, OUT_F32, OUT_S32 = 0, 1, 2
PATH_AUTO, PATH_TCGEN05, PATH_SIMT = 0, 1, 2
SCHEDULE_PERSISTENT, SCHEDULE_TILE_PER_CTA = 0, 1
CTA_GROUP_AUTO, CTA_GROUP_SINGLE, CTA_GROUP_PAIR = 0, 1, 2
LAUNCHED_NOTHING, LAUNCHED_TCGEN05, LAUNCHED_TCGEN05_PAIR, LAUNCHED_SIMT = 0, 1, 2, 3
ACCUMULATE_FUSED, ACCUMULATE_REFERENCE = 0, 1
A_OPERAND_AUTO, A_OPERAND_SMEM, A_OPERAND_TMEM = 0, 1, 2
TAIL_AUTO, TAIL_OFF, TAIL_ALWAYS = 0, 1, 2
WIDE_AUTO, WIDE_OFF, WIDE_ON = 0, 1, 2

# Order of roundings of subchannel dense launches made through the registry / public API: "fused" (default; the
# last multiply and the add of each K-group share one rounding) or "reference" (every rounding of the reference's
# PyTorch math: bit-identical to it, about a third slower on large problems).  See ``accumulation_order``.
_ACCUMULATION_ORDER = ACCUMULATE_FUSED


class accumulation_order:
    """Context manager (or plain call) that sets the order for subchannel dense launches of this process:
    ``with accumulation_order("reference"): mm(...)``."""

    def __init__(self, order: str) -> None:
        global _ACCUMULATION_ORDER
        if order not in ("fused", "reference"):
            raise ValueError("order must be 'fused' or 'reference'")
        self._previous = _ACCUMULATION_ORDER
        _ACCUMULATION_ORDER = ACCUMULATE_REFERENCE if order == "reference" else ACCUMULATE_FUSED

    def __enter__(self) -> "accumulation_order":
        return self

    def __exit__(self, *exc: object) -> None:
        global _ACCUMULATION_ORDER
        _ACCUMULATION_ORDER = self._previous

EXPORTED_SYMBOLS = (
    "b200_int4_gemms_dispatch_version",
    "b200_int4_gemms_has_compiled_kernels",
    "b200_int4_gemms_has_cuda_runtime",
    "b200_int4_gemms_has_linked_kernels",
    "b200_int4_gemms_last_error",
    "b200_int4_gemms_device_status",
    "b200_int4_gemms_reset_device_status",
    "b200_int4_gemms_launch_dense",
    "b200_int4_gemms_dense_workspace_bytes",
    "b200_int4_gemms_plan_dense",
    "b200_int4_gemms_last_launch_path",
    "b200_int4_gemms_launch_ragged_fwd",
    "b200_int4_gemms_launch_ragged_bwd",
    "b200_int4_gemms_unpack_int4",
    "b200_int4_gemms_group_info",
    "b200_int4_gemms_launch_ragged_fwd_device_tasks",
    "b200_int4_gemms_ragged_bwd_flat_workspace_bytes",
    "b200_int4_gemms_launch_ragged_bwd_flat",
    "b200_int4_gemms_launch_ragged_bwd_flat_static",
    "b200_int4_gemms_quantize",
    "b200_int4_gemms_repack_tokens",
)


class GemmVariant(ctypes.Structure):
    """``b200_gemm_variant`` of include/b200_int4_gemms.h."""

    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("layout", ctypes.c_int32),
        ("scale_mode", ctypes.c_int32),
        ("subchannel", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("split_k", ctypes.c_int32),
        ("path", ctypes.c_int32),
        ("group_m", ctypes.c_int32),
        ("schedule", ctypes.c_int32),
        ("cta_group", ctypes.c_int32),
        ("accumulate_order", ctypes.c_int32),
        ("a_operand", ctypes.c_int32),
        ("tail_balance", ctypes.c_int32),
        ("task_align", ctypes.c_int32),
        ("wide_tiles", ctypes.c_int32),
    ]


class DensePlan(ctypes.Structure):
    """``b200_dense_plan`` of include/b200_int4_gemms.h: what a dense launch would do."""

    _fields_ = [
        ("path", ctypes.c_int32),
        ("grid", ctypes.c_int32),
        ("tile_rows", ctypes.c_int32),
        ("tile_cols", ctypes.c_int32),
        ("group_m", ctypes.c_int32),
        ("split_k", ctypes.c_int32),
        ("tail_units", ctypes.c_int32),
        ("tiles_384", ctypes.c_int32),
    ]

    def as_tuple(self) -> tuple[int, int, int, int, int, int]:
        return (int(self.path), int(self.grid), int(self.tile_rows), int(self.tile_cols), int(self.group_m), int(self.split_k))


@dataclass(frozen=True, slots=True)
class NativeRuntimeStatus:
    library_path: Path
    dispatch_version: int
    has_compiled_code_objects: bool
    has_cuda_runtime: bool
    has_linked_kernels: bool

    @property
    def has_hip_runtime(self) -> bool:
        """Name the reference uses for "the GPU runtime is usable" (native.py:19-25)."""
        return self.has_cuda_runtime


def package_root() -> Path:
    return Path(__file__).resolve().parent


def native_library_path(*, root: str | Path | None = None) -> Path:
    base = Path(root) if root is not None else package_root() / "lib"
    return base / NATIVE_LIBRARY_NAME


_LIBRARIES: dict[str, ctypes.CDLL] = {}
_LIBRARIES_LOCK = threading.Lock()


def _declare(library: ctypes.CDLL) -> None:
    void_p, i32, i64, size_t = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
    variant_p = ctypes.POINTER(GemmVariant)
    for name in ("dispatch_version", "has_compiled_kernels", "has_cuda_runtime", "has_linked_kernels"):
        fn = getattr(library, f"b200_int4_gemms_{name}")
        fn.restype, fn.argtypes = ctypes.c_int, []
    library.b200_int4_gemms_last_error.restype = ctypes.c_char_p
    library.b200_int4_gemms_last_error.argtypes = []
    library.b200_int4_gemms_device_status.restype = ctypes.c_int
    library.b200_int4_gemms_device_status.argtypes = [ctypes.c_int, ctypes.POINTER(i32)]
    library.b200_int4_gemms_reset_device_status.restype = ctypes.c_int
    library.b200_int4_gemms_reset_device_status.argtypes = [ctypes.c_int]
    library.b200_int4_gemms_launch_dense.restype = ctypes.c_int
    library.b200_int4_gemms_launch_dense.argtypes = [
        variant_p, ctypes.c_int, size_t, void_p, void_p, void_p, void_p, void_p, void_p, size_t, i32, i32, i32,
    ]
    library.b200_int4_gemms_dense_workspace_bytes.restype = size_t
    library.b200_int4_gemms_dense_workspace_bytes.argtypes = [variant_p, i32, i32, i32]
    library.b200_int4_gemms_plan_dense.restype = ctypes.c_int
    library.b200_int4_gemms_plan_dense.argtypes = [variant_p, ctypes.c_int, i32, i32, i32, ctypes.POINTER(DensePlan)]
    library.b200_int4_gemms_last_launch_path.restype = ctypes.c_int
    library.b200_int4_gemms_last_launch_path.argtypes = []
    library.b200_int4_gemms_launch_ragged_fwd.restype = ctypes.c_int
    library.b200_int4_gemms_launch_ragged_fwd.argtypes = [variant_p, ctypes.c_int, size_t] + [void_p] * 9 + [i32] * 7
    library.b200_int4_gemms_launch_ragged_bwd.restype = ctypes.c_int
    library.b200_int4_gemms_launch_ragged_bwd.argtypes = [variant_p, ctypes.c_int, size_t] + [void_p] * 6 + [i32] * 5
    library.b200_int4_gemms_unpack_int4.restype = ctypes.c_int
    library.b200_int4_gemms_unpack_int4.argtypes = [ctypes.c_int, size_t, void_p, void_p, i64, i64]
    library.b200_int4_gemms_group_info.restype = ctypes.c_int
    library.b200_int4_gemms_group_info.argtypes = [ctypes.c_int, size_t, void_p, i32, i32, i32] + [void_p] * 4 + [i32, void_p, void_p]
    library.b200_int4_gemms_launch_ragged_fwd_device_tasks.restype = ctypes.c_int
    library.b200_int4_gemms_launch_ragged_fwd_device_tasks.argtypes = [variant_p, ctypes.c_int, size_t] + [void_p] * 11 + [i32] * 7
    library.b200_int4_gemms_ragged_bwd_flat_workspace_bytes.restype = size_t
    library.b200_int4_gemms_ragged_bwd_flat_workspace_bytes.argtypes = [i32]
    library.b200_int4_gemms_launch_ragged_bwd_flat.restype = ctypes.c_int
    library.b200_int4_gemms_launch_ragged_bwd_flat.argtypes = [variant_p, ctypes.c_int, size_t] + [void_p] * 7 + [size_t, i32, i32, i64, i32]
    library.b200_int4_gemms_launch_ragged_bwd_flat_static.restype = ctypes.c_int
    library.b200_int4_gemms_launch_ragged_bwd_flat_static.argtypes = [variant_p, ctypes.c_int, size_t] + [void_p] * 6 + [i32, i32, i64, i32]
    library.b200_int4_gemms_quantize.restype = ctypes.c_int
    library.b200_int4_gemms_quantize.argtypes = [ctypes.c_int, size_t, void_p, void_p, i64, i64, i32, ctypes.c_float]
    library.b200_int4_gemms_repack_tokens.restype = ctypes.c_int
    library.b200_int4_gemms_repack_tokens.argtypes = [ctypes.c_int, size_t, void_p, void_p, i64, i64]


def load_dispatch_library(path: str | Path | None = None) -> ctypes.CDLL:
    """dlopen the CUDA library (once per path) and declare its prototypes."""
    library_path = Path(path) if path is not None else native_library_path()
    key = str(library_path)
    with _LIBRARIES_LOCK:
        cached = _LIBRARIES.get(key)
        if cached is not None:
            return cached
        if not library_path.exists():
            raise RuntimeError(
                f"native dispatch library is not installed at {library_path}; "
                "build it with build.py (nvcc, sm_100a) - there is no fallback path"
            )
        library = ctypes.CDLL(key)
        _declare(library)
        _LIBRARIES[key] = library
        return library


def dispatch_runtime_status(path: str | Path | None = None) -> NativeRuntimeStatus:
    library_path = Path(path) if path is not None else native_library_path()
    library = load_dispatch_library(library_path)
    return NativeRuntimeStatus(
        library_path=library_path,
        dispatch_version=int(library.b200_int4_gemms_dispatch_version()),
        has_compiled_code_objects=bool(library.b200_int4_gemms_has_compiled_kernels()),
        has_cuda_runtime=bool(library.b200_int4_gemms_has_cuda_runtime()),
        has_linked_kernels=bool(library.b200_int4_gemms_has_linked_kernels()),
    )


def _library_last_error(library: ctypes.CDLL) -> str:
    raw = library.b200_int4_gemms_last_error()
    return raw.decode("utf-8", errors="replace") if raw else "unknown native dispatcher error"


def device_status(device_index: int = 0, *, library_path: str | Path | None = None) -> tuple[int, tuple[int, int, int]]:
    """(status, (block, wait site, spare)) reported by kernels on a device; 0 means clean.

    Does not synchronise: call after the stream has been synchronised.
    """
    library = load_dispatch_library(library_path)
    detail = (ctypes.c_int32 * 3)()
    status = int(library.b200_int4_gemms_device_status(int(device_index), detail))
    return status, (int(detail[0]), int(detail[1]), int(detail[2]))


def reset_device_status(device_index: int = 0, *, library_path: str | Path | None = None) -> None:
    load_dispatch_library(library_path).b200_int4_gemms_reset_device_status(int(device_index))


def _torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError("torch is required for native kernel dispatch") from exc
    return torch


def _stream_handle(torch: Any, tensor: Any, stream: Any | None) -> int:
    chosen = stream if stream is not None else torch.cuda.current_stream(tensor.device)
    return int(chosen.cuda_stream)


def _device_index(tensor: Any) -> int:
    return int(tensor.device.index or 0)


def _require_contiguous(name: str, tensor: Any) -> Any:
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous for native dispatch")
    return tensor


def _require_bfloat16_scale(torch: Any, name: str, tensor: Any) -> Any:
    if tensor.dtype != torch.bfloat16:
        raise ValueError(f"{name} must have dtype torch.bfloat16 for native dispatch; got {tensor.dtype}")
    return tensor


def _logical_problem_shape(kernel: KernelMetadata, a: Any, b: Any) -> tuple[int, int, int]:
    """(M, N, K) from operand shapes; packed int4 doubles the K extent; SwiGLU halves N."""
    k_scale = 2 if kernel.a_dtype is OperandDType.INT4 else 1
    layout = kernel.layout
    if layout not in (GemmLayout.NN, GemmLayout.NT, GemmLayout.TN):
        raise ValueError(f"native dispatch does not support layout={layout.value}")
    a_rows, a_cols = int(a.shape[-2]), int(a.shape[-1])
    b_rows, b_cols = int(b.shape[-2]), int(b.shape[-1])
    m, k_a = (a_cols, a_rows * k_scale) if layout is GemmLayout.TN else (a_rows, a_cols * k_scale)
    n, k_b = (b_rows, b_cols * k_scale) if layout is GemmLayout.NT else (b_cols, b_rows * k_scale)
    if kernel.epilogue is Epilogue.SWIGLU:
        if n % 2:
            raise ValueError("fused SwiGLU native dispatch requires the logical B output dimension to be even")
        n //= 2
    if k_a != k_b:
        raise ValueError(f"logical K mismatch for layout={layout.value}: A has {k_a}, B has {k_b}")
    return m, n, k_a


def _output_torch_dtype(torch: Any, kernel: KernelMetadata) -> Any:
    try:
        return {"bfloat16": torch.bfloat16, "float32": torch.float32}[kernel.output_dtype]
    except KeyError:
        raise ValueError(f"unsupported kernel output dtype: {kernel.output_dtype}") from None


def _scale_cols(scale: ScaleSpec, k: int) -> int:
    if scale.subchannel_size is None:
        raise ValueError("subchannel scale mode requires subchannel_size")
    return -(-k // scale.subchannel_size)


def _validate_scale_shapes(kernel: KernelMetadata, *, m: int, n: int, k: int, a_scale: Any, b_scale: Any) -> None:
    b_cols = 2 * n if kernel.epilogue is Epilogue.SWIGLU else n
    if kernel.scale.mode is ScaleMode.PER_CHANNEL:
        want_a, want_b = (m,), (b_cols,)
        if tuple(a_scale.shape) != want_a:
            raise ValueError(f"a_scale must have shape ({m},) for native dispatch; got {tuple(a_scale.shape)}")
        if tuple(b_scale.shape) != want_b:
            raise ValueError(f"b_scale must have shape ({b_cols},) for native dispatch; got {tuple(b_scale.shape)}")
        return
    groups = _scale_cols(kernel.scale, k)
    if tuple(a_scale.shape) != (m, groups):
        raise ValueError(f"a_scale must have shape ({m}, {groups}) for native dispatch; got {tuple(a_scale.shape)}")
    if tuple(b_scale.shape) != (groups, b_cols):
        raise ValueError(
            "subchannel b_scale must use weight-matched layout "
            f"{(groups, b_cols)} == (scale_cols, output_cols) for native dispatch; got {tuple(b_scale.shape)}. "
            f"If you have logical layout {(b_cols, groups)} == (output_cols, scale_cols), "
            "call pack_rhs_subchannel_scales(...) first."
        )


def launch_grid(kernel: KernelMetadata, m: int, n: int, *, num_sms: int = 148) -> tuple[int, int, int]:
    """Grid of a dense launch of ``kernel`` when every SM (pair of SMs) can hold a CTA (pair): informational,
    computed from the entry alone.  The library sizes the grid itself (``plan_dense`` asks it; the reference
    computed it in Python, native.py:306-332).  A ``STANDARD`` entry is counted in its single-CTA form."""
    tile_cols = 128 if kernel.epilogue is Epilogue.SWIGLU else 256
    pair = kernel.schedule is KernelSchedule.PERSISTENT_2CTA
    tile_rows, ctas = (256, 2) if pair else (128, 1)
    tiles = -(-m // tile_rows) * -(-n // tile_cols) * kernel.tile.split_k
    if kernel.schedule is KernelSchedule.TILE_PER_CTA:
        return (tiles * ctas, 1, 1)
    return (min(num_sms // ctas, tiles) * ctas, 1, 1)


def block_size(kernel: KernelMetadata) -> int:
    return kernel.tile.num_warps * THREADS_PER_WARP


SCHEDULE_LAUNCH = {
    # registry launch form -> (schedule, cta_group) of the C variant record
    KernelSchedule.STANDARD: (SCHEDULE_PERSISTENT, CTA_GROUP_AUTO),
    KernelSchedule.PERSISTENT: (SCHEDULE_PERSISTENT, CTA_GROUP_SINGLE),
    KernelSchedule.PERSISTENT_2CTA: (SCHEDULE_PERSISTENT, CTA_GROUP_PAIR),
    KernelSchedule.TILE_PER_CTA: (SCHEDULE_TILE_PER_CTA, CTA_GROUP_SINGLE),
}


def make_variant(
    *,
    dtype: OperandDType,
    layout: GemmLayout,
    scale: ScaleSpec,
    epilogue: Epilogue,
    out_dtype: int,
    split_k: int = 1,
    path: int = PATH_AUTO,
    group_m: int = 0,
    schedule: KernelSchedule = KernelSchedule.STANDARD,
    cta_group: int | None = None,
    accumulate_order: int | None = None,
    a_operand: int = A_OPERAND_AUTO,
    tail_balance: int = TAIL_AUTO,
    task_align: int = 0,
    wide_tiles: int = 0,
) -> GemmVariant:
    """The C variant record of one launch.  ``schedule`` is the registry's launch form; ``cta_group``
    (CTA_GROUP_*) overrides the form's CTA choice when given."""
    variant = GemmVariant()
    variant.dtype = DTYPE_CODES[dtype]
    variant.layout = LAYOUT_CODES[layout]
    variant.scale_mode = 1 if scale.mode is ScaleMode.SUBCHANNEL else 0
    variant.subchannel = int(scale.subchannel_size or 0)
    variant.epilogue = EPILOGUE_CODES[epilogue]
    variant.out_dtype = int(out_dtype)
    variant.split_k = int(split_k)
    variant.path = int(path)
    variant.group_m = int(group_m)
    variant.schedule, form_cta_group = SCHEDULE_LAUNCH[schedule]
    variant.cta_group = int(form_cta_group if cta_group is None else cta_group)
    variant.accumulate_order = int(_ACCUMULATION_ORDER if accumulate_order is None else accumulate_order)
    variant.a_operand = int(a_operand)
    variant.tail_balance = int(tail_balance)
    variant.wide_tiles = int(wide_tiles)   # WIDE_AUTO / WIDE_OFF / WIDE_ON: 256 x 512 tiles on CTA pairs
    variant.task_align = int(task_align)   # grouped forward: what the tasks' block starts are multiples of (0: not stated)
    return variant


def variant_for_kernel(kernel: KernelMetadata, *, out_dtype: int, path: int = PATH_AUTO) -> GemmVariant:
    """The variant record a registry entry launches with: its form, raster width and split factor."""
    return make_variant(
        dtype=kernel.a_dtype, layout=kernel.layout, scale=kernel.scale, epilogue=kernel.epilogue, out_dtype=out_dtype,
        split_k=kernel.tile.split_k, path=path, group_m=kernel.tile.group_size_m, schedule=kernel.schedule,
    )


def plan_dense(variant: GemmVariant, *, m: int, n: int, k: int, device_index: int = 0,
               library_path: str | Path | None = None) -> DensePlan:
    """What ``launch_dense`` would do for the variant and shape on the device (needs a CUDA device)."""
    library = load_dispatch_library(library_path)
    plan = DensePlan()
    rc = library.b200_int4_gemms_plan_dense(ctypes.byref(variant), int(device_index), int(m), int(n), int(k), ctypes.byref(plan))
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    return plan


def last_launch_path(*, library_path: str | Path | None = None) -> int:
    """LAUNCHED_* of the calling thread's most recent launch call."""
    return int(load_dispatch_library(library_path).b200_int4_gemms_last_launch_path())


_SLOW_PATH_WARNED: set[str] = set()


def _warn_if_cuda_core_path(library: ctypes.CDLL, what: str, requested_path: int = PATH_AUTO) -> None:
    """The reference raises where it has no kernel (api.py:136-138); this library has a CUDA-core kernel for
    the shapes and layouts its tensor-core kernel does not take.  It is correct and very slow: say so once."""
    if requested_path == PATH_SIMT or what in _SLOW_PATH_WARNED:
        return
    if int(library.b200_int4_gemms_last_launch_path()) != LAUNCHED_SIMT:
        return
    _SLOW_PATH_WARNED.add(what)
    import warnings

    warnings.warn(
        f"{what} ran on the CUDA-core kernel (no tensor cores): the tensor-core kernel needs 16-byte aligned operands "
        "and pitches and does not cover this layout / scale combination; pass path=PATH_TCGEN05 to fail instead",
        RuntimeWarning, stacklevel=3)


def launch_dense(
    variant: GemmVariant,
    *,
    device_index: int,
    stream_handle: int,
    a_ptr: int,
    b_ptr: int,
    a_scale_ptr: int,
    b_scale_ptr: int,
    c_ptr: int,
    m: int,
    n: int,
    k: int,
    workspace_ptr: int = 0,
    workspace_bytes: int = 0,
    library_path: str | Path | None = None,
) -> None:
    """Pointer-level dense launch (the reference's ``launch_hsaco``, native.py:335-381)."""
    library = load_dispatch_library(library_path)
    rc = library.b200_int4_gemms_launch_dense(
        ctypes.byref(variant), int(device_index), int(stream_handle),
        ctypes.c_void_p(int(a_ptr)), ctypes.c_void_p(int(b_ptr)),
        ctypes.c_void_p(int(a_scale_ptr)), ctypes.c_void_p(int(b_scale_ptr)),
        ctypes.c_void_p(int(c_ptr)), ctypes.c_void_p(int(workspace_ptr)), int(workspace_bytes),
        int(m), int(n), int(k),
    )
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    _warn_if_cuda_core_path(library, "a dense GEMM", int(variant.path))


def dense_workspace(variant: GemmVariant, *, m: int, n: int, k: int, device: Any, stream_handle: int,
                    library_path: str | Path | None = None) -> tuple[int, int]:
    """(pointer, bytes) of the scratch a launch can use (split-K slices, partial sums of the balanced tail); (0, 0)
    when the variant needs none.  The buffer is kept per (device, stream): launches that share it run in stream
    order and so never overlap."""
    library = load_dispatch_library(library_path)
    need = int(library.b200_int4_gemms_dense_workspace_bytes(ctypes.byref(variant), int(m), int(n), int(k)))
    if need == 0:
        return 0, 0
    torch = _torch()
    key = (int(device.index or 0), int(stream_handle), "dense_split_k")
    with _WORKSPACES_LOCK:
        scratch = _WORKSPACES.get(key)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                _RETIRED_WORKSPACES.append(scratch)
            scratch = torch.zeros(need, dtype=torch.uint8, device=device)  # the flag words of the balanced tail start out zero
            _WORKSPACES[key] = scratch
    return int(scratch.data_ptr()), int(scratch.numel())


def launch_generated_kernel(
    a: Any,
    b: Any,
    *,
    kernel: KernelMetadata,
    a_scale: Any,
    b_scale: Any,
    c: Any | None = None,
    gate: Any | None = None,
    root: str | Path | None = None,
    library_path: str | Path | None = None,
    stream: Any | None = None,
    path: int = PATH_AUTO,
) -> Any:
    """Run one registry entry on CUDA tensors and return the output tensor.

    Validation, allocation and error types follow the reference launcher
    (native.py:690-767): CUDA tensors and both scales required, operands contiguous, scales
    bf16, output dtype fixed by the entry, shape a multiple of the entry's tile record.
    """
    torch = _torch()
    if not torch.cuda.is_available():
        raise RuntimeError("native generated kernels require a CUDA torch device")
    if not getattr(a, "is_cuda", False):
        raise RuntimeError("native generated kernels require CUDA tensors")
    if a_scale is None or b_scale is None:
        raise ValueError("native generated kernels require a_scale and b_scale tensors")
    if kernel.epilogue is Epilogue.SWIGLU and gate is not None:
        raise ValueError("SwiGLU native dispatch uses fused up/gate columns; external gate is not supported")
    if kernel.epilogue is not Epilogue.NONE and kernel.tile.split_k != 1:
        raise ValueError(f"{kernel.epilogue.value} native dispatch currently supports SPLIT_K=1 only")
    if library_path is None and root is not None:
        library_path = native_library_path(root=root)

    a = _require_contiguous("a", a)
    b = _require_contiguous("b", b)
    a_scale = _require_bfloat16_scale(torch, "a_scale", _require_contiguous("a_scale", a_scale))
    b_scale = _require_bfloat16_scale(torch, "b_scale", _require_contiguous("b_scale", b_scale))
    m, n, k = _logical_problem_shape(kernel, a, b)
    want_dtype = _output_torch_dtype(torch, kernel)
    if c is None:
        c = torch.empty((m, n), device=a.device, dtype=want_dtype)
    c = _require_contiguous("c", c)
    if c.dtype != want_dtype:
        raise ValueError(f"output dtype must be {want_dtype}; got {c.dtype}")
    if tuple(c.shape[-2:]) != (m, n):
        raise ValueError(f"output shape must be {(m, n)}; got {tuple(c.shape[-2:])}")
    LaunchShape(m, n, k).validate_for(kernel)
    _validate_scale_shapes(kernel, m=m, n=n, k=k, a_scale=a_scale, b_scale=b_scale)

    variant = variant_for_kernel(kernel, out_dtype=OUT_F32 if want_dtype is torch.float32 else OUT_BF16, path=path)
    stream_handle = _stream_handle(torch, a, stream)
    workspace_ptr, workspace_bytes = dense_workspace(variant, m=m, n=n, k=k, device=a.device, stream_handle=stream_handle,
                                                     library_path=library_path)
    launch_dense(
        variant,
        device_index=_device_index(a),
        stream_handle=stream_handle,
        a_ptr=a.data_ptr(),
        b_ptr=b.data_ptr(),
        a_scale_ptr=a_scale.data_ptr(),
        b_scale_ptr=b_scale.data_ptr(),
        c_ptr=c.data_ptr(),
        m=m,
        n=n,
        k=k,
        workspace_ptr=workspace_ptr,
        workspace_bytes=workspace_bytes,
        library_path=library_path,
    )
    return c


def launch_accumulators(
    a: Any,
    b: Any,
    *,
    dtype: OperandDType,
    layout: GemmLayout = GemmLayout.NN,
    path: int = PATH_AUTO,
    library_path: str | Path | None = None,
    stream: Any | None = None,
) -> Any:
    """Raw int32 accumulators ``A_q @ B_q`` of the device path, for bit-exact checks."""
    torch = _torch()
    if not getattr(a, "is_cuda", False):
        raise RuntimeError("native generated kernels require CUDA tensors")
    probe = KernelMetadata(
        kernel_id="accumulators", arch="", a_dtype=dtype, b_dtype=dtype, acc_dtype="int32",
        output_dtype="int32", scale_dtype="bfloat16", scale=ScaleSpec(ScaleMode.PER_CHANNEL),
        epilogue=Epilogue.NONE, tile=None, device_kernel="", layout=layout,  # type: ignore[arg-type]
    )
    m, n, k = _logical_problem_shape(probe, _require_contiguous("a", a), _require_contiguous("b", b))
    c = torch.empty((m, n), device=a.device, dtype=torch.int32)
    variant = make_variant(dtype=dtype, layout=layout, scale=probe.scale, epilogue=Epilogue.NONE,
                           out_dtype=OUT_S32, path=path)
    launch_dense(
        variant, device_index=_device_index(a), stream_handle=_stream_handle(torch, a, stream),
        a_ptr=a.data_ptr(), b_ptr=b.data_ptr(), a_scale_ptr=0, b_scale_ptr=0, c_ptr=c.data_ptr(),
        m=m, n=n, k=k, library_path=library_path,
    )
    return c


def launch_ragged_fwd_kernel(
    lhs: Any,
    rhs: Any,
    *,
    group_info: Any,
    a_scale: Any,
    b_scale: Any,
    out: Any,
    scale: ScaleSpec,
    config: Any,
    layout: GemmLayout,
    variant: str = "",
    rows: int,
    cols: int,
    k_packed: int,
    scale_cols: int,
    root: str | Path | None = None,
    library_path: str | Path | None = None,
    stream: Any | None = None,
    path: int = PATH_AUTO,
    a_operand: int = A_OPERAND_AUTO,
    wide_tiles: int = WIDE_AUTO,
) -> Any:
    """Grouped forward launch over prebuilt row-block tasks (reference native.py:533-600)."""
    torch = _torch()
    if not torch.cuda.is_available() or not getattr(lhs, "is_cuda", False):
        raise RuntimeError("native ragged kernels require CUDA tensors")
    a_scale = _require_bfloat16_scale(torch, "a_scale", _require_contiguous("a_scale", a_scale))
    b_scale = _require_bfloat16_scale(torch, "b_scale", _require_contiguous("b_scale", b_scale))
    out = _require_contiguous("out", out)
    if group_info.num_tasks == 0:
        return out
    if library_path is None and root is not None:
        library_path = native_library_path(root=root)
    library = load_dispatch_library(library_path)
    record = make_variant(
        dtype=OperandDType.INT4, layout=layout, scale=scale, epilogue=Epilogue.NONE,
        out_dtype=OUT_F32 if out.dtype is torch.float32 else OUT_BF16, path=path, a_operand=a_operand, wide_tiles=wide_tiles,
        # a transposed lhs reaches the tensor cores only when every task starts on a multiple of 16 rows
        task_align=int(getattr(group_info, "align_tile", None) or 0),
    )
    groups = int(rhs.shape[0])
    task_arrays = (
        ctypes.c_void_p(group_info.group_id.data_ptr()), ctypes.c_void_p(group_info.block_start.data_ptr()),
        ctypes.c_void_p(group_info.actual_start.data_ptr()), ctypes.c_void_p(group_info.actual_end.data_ptr()),
    )
    operands = (
        ctypes.c_void_p(lhs.data_ptr()), ctypes.c_void_p(rhs.data_ptr()),
        ctypes.c_void_p(a_scale.data_ptr()), ctypes.c_void_p(b_scale.data_ptr()),
    )
    sizes = (int(rows), int(cols), int(k_packed), int(scale_cols), int(group_info.num_tasks), groups, int(config.block_m))
    device_count = getattr(group_info, "device_num_tasks", None)
    device_overflow = getattr(group_info, "device_overflow", None)
    if device_count is not None:
        # tasks built on the device: num_tasks is the capacity of the arrays, the real count stays on the GPU
        rc = library.b200_int4_gemms_launch_ragged_fwd_device_tasks(
            ctypes.byref(record), _device_index(lhs), _stream_handle(torch, lhs, stream), *operands, *task_arrays,
            ctypes.c_void_p(device_count.data_ptr()),
            ctypes.c_void_p(device_overflow.data_ptr() if device_overflow is not None else 0),
            ctypes.c_void_p(out.data_ptr()), *sizes)
    else:
        rc = library.b200_int4_gemms_launch_ragged_fwd(
            ctypes.byref(record), _device_index(lhs), _stream_handle(torch, lhs, stream), *operands, *task_arrays,
            ctypes.c_void_p(out.data_ptr()), *sizes)
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    _warn_if_cuda_core_path(library, f"a grouped forward dot (layout {layout.value})", path)
    return out


def launch_ragged_bwd_kernel(
    lhs: Any,
    rhs: Any,
    group_sizes: Any,
    *,
    a_scale: Any,
    b_scale: Any,
    out: Any,
    scale: ScaleSpec,
    config: Any,
    layout: GemmLayout,
    variant: str = "",
    rows: int,
    cols: int,
    k_packed: int,
    scale_cols: int,
    root: str | Path | None = None,
    library_path: str | Path | None = None,
    stream: Any | None = None,
    path: int = PATH_AUTO,
) -> Any:
    """Grouped K-ragged backward launch (reference native.py:603-667); ``group_sizes`` int64 on device."""
    torch = _torch()
    if not torch.cuda.is_available() or not getattr(lhs, "is_cuda", False):
        raise RuntimeError("native ragged kernels require CUDA tensors")
    a_scale = _require_bfloat16_scale(torch, "a_scale", _require_contiguous("a_scale", a_scale))
    b_scale = _require_bfloat16_scale(torch, "b_scale", _require_contiguous("b_scale", b_scale))
    out = _require_contiguous("out", out)
    if group_sizes.dtype != torch.int64 or not group_sizes.is_contiguous():
        group_sizes = group_sizes.to(torch.int64).contiguous()
    if library_path is None and root is not None:
        library_path = native_library_path(root=root)
    library = load_dispatch_library(library_path)
    pair_tiles = getattr(config, "pair_tiles", None)
    record = make_variant(
        dtype=OperandDType.INT4, layout=layout, scale=scale, epilogue=Epilogue.NONE, out_dtype=OUT_F32, path=path,
        cta_group=CTA_GROUP_AUTO if pair_tiles is None else (CTA_GROUP_PAIR if pair_tiles else CTA_GROUP_SINGLE),
    )
    groups = int(lhs.shape[0])
    if groups == 0 or rows == 0 or cols == 0:
        return out
    rc = library.b200_int4_gemms_launch_ragged_bwd(
        ctypes.byref(record), _device_index(lhs), _stream_handle(torch, lhs, stream),
        ctypes.c_void_p(lhs.data_ptr()), ctypes.c_void_p(rhs.data_ptr()),
        ctypes.c_void_p(a_scale.data_ptr()), ctypes.c_void_p(b_scale.data_ptr()),
        ctypes.c_void_p(group_sizes.data_ptr()), ctypes.c_void_p(out.data_ptr()),
        int(rows), int(cols), int(k_packed), int(scale_cols), groups,
    )
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    _warn_if_cuda_core_path(library, f"a grouped backward dot (layout {layout.value})", path)
    return out


def unpack_int4_on_device(packed: Any, *, library_path: str | Path | None = None, stream: Any | None = None) -> Any:
    """uint8 ``[rows, Kb]`` -> int8 ``[rows, 2*Kb]`` on the GPU (the pre-expand path of the A/B comparison)."""
    torch = _torch()
    if not getattr(packed, "is_cuda", False):
        raise RuntimeError("native kernels require CUDA tensors")
    packed = _require_contiguous("packed", packed)
    rows = int(packed.numel() // packed.shape[-1]) if packed.numel() else 0
    out = torch.empty((*packed.shape[:-1], packed.shape[-1] * 2), device=packed.device, dtype=torch.int8)
    library = load_dispatch_library(library_path)
    rc = library.b200_int4_gemms_unpack_int4(
        _device_index(packed), _stream_handle(torch, packed, stream),
        ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, int(packed.shape[-1]),
    )
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    return out


# device scratch kept per (device, stream, purpose); a buffer that was outgrown stays alive because a
# kernel launched earlier may still be using it
_WORKSPACES: dict[tuple[int, int, str], Any] = {}
_RETIRED_WORKSPACES: list[Any] = []
_WORKSPACES_LOCK = threading.Lock()


def group_info_on_device(
    group_sizes: Any, tile: int, *, align_tile: int = 8, max_tasks: int,
    library_path: str | Path | None = None, stream: Any | None = None,
) -> tuple[Any, Any, Any, Any, Any, Any]:
    """Task arrays of the grouped forward pass built by ``b200_int4_gemms_group_info``.

    Returns ``(group_id, block_start, actual_start, actual_end, num_tasks, overflow)``: four int64
    tensors of ``max_tasks`` entries and two int32 one-element tensors, all on the device of
    ``group_sizes``.  Nothing is copied to the host.
    """
    torch = _torch()
    if not getattr(group_sizes, "is_cuda", False):
        raise RuntimeError("group_info_on_device requires a CUDA group_sizes tensor")
    library = load_dispatch_library(library_path)
    sizes = group_sizes.to(torch.int64).contiguous()
    arrays = [torch.empty(int(max_tasks), device=sizes.device, dtype=torch.int64) for _ in range(4)]
    counters = torch.empty(2, device=sizes.device, dtype=torch.int32)
    rc = library.b200_int4_gemms_group_info(
        _device_index(sizes), _stream_handle(torch, sizes, stream), ctypes.c_void_p(sizes.data_ptr()),
        int(sizes.numel()), int(tile), int(align_tile), *[ctypes.c_void_p(t.data_ptr()) for t in arrays],
        int(max_tasks), ctypes.c_void_p(counters[0:1].data_ptr()), ctypes.c_void_p(counters[1:2].data_ptr()))
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    return arrays[0], arrays[1], arrays[2], arrays[3], counters[0:1], counters[1:2]


STATIC_SCRATCH_MAX_GROUPS = 4096  # B200_STATIC_SCRATCH_MAX_GROUPS of the header


def launch_ragged_bwd_flat_kernel(
    lhs: Any, rhs: Any, group_sizes: Any, *, a_scale: Any, b_scale: Any, out: Any, tokens: int,
    library_path: str | Path | None = None, stream: Any | None = None, path: int = PATH_AUTO,
    static_scratch: bool = False,
) -> Any:
    """Grouped backward launch over flat token-packed operands (``b200_int4_gemms_launch_ragged_bwd_flat``).

    ``static_scratch=True`` goes through ``b200_int4_gemms_launch_ragged_bwd_flat_static``: no workspace
    tensor is made here and the library allocates nothing; ``group_sizes`` must already be a contiguous
    int64 CUDA tensor (converting it would allocate)."""
    torch = _torch()
    if not torch.cuda.is_available() or not getattr(lhs, "is_cuda", False):
        raise RuntimeError("native ragged kernels require CUDA tensors")
    a_scale = _require_bfloat16_scale(torch, "a_scale", _require_contiguous("a_scale", a_scale))
    b_scale = _require_bfloat16_scale(torch, "b_scale", _require_contiguous("b_scale", b_scale))
    library = load_dispatch_library(library_path)
    record = make_variant(dtype=OperandDType.INT4, layout=GemmLayout.TN, scale=ScaleSpec(ScaleMode.PER_CHANNEL),
                          epilogue=Epilogue.NONE, out_dtype=OUT_F32, path=path)
    groups = int(group_sizes.numel())
    device_index, stream_handle = _device_index(lhs), _stream_handle(torch, lhs, stream)
    if static_scratch:
        if group_sizes.dtype is not torch.int64 or not group_sizes.is_contiguous() or not group_sizes.is_cuda:
            raise ValueError("static_scratch=True requires group_sizes as a contiguous int64 CUDA tensor")
        rc = library.b200_int4_gemms_launch_ragged_bwd_flat_static(
            ctypes.byref(record), device_index, stream_handle,
            ctypes.c_void_p(lhs.data_ptr()), ctypes.c_void_p(rhs.data_ptr()),
            ctypes.c_void_p(a_scale.data_ptr()), ctypes.c_void_p(b_scale.data_ptr()),
            ctypes.c_void_p(group_sizes.data_ptr()), ctypes.c_void_p(out.data_ptr()),
            int(lhs.shape[1]), int(rhs.shape[1]), int(tokens), groups)
        if rc != 0:
            raise RuntimeError(_library_last_error(library))
        return out
    need = int(library.b200_int4_gemms_ragged_bwd_flat_workspace_bytes(groups))
    key = (device_index, stream_handle, "bwd_flat")
    with _WORKSPACES_LOCK:  # one scratch buffer per (device, stream): calls that share one must not overlap
        scratch = _WORKSPACES.get(key)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                _RETIRED_WORKSPACES.append(scratch)
            scratch = torch.empty(max(need, 4096), dtype=torch.uint8, device=lhs.device)
            _WORKSPACES[key] = scratch
    sizes = group_sizes.to(torch.int64).contiguous()
    rc = library.b200_int4_gemms_launch_ragged_bwd_flat(
        ctypes.byref(record), device_index, stream_handle,
        ctypes.c_void_p(lhs.data_ptr()), ctypes.c_void_p(rhs.data_ptr()),
        ctypes.c_void_p(a_scale.data_ptr()), ctypes.c_void_p(b_scale.data_ptr()),
        ctypes.c_void_p(sizes.data_ptr()), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_void_p(scratch.data_ptr()), int(scratch.numel()),
        int(lhs.shape[1]), int(rhs.shape[1]), int(tokens), groups)
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    return out


def quantize_on_device(x: Any, *, bits: int, scale: float, library_path: str | Path | None = None,
                       stream: Any | None = None) -> Any:
    """bf16 ``[..., cols]`` -> packed int4 ``[..., ceil(cols/2)]`` uint8 (bits=4) or int8 codes (bits=8)."""
    torch = _torch()
    if not getattr(x, "is_cuda", False) or x.dtype is not torch.bfloat16:
        raise RuntimeError("quantize_on_device requires a CUDA bfloat16 tensor")
    x = _require_contiguous("x", x)
    cols = int(x.shape[-1])
    rows = int(x.numel() // cols) if cols else 0
    if bits == 4:
        out = torch.empty((*x.shape[:-1], (cols + 1) // 2), device=x.device, dtype=torch.uint8)
    else:
        out = torch.empty(x.shape, device=x.device, dtype=torch.int8)
    library = load_dispatch_library(library_path)
    rc = library.b200_int4_gemms_quantize(_device_index(x), _stream_handle(torch, x, stream), ctypes.c_void_p(x.data_ptr()),
                                          ctypes.c_void_p(out.data_ptr()), rows, cols, int(bits), float(scale))
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    return out


def repack_tokens_on_device(packed: Any, *, library_path: str | Path | None = None, stream: Any | None = None) -> Any:
    """int4 packed along features ``[rows, cols/2]`` -> packed along tokens ``[ceil(rows/2), cols]``."""
    torch = _torch()
    if not getattr(packed, "is_cuda", False) or packed.dtype is not torch.uint8 or packed.ndim != 2:
        raise RuntimeError("repack_tokens_on_device requires a 2-D CUDA uint8 tensor")
    packed = _require_contiguous("packed", packed)
    rows, cols = int(packed.shape[0]), 2 * int(packed.shape[1])
    out = torch.empty(((rows + 1) // 2, cols), device=packed.device, dtype=torch.uint8)
    library = load_dispatch_library(library_path)
    rc = library.b200_int4_gemms_repack_tokens(_device_index(packed), _stream_handle(torch, packed, stream),
                                               ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, cols)
    if rc != 0:
        raise RuntimeError(_library_last_error(library))
    return out
