"""Benchmark-and-pick for dense registry entries and for grouped-dot launch configurations.

Surface of the reference's ``autotune.py``: ``autotune`` (:148-220), ``find_autotune_candidates``
(:115-145), ``AutotuneResult`` (:47-54), ``autotune_ragged_dot`` (:259-386),
``default_ragged_dot_candidates`` (:223-256), ``RaggedAutotuneCandidate`` / ``RaggedAutotuneResult``
/ ``RaggedDotMode`` (:40-88), ``generated_shape_for_kernel`` (:91-99).  Both tuners accept an
injected ``benchmark_runner`` so their bookkeeping can be exercised without a GPU.

Device timing uses CUDA events (see :mod:`benchmarking`).  TOPS conventions are the
reference's: ``2*M*N*K / t``; a fused SwiGLU counts both projections (x2); the backward grouped
dot uses ``K = sum(group_sizes)``.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Iterable, Sequence

from .api import explicit_mm
from .benchmarking import (
    BenchmarkDatabase,
    BenchmarkRecord,
    BenchmarkShape,
    benchmark_device_callable,
    tops_for_runtime,
)
from .heuristics import kernel_supports_shape
from .metadata import Epilogue, GemmLayout, KernelMetadata, KernelSchedule, OperandDType, ScaleMode, ScaleSpec
from .native import launch_generated_kernel
from .quant import pack_int4_k_major
from .ragged import (
    RaggedBwdDotConfig,
    RaggedDotConfig,
    _check_layout,
    ragged_config_label,
    ragged_dot_int4,
    ragged_dot_int4_bwd,
)
from .registry import KernelRegistry, default_registry, launch_signature

BenchmarkRunner = Callable[[KernelMetadata, BenchmarkShape], BenchmarkRecord]
RaggedBenchmarkRunner = Callable[["RaggedAutotuneCandidate", BenchmarkShape], BenchmarkRecord]


class RaggedDotMode(str, Enum):
    """Which grouped dot to tune."""

    FWD = "fwd"
    BWD = "bwd"


@dataclass(frozen=True, slots=True)
class AutotuneResult:
    shape: BenchmarkShape
    candidates: tuple[KernelMetadata, ...]
    records: tuple[BenchmarkRecord, ...]
    best_kernel: KernelMetadata
    best_record: BenchmarkRecord
    benchmark_db: BenchmarkDatabase


@dataclass(frozen=True, slots=True)
class RaggedAutotuneCandidate:
    """One grouped-dot launch configuration under test."""

    mode: RaggedDotMode
    layout: GemmLayout
    scale: ScaleSpec
    config: RaggedDotConfig | RaggedBwdDotConfig

    @property
    def config_label(self) -> str:
        return ragged_config_label(self.config)

    @property
    def kernel_id(self) -> str:
        parts = ("ragged_dot_int4", self.mode.value, self.layout.value, self.scale.label.lower(), self.config_label.lower())
        return "_".join(parts)


@dataclass(frozen=True, slots=True)
class RaggedAutotuneResult:
    shape: BenchmarkShape
    mode: RaggedDotMode
    layout: GemmLayout
    scale: ScaleSpec
    group_sizes: tuple[int, ...]
    candidates: tuple[RaggedAutotuneCandidate, ...]
    records: tuple[BenchmarkRecord, ...]
    best_candidate: RaggedAutotuneCandidate
    best_record: BenchmarkRecord
    benchmark_db: BenchmarkDatabase


def generated_shape_for_kernel(kernel: KernelMetadata, *, root: str | Path | None = None) -> BenchmarkShape | None:
    """Shape a variant was specialised for.  The sm_100a kernels take their sizes at run time,
    so no entry has one and this always answers ``None`` (the reference read it from a
    per-kernel JSON record)."""
    del kernel, root
    return None


def find_autotune_candidates(
    *,
    m: int,
    n: int,
    k: int,
    dtype: OperandDType,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec,
    epilogue: Epilogue,
    schedule: KernelSchedule | None = None,
    registry: KernelRegistry = default_registry,
    root: str | Path | None = None,
    require_exact_generated_shape: bool = True,
) -> tuple[KernelMetadata, ...]:
    """Entries of the requested cell that accept the shape and launch differently from one another.

    ``schedule=None`` (the default) spans every launch form: the library's own choice, one CTA per tile,
    CTA pairs, one CTA per tile without the persistent grid, each with its raster widths and split-K factors.
    Entries that differ only in the shape multiples they are registered for run the same launch, so one per
    launch signature is kept (the one with the largest multiples).  ``root`` and
    ``require_exact_generated_shape`` are accepted for compatibility; every entry is compiled into the
    library and none is tied to a single shape.
    """
    del root, require_exact_generated_shape
    kept: dict[tuple, KernelMetadata] = {}
    for kernel in registry.all():
        if not (kernel.a_dtype is dtype and kernel.b_dtype is dtype and kernel.layout is layout and kernel.scale == scale
                and kernel.epilogue is epilogue and (schedule is None or kernel.schedule is schedule)
                and kernel_supports_shape(kernel, m=m, n=n, k=k)):
            continue
        signature = launch_signature(kernel)
        held = kept.get(signature)
        if held is None or kernel.tile.block_m * kernel.tile.block_n > held.tile.block_m * held.tile.block_n:
            kept[signature] = kernel
    return tuple(kept.values())


def _load_db(benchmark_db: BenchmarkDatabase | None, path: str | Path | None) -> tuple[BenchmarkRecord, ...]:
    if benchmark_db is None and path is not None and Path(path).exists():
        benchmark_db = BenchmarkDatabase.load(Path(path))
    return tuple(benchmark_db.records()) if benchmark_db is not None else ()


def autotune(
    *,
    m: int,
    n: int,
    k: int,
    dtype: OperandDType,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec,
    epilogue: Epilogue,
    schedule: KernelSchedule | None = None,
    registry: KernelRegistry = default_registry,
    benchmark_db: BenchmarkDatabase | None = None,
    benchmark_db_path: str | Path | None = None,
    root: str | Path | None = None,
    library_path: str | Path | None = None,
    warmup_ms: int = 25,
    rep_ms: int = 100,
    validate: bool = False,
    benchmark_runner: BenchmarkRunner | None = None,
) -> AutotuneResult:
    """Time every candidate entry on seeded synthetic operands and return the fastest.

    The candidates are launches that differ (see ``find_autotune_candidates``): with ``schedule=None`` the
    result says which launch form, raster width and split factor is fastest for the shape."""
    shape = BenchmarkShape(m, n, k)
    candidates = find_autotune_candidates(
        m=m, n=n, k=k, dtype=dtype, layout=layout, scale=scale, epilogue=epilogue,
        schedule=schedule, registry=registry, root=root,
    )
    if not candidates:
        raise LookupError(
            f"no pregenerated kernels match dtype={dtype.value}, layout={layout.value}, scale={scale.label}, "
            f"epilogue={epilogue.value}, schedule={schedule.value if schedule is not None else 'any'}, shape=({m}, {n}, {k})"
        )
    earlier = _load_db(benchmark_db, benchmark_db_path)

    def default_runner(kernel: KernelMetadata, tuned: BenchmarkShape) -> BenchmarkRecord:
        return _benchmark_native_kernel(
            kernel, tuned, root=root, library_path=library_path, warmup_ms=warmup_ms, rep_ms=rep_ms, validate=validate
        )

    run = benchmark_runner or default_runner
    records = tuple(run(kernel, shape) for kernel in candidates)
    if not records:
        raise RuntimeError("autotune produced no benchmark records")
    good = [record for record in records if record.success]
    if not good:
        raise RuntimeError("autotune produced no successful benchmark records")
    best_record = max(good, key=lambda record: record.tops)
    best_kernel = next(kernel for kernel in candidates if kernel.kernel_id == best_record.kernel_id)
    merged = BenchmarkDatabase((*earlier, *records))
    if benchmark_db_path is not None:
        merged.save(Path(benchmark_db_path))
    return AutotuneResult(shape, candidates, records, best_kernel, best_record, merged)


def _check_ragged_mode(mode: RaggedDotMode) -> RaggedDotMode:
    if type(mode) is not RaggedDotMode:
        raise TypeError(f"mode must be a RaggedDotMode, got {type(mode).__name__}")
    return mode


# Task heights of the forward kernel (rows per task, column tile, K stage, tasks per raster group): 256-row tasks
# run on CTA pairs, the others on single CTAs.
_FWD_SEEDS = ((256, 256, 128, 1), (128, 256, 128, 1), (64, 256, 128, 1), (32, 256, 128, 1))
_BWD_SEEDS = ((128, 256, 128),)


def default_ragged_dot_candidates(
    mode: RaggedDotMode,
    *,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec = ScaleSpec(ScaleMode.PER_CHANNEL),
    split_ks: Iterable[int] = (1, 2),
) -> tuple[RaggedAutotuneCandidate, ...]:
    """Launch configurations worth timing: task heights for the forward dot, split factors for the backward one."""
    mode = _check_ragged_mode(mode)
    layout = _check_layout(layout)
    if mode is RaggedDotMode.FWD:
        # pair_tasks=False: a candidate runs with the task height it names (the default would widen 128 to 256)
        pair_ok = layout is GemmLayout.NN and (scale.mode is ScaleMode.PER_CHANNEL or (scale.subchannel_size or 0) >= 128)
        configs: list[Any] = [
            RaggedDotConfig(block_m=bm, block_n=bn, block_k=bk, group_size_tasks=gst, pair_tasks=False)
            for bm, bn, bk, gst in _FWD_SEEDS
            if bm <= 128 or pair_ok
        ]
    else:
        configs = [
            RaggedBwdDotConfig(block_m=bm, block_n=bn, block_k=bk, split_k=split)
            for bm, bn, bk in _BWD_SEEDS
            for split in tuple(split_ks)
        ]
    return tuple(RaggedAutotuneCandidate(mode=mode, layout=layout, scale=scale, config=cfg) for cfg in configs)


def _balanced_sizes(total: int, groups: int) -> tuple[int, ...]:
    if groups <= 0:
        raise ValueError("groups must be positive")
    share, extra = divmod(total, groups)
    return tuple(share + (1 if index < extra else 0) for index in range(groups))


def _normalize_ragged_group_sizes(
    *, mode: RaggedDotMode, group_sizes: Sequence[int] | Any | None, groups: int, m: int, k: int
) -> tuple[int, ...]:
    total = m if mode is RaggedDotMode.FWD else k
    if group_sizes is None:
        values = _balanced_sizes(total, groups)
    else:
        raw = group_sizes
        for method in ("detach", "cpu", "tolist"):
            if hasattr(raw, method):
                raw = getattr(raw, method)()
        values = tuple(int(value) for value in raw)
    if not values:
        raise ValueError("group_sizes must contain at least one group")
    if min(values) < 0:
        raise ValueError("group_sizes must be non-negative")
    if sum(values) != total:
        if mode is RaggedDotMode.FWD:
            raise ValueError(f"forward group_sizes must sum to M={m}; got {sum(values)}")
        raise ValueError(f"backward group_sizes must sum to K={k}; got {sum(values)}")
    return values


def _normalize_ragged_k_capacity(
    *, mode: RaggedDotMode, k: int, k_capacity: int | None, group_sizes: tuple[int, ...]
) -> int:
    if mode is RaggedDotMode.FWD:
        if k_capacity is not None and k_capacity != k:
            raise ValueError("k_capacity is only configurable for backward ragged dot")
        return k
    longest = max(group_sizes)
    capacity = longest if k_capacity is None else int(k_capacity)
    if capacity <= 0:
        raise ValueError("k_capacity must be positive")
    if capacity < longest:
        raise ValueError(f"backward k_capacity must be >= max(group_sizes)={longest}; got {capacity}")
    return capacity


def _normalize_ragged_candidates(
    *,
    mode: RaggedDotMode,
    layout: GemmLayout,
    scale: ScaleSpec,
    candidates: Iterable[RaggedAutotuneCandidate | RaggedDotConfig | RaggedBwdDotConfig] | None,
    split_ks: Iterable[int],
) -> tuple[RaggedAutotuneCandidate, ...]:
    if candidates is None:
        return default_ragged_dot_candidates(mode, layout=layout, scale=scale, split_ks=split_ks)
    wanted_config = RaggedDotConfig if mode is RaggedDotMode.FWD else RaggedBwdDotConfig
    out: list[RaggedAutotuneCandidate] = []
    for item in candidates:
        if isinstance(item, RaggedAutotuneCandidate):
            if item.mode is not mode:
                raise ValueError(f"candidate mode {item.mode.value} does not match requested {mode.value}")
            if item.layout is not layout:
                raise ValueError(f"candidate layout {item.layout.value} does not match requested {layout.value}")
            if item.scale != scale:
                raise ValueError(f"candidate scale {item.scale.label} does not match requested {scale.label}")
            if not isinstance(item.config, wanted_config):
                side = "forward" if mode is RaggedDotMode.FWD else "backward"
                raise TypeError(f"{side} ragged-dot candidates must use {wanted_config.__name__}")
            out.append(item)
        elif isinstance(item, wanted_config):
            out.append(RaggedAutotuneCandidate(mode=mode, layout=layout, scale=scale, config=item))
        else:
            raise TypeError(f"unsupported ragged autotune candidate {item!r}")
    return tuple(out)


def _ragged_record_metadata(
    *, candidate: RaggedAutotuneCandidate, group_sizes: tuple[int, ...], k_capacity: int, warmup_ms: int, rep_ms: int
) -> dict[str, Any]:
    return {
        "family": "ragged_dot_int4",
        "mode": candidate.mode.value,
        "layout": candidate.layout.value,
        "scale": candidate.scale.label,
        "config": candidate.config_label,
        "group_sizes": list(group_sizes),
        "groups": len(group_sizes),
        "k_capacity": k_capacity,
        "warmup_ms": warmup_ms,
        "rep_ms": rep_ms,
    }


def autotune_ragged_dot(
    *,
    mode: RaggedDotMode,
    m: int,
    n: int,
    k: int,
    k_capacity: int | None = None,
    group_sizes: Sequence[int] | Any | None = None,
    groups: int = 8,
    layout: GemmLayout = GemmLayout.NN,
    scale: ScaleSpec = ScaleSpec(ScaleMode.PER_CHANNEL),
    candidates: Iterable[RaggedAutotuneCandidate | RaggedDotConfig | RaggedBwdDotConfig] | None = None,
    split_ks: Iterable[int] = (1, 2),
    benchmark_db: BenchmarkDatabase | None = None,
    benchmark_db_path: str | Path | None = None,
    warmup_ms: int = 25,
    rep_ms: int = 100,
    continue_on_error: bool = True,
    benchmark_runner: RaggedBenchmarkRunner | None = None,
) -> RaggedAutotuneResult:
    """Time grouped-dot configurations for one run-time shape.

    Forward: ``group_sizes`` partitions the ``M`` rows.  Backward: it partitions the reduction
    work ``K`` between groups, and synthetic operands are padded to ``k_capacity`` per group
    (default: the longest group).
    """
    if min(m, n, k) <= 0:
        raise ValueError("m, n, and k must be positive")
    if warmup_ms < 0:
        raise ValueError("warmup_ms must be non-negative")
    if rep_ms <= 0:
        raise ValueError("rep_ms must be positive")
    mode = _check_ragged_mode(mode)
    layout = _check_layout(layout)
    sizes = _normalize_ragged_group_sizes(mode=mode, group_sizes=group_sizes, groups=groups, m=m, k=k)
    capacity = _normalize_ragged_k_capacity(mode=mode, k=k, k_capacity=k_capacity, group_sizes=sizes)
    shape = BenchmarkShape(m=m, n=n, k=k)
    pool = _normalize_ragged_candidates(mode=mode, layout=layout, scale=scale, candidates=candidates, split_ks=split_ks)
    if not pool:
        raise LookupError(f"no ragged-dot autotune candidates for mode={mode.value}, layout={layout.value}")
    earlier = _load_db(benchmark_db, benchmark_db_path)

    def default_runner(candidate: RaggedAutotuneCandidate, record_shape: BenchmarkShape) -> BenchmarkRecord:
        return _benchmark_ragged_candidate(
            candidate, record_shape, m=m, n=n, k_capacity=capacity, group_sizes=sizes, warmup_ms=warmup_ms, rep_ms=rep_ms
        )

    run = benchmark_runner or default_runner
    records: list[BenchmarkRecord] = []
    for candidate in pool:
        try:
            records.append(run(candidate, shape))
        except Exception as exc:
            if not continue_on_error:
                raise
            info = _ragged_record_metadata(
                candidate=candidate, group_sizes=sizes, k_capacity=capacity, warmup_ms=warmup_ms, rep_ms=rep_ms
            )
            records.append(
                BenchmarkRecord(
                    kernel_id=candidate.kernel_id, shape=shape, runtime_ms=float("inf"), tops=0.0, iterations=0,
                    warmup=warmup_ms, success=False, notes="ragged-dot autotune candidate failed",
                    metadata={"error": repr(exc), **info},
                )
            )
    good = [record for record in records if record.success]
    if not good:
        raise RuntimeError("ragged-dot autotune produced no successful benchmark records")
    best_record = max(good, key=lambda record: record.tops)
    best_candidate = next(c for c in pool if c.kernel_id == best_record.kernel_id)
    merged = BenchmarkDatabase((*earlier, *records))
    if benchmark_db_path is not None:
        merged.save(Path(benchmark_db_path))
    return RaggedAutotuneResult(
        shape=shape, mode=mode, layout=layout, scale=scale, group_sizes=sizes, candidates=pool,
        records=tuple(records), best_candidate=best_candidate, best_record=best_record, benchmark_db=merged,
    )


# ----------------------------------------------------------------------------------------------
# seeded synthetic operands
# ----------------------------------------------------------------------------------------------
def _stable_seed(text: str) -> int:
    return int.from_bytes(hashlib.sha256(text.encode()).digest()[:4], "little")


def _random_codes(torch: Any, shape: tuple[int, ...], dtype: OperandDType, generator: Any) -> Any:
    low, high = (-8, 8) if dtype is OperandDType.INT4 else (-127, 128)
    return torch.randint(low, high, shape, generator=generator, dtype=torch.int8)


def _random_scales(torch: Any, shape: tuple[int, ...], generator: Any) -> Any:
    return ((torch.rand(shape, generator=generator) + 0.5) * 0.05).to(torch.bfloat16)


def _store_operand(codes: Any, *, int4: bool, k_last: bool) -> Any:
    """``codes`` is logical with K as its last axis.  Pack along K, then put K where the layout wants it."""
    stored = pack_int4_k_major(codes) if int4 else codes
    return stored.contiguous() if k_last else stored.transpose(-2, -1).contiguous()


def make_dense_inputs(kernel: KernelMetadata, shape: BenchmarkShape, *, seed: int | None = None) -> tuple[Any, Any, Any, Any]:
    """CPU tensors ``(a, b, a_scale, b_scale)`` in ``kernel``'s layout: uniform codes, scales in [0.025, 0.075)."""
    import torch

    generator = torch.Generator().manual_seed(_stable_seed(kernel.kernel_id) if seed is None else seed)
    int4 = kernel.a_dtype is OperandDType.INT4
    out_cols = 2 * shape.n if kernel.epilogue is Epilogue.SWIGLU else shape.n
    a_codes = _random_codes(torch, (shape.m, shape.k), kernel.a_dtype, generator)        # [M, K]
    b_codes_t = _random_codes(torch, (out_cols, shape.k), kernel.a_dtype, generator)     # [N, K]
    a = _store_operand(a_codes, int4=int4, k_last=kernel.layout is not GemmLayout.TN)
    b = _store_operand(b_codes_t, int4=int4, k_last=kernel.layout is GemmLayout.NT)
    if kernel.scale.mode is ScaleMode.PER_CHANNEL:
        a_scale = _random_scales(torch, (shape.m,), generator)
        b_scale = _random_scales(torch, (out_cols,), generator)
    else:
        groups = -(-shape.k // int(kernel.scale.subchannel_size or 1))
        a_scale = _random_scales(torch, (shape.m, groups), generator)
        b_scale = _random_scales(torch, (groups, out_cols), generator)
    return a, b, a_scale, b_scale


def _validation_tolerances(kernel: KernelMetadata) -> tuple[float, float]:
    """(rtol, atol) against the PyTorch reference math; the reference's values (autotune.py:889-893)."""
    if kernel.output_dtype == "bfloat16":
        return 8.0e-3, 1.0e-2
    return 1.0e-4, (1.0e-3 if kernel.epilogue is Epilogue.NONE else 1.0e-2)


def _max_diffs(torch: Any, actual: Any, expected: Any) -> tuple[float, float]:
    delta = (actual.float() - expected.float()).abs()
    rel = delta / expected.float().abs().clamp_min(1.0e-12)
    return float(delta.max().item()), float(rel.max().item())


def _benchmark_native_kernel(
    kernel: KernelMetadata,
    shape: BenchmarkShape,
    *,
    root: str | Path | None,
    library_path: str | Path | None,
    warmup_ms: int,
    rep_ms: int,
    validate: bool,
) -> BenchmarkRecord:
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("autotuning native kernels requires a CUDA device")
    a, b, a_scale, b_scale = make_dense_inputs(kernel, shape)
    expected = None
    if validate:
        expected = explicit_mm(a, b, kernel=kernel, a_scale=a_scale, b_scale=b_scale, use_reference=True)
    dev = [t.to("cuda") for t in (a, b, a_scale, b_scale)]
    out_dtype = torch.bfloat16 if kernel.output_dtype == "bfloat16" else torch.float32
    c = torch.empty((shape.m, shape.n), device="cuda", dtype=out_dtype)

    def run() -> Any:
        return launch_generated_kernel(
            dev[0], dev[1], kernel=kernel, a_scale=dev[2], b_scale=dev[3], c=c, root=root, library_path=library_path
        )

    max_abs = max_rel = None
    if validate:
        got = run()
        torch.cuda.synchronize()
        got = got.cpu()
        rtol, atol = _validation_tolerances(kernel)
        torch.testing.assert_close(got, expected, rtol=rtol, atol=atol)
        max_abs, max_rel = _max_diffs(torch, got, expected)
    timed = benchmark_device_callable(
        kernel=kernel, shape=shape, fn=run, warmup_ms=warmup_ms, rep_ms=rep_ms,
        notes="autotuned sm_100a kernel, CUDA-event device timing",
        metadata={
            "arch": kernel.arch, "dtype": kernel.a_dtype.value, "layout": kernel.layout.value,
            "scale": kernel.scale.label, "epilogue": kernel.epilogue.value, "output_dtype": kernel.output_dtype,
            "tile": kernel.tile.label, "even_k": kernel.tile.even_k, "split_k": kernel.tile.split_k,
            "validated": validate, "torch_version": str(torch.__version__), "device": torch.cuda.get_device_name(),
        },
    )
    factor = 2.0 if kernel.epilogue is Epilogue.SWIGLU else 1.0  # up and gate projections both count
    return BenchmarkRecord(
        kernel_id=timed.kernel_id, shape=timed.shape, runtime_ms=timed.runtime_ms, tops=timed.tops * factor,
        iterations=timed.iterations, warmup=timed.warmup, success=timed.success,
        max_abs_diff=max_abs, max_rel_diff=max_rel, notes=timed.notes, metadata=timed.metadata,
    )


def make_ragged_fwd_inputs(
    *, m: int, n: int, k: int, group_sizes: Sequence[int], layout: GemmLayout, scale: ScaleSpec, seed: int = 0
) -> dict[str, Any]:
    """CPU operands of a forward grouped dot plus their logical int8 forms (``x``, ``w``)."""
    import torch

    generator = torch.Generator().manual_seed(seed)
    groups = len(group_sizes)
    x = _random_codes(torch, (m, k), OperandDType.INT4, generator)               # [M, K]
    w_t = _random_codes(torch, (groups, n, k), OperandDType.INT4, generator)     # [G, N, K]
    lhs = _store_operand(x, int4=True, k_last=layout in (GemmLayout.NN, GemmLayout.NT))
    rhs = _store_operand(w_t, int4=True, k_last=layout in (GemmLayout.NT, GemmLayout.TT))
    if scale.mode is ScaleMode.PER_CHANNEL:
        a_scale = _random_scales(torch, (m,), generator)
        b_scale = _random_scales(torch, (groups, n), generator)
    else:
        cols = -(-k // int(scale.subchannel_size or 1))
        a_scale = _random_scales(torch, (m, cols), generator)
        b_scale = _random_scales(torch, (groups, cols, n), generator)
    return {
        "lhs": lhs, "rhs": rhs, "a_scale": a_scale, "b_scale": b_scale,
        "group_sizes": torch.tensor(list(group_sizes), dtype=torch.int64), "x": x, "w": w_t.transpose(1, 2),
    }


def make_ragged_bwd_inputs(
    *, m: int, n: int, k_capacity: int, group_sizes: Sequence[int], layout: GemmLayout, scale: ScaleSpec, seed: int = 0
) -> dict[str, Any]:
    """CPU operands of a backward grouped dot, every group padded to ``k_capacity`` (rounded up to even)."""
    import torch

    generator = torch.Generator().manual_seed(seed)
    groups = len(group_sizes)
    cap = k_capacity + (k_capacity & 1)
    a = _random_codes(torch, (groups, m, cap), OperandDType.INT4, generator)     # [G, M, K]
    b_t = _random_codes(torch, (groups, n, cap), OperandDType.INT4, generator)   # [G, N, K]
    lhs = _store_operand(a, int4=True, k_last=layout in (GemmLayout.NN, GemmLayout.NT))
    rhs = _store_operand(b_t, int4=True, k_last=layout in (GemmLayout.NT, GemmLayout.TT))
    if scale.mode is ScaleMode.PER_CHANNEL:
        a_scale = _random_scales(torch, (groups, m), generator)
        b_scale = _random_scales(torch, (groups, n), generator)
    else:
        cols = -(-cap // int(scale.subchannel_size or 1))
        a_scale = _random_scales(torch, (groups, m, cols), generator)
        b_scale = _random_scales(torch, (groups, cols, n), generator)
    return {
        "lhs": lhs, "rhs": rhs, "a_scale": a_scale, "b_scale": b_scale,
        "group_sizes": torch.tensor(list(group_sizes), dtype=torch.int64), "a": a, "b": b_t.transpose(1, 2),
    }


def _benchmark_ragged_candidate(
    candidate: RaggedAutotuneCandidate,
    shape: BenchmarkShape,
    *,
    m: int,
    n: int,
    k_capacity: int,
    group_sizes: tuple[int, ...],
    warmup_ms: int,
    rep_ms: int,
) -> BenchmarkRecord:
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("autotuning ragged kernels requires a CUDA device")
    if candidate.mode is RaggedDotMode.FWD:
        data = make_ragged_fwd_inputs(
            m=m, n=n, k=k_capacity, group_sizes=group_sizes, layout=candidate.layout, scale=candidate.scale,
            seed=_stable_seed(candidate.kernel_id),
        )
        dev = {name: data[name].to("cuda") for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
        out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)

        def run() -> Any:
            return ragged_dot_int4(
                dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                scale=candidate.scale, config=candidate.config, layout=candidate.layout, out=out, use_native=True,
            )
    else:
        data = make_ragged_bwd_inputs(
            m=m, n=n, k_capacity=k_capacity, group_sizes=group_sizes, layout=candidate.layout, scale=candidate.scale,
            seed=_stable_seed(candidate.kernel_id),
        )
        dev = {name: data[name].to("cuda") for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
        out = torch.empty((len(group_sizes), m, n), device="cuda", dtype=torch.float32)

        def run() -> Any:
            return ragged_dot_int4_bwd(
                dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                scale=candidate.scale, config=candidate.config, layout=candidate.layout, out=out, use_native=True,
            )

    probe = KernelMetadata(
        kernel_id=candidate.kernel_id, arch="sm_100a", a_dtype=OperandDType.INT4, b_dtype=OperandDType.INT4,
        acc_dtype="int32", output_dtype="bfloat16" if candidate.mode is RaggedDotMode.FWD else "float32",
        scale_dtype="bfloat16", scale=candidate.scale, epilogue=Epilogue.NONE, tile=None,  # type: ignore[arg-type]
        device_kernel="b200::gemm_i8_tcgen05_kernel", layout=candidate.layout,
    )
    info = _ragged_record_metadata(
        candidate=candidate, group_sizes=group_sizes, k_capacity=k_capacity, warmup_ms=warmup_ms, rep_ms=rep_ms
    )
    return benchmark_device_callable(
        kernel=probe, shape=shape, fn=run, warmup_ms=warmup_ms, rep_ms=rep_ms, metadata=info,
        notes="grouped int4 dot through the public API (task building and validation inside the timed call)",
    )


__all__ = [
    "AutotuneResult",
    "RaggedAutotuneCandidate",
    "RaggedAutotuneResult",
    "RaggedDotMode",
    "autotune",
    "autotune_ragged_dot",
    "default_ragged_dot_candidates",
    "find_autotune_candidates",
    "generated_shape_for_kernel",
    "make_dense_inputs",
    "make_ragged_bwd_inputs",
    "make_ragged_fwd_inputs",
    "tops_for_runtime",
]
