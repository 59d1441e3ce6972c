"""TOPS arithmetic, sample summaries and the record database (CPU).  Reference: tests/test_benchmarking.py."""
import json

import numpy as np
import pytest

from strix_halo_int4_gemms_b200.benchmarking import (
    BenchmarkDatabase,
    BenchmarkRecord,
    BenchmarkShape,
    benchmark_callable,
    gemm_ops,
    summarize_runtime_samples,
    tops_for_runtime,
)


def test_tops_definition():
    shape = BenchmarkShape(1024, 1024, 1024)
    assert gemm_ops(shape) == 2 * 1024 ** 3
    assert tops_for_runtime(shape, 1.0) == pytest.approx(2.147483648)
    with pytest.raises(ValueError, match="runtime_ms must be positive"):
        tops_for_runtime(shape, 0.0)


def test_summary_matches_reference_fixture(golden):
    summary = summarize_runtime_samples([3.0, 1.0, 0.0, 2.0, 10.0, -1.0])
    keys = [str(k) for k in golden["metric/summary_keys"]]
    assert sorted(summary) == keys
    np.testing.assert_allclose([float(summary[k]) for k in keys], golden["metric/summary_values"], rtol=0, atol=1e-12)
    assert summary["sample_count"] == 4 and summary["dropped_nonpositive_sample_count"] == 2
    assert summary["runtime_ms_median"] == 2.5 and summary["runtime_ms_p20"] == pytest.approx(1.6)
    with pytest.raises(ValueError, match="at least one runtime sample"):
        summarize_runtime_samples([])
    with pytest.raises(ValueError, match="positive runtime sample"):
        summarize_runtime_samples([0.0, -2.0])


def test_database_round_trip(pkg, tmp_path):
    kernel = pkg.default_registry.all()[0]
    shape = BenchmarkShape(128, 256, 64)
    slow = BenchmarkRecord(kernel.kernel_id, shape, 2.0, 1.0, 10, 3)
    fast = BenchmarkRecord(kernel.kernel_id, shape, 1.0, 2.0, 10, 3, metadata={"note": 1})
    failed = BenchmarkRecord(kernel.kernel_id, shape, 0.5, 9.0, 10, 3, success=False)
    other = BenchmarkRecord(kernel.kernel_id, BenchmarkShape(1, 1, 1), 1.0, 5.0, 10, 3)
    db = BenchmarkDatabase([slow, fast, failed, other])
    assert db.best_record(kernel, shape) == fast
    assert db.matching_records(kernel, shape) == (slow, fast)
    assert db.best_record(kernel, BenchmarkShape(2, 2, 2)) is None
    path = tmp_path / "nested" / "db.json"
    db.save(path)
    assert json.loads(path.read_text())["records"][1]["metadata"] == {"note": 1}
    assert BenchmarkDatabase.load(path).records() == db.records()


def test_wall_clock_benchmark(pkg):
    kernel = pkg.default_registry.all()[0]
    calls = []
    record = benchmark_callable(kernel=kernel, shape=BenchmarkShape(8, 8, 8), fn=lambda: calls.append(1), warmup=2, iterations=5)
    assert len(calls) == 7 and record.iterations == 5 and record.runtime_ms > 0
    with pytest.raises(ValueError, match="iterations must be positive"):
        benchmark_callable(kernel=kernel, shape=BenchmarkShape(8, 8, 8), fn=lambda: None, iterations=0)
