#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5fwd|c5bwd|c5bwd_flat] [--impl ours|reference]

Prints ONE JSON line (rank 0).  Default workload is the headline one: int4 x int4 per-channel GEMM at
M = N = K = 4096 (metric: TOPS = 2*M*N*K / t).  One *step* is one pass over a batch of ``--batch``
independent problems of that shape, each with its own operands and output, so that the operand bytes
touched between two uses of the same buffer exceed the 126 MB L2 (stated in ``config.l2``).

Multi-GPU (launched by torchrun, one rank per GPU): every rank runs the same per-GPU problem on its own
shard - dense workloads are column-parallel along N (global N = N_per_gpu * world), grouped workloads are
expert-parallel - with no collective on the data path; time is the max over ranks; ``scaling`` is weak.

Timing: CUDA events on the launching stream around exactly K steps, barrier + synchronize on both sides,
SM clock and throttle reasons polled through NVML during the timed region.

``e2e`` is the same metric through the public Python API with HOST operands: every step copies the
operands from pinned host memory, runs the op, and copies the result back, all inside the timed region.

``--impl reference`` times the reference's own CPU path for the workload (the oracle port of its PyTorch
int32-matmul math; the reference package is Python and is not present on the GPU box) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_INT8_TOPS = 4500.0   # dense int8 tensor peak of a B200 (public figure)
L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------
WORKLOADS = {
    "c2": dict(kind="dense", m=4096, n=4096, k=4096, dtype="int4", sub=0, epilogue="none",
               name="int4 x int4 per-channel GEMM, M=N=K=4096, bf16 out (BASELINE config 2)",
               metric="W4A4 GEMM TOPS @4096^3"),
    "c3": dict(kind="dense", m=8192, n=8192, k=8192, dtype="int8", sub=0, epilogue="relu2",
               name="int8 x int8 per-channel GEMM + ReLU^2, M=N=K=8192 (BASELINE config 3)",
               metric="W8A8 ReLU2 GEMM TOPS @8192^3"),
    "c4": dict(kind="dense", m=4096, n=14336, k=4096, dtype="int4", sub=256, epilogue="swiglu",
               name="int4 sc256 fused SwiGLU up/gate, M=4096 K=4096 D=14336 (BASELINE config 4)",
               metric="W4A4 SC256 SwiGLU TOPS"),
    "c5fwd": dict(kind="ragged_fwd", rows=32768, k=2048, n=1408, groups=64,
                  name="ragged_dot_int4 forward, 64 groups, 32768 rows, K=2048, N=1408 (BASELINE config 5)",
                  metric="ragged_dot_int4 fwd TOPS"),
    "c5bwd": dict(kind="ragged_bwd", rows=32768, m=2048, n=1408, groups=64,
                  name="ragged_dot_int4_bwd, 64 groups, 32768 tokens, out [64,2048,1408] fp32 (BASELINE config 5)",
                  metric="ragged_dot_int4 bwd TOPS"),
    # the same grouped backward over FLAT token-packed operands (no per-group padding; not in the reference API)
    "c5bwd_flat": dict(kind="ragged_bwd", flat=True, rows=32768, m=2048, n=1408, groups=64,
                       name="ragged_dot_int4_bwd_flat, 64 groups, 32768 tokens back to back, out [64,2048,1408] fp32 (BASELINE config 5, flat dy)",
                       metric="ragged_dot_int4 bwd TOPS"),
}


def config5_group_sizes(torch):
    """Dirichlet(0.5) proportions over 64 groups, 3 forced empty, multinomial over 32768 rows (seed 0)."""
    g = torch.Generator().manual_seed(0)
    probs = torch._sample_dirichlet(torch.full((64,), 0.5), generator=g)
    probs[torch.randperm(64, generator=g)[:3]] = 0
    draws = torch.multinomial(probs / probs.sum(), 32768, replacement=True, generator=g)
    return torch.bincount(draws, minlength=64)


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the workload's GEMM kernel, from one `ncu --set full`
# capture of the same command at 1 GPU (summaries under profiles/).  Smaller than the algorithmic bytes where the
# result is still in the 126 MB L2 when the kernel ends.
NCU_DRAM_TRAFFIC_BYTES = {
    "c2": 17.08e6, "c3": 358.7e6, "c4": 147.2e6, "c5fwd": 175.2e6, "c5bwd": 749.2e6, "c5bwd_flat": 742.7e6,
}
VENDOR_INT8_GEMM_TOPS = 2973.1  # torch._int_mm (cuBLASLt) int8 8192^3 on this pool's B200: `bench.py --probe-int8-peak`


def workload_ops(w, sizes=None) -> float:
    if w["kind"] == "dense":
        cols = 2 * w["n"] if w["epilogue"] == "swiglu" else w["n"]
        return 2.0 * w["m"] * cols * w["k"]
    if w["kind"] == "ragged_fwd":
        return 2.0 * w["rows"] * w["k"] * w["n"]
    return 2.0 * w["m"] * w["n"] * w["rows"]  # backward: K = sum(group_sizes)


def workload_bytes(w) -> float:
    """Algorithmic HBM bytes of one problem: every operand read once, the result written once."""
    if w["kind"] == "dense":
        cols = 2 * w["n"] if w["epilogue"] == "swiglu" else w["n"]
        kb = w["k"] // 2 if w["dtype"] == "int4" else w["k"]
        groups = max(1, w["k"] // w["sub"]) if w["sub"] else 1
        return w["m"] * kb + kb * cols + 2 * groups * (w["m"] + cols) + 2 * w["m"] * w["n"]
    if w["kind"] == "ragged_fwd":
        return w["rows"] * w["k"] // 2 + w["groups"] * (w["k"] // 2) * w["n"] + 2 * (w["rows"] + w["groups"] * w["n"]) + 2 * w["rows"] * w["n"]
    return w["rows"] // 2 * (w["m"] + w["n"]) + 2 * w["groups"] * (w["m"] + w["n"]) + 4 * w["groups"] * w["m"] * w["n"]


# ----------------------------------------------------------------------------------------------
# clock sampling through NVML (read-only)
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
    }

    def __init__(self, device_index: int) -> None:
        self.samples: list[int] = []
        self.reason_bits = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _poll(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        ordered = sorted(self.samples)
        reasons = [name for bit, name in self.REASONS.items() if self.reason_bits & bit]
        return {"sm_mhz": ordered[len(ordered) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons), "samples": len(ordered)}


def visible_device_index(local_rank: int) -> int:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        parts = [p for p in visible.split(",") if p.strip()]
        try:
            return int(parts[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
def build_problem_set(torch, pkg, w, batch: int, seed: int, device):
    """``batch`` independent problems on ``device`` (operands generated there as random codes)."""
    from strix_halo_int4_gemms_b200 import native

    gen = torch.Generator(device=device).manual_seed(seed)
    cpu_gen = torch.Generator().manual_seed(seed)

    def scales(shape, mult=0.05):
        return ((torch.rand(shape, generator=cpu_gen) + 0.5) * mult).to(torch.bfloat16).to(device)

    def codes(shape, int4=True):
        if int4:
            return torch.randint(0, 256, shape, generator=gen, device=device, dtype=torch.uint8)
        return torch.randint(-127, 128, shape, generator=gen, device=device, dtype=torch.int8)

    problems = []
    for _ in range(batch):
        if w["kind"] == "dense":
            int4 = w["dtype"] == "int4"
            cols = 2 * w["n"] if w["epilogue"] == "swiglu" else w["n"]
            kb = w["k"] // 2 if int4 else w["k"]
            mult = 0.05 if int4 else 0.01
            groups = w["k"] // w["sub"] if w["sub"] else 0
            problems.append(dict(
                a=codes((w["m"], kb), int4), b=codes((kb, cols), int4),
                a_scale=scales((w["m"], groups) if groups else (w["m"],), mult),
                b_scale=scales((groups, cols) if groups else (cols,), mult),
                out=torch.empty((w["m"], w["n"]), device=device, dtype=torch.bfloat16),
            ))
        elif w["kind"] == "ragged_fwd":
            sizes = w["sizes"]
            problems.append(dict(
                lhs=codes((int(sizes.sum()), w["k"] // 2)), rhs=codes((len(sizes), w["k"] // 2, w["n"])),
                a_scale=scales((int(sizes.sum()),)), b_scale=scales((len(sizes), w["n"])),
                group_sizes=sizes.to(device), out=torch.empty((int(sizes.sum()), w["n"]), device=device, dtype=torch.bfloat16),
            ))
        elif w.get("flat"):
            sizes = w["sizes"]
            pairs = (int(sizes.sum()) + 1) // 2
            problems.append(dict(
                lhs=codes((pairs, w["m"])), rhs=codes((pairs, w["n"])),
                a_scale=scales((len(sizes), w["m"])), b_scale=scales((len(sizes), w["n"])),
                group_sizes=sizes.to(device), out=torch.empty((len(sizes), w["m"], w["n"]), device=device, dtype=torch.float32),
            ))
        else:
            sizes = w["sizes"]
            cap = int(sizes.max()) if len(sizes) else 2
            cap = max(32, cap + (-cap) % 32)
            problems.append(dict(
                lhs=codes((len(sizes), cap // 2, w["m"])), rhs=codes((len(sizes), cap // 2, w["n"])),
                a_scale=scales((len(sizes), w["m"])), b_scale=scales((len(sizes), w["n"])),
                group_sizes=sizes.to(device), out=torch.empty((len(sizes), w["m"], w["n"]), device=device, dtype=torch.float32),
            ))
    return problems


def make_runner(torch, pkg, w, problems):
    """A zero-argument callable that launches one step (all problems) with as little host work as possible."""
    from strix_halo_int4_gemms_b200 import native
    from strix_halo_int4_gemms_b200.ragged import RaggedBwdDotConfig, RaggedDotConfig

    device_index = torch.cuda.current_device()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    if w["kind"] == "dense":
        scale = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, w["sub"]) if w["sub"] else pc
        variant = native.make_variant(dtype=pkg.OperandDType(w["dtype"]), layout=pkg.GemmLayout.NN, scale=scale,
                                      epilogue=pkg.Epilogue(w["epilogue"]), out_dtype=native.OUT_BF16)
        args = [dict(a_ptr=p["a"].data_ptr(), b_ptr=p["b"].data_ptr(), a_scale_ptr=p["a_scale"].data_ptr(),
                     b_scale_ptr=p["b_scale"].data_ptr(), c_ptr=p["out"].data_ptr()) for p in problems]

        def step():
            for ptrs in args:
                # the stream is looked up per call: under CUDA-graph capture the current stream is the capturing one
                native.launch_dense(variant, device_index=device_index, stream_handle=torch.cuda.current_stream().cuda_stream,
                                    m=w["m"], n=w["n"], k=w["k"], **ptrs)
        return step, len(problems)
    if w["kind"] == "ragged_fwd":
        # the task height ragged_dot_int4 itself picks for groups this large: 256-row tasks on pairs of SMs
        from strix_halo_int4_gemms_b200.ragged import PAIR_MIN_MEAN_GROUP_ROWS, PAIR_TASK_ROWS
        rows, groups = problems[0]["lhs"].shape[0], len(problems[0]["group_sizes"])
        cfg = RaggedDotConfig(block_m=PAIR_TASK_ROWS if rows >= PAIR_MIN_MEAN_GROUP_ROWS * groups else 128)
        infos = [pkg.calculate_group_info(p["group_sizes"], cfg.block_m, align_tile=cfg.align_tile) for p in problems]

        def step():
            for p, info in zip(problems, infos):
                native.launch_ragged_fwd_kernel(p["lhs"], p["rhs"], group_info=info, a_scale=p["a_scale"], b_scale=p["b_scale"], out=p["out"],
                                                scale=pc, config=cfg, layout=pkg.GemmLayout.NN, rows=p["lhs"].shape[0], cols=w["n"],
                                                k_packed=w["k"] // 2, scale_cols=1)
        return step, len(problems)
    cfg = RaggedBwdDotConfig()
    if w.get("flat"):
        tokens = [int(p["group_sizes"].sum()) for p in problems]

        def step():
            for p, t in zip(problems, tokens):
                native.launch_ragged_bwd_flat_kernel(p["lhs"], p["rhs"], p["group_sizes"], a_scale=p["a_scale"], b_scale=p["b_scale"],
                                                     out=p["out"], tokens=t)
        return step, 2 * len(problems)  # the group-start scan + the GEMM kernel per problem

    def step():
        for p in problems:
            native.launch_ragged_bwd_kernel(p["lhs"], p["rhs"], p["group_sizes"], a_scale=p["a_scale"], b_scale=p["b_scale"], out=p["out"],
                                            scale=pc, config=cfg, layout=pkg.GemmLayout.TN, rows=w["m"], cols=w["n"],
                                            k_packed=p["lhs"].shape[1], scale_cols=1)
    return step, len(problems)


def make_e2e_runner(torch, pkg, w, problem):
    """One step through the PUBLIC API from pinned host buffers and back; returns (callable, h2d, d2h bytes).

    Every step uploads its operands, calls the API and downloads the result.  Steps alternate between two
    streams with their own device and host buffers, the way a host pipeline would run them, so that one step's
    upload overlaps the previous step's download (PCIe is full duplex); the work of each step is unchanged.
    ``step.finish()`` joins both streams into the current one (called before the stop event is recorded)."""
    lanes = 2
    streams = [torch.cuda.Stream() for _ in range(lanes)]
    host = {k: v.cpu().pin_memory() for k, v in problem.items() if k != "out"}
    out_host = [torch.empty(problem["out"].shape, dtype=problem["out"].dtype).pin_memory() for _ in range(lanes)]
    dev_sets = [{k: torch.empty_like(v, device="cuda") for k, v in host.items()} for _ in range(lanes)]
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host[0].numel() * out_host[0].element_size()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    state = {"i": 0}

    def step():
        lane = state["i"] % lanes
        state["i"] += 1
        stream, dev = streams[lane], dev_sets[lane]
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for k, v in host.items():
                dev[k].copy_(v, non_blocking=True)
            if w["kind"] == "dense":
                scale = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, w["sub"]) if w["sub"] else pc
                if w["epilogue"] == "swiglu":
                    out = pkg.fused_swiglu_up_gate(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], scale=scale,
                                                   dtype=pkg.OperandDType(w["dtype"]))
                else:
                    out = pkg.mm(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], scale=scale,
                                 dtype=pkg.OperandDType(w["dtype"]), epilogue=pkg.Epilogue(w["epilogue"]), schedule=pkg.KernelSchedule.PERSISTENT)
            elif w["kind"] == "ragged_fwd":
                out = pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
            elif w.get("flat"):
                out = pkg.ragged_dot_int4_bwd_flat(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
            else:
                out = pkg.ragged_dot_int4_bwd(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                                              layout=pkg.GemmLayout.TN)
            out_host[lane].copy_(out, non_blocking=True)

    def finish():
        for stream in streams:
            torch.cuda.current_stream().wait_stream(stream)

    step.finish = finish
    return step, h2d, d2h


def timed_region(torch, dist, world, step, steps: int, warmup: int, sampler=None) -> float:
    """ms for exactly ``steps`` steps, max over ranks, CUDA events on the current stream."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        start.record()
        for _ in range(steps):
            step()
        finish = getattr(step, "finish", None)
        if finish is not None:
            finish()  # steps that run on side streams: the stop event must come after all of them
        stop.record()
        stop.synchronize()
    torch.cuda.synchronize()
    ms = float(start.elapsed_time(stop))
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's PyTorch math (oracle port), bounded sample
# ----------------------------------------------------------------------------------------------
def make_cpu_step(w):
    """``run(rows) -> (seconds, ops)``: the reference CPU path on ``rows`` rows of the workload.

    The reference computes ``torch.matmul`` on int32 operands and scales in fp32 (api.py:299-325; the
    grouped references of tests/test_ragged_dot.py:19-117 for config 5).  The oracle's ``torch_int32``
    engine is that arithmetic.  Rows (tokens, for the backward dot) are independent, so throughput on a
    row sample is the throughput of the whole job.
    """
    import numpy as np
    import torch

    from oracle import reference_math as oracle

    torch.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    bits = 0x3D4D  # bf16(0.05)
    if w["kind"] == "dense":
        int4 = w["dtype"] == "int4"
        cols = 2 * w["n"] if w["epilogue"] == "swiglu" else w["n"]
        k = w["k"]
        lo, hi = (-8, 8) if int4 else (-127, 128)
        b = rng.integers(lo, hi, (k, cols), dtype=np.int8)
        groups = k // w["sub"] if w["sub"] else 0
        sb = oracle.bf16_bits_to_f32(np.full((groups, cols) if groups else (cols,), bits, dtype=np.uint16))

        def run(rows):
            a = rng.integers(lo, hi, (rows, k), dtype=np.int8)
            sa = oracle.bf16_bits_to_f32(np.full((rows, groups) if groups else (rows,), bits, dtype=np.uint16))
            t0 = time.perf_counter()
            out = oracle.scaled_matmul(a, b, sa, sb, subchannel=w["sub"], engine="torch_int32")
            oracle.round_to_bf16(oracle.apply_epilogue(out, w["epilogue"]))
            return time.perf_counter() - t0, 2.0 * rows * cols * k
        return run, w["m"]
    n = w["n"]
    if w["kind"] == "ragged_fwd":
        k = w["k"]
        wg = rng.integers(-8, 8, (k, n), dtype=np.int8)

        def run(rows):
            x = rng.integers(-8, 8, (rows, k), dtype=np.int8)
            t0 = time.perf_counter()
            oracle.round_to_bf16(oracle.scaled_matmul(x, wg, np.ones(rows, np.float32), np.ones(n, np.float32), engine="torch_int32"))
            return time.perf_counter() - t0, 2.0 * rows * k * n
        return run, w["rows"]
    m = w["m"]

    def run(rows):  # rows = tokens of one group: out[g] = x_g^T [m, rows] @ dy_g [rows, n]
        xt = rng.integers(-8, 8, (m, rows), dtype=np.int8)
        dy = rng.integers(-8, 8, (rows, n), dtype=np.int8)
        t0 = time.perf_counter()
        oracle.scaled_matmul(xt, dy, np.ones(m, np.float32), np.ones(n, np.float32), engine="torch_int32")
        return time.perf_counter() - t0, 2.0 * m * n * rows
    return run, w["rows"]


def pick_sample_rows(run, limit: int, budget_s: float) -> tuple[int, float, float]:
    """Largest power-of-two row count (<= limit) whose single run stays within ``budget_s``."""
    rows = 16
    run(rows)  # warms the thread pool
    seconds, ops = run(rows)
    while rows * 2 <= limit and seconds * 2.2 <= budget_s:
        rows *= 2
        seconds, ops = run(rows)
    return rows, seconds, ops


def cpu_reference_sample(w, *, budget_s: float = 12.0):
    """(TOPS, rows, seconds, threads) of one bounded run of the reference CPU path."""
    import torch

    run, limit = make_cpu_step(w)
    rows, seconds, ops = pick_sample_rows(run, limit, budget_s)
    return ops / seconds / 1e12, rows, seconds, torch.get_num_threads()


def run_reference_arm(args, w) -> dict:
    """--impl reference: exactly K timed steps of the CPU path, each step one bounded row sample."""
    import torch

    run, limit = make_cpu_step(w)
    per_step_budget = max(0.05, min(2.0, 150.0 / (args.steps + args.warmup)))
    rows, _seconds, _ops = pick_sample_rows(run, limit, per_step_budget)
    for _ in range(args.warmup):
        run(rows)
    total_s = total_ops = 0.0
    for _ in range(args.steps):
        seconds, ops = run(rows)
        total_s += seconds
        total_ops += ops
    value = total_ops / total_s / 1e12
    cores = torch.get_num_threads()
    sample = f"{rows} rows of the workload per step, {args.steps} steps; rows are independent"
    return {
        "impl": "reference", "metric": w["metric"], "value": value, "unit": "TOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32 matmul + fp32 scale (CPU)", "data": "synthetic",
        "config": {"workload": w["name"], "engine": "oracle port of the reference's PyTorch CPU math (torch.matmul on int32)"},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ----------------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="independent problems per step (0 = enough to exceed L2 twice over)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--probe-int8-peak", action="store_true",
                    help="time the vendor library's int8 GEMM (torch._int_mm, 8192^3, best of 10) and print it: "
                         "a measured int8 figure to set beside the nominal 4500 TOPS; not a bench line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from Python instead of replaying a CUDA graph of one step")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = dict(WORKLOADS[args.workload])

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference_arm(args, w)), flush=True)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import strix_halo_int4_gemms_b200 as pkg
    from strix_halo_int4_gemms_b200 import distributed as shard
    from strix_halo_int4_gemms_b200 import native

    if args.probe_int8_peak:
        n = 8192
        a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8).t()   # column-major B, as cuBLASLt wants it
        for _ in range(3):
            torch._int_mm(a, b)
        best = float("inf")
        for _ in range(10):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            torch._int_mm(a, b)
            stop.record()
            stop.synchronize()
            best = min(best, float(start.elapsed_time(stop)))
        print(json.dumps({"probe": "torch._int_mm int8 8192^3 -> int32, best of 10", "ms": best,
                          "tops": 2.0 * n ** 3 / (best * 1e-3) / 1e12}), flush=True)
        return

    status = pkg.dispatch_runtime_status()
    if not status.has_linked_kernels:
        raise SystemExit(f"CUDA library at {status.library_path} cannot run here: {status}")

    imbalance = 1.0
    if w["kind"] != "dense":
        sizes = config5_group_sizes(torch)
        if world > 1:
            # expert-parallel: the global problem has 64 * world groups (weak scaling), LPT-assigned
            all_sizes = torch.cat([sizes[torch.randperm(64, generator=torch.Generator().manual_seed(r))] for r in range(world)])
            plan = shard.assign_groups(all_sizes.tolist(), world)
            imbalance = shard.load_imbalance(all_sizes.tolist(), plan)
            sizes = all_sizes[plan[rank]]
        w["sizes"] = sizes
        w["rows_local"] = int(sizes.sum())
    per_problem_bytes = workload_bytes(w)
    batch = args.batch or max(2, int(-(-2.2 * L2_BYTES // per_problem_bytes)))
    problems = build_problem_set(torch, pkg, w, batch, seed=1234 + rank, device=torch.device("cuda", local_rank))
    step, launches_per_step = make_runner(torch, pkg, w, problems)

    if w["kind"] == "dense":
        ops_per_step_rank = workload_ops(w) * batch
    elif w["kind"] == "ragged_fwd":
        ops_per_step_rank = 2.0 * w["rows_local"] * w["k"] * w["n"] * batch
    else:
        ops_per_step_rank = 2.0 * w["m"] * w["n"] * w["rows_local"] * batch
    ops_t = torch.tensor([ops_per_step_rank], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ops_t)
    ops_per_step = float(ops_t.item())

    # One step (its `launches_per_step` kernels) is captured into a CUDA graph and replayed: at 60 us per kernel the
    # Python launch loop is otherwise the bottleneck as soon as several ranks share the host's cores.
    graphed = False
    if not args.no_graph:
        step()  # first-call set-up of the library happens outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        step = graph.replay
        graphed = True
    sampler = ClockSampler(visible_device_index(local_rank))
    native.reset_device_status(local_rank)
    ms = timed_region(torch, dist, world, step, args.steps, args.warmup, sampler)
    dev_status = native.device_status(local_rank)
    if dev_status[0] != 0:
        raise SystemExit(f"a kernel reported status {dev_status}")
    ms_per_step = ms / args.steps
    value = ops_per_step / (ms_per_step * 1e-3) / 1e12
    # duration of the dominant (GEMM) kernel: one per problem; the flat backward's group-start scan (one tiny
    # CTA per problem, counted in gpu_launches) rides along inside it
    kernel_us = ms_per_step * 1e3 / batch

    e2e = None
    if not args.no_e2e:
        e2e_step, h2d, d2h = make_e2e_runner(torch, pkg, w, problems[0])
        e2e_steps = max(3, min(args.steps, 20))
        e2e_ms = timed_region(torch, dist, world, e2e_step, e2e_steps, 3) / e2e_steps
        e2e = {"value": (ops_per_step / batch) / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": e2e_steps,
               "note": "one problem per step through the public API; pinned host operands in, result out, copies inside the timed region; "
                       "steps alternate between two streams so that uploads overlap the previous step's download"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_source = load_peaks()
    timed_s = ms / 1e3
    bf16_peak = peaks["bf16_tflops_sustained"] if timed_s > 1.0 and "bf16_tflops_sustained" in peaks else peaks["bf16_tflops"]
    hbm_bound = args.workload in ("c5bwd", "c5bwd_flat")
    per_gpu_tops = value / world
    traffic = NCU_DRAM_TRAFFIC_BYTES.get(args.workload) if world == 1 else None
    if hbm_bound:
        achieved = per_problem_bytes / (kernel_us * 1e-6) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "traffic": traffic, "peak_source": f"{peak_source} STREAM-style copy",
                    "algorithmic_bytes_per_launch": per_problem_bytes, "kernel_us": kernel_us}
    else:
        peak = 2.0 * bf16_peak
        roofline = {"bound": "tensor", "achieved": per_gpu_tops, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu_tops / peak, "traffic": traffic,
                    "peak_source": f"2 x {peak_source} cuBLAS bf16 {'sustained' if bf16_peak != peaks['bf16_tflops'] else 'burst'} "
                                   f"({bf16_peak} TFLOP/s): kind::i8 runs at twice the bf16 rate",
                    "frac_of_nominal_int8_4500": per_gpu_tops / NOMINAL_INT8_TOPS,
                    "frac_of_vendor_int8_gemm": per_gpu_tops / VENDOR_INT8_GEMM_TOPS,
                    "algorithmic_bytes_per_launch": per_problem_bytes, "kernel_us": kernel_us}

    line = {
        "metric": w["metric"], "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s32 accumulate of int8 tensor-core products (int4 or int8 operands), fp32 scale, bf16/fp32 store",
        "data": "synthetic",
        "config": {
            "workload": w["name"], "problems_per_step": batch,
            "launch": "one CUDA graph replay per step" if graphed else "one Python call per kernel",
            "l2": f"{batch} independent operand/output sets per step, {batch * per_problem_bytes / 1e6:.0f} MB touched between reuses (> 126 MB L2)",
            "parallelism": "none" if world == 1 else ("column-parallel along N, one shard per GPU" if w["kind"] == "dense" else f"expert-parallel, LPT assignment, max/mean load {imbalance:.3f}"),
            "per_gpu_problem": "same as 1-GPU (weak scaling)",
        },
        "clocks": sampler.summary(),
        "gpu_launches": launches_per_step * args.steps,
        "roofline": roofline,
        "pct_of_nominal_int8_peak": 100.0 * per_gpu_tops / NOMINAL_INT8_TOPS,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if not args.no_cpu_baseline:
        tops, rows, seconds, cores = cpu_reference_sample(w, budget_s=12.0)
        line["cpu_baseline"] = {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
                                "sample": f"{rows} rows of the same workload in {seconds:.1f} s (reference PyTorch int32-matmul math)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
