#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5fwd|c5bwd|c5bwd_flat] [--impl ours|reference]

Prints ONE JSON line (rank 0).  The headline workload (default c2) is the int4 x int4 per-channel GEMM at
M = N = K = 4096 (metric: TOPS = 2*M*N*K / t).  One *pass* runs ``problems_per_step`` independent problems of
that shape, each with its own operands and output, so that the bytes touched between two uses of a buffer exceed
the 126 MB L2; one *step* is ``passes_per_step`` passes, chosen so that the K timed steps last at least a second
(a sustained figure, with the SM clock sampled throughout); the short first-touch figure is kept as ``burst``.

The same line carries ``workloads``: the other BASELINE configurations (c1 as a latency, c3, c4, c5 forward and
backward), each measured the same way in the same run, with its own roofline fraction, clocks and end-to-end
figure.

Multi-GPU (launched by torchrun, one rank per GPU, no collective on the data path, time = max over ranks):
  * the headline is weak scaling: dense workloads are column-parallel along N with a global N of N_per_gpu * world,
    every rank taking its columns of the global B through ``distributed.shard_dense_rhs``; grouped workloads are
    expert-parallel with 64 * world groups assigned by ``distributed.assign_groups``;
  * ``strong`` holds the BASELINE problems themselves split over the ranks: c2 and c4 column-parallel, c5 forward
    and backward expert-parallel over the actual 64 groups (with the load imbalance of the assignment), and the
    NCCL all-gather of the output timed separately.

Timing: CUDA events on the launching stream around exactly K steps, barrier + synchronize on both sides, SM clock
and throttle reasons polled through NVML during the timed region.

``e2e`` is the same metric through the public Python API, called with default arguments, with HOST operands: every
step copies the operands from pinned host memory, runs the op, and copies the result back, all inside the timed
region.

``--impl reference`` times the reference's own CPU path for the workload (the oracle port of its PyTorch
int32-matmul math; the reference package is Python and is not present on the GPU box) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_INT8_TOPS = 4500.0   # dense int8 tensor peak of a B200 (public figure)
NOMINAL_HBM_GBS = 8000.0     # public HBM3e figure the brief quotes
L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
SUSTAINED_SECONDS = 1.05     # the timed steps of every workload last at least this long


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------
WORKLOADS = {
    "c1": dict(kind="dense", m=128, n=1024, k=64, dtype="int4", sub=0, epilogue="none",
               name="quick-start int4 x int4 per-channel GEMM, M=128 N=1024 K=64 (BASELINE config 1)",
               metric="W4A4 GEMM latency @128x1024x64"),
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
SUB_WORKLOADS = ("c1", "c3", "c4", "c5fwd", "c5bwd")      # reported beside the headline at one GPU
STRONG_WORKLOADS = ("c2", "c4", "c5fwd", "c5bwd")         # the given problems split over the ranks


def config5_group_sizes(torch):
    """Dirichlet(0.5) proportions over 64 groups, 3 forced empty, multinomial over 32768 rows (seed 0)."""
    g = torch.Generator().manual_seed(0)
    probs = torch._sample_dirichlet(torch.full((64,), 0.5), generator=g)
    probs[torch.randperm(64, generator=g)[:3]] = 0
    draws = torch.multinomial(probs / probs.sum(), 32768, replacement=True, generator=g)
    return torch.bincount(draws, minlength=64)


def load_measured_traffic() -> dict:
    """DRAM read + write bytes of one launch per workload, from the ncu captures summarised in
    ``profiles/dram_traffic.txt`` (lines ``<workload> <bytes> <capture>``).  Absent file or workload: no figure."""
    found = {}
    path = ROOT / "profiles" / "dram_traffic.txt"
    if path.exists():
        for line in path.read_text().splitlines():
            parts = line.split(None, 2)
            if len(parts) >= 2 and not line.startswith("#"):
                try:
                    found[parts[0]] = {"bytes": float(parts[1]), "source": parts[2] if len(parts) > 2 else ""}
                except ValueError:
                    pass
    return found


def dense_ops(w, n=None) -> float:
    n = w["n"] if n is None else n
    cols = 2 * n if w["epilogue"] == "swiglu" else n
    return 2.0 * w["m"] * cols * w["k"]


def dense_bytes(w, n=None) -> float:
    n = w["n"] if n is None else n
    cols = 2 * n if w["epilogue"] == "swiglu" else n
    kb = w["k"] // 2 if w["dtype"] == "int4" else w["k"]
    groups = max(1, w["k"] // w["sub"]) if w["sub"] else 1
    return w["m"] * kb + kb * cols + 2 * groups * (w["m"] + cols) + 2 * w["m"] * n


def ragged_ops(w, rows) -> float:
    if w["kind"] == "ragged_fwd":
        return 2.0 * rows * w["k"] * w["n"]
    return 2.0 * w["m"] * w["n"] * rows  # backward: K = sum(group_sizes)


def ragged_bytes(w, rows, groups) -> float:
    """Algorithmic HBM bytes of one problem: every operand read once, the result written once."""
    if w["kind"] == "ragged_fwd":
        return rows * w["k"] // 2 + groups * (w["k"] // 2) * w["n"] + 2 * (rows + groups * w["n"]) + 2 * rows * w["n"]
    return rows // 2 * (w["m"] + w["n"]) + 2 * groups * (w["m"] + w["n"]) + 4 * groups * w["m"] * w["n"]


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
        self.power_w: list[float] = []
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
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0)
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
        out = {"sm_mhz": ordered[len(ordered) // 2], "sm_mhz_min": ordered[0], "sm_max_mhz": self.max_mhz,
               "reasons": sorted(reasons), "samples": len(ordered)}
        if self.power_w:
            out["power_w_max"] = round(max(self.power_w), 1)
        return out


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


def host_numa_nodes() -> list[int]:
    """NUMA nodes of the CPUs this process may run on (where its pinned host buffers are first touched)."""
    try:
        allowed = os.sched_getaffinity(0)
    except AttributeError:
        return []
    nodes = []
    base = Path("/sys/devices/system/node")
    if not base.exists():
        return []
    for node in sorted(base.glob("node[0-9]*")):
        cpus = set()
        try:
            for part in (node / "cpulist").read_text().strip().split(","):
                if "-" in part:
                    lo, hi = part.split("-")
                    cpus.update(range(int(lo), int(hi) + 1))
                elif part:
                    cpus.add(int(part))
        except Exception:
            continue
        if cpus & allowed:
            nodes.append(int(node.name[4:]))
    return nodes


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
class Ctx:
    """What every measurement needs: modules, rank layout, device."""

    def __init__(self, torch, dist, pkg, native, shard, rank, local_rank, world):
        self.torch, self.dist, self.pkg, self.native, self.shard = torch, dist, pkg, native, shard
        self.rank, self.local_rank, self.world = rank, local_rank, world
        self.device = torch.device("cuda", local_rank)

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = self.torch.tensor([value], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = self.torch.tensor([value], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t)
        return float(t.item())

    def gather(self, value) -> list:
        if self.world == 1:
            return [value]
        out = [None] * self.world
        self.dist.all_gather_object(out, value)
        return out


def _scales(torch, shape, gen, device, mult=0.05):
    return ((torch.rand(shape, generator=gen) + 0.5) * mult).to(torch.bfloat16).to(device)


def _codes(torch, shape, gen, device, int4=True):
    if int4:
        return torch.randint(0, 256, shape, generator=gen, device=device, dtype=torch.uint8)
    return torch.randint(-127, 128, shape, generator=gen, device=device, dtype=torch.int8)


def build_dense_problems(ctx: Ctx, w, batch: int, *, seed: int, split: str | None):
    """``batch`` dense problems on this rank.  ``split`` None: the workload as given; "weak": this rank's columns of
    a global problem with N * world columns; "strong": this rank's columns of the given problem.  A sharded problem
    is generated whole (same seed on every rank) and cut by ``distributed.shard_dense_rhs``."""
    torch, pkg = ctx.torch, ctx.pkg
    int4 = w["dtype"] == "int4"
    swiglu = w["epilogue"] == "swiglu"
    kb = w["k"] // 2 if int4 else w["k"]
    mult = 0.05 if int4 else 0.01
    groups = w["k"] // w["sub"] if w["sub"] else 0
    n_global = w["n"] * ctx.world if split == "weak" else w["n"]
    cols_global = 2 * n_global if swiglu else n_global
    shared = torch.Generator(device=ctx.device).manual_seed(seed)          # same stream on every rank
    shared_cpu = torch.Generator().manual_seed(seed)
    problems = []
    for _ in range(batch):
        a = _codes(torch, (w["m"], kb), shared, ctx.device, int4)
        a_scale = _scales(torch, (w["m"], groups) if groups else (w["m"],), shared_cpu, ctx.device, mult)
        b = _codes(torch, (kb, cols_global), shared, ctx.device, int4)
        b_scale = _scales(torch, (groups, cols_global) if groups else (cols_global,), shared_cpu, ctx.device, mult)
        columns = (0, n_global)
        if split is not None and ctx.world > 1:
            b, b_scale, columns = ctx.shard.shard_dense_rhs(b, b_scale, layout=pkg.GemmLayout.NN, world_size=ctx.world,
                                                            rank=ctx.rank, swiglu=swiglu)
        n_local = columns[1] - columns[0]
        problems.append(dict(a=a, b=b, a_scale=a_scale, b_scale=b_scale, n=n_local, columns=columns,
                             out=torch.empty((w["m"], n_local), device=ctx.device, dtype=torch.bfloat16)))
    return problems


def build_ragged_problems(ctx: Ctx, w, batch: int, *, seed: int, sizes, owned):
    """``batch`` grouped problems holding the groups ``owned`` (indices into ``sizes``) of a global problem that is
    generated whole with the same seed on every rank and cut by ``distributed.shard_ragged_fwd`` / ``_bwd``."""
    torch, pkg = ctx.torch, ctx.pkg
    shared = torch.Generator(device=ctx.device).manual_seed(seed)
    shared_cpu = torch.Generator().manual_seed(seed)
    total, groups = int(sizes.sum()), len(sizes)
    whole = len(owned) == groups
    problems = []
    for _ in range(batch):
        if w["kind"] == "ragged_fwd":
            lhs = _codes(torch, (total, w["k"] // 2), shared, ctx.device)
            rhs = _codes(torch, (groups, w["k"] // 2, w["n"]), shared, ctx.device)
            a_scale = _scales(torch, (total,), shared_cpu, ctx.device)
            b_scale = _scales(torch, (groups, w["n"]), shared_cpu, ctx.device)
            if whole:
                local = dict(lhs=lhs, rhs=rhs, a_scale=a_scale, b_scale=b_scale, group_sizes=sizes.to(ctx.device), row_index=None)
            else:
                part = ctx.shard.shard_ragged_fwd(lhs, rhs, a_scale, b_scale, sizes, owned)
                local = dict(lhs=part.lhs, rhs=part.rhs, a_scale=part.a_scale, b_scale=part.b_scale,
                             group_sizes=part.group_sizes.to(ctx.device), row_index=part.row_index)
            local["out"] = torch.empty((local["lhs"].shape[0], w["n"]), device=ctx.device, dtype=torch.bfloat16)
        elif w.get("flat"):
            mine = sizes[list(owned)]
            pairs = (int(mine.sum()) + 1) // 2
            local = dict(lhs=_codes(torch, (pairs, w["m"]), shared, ctx.device), rhs=_codes(torch, (pairs, w["n"]), shared, ctx.device),
                         a_scale=_scales(torch, (len(mine), w["m"]), shared_cpu, ctx.device),
                         b_scale=_scales(torch, (len(mine), w["n"]), shared_cpu, ctx.device), group_sizes=mine.to(ctx.device))
            local["out"] = torch.empty((len(mine), w["m"], w["n"]), device=ctx.device, dtype=torch.float32)
        else:
            cap = int(sizes.max()) if groups else 2
            cap = max(32, cap + (-cap) % 32)
            lhs = _codes(torch, (groups, cap // 2, w["m"]), shared, ctx.device)
            rhs = _codes(torch, (groups, cap // 2, w["n"]), shared, ctx.device)
            a_scale = _scales(torch, (groups, w["m"]), shared_cpu, ctx.device)
            b_scale = _scales(torch, (groups, w["n"]), shared_cpu, ctx.device)
            gs = sizes.to(ctx.device)
            if not whole:
                lhs, rhs, a_scale, b_scale, gs = ctx.shard.shard_ragged_bwd(lhs, rhs, a_scale, b_scale, gs, owned)
            local = dict(lhs=lhs, rhs=rhs, a_scale=a_scale, b_scale=b_scale, group_sizes=gs)
            local["out"] = torch.empty((len(owned), w["m"], w["n"]), device=ctx.device, dtype=torch.float32)
        problems.append(local)
    return problems


def make_pass(ctx: Ctx, w, problems):
    """``(callable, launches)``: one pass over all problems through the pointer-level binding of the C ABI."""
    torch, pkg, native = ctx.torch, ctx.pkg, ctx.native
    from strix_halo_int4_gemms_b200.ragged import PAIR_MIN_MEAN_GROUP_ROWS, PAIR_TASK_ROWS, RaggedBwdDotConfig, RaggedDotConfig

    device_index = torch.cuda.current_device()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    if w["kind"] == "dense":
        scale = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, w["sub"]) if w["sub"] else pc
        variant = native.make_variant(dtype=pkg.OperandDType(w["dtype"]), layout=pkg.GemmLayout.NN, scale=scale,
                                      epilogue=pkg.Epilogue(w["epilogue"]), out_dtype=native.OUT_BF16)
        # the scratch the library asks for (partial sums of the balanced tail); one buffer: the launches of a pass run in
        # stream order
        scratch = max(int(native.load_dispatch_library().b200_int4_gemms_dense_workspace_bytes(
            __import__("ctypes").byref(variant), w["m"], p["n"], w["k"])) for p in problems)
        workspace = torch.zeros(max(scratch, 16), dtype=torch.uint8, device=ctx.device)  # flag words start out zero
        args = [dict(a_ptr=p["a"].data_ptr(), b_ptr=p["b"].data_ptr(), a_scale_ptr=p["a_scale"].data_ptr(),
                     b_scale_ptr=p["b_scale"].data_ptr(), c_ptr=p["out"].data_ptr(), n=p["n"],
                     workspace_ptr=workspace.data_ptr() if scratch else 0, workspace_bytes=scratch) for p in problems]
        run_keepalive = workspace

        def run():
            for ptrs in args:
                # the stream is looked up per call: under CUDA-graph capture the current stream is the capturing one
                native.launch_dense(variant, device_index=device_index, stream_handle=torch.cuda.current_stream().cuda_stream,
                                    m=w["m"], k=w["k"], **ptrs)
        run.workspace = run_keepalive   # keeps the scratch alive as long as the callable
        return run, len(problems)
    if w["kind"] == "ragged_fwd":
        # the task height ragged_dot_int4 itself picks for groups this large: 256-row tasks on pairs of SMs
        rows, groups = problems[0]["lhs"].shape[0], len(problems[0]["group_sizes"])
        cfg = RaggedDotConfig(block_m=PAIR_TASK_ROWS if rows >= PAIR_MIN_MEAN_GROUP_ROWS * max(groups, 1) else 128)
        infos = [pkg.calculate_group_info(p["group_sizes"], cfg.block_m, align_tile=cfg.align_tile) for p in problems]

        def run():
            for p, info in zip(problems, infos):
                native.launch_ragged_fwd_kernel(p["lhs"], p["rhs"], group_info=info, a_scale=p["a_scale"], b_scale=p["b_scale"], out=p["out"],
                                                scale=pc, config=cfg, layout=pkg.GemmLayout.NN, rows=p["lhs"].shape[0], cols=w["n"],
                                                k_packed=w["k"] // 2, scale_cols=1)
        return run, len(problems)
    cfg = RaggedBwdDotConfig()
    if w.get("flat"):
        tokens = [int(p["group_sizes"].sum()) for p in problems]

        def run():
            for p, t in zip(problems, tokens):
                native.launch_ragged_bwd_flat_kernel(p["lhs"], p["rhs"], p["group_sizes"], a_scale=p["a_scale"], b_scale=p["b_scale"],
                                                     out=p["out"], tokens=t)
        return run, 2 * len(problems)  # the group-start scan + the GEMM kernel per problem

    def run():
        for p in problems:
            native.launch_ragged_bwd_kernel(p["lhs"], p["rhs"], p["group_sizes"], a_scale=p["a_scale"], b_scale=p["b_scale"], out=p["out"],
                                            scale=pc, config=cfg, layout=pkg.GemmLayout.TN, rows=w["m"], cols=w["n"],
                                            k_packed=p["lhs"].shape[1], scale_cols=1)
    return run, len(problems)


def make_e2e_runner(ctx: Ctx, w, problem):
    """One step through the PUBLIC API, default arguments, from pinned host buffers and back; returns
    ``(callable, h2d bytes, d2h bytes)``.

    Every step uploads its operands, calls the API and downloads the result.  Steps alternate between two
    streams with their own device and host buffers, the way a host pipeline would run them, so that one step's
    upload overlaps the previous step's download (PCIe is full duplex); the work of each step is unchanged.
    ``step.finish()`` joins both streams into the current one (called before the stop event is recorded)."""
    torch, pkg = ctx.torch, ctx.pkg
    lanes = 2
    streams = [torch.cuda.Stream() for _ in range(lanes)]
    names = ("a", "b", "a_scale", "b_scale") if w["kind"] == "dense" else ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")
    host = {k: problem[k].cpu().pin_memory() for k in names}
    out_host = [torch.empty(problem["out"].shape, dtype=problem["out"].dtype).pin_memory() for _ in range(lanes)]
    dev_sets = [{k: torch.empty_like(v, device="cuda") for k, v in host.items()} for _ in range(lanes)]
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host[0].numel() * out_host[0].element_size()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    state = {"i": 0}

    def call_api(dev):
        if w["kind"] == "dense":
            scale = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, w["sub"]) if w["sub"] else pc
            if w["epilogue"] == "swiglu":
                return pkg.fused_swiglu_up_gate(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], scale=scale,
                                                dtype=pkg.OperandDType(w["dtype"]))
            return pkg.mm(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], scale=scale,
                          dtype=pkg.OperandDType(w["dtype"]), epilogue=pkg.Epilogue(w["epilogue"]))
        if w["kind"] == "ragged_fwd":
            return pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
        if w.get("flat"):
            return pkg.ragged_dot_int4_bwd_flat(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
        return pkg.ragged_dot_int4_bwd(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                                       layout=pkg.GemmLayout.TN)

    def step():
        lane = state["i"] % lanes
        state["i"] += 1
        stream, dev = streams[lane], dev_sets[lane]
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for k, v in host.items():
                dev[k].copy_(v, non_blocking=True)
            out = call_api(dev)
            out_host[lane].copy_(out, non_blocking=True)

    def finish():
        for stream in streams:
            torch.cuda.current_stream().wait_stream(stream)

    def copy_rates(reps: int = 3) -> dict:
        """GB/s of the upload and of the download alone (pinned host memory, this rank)."""
        rates = {}
        for name, fn, nbytes in (("h2d_gbs", lambda: [dev_sets[0][k].copy_(v, non_blocking=True) for k, v in host.items()], h2d),
                                 ("d2h_gbs", lambda: out_host[0].copy_(problem["out"], non_blocking=True), d2h)):
            fn()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(reps):
                fn()
            stop.record()
            stop.synchronize()
            rates[name] = round(nbytes * reps / (start.elapsed_time(stop) * 1e-3) / 1e9, 2)
        return rates

    step.finish = finish
    step.copy_rates = copy_rates
    return step, h2d, d2h


def timed_region(ctx: Ctx, step, steps: int, warmup: int, sampler=None) -> float:
    """ms for exactly ``steps`` steps, max over ranks, CUDA events on the current stream."""
    torch = ctx.torch
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with (sampler if sampler is not None else _Null()):
        start.record()
        for _ in range(steps):
            step()
        finish = getattr(step, "finish", None)
        if finish is not None:
            finish()  # steps that run on side streams: the stop event must come after all of them
        stop.record()
        stop.synchronize()
    torch.cuda.synchronize()
    ms = ctx.max_over_ranks(float(start.elapsed_time(stop)))
    if ctx.world > 1:
        ctx.dist.barrier()
    return ms


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def measure(ctx: Ctx, key: str, w, problems, *, ops_per_pass_rank: float, bytes_per_problem: float, steps: int, warmup: int,
            graph: bool, sustained_s: float, passes_override: int, e2e: bool, peaks, peak_source, traffic, vendor_tops,
            warm_steps: int = 1) -> dict:
    """Burst and sustained device-timed throughput of one workload on this rank's problems, its roofline fraction,
    clocks and (optionally) the end-to-end figure.  Every rank calls it; the numbers are whole-job (all ranks)."""
    torch, native = ctx.torch, ctx.native
    run_pass, launches_per_pass = make_pass(ctx, w, problems)
    batch = len(problems)
    run_pass()  # first-call set-up of the library happens outside any capture
    torch.cuda.synchronize()
    replay = run_pass
    if graph:
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            run_pass()
        replay = captured.replay
    native.reset_device_status(ctx.local_rank)
    ops_per_pass = ctx.sum_over_ranks(ops_per_pass_rank)

    # burst: a short region once the clocks have come up from idle (about 50 ms of replays), before the part has
    # drawn power for long
    first_ms = timed_region(ctx, replay, 2, max(warmup, 3)) / 2
    ramp = max(3, min(2000, int(50.0 / max(first_ms, 1e-3))))
    burst_passes = max(5, min(200, int(10.0 / max(first_ms, 1e-3))))
    if passes_override > 0:  # a short run was asked for (profiling): no ramp either
        ramp, burst_passes = 3, 2
    burst_ms = timed_region(ctx, replay, burst_passes, ramp) / burst_passes
    if passes_override > 0:
        passes = passes_override
    else:
        passes = max(1, math.ceil(1.1 * sustained_s * 1e3 / (steps * burst_ms)))

    def step():
        for _ in range(passes):
            replay()

    sampler = ClockSampler(visible_device_index(ctx.local_rank))
    ms = timed_region(ctx, step, steps, warm_steps, sampler)
    status = native.device_status(ctx.local_rank)
    if status[0] != 0:
        raise SystemExit(f"{key}: a kernel reported status {status}")
    ms_per_step = ms / steps
    ms_per_pass = ms_per_step / passes
    value = ops_per_pass / (ms_per_pass * 1e-3) / 1e12
    kernel_us = ms_per_pass * 1e3 / batch
    clocks = sampler.summary()
    per_gpu_tops = value / ctx.world
    sustained = ms >= 1000.0
    record = {
        "workload": w["name"], "metric": w["metric"], "value": value, "unit": "TOPS", "kernel_us": kernel_us,
        "ms_per_step": ms_per_step, "steps": steps, "passes_per_step": passes, "problems_per_pass": batch, "timed_region_s": ms / 1e3,
        "gpu_launches": launches_per_pass * passes * steps,
        "burst": {"value": ops_per_pass / (burst_ms * 1e-3) / 1e12, "unit": "TOPS", "kernel_us": burst_ms * 1e3 / batch,
                  "passes": burst_passes, "note": "first passes after warm-up, before the power cap settles the clock"},
        "clocks": clocks,
        "kernel_us_x_sm_mhz": kernel_us * clocks["sm_mhz"] if clocks.get("sm_mhz") else None,
    }
    bf16_peak = peaks["bf16_tflops_sustained"] if sustained and "bf16_tflops_sustained" in peaks else peaks["bf16_tflops"]
    which = "sustained" if bf16_peak != peaks["bf16_tflops"] else "burst"
    info = traffic.get(key) if ctx.world == 1 else None
    if w["kind"] == "ragged_bwd":
        achieved = bytes_per_problem / (kernel_us * 1e-6) / 1e9
        record["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                              "traffic": info["bytes"] if info else None, "traffic_source": info["source"] if info else None,
                              "peak_source": f"{peak_source} STREAM-style copy", "frac_of_nominal_hbm_8000": achieved / NOMINAL_HBM_GBS,
                              "algorithmic_bytes_per_launch": bytes_per_problem, "kernel_us": kernel_us}
    else:
        peak = 2.0 * bf16_peak
        record["roofline"] = {"bound": "tensor", "achieved": per_gpu_tops, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu_tops / peak,
                              "traffic": info["bytes"] if info else None, "traffic_source": info["source"] if info else None,
                              "peak_source": f"2 x {peak_source} cuBLAS bf16 {which} ({bf16_peak} TFLOP/s): kind::i8 runs at twice the bf16 rate",
                              "frac_of_nominal_int8_4500": per_gpu_tops / NOMINAL_INT8_TOPS,
                              "frac_of_nominal_at_sampled_clock": (per_gpu_tops / (NOMINAL_INT8_TOPS * clocks["sm_mhz"] / clocks["sm_max_mhz"])
                                                                   if clocks.get("sm_mhz") and clocks.get("sm_max_mhz") else None),
                              "algorithmic_bytes_per_launch": bytes_per_problem, "kernel_us": kernel_us}
        if vendor_tops:
            record["roofline"]["frac_of_vendor_int8_gemm"] = per_gpu_tops / vendor_tops[which]
    if key == "c1":
        record["latency_us"] = kernel_us
        record["note"] = "16.8 MOP on 4 tiles: launch-latency bound; kernel_us is the time per launch of back-to-back launches replayed from a CUDA graph"
    if e2e:
        e2e_step, h2d, d2h = make_e2e_runner(ctx, w, problems[0])
        e2e_steps = max(3, min(steps, 10))
        e2e_ms = timed_region(ctx, e2e_step, e2e_steps, 3) / e2e_steps
        rates = e2e_step.copy_rates()
        record["e2e"] = {"value": (ops_per_pass / batch) / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "h2d_bytes_per_step": int(h2d),
                         "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": e2e_steps,
                         "per_rank_copy_gbs": ctx.gather(rates), "host_numa_nodes_per_rank": ctx.gather(host_numa_nodes()),
                         "note": "one problem per step through the public API with default arguments; pinned host operands in, result out, "
                                 "copies inside the timed region; steps alternate between two streams so that uploads overlap the previous "
                                 "step's download.  Bound by the host link: with several ranks the copies of all GPUs share one socket's memory"}
    return record


def vendor_int8_probe(torch) -> dict:
    """The vendor library's int8 GEMM (torch._int_mm -> cuBLASLt) at 8192^3 in this run: best of 10 launches and a
    back-to-back loop of about half a second.  A measured int8 figure to set beside the nominal 4500 TOPS."""
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
    reps = max(10, int(500.0 / best))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        torch._int_mm(a, b)
    stop.record()
    stop.synchronize()
    loop = float(start.elapsed_time(stop)) / reps
    ops = 2.0 * n ** 3 / 1e12
    return {"probe": "torch._int_mm int8 8192^3 -> int32", "burst": ops / (best * 1e-3), "sustained": ops / (loop * 1e-3), "loop_reps": reps}


def batch_for(bytes_per_problem: float) -> int:
    return max(2, int(-(-2.2 * L2_BYTES // bytes_per_problem)))


def plan_problem(ctx: Ctx, key: str, *, split: str | None, batch_override: int, seed: int):
    """Problems of workload ``key`` for this rank and their per-pass ops / per-problem bytes.
    Returns ``(w, problems, ops_per_pass_rank, bytes_per_problem, extra_config)``."""
    torch, shard = ctx.torch, ctx.shard
    w = dict(WORKLOADS[key])
    extra = {}
    if w["kind"] == "dense":
        n_local = w["n"]
        if split == "strong" and ctx.world > 1:
            lo, hi = shard.column_block(w["n"], ctx.world, ctx.rank)
            n_local = hi - lo
        per_problem = dense_bytes(w, n_local)
        # every rank runs the same number of problems per pass (the smallest shard decides: its sets must still
        # exceed L2 between reuses)
        widths = ([hi - lo for lo, hi in (shard.column_block(w["n"], ctx.world, r) for r in range(ctx.world))]
                  if split == "strong" and ctx.world > 1 else [n_local])
        batch = batch_override or min(max(batch_for(dense_bytes(w, n)) for n in widths), 1024)
        problems = build_dense_problems(ctx, w, batch, seed=seed, split=split)
        ops = sum(dense_ops(w, p["n"]) for p in problems)
        return w, problems, ops, per_problem, extra
    sizes = config5_group_sizes(torch)
    if split == "weak" and ctx.world > 1:
        # expert-parallel, weak scaling: the global problem has 64 * world groups
        sizes = torch.cat([sizes[torch.randperm(64, generator=torch.Generator().manual_seed(r))] for r in range(ctx.world)])
    # the backward dot writes a [M, N] fp32 slab per group whatever the group's size: groups count as two mean groups' rows
    slab_rows = 2 * int(sizes.sum()) // max(len(sizes), 1) if w["kind"] == "ragged_bwd" else 0
    plan = (shard.assign_groups(sizes.tolist(), ctx.world, per_group_cost=slab_rows) if (split and ctx.world > 1)
            else [list(range(len(sizes)))])
    owned = plan[ctx.rank] if (split and ctx.world > 1) else plan[0]
    if split and ctx.world > 1:
        extra["load_imbalance_max_over_mean"] = shard.load_imbalance(sizes.tolist(), plan)
    rows_local = int(sizes[list(owned)].sum())
    per_problem = ragged_bytes(w, rows_local, len(owned))
    # the same number of problems per pass on every rank, decided by the rank with the smallest shard
    batch = batch_override or max(batch_for(ragged_bytes(w, int(sizes[list(groups)].sum()), len(groups))) for groups in plan)
    problems = build_ragged_problems(ctx, w, batch, seed=seed, sizes=sizes, owned=owned)
    w["plan"], w["sizes"] = plan, sizes
    return w, problems, ragged_ops(w, rows_local) * batch, per_problem, extra


def time_all_gather(ctx: Ctx, w, problem, reps: int = 10) -> dict | None:
    """The NCCL all-gather that assembles the full result from the ranks' local outputs, timed on its own."""
    torch, shard, dist = ctx.torch, ctx.shard, ctx.dist
    if ctx.world == 1 or w["kind"] == "ragged_bwd":
        return None  # backward outputs are whole [g] slabs that stay with their expert
    if w["kind"] == "dense":
        ranges = [shard.column_block(w["n"], ctx.world, r) for r in range(ctx.world)]
        fn = lambda: shard.all_gather_columns(problem["out"], ranges)
        nbytes = 2 * w["m"] * w["n"]
    else:
        sizes, plan = w["sizes"], w["plan"]
        ends = torch.cumsum(sizes, 0)
        starts = ends - sizes
        indices = [torch.cat([torch.arange(int(starts[g]), int(ends[g])) for g in groups]) if groups else torch.zeros(0, dtype=torch.int64)
                   for groups in plan]
        indices = [idx.to(ctx.device) for idx in indices]
        fn = lambda: shard.all_gather_rows(problem["out"], indices, int(sizes.sum()))
        nbytes = 2 * int(sizes.sum()) * w["n"]
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    stop.synchronize()
    us = ctx.max_over_ranks(float(start.elapsed_time(stop))) / reps * 1e3
    return {"us": us, "gathered_bytes": nbytes, "backend": "nccl all_gather_into_tensor + local placement", "reps": reps}


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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="independent problems per pass (0 = enough to exceed L2 twice over)")
    ap.add_argument("--passes", type=int, default=0, help="passes per step (0 = enough for the timed steps to last a second)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every pass from Python instead of replaying a CUDA graph of one pass")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="measure the headline workload only (no `workloads` / `strong` records, no vendor probe)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    head = dict(WORKLOADS[args.workload])

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference_arm(args, head)), flush=True)
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

    status = pkg.dispatch_runtime_status()
    if not status.has_linked_kernels:
        raise SystemExit(f"CUDA library at {status.library_path} cannot run here: {status}")
    ctx = Ctx(torch, dist, pkg, native, shard, rank, local_rank, world)
    peaks, peak_source = load_peaks()
    traffic = load_measured_traffic()
    vendor = None
    if not args.no_sub and world == 1:
        vendor = vendor_int8_probe(torch)
    common = dict(steps=args.steps, warmup=args.warmup, graph=not args.no_graph, sustained_s=SUSTAINED_SECONDS,
                  passes_override=args.passes, peaks=peaks, peak_source=peak_source, traffic=traffic, vendor_tops=vendor)

    # ---- headline (weak scaling at N > 1)
    w, problems, ops, per_problem, extra = plan_problem(ctx, args.workload, split="weak" if world > 1 else None,
                                                        batch_override=args.batch, seed=1234)
    headline = measure(ctx, args.workload, w, problems, ops_per_pass_rank=ops, bytes_per_problem=per_problem, e2e=not args.no_e2e,
                       warm_steps=args.warmup, **common)
    batch = len(problems)
    del problems
    torch.cuda.empty_cache()

    # ---- the other BASELINE configurations (one GPU) / the given problems split over the ranks (N > 1)
    workloads, strong = {}, {}
    if not args.no_sub:
        if world == 1:
            for key in SUB_WORKLOADS:
                if key == args.workload:
                    continue
                ws, ps, ops_s, bytes_s, _ = plan_problem(ctx, key, split=None, batch_override=0, seed=4321)
                workloads[key] = measure(ctx, key, ws, ps, ops_per_pass_rank=ops_s, bytes_per_problem=bytes_s, e2e=not args.no_e2e, **common)
                del ps
                torch.cuda.empty_cache()
        else:
            for key in STRONG_WORKLOADS:
                ws, ps, ops_s, bytes_s, extra_s = plan_problem(ctx, key, split="strong", batch_override=0, seed=4321)
                rec = measure(ctx, key, ws, ps, ops_per_pass_rank=ops_s, bytes_per_problem=bytes_s, e2e=False, **common)
                rec.update(extra_s)
                rec["scaling"] = "strong"
                rec["parallelism"] = ("column-parallel along N through distributed.shard_dense_rhs (A replicated, [M, N/ranks] local output)"
                                      if ws["kind"] == "dense" else "expert-parallel over the 64 groups, distributed.assign_groups (LPT)")
                gather = time_all_gather(ctx, ws, ps[0])
                if gather is not None:
                    rec["all_gather"] = gather
                strong[key] = rec
                del ps
                torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    line = {
        "metric": w["metric"], "value": headline["value"], "unit": "TOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": headline["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s32 accumulate of int8 tensor-core products (int4 or int8 operands), fp32 scale, bf16/fp32 store",
        "data": "synthetic",
        "config": {
            "workload": w["name"], "problems_per_step": batch * headline["passes_per_step"], "problems_per_pass": batch,
            "passes_per_step": headline["passes_per_step"],
            "launch": "one CUDA graph replay per pass" if not args.no_graph else "one Python call per kernel",
            "l2": f"{batch} independent operand/output sets per pass, {batch * per_problem / 1e6:.0f} MB touched between reuses (> 126 MB L2)",
            "parallelism": "none" if world == 1 else (
                "column-parallel along N: global N = N x ranks, each rank's columns of the global B cut by distributed.shard_dense_rhs"
                if w["kind"] == "dense" else
                f"expert-parallel: 64 x ranks groups, distributed.assign_groups (LPT), max/mean load {extra.get('load_imbalance_max_over_mean', 1.0):.3f}"),
            "per_gpu_problem": "same as 1-GPU (weak scaling)",
        },
        "timed_region_s": headline["timed_region_s"],
        "clocks": headline["clocks"],
        "gpu_launches": headline["gpu_launches"],
        "kernel_us": headline["kernel_us"],
        "kernel_us_x_sm_mhz": headline["kernel_us_x_sm_mhz"],
        "burst": headline["burst"],
        "roofline": headline["roofline"],
        "pct_of_nominal_int8_peak": 100.0 * headline["value"] / world / NOMINAL_INT8_TOPS,
    }
    if "e2e" in headline:
        line["e2e"] = headline["e2e"]
    if vendor is not None:
        line["vendor_int8_gemm"] = vendor
    if workloads:
        line["workloads"] = workloads
    if strong:
        line["strong"] = strong
    if not args.no_cpu_baseline:
        tops, rows, seconds, cores = cpu_reference_sample(head, budget_s=12.0)
        line["cpu_baseline"] = {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
                                "sample": f"{rows} rows of the same workload in {seconds:.1f} s (reference PyTorch int32-matmul math)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
