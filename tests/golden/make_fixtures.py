"""Generate golden fixtures by running the REFERENCE package on CPU.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_fixtures.py <path of the reference checkout>

It imports ``amd_strix_halo_kernels`` from ``<reference>/src`` and the grouped-dot reference
functions from ``<reference>/tests/test_ragged_dot.py`` (the package itself has no reference mode
for the grouped dots), feeds them seeded inputs and stores inputs and outputs in
``tests/golden/reference_vectors.npz``.  bf16 tensors are stored as uint16 bit patterns.

The tests never import the reference; they read the ``.npz`` only.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "reference_vectors.npz"


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(reference_root: str) -> None:
    root = Path(reference_root)
    sys.path.insert(0, str(root / "src"))
    import amd_strix_halo_kernels as ref
    from amd_strix_halo_kernels.api import explicit_mm, fused_swiglu_up_gate, mm
    from amd_strix_halo_kernels.quant import (
        fake_quant_int,
        pack_int4_k_major,
        pack_rhs_subchannel_scales,
        unpack_int4_k_major,
    )

    spec = importlib.util.spec_from_file_location("ref_test_ragged", root / "tests" / "test_ragged_dot.py")
    ragged_tests = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ragged_tests)

    store: dict[str, np.ndarray] = {}
    gen = torch.Generator().manual_seed(20240607)

    # ---- operand format ---------------------------------------------------------------------
    for name, shape in (("even", (5, 12)), ("odd", (3, 7)), ("batched", (2, 3, 6))):
        x = torch.randint(-8, 8, shape, generator=gen, dtype=torch.int8)
        p = pack_int4_k_major(x)
        store[f"pack/{name}/x"] = x.numpy()
        store[f"pack/{name}/packed"] = p.numpy()
        store[f"pack/{name}/unpacked"] = unpack_int4_k_major(p).numpy()
    xf = (torch.randn((6, 33), generator=gen) * 0.3).to(torch.bfloat16)
    store["fake_quant/x_bits"] = bits(xf)
    store["fake_quant/q4_scale0p1"] = fake_quant_int(xf, bits=4, scale=0.1).numpy()
    store["fake_quant/q8_scale0p01"] = fake_quant_int(xf, bits=8, scale=0.01).numpy()
    sc = torch.arange(2 * 3 * 4, dtype=torch.bfloat16).reshape(2, 3, 4)
    store["scale_pack/in_bits"] = bits(sc)
    store["scale_pack/out_bits"] = bits(pack_rhs_subchannel_scales(sc))

    # ---- dense reference math -----------------------------------------------------------------
    M, D, K = 24, 32, 96
    reg = ref.default_registry
    names = []
    for dtype in (ref.OperandDType.INT4, ref.OperandDType.INT8):
        lo, hi = (-8, 8) if dtype is ref.OperandDType.INT4 else (-127, 128)
        for layout in (ref.GemmLayout.NN, ref.GemmLayout.NT, ref.GemmLayout.TN):
            for scale in (
                ref.ScaleSpec(ref.ScaleMode.PER_CHANNEL),
                ref.ScaleSpec(ref.ScaleMode.SUBCHANNEL, 32),
                ref.ScaleSpec(ref.ScaleMode.SUBCHANNEL, 64),
            ):
                for epilogue in (ref.Epilogue.NONE, ref.Epilogue.RELU2, ref.Epilogue.SWIGLU):
                    cols = 2 * D if epilogue is ref.Epilogue.SWIGLU else D
                    a_q = torch.randint(lo, hi, (M, K), generator=gen, dtype=torch.int8)
                    b_q = torch.randint(lo, hi, (K, cols), generator=gen, dtype=torch.int8)
                    kernel = reg.select_reference(dtype=dtype, layout=layout, scale=scale, epilogue=epilogue)
                    a_arg, b_arg = ragged_tests_kernel_args(ref, a_q, b_q, kernel)
                    if scale.mode is ref.ScaleMode.PER_CHANNEL:
                        sa = ((torch.rand((M,), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                        sb = ((torch.rand((cols,), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                    else:
                        groups = -(-K // scale.subchannel_size)
                        sa = ((torch.rand((M, groups), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                        sb = ((torch.rand((groups, cols), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                    out = explicit_mm(a_arg, b_arg, kernel=kernel, a_scale=sa, b_scale=sb, use_reference=True)
                    key = f"dense/{dtype.value}_{layout.value}_{scale.label}_{epilogue.value}"
                    names.append(key)
                    store[f"{key}/a"] = a_arg.numpy()
                    store[f"{key}/b"] = b_arg.numpy()
                    store[f"{key}/a_scale_bits"] = bits(sa)
                    store[f"{key}/b_scale_bits"] = bits(sb)
                    store[f"{key}/out_bits"] = bits(out)
    store["dense/names"] = np.array(names)

    # float32 output (split-K metadata) and unscaled accumulators
    a_q = torch.randint(-8, 8, (16, 64), generator=gen, dtype=torch.int8)
    b_q = torch.randint(-8, 8, (64, 24), generator=gen, dtype=torch.int8)
    ap = pack_int4_k_major(a_q)
    bp = pack_int4_k_major(b_q.t()).t().contiguous()
    k32 = reg.select_reference(
        dtype=ref.OperandDType.INT4, scale=ref.ScaleSpec(ref.ScaleMode.PER_CHANNEL), epilogue=ref.Epilogue.NONE, split_k=2
    )
    sa = ((torch.rand((16,), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
    sb = ((torch.rand((24,), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
    store["dense_f32/a"] = ap.numpy()
    store["dense_f32/b"] = bp.numpy()
    store["dense_f32/a_scale_bits"] = bits(sa)
    store["dense_f32/b_scale_bits"] = bits(sb)
    store["dense_f32/out"] = explicit_mm(ap, bp, kernel=k32, a_scale=sa, b_scale=sb, use_reference=True).numpy()
    store["dense_f32/acc"] = torch.matmul(a_q.to(torch.int32), b_q.to(torch.int32)).numpy()

    # ---- the quick-start configuration (README: M=128, N=1024, K=64, bf16 ones scales) ---------
    torch.manual_seed(0)
    a = torch.randn((128, 64), dtype=torch.bfloat16) * 0.1
    b = torch.randn((64, 1024), dtype=torch.bfloat16) * 0.1
    a_q = fake_quant_int(a, bits=4, scale=0.1)
    b_q = fake_quant_int(b, bits=4, scale=0.1)
    ap = pack_int4_k_major(a_q)
    bp = pack_int4_k_major(b_q.t()).t().contiguous()
    ones_a = torch.ones((128,), dtype=torch.bfloat16)
    ones_b = torch.ones((1024,), dtype=torch.bfloat16)
    out = mm(ap, bp, a_scale=ones_a, b_scale=ones_b, use_reference=True)
    store["quickstart/a"] = ap.numpy()
    store["quickstart/b"] = bp.numpy()
    store["quickstart/out_bits"] = bits(out)

    # ---- calculate_group_info ------------------------------------------------------------------
    gi_cases = [
        ([17, 31, 24], 32, 8, None),
        ([2, 0, 7], 16, 8, 4),
        ([0, 0, 0], 64, 8, None),
        ([300, 1, 0, 129, 64], 128, 8, None),
        ([5, 250, 3, 0, 77], 64, 16, 12),
        ([128, 128], 128, 128, None),
    ]
    for i, (sizes, tile, align, tid) in enumerate(gi_cases):
        info = ref.calculate_group_info(torch.tensor(sizes, dtype=torch.int64), tile, tid_size=tid, align_tile=align)
        store[f"group_info/{i}/sizes"] = np.array(sizes, dtype=np.int64)
        store[f"group_info/{i}/params"] = np.array([tile, align, -1 if tid is None else tid, info.num_tasks], dtype=np.int64)
        for field in ("group_id", "block_start", "actual_start", "actual_end", "start_within_block", "actual_size"):
            store[f"group_info/{i}/{field}"] = getattr(info, field).numpy()
    store["group_info/count"] = np.array(len(gi_cases))

    # ---- grouped dots (reference test helpers) -------------------------------------------------
    layouts = {"nn": ref.GemmLayout.NN, "nt": ref.GemmLayout.NT, "tn": ref.GemmLayout.TN, "tt": ref.GemmLayout.TT}
    sizes_fwd = [17, 0, 31, 24]
    Mf, Kf, Nf = sum(sizes_fwd), 40, 48
    for lname, layout in layouts.items():
        for sub in (0, 32):
            a_q = torch.randint(-8, 8, (Mf, Kf), generator=gen, dtype=torch.int8)
            b_q = torch.randint(-8, 8, (len(sizes_fwd), Kf, Nf), generator=gen, dtype=torch.int8)
            lhs, rhs = ragged_tests._pack_forward_args(a_q, b_q, layout)
            gs = torch.tensor(sizes_fwd, dtype=torch.int64)
            if sub == 0:
                sa = ((torch.rand((Mf,), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                sb = ((torch.rand((len(sizes_fwd), Nf), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                out = ragged_tests._manual_grouped_reference(a_q, b_q, gs, sa, sb)
            else:
                cols = -(-Kf // sub)
                sa = ((torch.rand((Mf, cols), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                sb = ((torch.rand((len(sizes_fwd), cols, Nf), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                out = ragged_tests._manual_grouped_subchannel_reference(a_q, b_q, gs, sa, sb, sub)
            # rows of empty groups are never written by the reference helper (torch.empty); none here
            key = f"ragged_fwd/{lname}_{'pc' if sub == 0 else 'sc32'}"
            store[f"{key}/lhs"] = lhs.numpy()
            store[f"{key}/rhs"] = rhs.numpy()
            store[f"{key}/group_sizes"] = gs.numpy()
            store[f"{key}/a_scale_bits"] = bits(sa)
            store[f"{key}/b_scale_bits"] = bits(sb)
            store[f"{key}/out_f32"] = out.numpy()
    sizes_bwd = [37, 0, 64, 5]
    Mb, Nb, cap = 24, 40, 64
    for lname, layout in layouts.items():
        for sub in (0, 32):
            a_q = torch.randint(-8, 8, (len(sizes_bwd), Mb, cap), generator=gen, dtype=torch.int8)
            b_q = torch.randint(-8, 8, (len(sizes_bwd), cap, Nb), generator=gen, dtype=torch.int8)
            lhs, rhs = ragged_tests._pack_bwd_args(a_q, b_q, layout)
            gs = torch.tensor(sizes_bwd, dtype=torch.int64)
            if sub == 0:
                sa = ((torch.rand((len(sizes_bwd), Mb), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                sb = ((torch.rand((len(sizes_bwd), Nb), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                out = ragged_tests._manual_bwd_reference(a_q, b_q, gs, sa, sb)
            else:
                cols = -(-cap // sub)
                sa = ((torch.rand((len(sizes_bwd), Mb, cols), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                sb = ((torch.rand((len(sizes_bwd), cols, Nb), generator=gen) + 0.5) * 0.05).to(torch.bfloat16)
                out = ragged_tests._manual_bwd_subchannel_reference(a_q, b_q, gs, sa, sb, sub)
            key = f"ragged_bwd/{lname}_{'pc' if sub == 0 else 'sc32'}"
            store[f"{key}/lhs"] = lhs.numpy()
            store[f"{key}/rhs"] = rhs.numpy()
            store[f"{key}/group_sizes"] = gs.numpy()
            store[f"{key}/a_scale_bits"] = bits(sa)
            store[f"{key}/b_scale_bits"] = bits(sb)
            store[f"{key}/out_f32"] = out.numpy()

    # ---- metric --------------------------------------------------------------------------------
    from amd_strix_halo_kernels.benchmarking import BenchmarkShape, summarize_runtime_samples, tops_for_runtime

    store["metric/tops_1024_1ms"] = np.array(tops_for_runtime(BenchmarkShape(1024, 1024, 1024), 1.0))
    summary = summarize_runtime_samples([3.0, 1.0, 0.0, 2.0, 10.0, -1.0])
    store["metric/summary_keys"] = np.array(sorted(summary))
    store["metric/summary_values"] = np.array([float(summary[k]) for k in sorted(summary)])

    np.savez_compressed(OUT, **store)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(store)} arrays)")


def ragged_tests_kernel_args(ref, a_q, b_q, kernel):
    """Logical ``A[M,K]``, ``B[K,N]`` -> stored operands in ``kernel``'s layout (the reference's
    tests/test_quant.py:113-129, restated with the reference's own pack function)."""
    from amd_strix_halo_kernels.quant import pack_int4_k_major

    a_t = kernel.layout in (ref.GemmLayout.TN, ref.GemmLayout.TT)
    b_t = kernel.layout in (ref.GemmLayout.NT, ref.GemmLayout.TT)
    if kernel.a_dtype is ref.OperandDType.INT4:
        a = pack_int4_k_major(a_q)
        a = a.transpose(0, 1).contiguous() if a_t else a
        b = pack_int4_k_major(b_q.transpose(0, 1))
        b = b.contiguous() if b_t else b.transpose(0, 1).contiguous()
        return a, b
    a = a_q.transpose(0, 1).contiguous() if a_t else a_q
    b = b_q.transpose(0, 1).contiguous() if b_t else b_q
    return a, b


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_fixtures.py <path of the reference checkout>")
    main(sys.argv[1])
