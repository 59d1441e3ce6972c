"""Split-K (b200_gemm_variant.split_k = 2, 4, 8): K slices reduced by different CTAs into a workspace, then added in a
fixed order by a second kernel.  Per-channel scales: exact s32 partial sums, so the result is bit-identical to the
single-pass kernel and to the oracle.  Subchannel scales: fp32 partial sums added in slice order, deterministic and
within the bf16 output bar of the oracle.  Reference: the SPLIT_K kernels of scripts/generate_amdgcn.py:189-192."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import as_f32, assert_close_rms, dense_case, oracle_dense, scale_spec

pytestmark = pytest.mark.gpu


def _split_launch(pkg, case, *, m, n, k, dtype="int4", layout="nn", sub=0, split_k=2, cta_group=None, workspace=True, order="fused"):
    from strix_halo_int4_gemms_b200 import native

    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    variant = native.make_variant(dtype=pkg.OperandDType(dtype), layout=getattr(pkg.GemmLayout, layout.upper()), scale=scale_spec(pkg, sub),
                                  epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_F32, split_k=split_k, cta_group=cta_group,
                                  accumulate_order=native.ACCUMULATE_REFERENCE if order == "reference" else native.ACCUMULATE_FUSED)
    stream = torch.cuda.current_stream().cuda_stream
    ptr, size = native.dense_workspace(variant, m=m, n=n, k=k, device=out.device, stream_handle=stream) if workspace else (0, 0)
    native.launch_dense(variant, device_index=0, stream_handle=stream, a_ptr=dev["a"].data_ptr(), b_ptr=dev["b"].data_ptr(),
                        a_scale_ptr=dev["a_scale"].data_ptr(), b_scale_ptr=dev["b_scale"].data_ptr(), c_ptr=out.data_ptr(),
                        m=m, n=n, k=k, workspace_ptr=ptr, workspace_bytes=size)
    torch.cuda.synchronize()
    status, detail = native.device_status(0)
    assert status == 0, (status, detail)
    return out


@pytest.mark.parametrize("dtype", ["int4", "int8"])
@pytest.mark.parametrize("layout", ["nn", "nt"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 1024), (128, 1024, 4096), (200, 300 // 4 * 16, 1152), (512, 512, 2048)])
def test_per_channel_split_is_bit_identical_to_the_oracle(pkg, dtype, layout, m, n, k):
    case = dense_case(pkg, m=m, n=n, k=k, dtype=dtype, layout=layout, seed=m + k)
    want = oracle_dense(case, dtype=dtype, layout=layout, out_bf16=False)
    for split in (2, 4, 8):
        got = _split_launch(pkg, case, m=m, n=n, k=k, dtype=dtype, layout=layout, split_k=split)
        np.testing.assert_array_equal(got.cpu().numpy(), want, err_msg=f"split_k={split}")


def test_split_on_cta_pairs_and_plan(pkg):
    from strix_halo_int4_gemms_b200 import native

    m, n, k = 512, 512, 4096
    case = dense_case(pkg, m=m, n=n, k=k, seed=5)
    want = oracle_dense(case, out_bf16=False)
    for cta_group, path in ((native.CTA_GROUP_PAIR, native.LAUNCHED_TCGEN05_PAIR), (native.CTA_GROUP_SINGLE, native.LAUNCHED_TCGEN05)):
        got = _split_launch(pkg, case, m=m, n=n, k=k, split_k=4, cta_group=cta_group)
        assert native.last_launch_path() == path
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    pc = scale_spec(pkg, 0)
    split = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE,
                                out_dtype=native.OUT_F32, split_k=8)
    plain = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE,
                                out_dtype=native.OUT_F32, tail_balance=native.TAIL_OFF)
    # a skinny problem: 4 tiles without the split, 32 CTAs with it; a short K gives fewer slices than asked for
    assert native.plan_dense(plain, m=128, n=1024, k=8192).as_tuple()[:2] == (native.LAUNCHED_TCGEN05, 4)
    assert native.plan_dense(split, m=128, n=1024, k=8192).as_tuple() == (native.LAUNCHED_TCGEN05, 32, 128, 256, 8, 8)
    assert native.plan_dense(split, m=128, n=1024, k=256).split_k == 2
    assert native.plan_dense(split, m=128, n=1024, k=64).split_k == 1


@pytest.mark.parametrize("sub", [256, 128, 64, 32])
@pytest.mark.parametrize("layout", ["nn", "nt"])
def test_subchannel_split_is_deterministic_and_within_tolerance(pkg, sub, layout):
    m, n, k = 256, 512, 2048
    case = dense_case(pkg, m=m, n=n, k=k, layout=layout, sub=sub, seed=sub)
    want = oracle_dense(case, layout=layout, sub=sub, out_bf16=False)
    first = _split_launch(pkg, case, m=m, n=n, k=k, layout=layout, sub=sub, split_k=4)
    assert_close_rms(first.cpu().numpy(), want, rtol=1e-4, atol_rms=1e-5, what=f"sc{sub} split 4")
    for _ in range(2):
        assert torch.equal(first, _split_launch(pkg, case, m=m, n=n, k=k, layout=layout, sub=sub, split_k=4))
    # one slice (K of a single K-group multiple): exactly the single-pass kernel
    short = dense_case(pkg, m=128, n=256, k=sub if sub >= 128 else 128, layout=layout, sub=sub, seed=1)
    got = _split_launch(pkg, short, m=128, n=256, k=sub if sub >= 128 else 128, layout=layout, sub=sub, split_k=8, order="reference")
    np.testing.assert_array_equal(got.cpu().numpy(), oracle_dense(short, layout=layout, sub=sub, out_bf16=False))


def test_split_through_the_registry_and_api(pkg):
    """explicit_mm with a split-K entry: the workspace is the binding's business, the result float32."""
    m, n, k = 128, 1024, 8192
    case = dense_case(pkg, m=m, n=n, k=k, seed=9)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    want = oracle_dense(case, out_bf16=False)
    for schedule in (pkg.KernelSchedule.STANDARD, pkg.KernelSchedule.PERSISTENT):
        kernel = pkg.default_registry.select(dtype=pkg.OperandDType.INT4, scale=scale_spec(pkg, 0), epilogue=pkg.Epilogue.NONE,
                                             m=m, n=n, k=k, split_k=8, schedule=schedule)
        got = pkg.explicit_mm(dev["a"], dev["b"], kernel=kernel, a_scale=dev["a_scale"], b_scale=dev["b_scale"])
        assert got.dtype is torch.float32
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    run_twice = [pkg.explicit_mm(dev["a"], dev["b"], kernel=kernel, a_scale=dev["a_scale"], b_scale=dev["b_scale"]) for _ in range(2)]
    assert torch.equal(run_twice[0], run_twice[1])


def test_split_needs_a_workspace_and_a_kernel(pkg):
    case = dense_case(pkg, m=128, n=256, k=1024, seed=2)
    with pytest.raises(RuntimeError, match="split_k > 1 needs a 16-byte aligned workspace"):
        _split_launch(pkg, case, m=128, n=256, k=1024, split_k=2, workspace=False)
    tn = dense_case(pkg, m=128, n=256, k=1024, layout="tn", seed=2)
    with pytest.raises(RuntimeError, match="split_k > 1 runs on the tensor-core kernel only"):
        _split_launch(pkg, tn, m=128, n=256, k=1024, layout="tn", split_k=2)


def test_split_k_pays_on_skinny_shapes(pkg):
    """M = 128, N = 1024: four tiles without a split.  With a long K the split must be at least twice as fast."""
    from strix_halo_int4_gemms_b200 import native

    m, n, k = 128, 1024, 32768
    case = dense_case(pkg, m=m, n=n, k=k, seed=3)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    out = torch.empty((m, n), device="cuda", dtype=torch.float32)
    times = {}
    for split in (1, 8):
        variant = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0),
                                      epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_F32, split_k=split, tail_balance=native.TAIL_OFF)
        ptr, size = native.dense_workspace(variant, m=m, n=n, k=k, device=out.device, stream_handle=torch.cuda.current_stream().cuda_stream)

        def run():
            native.launch_dense(variant, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=dev["a"].data_ptr(), b_ptr=dev["b"].data_ptr(),
                                a_scale_ptr=dev["a_scale"].data_ptr(), b_scale_ptr=dev["b_scale"].data_ptr(), c_ptr=out.data_ptr(),
                                m=m, n=n, k=k, workspace_ptr=ptr, workspace_bytes=size)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()          # GPU time, not the host's launch rate
        with torch.cuda.graph(graph):
            for _ in range(20):
                run()
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(3):
            graph.replay()
        stop.record()
        stop.synchronize()
        times[split] = start.elapsed_time(stop) / 60
    assert times[8] * 2.0 <= times[1], times
