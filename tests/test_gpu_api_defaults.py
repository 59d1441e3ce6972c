"""What a drop-in caller gets: mm() / fused_swiglu_up_gate() with default arguments must reach the same kernel form,
and the same speed, as the pointer-level launch the benchmark times; launches that go to the CUDA-core kernel say so."""
import warnings

import pytest
import torch

from helpers import dense_case, scale_spec

pytestmark = pytest.mark.gpu


def _time(fn, reps=10):
    """GPU time per call of ``fn``: ``reps`` calls captured into a CUDA graph and replayed, so that host-side work
    (argument checks, registry look-up, output allocation) is not part of what is compared."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(3):
        graph.replay()
    stop.record()
    stop.synchronize()
    return start.elapsed_time(stop) / (3 * reps)


def _random_problem(m, n, k, *, sub=0, swiglu=False, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    cols = 2 * n if swiglu else n
    a = torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.uint8)
    b = torch.randint(0, 256, (k // 2, cols), generator=g, device="cuda", dtype=torch.uint8)
    groups = k // sub if sub else 0
    sa = ((torch.rand((m, groups) if groups else (m,), device="cuda", generator=g) + 0.5) * 0.05).bfloat16()
    sb = ((torch.rand((groups, cols) if groups else (cols,), device="cuda", generator=g) + 0.5) * 0.05).bfloat16()
    return a, b, sa, sb


def test_defaults_reach_cta_pairs_at_4096_cubed_and_a_single_cta_at_the_quick_start_shape(pkg):
    from strix_halo_int4_gemms_b200 import native

    a, b, sa, sb = _random_problem(4096, 4096, 4096)
    pkg.mm(a, b, a_scale=sa, b_scale=sb)
    assert native.last_launch_path() == native.LAUNCHED_TCGEN05_PAIR
    a, b, sa, sb = _random_problem(128, 1024, 64)
    pkg.mm(a, b, a_scale=sa, b_scale=sb)
    assert native.last_launch_path() == native.LAUNCHED_TCGEN05
    a, b, sa, sb = _random_problem(512, 1024, 1024, sub=256, swiglu=True)
    pkg.fused_swiglu_up_gate(a, b, a_scale=sa, b_scale=sb, scale=scale_spec(pkg, 256))
    assert native.last_launch_path() == native.LAUNCHED_TCGEN05_PAIR
    torch.cuda.synchronize()


@pytest.mark.parametrize("name,m,n,k,sub,swiglu", [("4096^3 per-channel", 4096, 4096, 4096, 0, False),
                                                   ("sc256 SwiGLU 4096 x 14336 x 4096", 4096, 14336, 4096, 256, True)])
def test_default_arguments_run_as_fast_as_the_pointer_level_launch(pkg, name, m, n, k, sub, swiglu):
    from strix_halo_int4_gemms_b200 import native

    a, b, sa, sb = _random_problem(m, n, k, sub=sub, swiglu=swiglu)
    scale = scale_spec(pkg, sub)
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    variant = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=scale,
                                  epilogue=pkg.Epilogue.SWIGLU if swiglu else pkg.Epilogue.NONE, out_dtype=native.OUT_BF16)

    def direct():
        native.launch_dense(variant, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=a.data_ptr(),
                            b_ptr=b.data_ptr(), a_scale_ptr=sa.data_ptr(), b_scale_ptr=sb.data_ptr(), c_ptr=out.data_ptr(), m=m, n=n, k=k)

    def api():
        if swiglu:
            return pkg.fused_swiglu_up_gate(a, b, a_scale=sa, b_scale=sb, scale=scale)
        return pkg.mm(a, b, a_scale=sa, b_scale=sb, scale=scale)

    assert torch.equal(api(), (direct(), out)[1])
    t_direct, t_api = _time(direct), _time(api)
    # the API allocates its output and validates shapes; at these sizes that must vanish beside the kernel
    assert t_api <= 1.05 * t_direct, f"{name}: api {t_api:.4f} ms vs direct {t_direct:.4f} ms"


def test_cuda_core_route_is_reported(pkg):
    from strix_halo_int4_gemms_b200 import native

    native._SLOW_PATH_WARNED.clear()
    case = dense_case(pkg, m=32, n=64, k=78, seed=1)          # K = 78: a 39-byte pitch, nothing TMA can describe
    kernel = pkg.default_registry.select_reference(dtype=pkg.OperandDType.INT4, scale=scale_spec(pkg, 0), epilogue=pkg.Epilogue.NONE)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    with pytest.warns(RuntimeWarning, match="ran on the CUDA-core kernel"):
        out = torch.empty((32, 64), device="cuda", dtype=torch.bfloat16)
        variant = native.variant_for_kernel(kernel, out_dtype=native.OUT_BF16)
        native.launch_dense(variant, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream,
                            a_ptr=dev["a"].data_ptr(), b_ptr=dev["b"].data_ptr(), a_scale_ptr=dev["a_scale"].data_ptr(),
                            b_scale_ptr=dev["b_scale"].data_ptr(), c_ptr=out.data_ptr(), m=32, n=64, k=78)
    assert native.last_launch_path() == native.LAUNCHED_SIMT
    torch.cuda.synchronize()
    with warnings.catch_warnings():
        warnings.simplefilter("error")                         # asked for by name: no warning
        forced = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0),
                                     epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16, path=native.PATH_SIMT)
        a, b, sa, sb = _random_problem(128, 256, 128)
        c = torch.empty((128, 256), device="cuda", dtype=torch.bfloat16)
        native.launch_dense(forced, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=a.data_ptr(), b_ptr=b.data_ptr(),
                            a_scale_ptr=sa.data_ptr(), b_scale_ptr=sb.data_ptr(), c_ptr=c.data_ptr(), m=128, n=256, k=128)
    torch.cuda.synchronize()


def test_autotune_tells_the_forms_apart(pkg):
    """At 4096^3 the CTA-pair launch wins, at the quick-start shape a single-CTA one; the records differ by more than noise."""
    pc = scale_spec(pkg, 0)
    big = pkg.autotune(m=4096, n=4096, k=4096, dtype=pkg.OperandDType.INT4, scale=pc, epilogue=pkg.Epilogue.RELU2, warmup_ms=5, rep_ms=30)
    forms = {k.kernel_id: k.schedule for k in big.candidates}
    by_form = {}
    for record in big.records:
        by_form.setdefault(forms[record.kernel_id], []).append(record.runtime_ms)
    assert big.best_kernel.schedule in (pkg.KernelSchedule.PERSISTENT_2CTA, pkg.KernelSchedule.STANDARD)
    assert min(by_form[pkg.KernelSchedule.PERSISTENT]) > 1.10 * min(by_form[pkg.KernelSchedule.PERSISTENT_2CTA])
    small = pkg.autotune(m=128, n=1024, k=64, dtype=pkg.OperandDType.INT4, scale=pc, epilogue=pkg.Epilogue.RELU2, warmup_ms=2, rep_ms=10)
    assert small.best_kernel.schedule is not pkg.KernelSchedule.PERSISTENT_2CTA


def test_reference_accumulation_order_on_request(pkg):
    """Subchannel launches through the API use the fused order; ``accumulation_order("reference")`` gives the
    reference's order of roundings, bit-identical to its PyTorch math."""
    case = dense_case(pkg, m=256, n=512, k=1024, sub=256, epilogue="relu2", seed=8)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    kw = dict(a_scale=dev["a_scale"], b_scale=dev["b_scale"], scale=scale_spec(pkg, 256), epilogue=pkg.Epilogue.RELU2)
    want = pkg.mm(case["a"], case["b"], a_scale=case["a_scale"], b_scale=case["b_scale"], scale=scale_spec(pkg, 256),
                  epilogue=pkg.Epilogue.RELU2, use_reference=True)
    fused = pkg.mm(dev["a"], dev["b"], **kw).cpu()
    with pkg.accumulation_order("reference"):
        exact = pkg.mm(dev["a"], dev["b"], **kw).cpu()
    again = pkg.mm(dev["a"], dev["b"], **kw).cpu()
    assert torch.equal(exact, want) and torch.equal(fused, again)
    assert float((fused == want).float().mean()) > 0.95
    torch.testing.assert_close(fused.float(), want.float(), rtol=8e-3, atol=1e-2)
