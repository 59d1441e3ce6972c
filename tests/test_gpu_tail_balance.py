"""The balanced tail of dense per-channel launches: when the last wave of the persistent grid fills at most half of
the CTAs (CTA pairs), its tiles are cut along K into 2 .. 4 parts that run side by side; one part owns the tile and
starts from (or, when there is no full wave before it, ends by adding) the other parts' exact s32 partial sums.
Results must be bit-identical to the whole-tile schedule (which the other test files pin to the oracle), for every
kernel form and output type."""
import numpy as np
import pytest
import torch

from helpers import abi_dense, as_f32, dense_case, oracle_dense, scale_spec
from oracle import reference_math as oracle

pytestmark = pytest.mark.gpu
SINGLE, PAIR = 1, 2


def _plan(pkg, *, m, n, k, dtype="int4", epilogue="none", cta_group=0, tail=True):
    from strix_halo_int4_gemms_b200 import native

    variant = native.make_variant(dtype=pkg.OperandDType(dtype), layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0),
                                  epilogue=pkg.Epilogue(epilogue), out_dtype=native.OUT_BF16, cta_group=cta_group,
                                  tail_balance={True: native.TAIL_ALWAYS, False: native.TAIL_OFF, None: native.TAIL_AUTO}[tail])
    return native.plan_dense(variant, m=m, n=n, k=k)


def test_plan_uses_the_balanced_tail_only_for_a_thin_last_wave(pkg):
    plan = _plan(pkg, m=4096, n=4096, k=4096)                        # 256 pair tiles on 74 pairs: 3 waves + 34 tiles
    assert plan.tail_units > 0 and plan.tail_units == plan.grid // 2
    assert _plan(pkg, m=4096, n=4096, k=4096, tail=False).tail_units == 0
    assert _plan(pkg, m=4096, n=4096, k=256).tail_units == 0        # two K blocks per tile: nothing to cut
    assert _plan(pkg, m=4096, n=2048 + 1024, k=4096).tail_units == 0  # 192 tiles: the last wave (44 of 74) is more than half full
    small = _plan(pkg, m=1024, n=2048, k=8192)                      # 32 tiles, no full wave: two parts each, on 64 pairs
    assert small.tail_units == 64 and small.grid == 128
    assert _plan(pkg, m=1024, n=2048, k=4096).tail_units == 0       # ... which pays only for long reductions
    assert _plan(pkg, m=1024, n=2048, k=8192, tail=None).tail_units == 64      # the library's own choice: no full wave
    assert _plan(pkg, m=4096, n=4096, k=4096, tail=None).tail_units == 0       # ... but not behind full waves
    single = _plan(pkg, m=4096, n=4096, k=4096, cta_group=SINGLE)
    assert single.tail_units == single.grid                          # 512 tiles on one CTA per SM: 3 waves + 68 tiles


@pytest.mark.parametrize("cta_group", [PAIR, SINGLE])
@pytest.mark.parametrize("dtype,a_operand", [("int4", 0), ("int8", 0)])
@pytest.mark.parametrize("m,n,k", [
    (4096, 4096, 1024),                   # 3 waves + 34 tiles: two parts, the owner preloaded
    (2048 + 256, 4096 + 256, 1536),       # 153 pair tiles: 5 rest tiles in three parts; partial tiles in M and N
    (4096, 5120, 1000 // 32 * 32),        # a K that ends inside the last K block of the second part
    (1024, 1024, 8192),                   # fewer tiles than units: no full wave, the parts are added after the MMAs
])
def test_balanced_tail_is_bit_identical_to_whole_tiles(pkg, cta_group, dtype, a_operand, m, n, k):
    case = dense_case(pkg, m=m, n=n, k=k, dtype=dtype, seed=n + k)
    kw = dict(m=m, n=n, k=k, dtype=dtype, cta_group=cta_group, a_operand=a_operand, path=1)
    for out in ("s32", "bf16"):
        balanced = abi_dense(pkg, case, out=out, tail=True, **kw)
        whole = abi_dense(pkg, case, out=out, tail=False, **kw)
        assert torch.equal(balanced, whole), out
        again = abi_dense(pkg, case, out=out, tail=True, **kw)
        assert torch.equal(balanced, again), out                    # the neighbour's partial sum is waited for, not raced
    rows = torch.cat([torch.arange(0, 32), torch.arange(m - 32, m)])
    sample = {"a": case["a"][rows], "b": case["b"], "a_scale": case["a_scale"][rows], "b_scale": case["b_scale"]}
    np.testing.assert_array_equal(as_f32(balanced[rows.cuda()]), oracle_dense(sample, dtype=dtype))


@pytest.mark.parametrize("epilogue", ["relu2", "swiglu"])
def test_balanced_tail_with_fused_activations(pkg, epilogue):
    m, n, k = 4096, 2560, 1024      # SwiGLU: 16 x 20 pair tiles of 128 output columns
    case = dense_case(pkg, m=m, n=n, k=k, epilogue=epilogue, seed=3)
    assert _plan(pkg, m=m, n=n, k=k, epilogue=epilogue).tail_units > 0
    balanced = abi_dense(pkg, case, m=m, n=n, k=k, epilogue=epilogue, tail=True)
    whole = abi_dense(pkg, case, m=m, n=n, k=k, epilogue=epilogue, tail=False)
    assert torch.equal(balanced, whole)


def test_balanced_tail_through_the_public_api_and_without_a_workspace(pkg):
    """mm() brings the workspace itself; a pointer-level caller that passes none gets whole tiles: same bits."""
    from strix_halo_int4_gemms_b200 import native

    m, n, k = 4096, 4096, 1024
    case = dense_case(pkg, m=m, n=n, k=k, seed=5)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    api = pkg.mm(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
    plain = abi_dense(pkg, case, m=m, n=n, k=k, tail=None)
    assert torch.equal(api, plain)
    m, n, k = 512, 512, 8192        # few tiles, long K: mm() takes the balanced tail by itself
    case = dense_case(pkg, m=m, n=n, k=k, seed=6)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    api = pkg.mm(dev["a"], dev["b"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
    assert torch.equal(api, abi_dense(pkg, case, m=m, n=n, k=k, tail=False))
    assert native.device_status(0)[0] == 0


def test_balanced_tail_pays_on_few_tiles_with_a_long_reduction(pkg):
    """512 x 512 x 16384: four pair tiles on 74 CTA pairs.  Cut four ways along K (16 pairs busy) the launch must be
    faster than with whole tiles (by a tenth at least), with the same bits."""
    from strix_halo_int4_gemms_b200 import native

    m, n, k = 512, 512, 16384
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.uint8)
    b = torch.randint(0, 256, (k // 2, n), generator=g, device="cuda", dtype=torch.uint8)
    sa = ((torch.rand(m, device="cuda", generator=g) + 0.5) * 0.05).bfloat16()
    sb = ((torch.rand(n, device="cuda", generator=g) + 0.5) * 0.05).bfloat16()
    times, outs = {}, {}
    for tail in (native.TAIL_AUTO, native.TAIL_OFF):
        variant = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0),
                                      epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16, tail_balance=tail)
        out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
        ptr, size = native.dense_workspace(variant, m=m, n=n, k=k, device=out.device, stream_handle=torch.cuda.current_stream().cuda_stream)
        assert (native.plan_dense(variant, m=m, n=n, k=k).tail_units > 0) == (tail == native.TAIL_AUTO)   # the library's own choice here

        def run():
            native.launch_dense(variant, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=a.data_ptr(), b_ptr=b.data_ptr(),
                                a_scale_ptr=sa.data_ptr(), b_scale_ptr=sb.data_ptr(), c_ptr=out.data_ptr(), m=m, n=n, k=k,
                                workspace_ptr=ptr, workspace_bytes=size)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
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
        times[tail], outs[tail] = start.elapsed_time(stop) / 60, out
    assert torch.equal(outs[native.TAIL_AUTO], outs[native.TAIL_OFF])
    assert times[native.TAIL_AUTO] * 1.1 <= times[native.TAIL_OFF], times
