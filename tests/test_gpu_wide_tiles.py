"""Tiles of 256 x 512 on CTA pairs (per-channel int4, B stored [K, N], bf16 output): each CTA unpacks its rows of A once
per K block for two blocks of B.  Results must be bit-identical to the 256 x 256 tiles and to the CUDA-core kernel
(which the other files pin to the oracle); the plan says which tile a launch uses; at 4096^3 the wide tiles must be
faster."""
import numpy as np
import pytest
import torch

from helpers import abi_dense, as_f32, dense_case, oracle_dense, scale_spec

pytestmark = pytest.mark.gpu
SIMT, TCGEN05 = 2, 1


def _plan(pkg, *, m, n, k, dtype="int4", epilogue="none", wide=None, sub=0, layout="nn"):
    from strix_halo_int4_gemms_b200 import native

    variant = native.make_variant(dtype=pkg.OperandDType(dtype), layout=getattr(pkg.GemmLayout, layout.upper()), scale=scale_spec(pkg, sub),
                                  epilogue=pkg.Epilogue(epilogue), out_dtype=native.OUT_BF16,
                                  wide_tiles=native.WIDE_OFF if wide is False else (native.WIDE_ON if wide is True else native.WIDE_AUTO))
    return native.plan_dense(variant, m=m, n=n, k=k)


def test_plan_takes_wide_tiles_when_their_waves_need_less_time(pkg):
    plan = _plan(pkg, m=4096, n=4096, k=4096)                            # 128 wide tiles in 2 waves against 256 in 4 ...
    assert plan.tile_cols == 512 and plan.tiles_384 == 72 and plan.grid == 148   # ... recut as 74 of 512 and 72 of 384 columns
    assert _plan(pkg, m=8192, n=8192, k=8192).tiles_384 == 0              # 6.9 waves: the last one is full enough
    assert _plan(pkg, m=3840, n=4096, k=4096).tiles_384 == 64             # 120 tiles: 46 past the wave, 16 swaps, two of them early
    assert _plan(pkg, m=2560, n=4096, k=4096).tile_cols == 256            # 160 narrow tiles in 3 waves beat 80 wide ones in 2
    assert _plan(pkg, m=2560, n=4096, k=4096, wide=True).tiles_384 == 8   # forced: 80 tiles, two swaps in the first two row tiles
    assert _plan(pkg, m=8192, n=8192, k=8192).tile_cols == 512            # also where A through TMEM used to be chosen
    assert _plan(pkg, m=4096, n=4096, k=4096, wide=False).tile_cols == 256
    assert _plan(pkg, m=1024, n=2048, k=4096).tile_cols == 256            # 32 tiles: one wave either way
    assert _plan(pkg, m=1024, n=2048, k=4096, wide=True).tile_cols == 512
    assert _plan(pkg, m=4096, n=4096, k=4096, dtype="int8").tile_cols == 256          # nothing to unpack: no wide kernel
    assert _plan(pkg, m=4096, n=4096, k=4096, sub=256).tile_cols == 256               # subchannel: two accumulators alternate
    assert _plan(pkg, m=4096, n=4096, k=4096, layout="nt").tile_cols == 256
    assert _plan(pkg, m=4096, n=4096, k=4096, epilogue="swiglu", wide=True).tile_cols == 128


@pytest.mark.parametrize("m,n,k", [
    (512, 1024, 512),           # whole wide tiles
    (2048 + 128, 2560, 384),    # five wide column tiles, a half-empty last row of tiles
    (768, 512 + 48, 256),       # the second wide tile holds 48 columns
    (256, 256 + 16, 1024),      # a wide tile with little more than its first half
    (4096, 4096, 640),          # two waves on the whole GPU: 74 tiles of 512 columns, then 72 of 384
    (3840, 4096, 512),          # 72 + 64: two 384-column tiles end the first wave
    (2560, 4096, 384),          # 74 + 8: only the first two row tiles are recut
    (2560 - 128, 4096, 256),    # the same with a half-empty last row of tiles
])
@pytest.mark.parametrize("epilogue", ["none", "relu2"])
def test_wide_tiles_equal_narrow_tiles_and_the_cuda_core_kernel(pkg, m, n, k, epilogue):
    case = dense_case(pkg, m=m, n=n, k=k, epilogue=epilogue, seed=m + n + k)
    assert _plan(pkg, m=m, n=n, k=k, epilogue=epilogue, wide=True).tile_cols == 512
    kw = dict(m=m, n=n, k=k, epilogue=epilogue)
    wide = abi_dense(pkg, case, path=TCGEN05, wide=True, **kw)
    narrow = abi_dense(pkg, case, path=TCGEN05, wide=False, **kw)
    assert torch.equal(wide, narrow)
    if m * n <= 1 << 21:
        assert torch.equal(wide, abi_dense(pkg, case, path=SIMT, **kw))
    rows = torch.cat([torch.arange(0, 32), torch.arange(m - 32, m)])
    sample = {"a": case["a"][rows], "b": case["b"], "a_scale": case["a_scale"][rows], "b_scale": case["b_scale"]}
    np.testing.assert_array_equal(as_f32(wide[rows.cuda()]), oracle_dense(sample, epilogue=epilogue))
    again = abi_dense(pkg, case, path=TCGEN05, wide=True, **kw)
    assert torch.equal(wide, again)


def test_grouped_forward_on_wide_tiles(pkg):
    """256-row tasks x 512-column tiles, N = 1408 (2.75 wide tiles): forced wide against forced narrow and the CUDA cores."""
    from strix_halo_int4_gemms_b200 import native

    g = torch.Generator().manual_seed(5)
    groups, k, n = 6, 512, 1408
    sizes = torch.tensor([700, 0, 300, 1, 535, 256])
    rows = int(sizes.sum())
    lhs = torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8).cuda()
    rhs = torch.randint(0, 256, (groups, k // 2, n), generator=g, dtype=torch.uint8).cuda()
    sa = ((torch.rand((rows,), generator=g) + 0.5) * 0.05).bfloat16().cuda()
    sb = ((torch.rand((groups, n), generator=g) + 0.5) * 0.05).bfloat16().cuda()
    config = pkg.RaggedDotConfig(block_m=256)
    info = pkg.calculate_group_info(sizes.cuda(), config.block_m, align_tile=config.align_tile)
    results = []
    for path, wide in ((native.PATH_TCGEN05, native.WIDE_ON), (native.PATH_TCGEN05, native.WIDE_OFF), (native.PATH_SIMT, native.WIDE_AUTO)):
        out = torch.full((rows, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        native.launch_ragged_fwd_kernel(lhs, rhs, group_info=info, a_scale=sa, b_scale=sb, out=out, scale=scale_spec(pkg, 0), config=config,
                                        layout=pkg.GemmLayout.NN, rows=rows, cols=n, k_packed=k // 2, scale_cols=1, path=path, wide_tiles=wide)
        torch.cuda.synchronize()
        assert native.device_status(0)[0] == 0
        results.append(out)
    assert not bool(torch.isnan(results[0]).any())
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])


def test_wide_tiles_are_faster_at_4096_cubed(pkg):
    from strix_halo_int4_gemms_b200 import native

    m = n = k = 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    sets = []
    for _ in range(6):           # rotate operand sets larger than L2 together
        sets.append(dict(a=torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.uint8),
                         b=torch.randint(0, 256, (k // 2, n), generator=g, device="cuda", dtype=torch.uint8),
                         sa=((torch.rand((m,), device="cuda", generator=g) + 0.5) * 0.05).bfloat16(),
                         sb=((torch.rand((n,), device="cuda", generator=g) + 0.5) * 0.05).bfloat16(),
                         c=torch.empty((m, n), device="cuda", dtype=torch.bfloat16)))
    times = {}
    for wide in (native.WIDE_OFF, native.WIDE_AUTO):
        variant = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0),
                                      epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16, wide_tiles=wide)

        def run():
            for d in sets:
                native.launch_dense(variant, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=d["a"].data_ptr(),
                                    b_ptr=d["b"].data_ptr(), a_scale_ptr=d["sa"].data_ptr(), b_scale_ptr=d["sb"].data_ptr(),
                                    c_ptr=d["c"].data_ptr(), m=m, n=n, k=k)
        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(5):
                run()
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(10):
            graph.replay()
        stop.record()
        stop.synchronize()
        times[wide] = start.elapsed_time(stop) / 300
    assert times[native.WIDE_AUTO] <= 0.97 * times[native.WIDE_OFF], times
