"""Device kernels either side of the GEMM path, on a B200, against the oracle: quantise + pack, token
repack, task building on the device with the sync-free grouped forward launch, and the grouped
backward pass over flat token-packed operands.  Everything here is integer / byte work or fp32 with
a fully specified order: the bar is bit equality."""
import numpy as np
import pytest
import torch

from helpers import as_f32, bf16_bits, scale_spec
from oracle import reference_math as oracle
from strix_halo_int4_gemms_b200.autotune import make_ragged_fwd_inputs

pytestmark = pytest.mark.gpu


def _status_clean():
    from strix_halo_int4_gemms_b200 import native

    torch.cuda.synchronize()
    status, detail = native.device_status(0)
    assert status == 0, (status, detail)


@pytest.mark.parametrize("shape", [(128, 64), (3, 7), (257, 1000), (1, 1), (64, 4096)])
@pytest.mark.parametrize("bits", [4, 8])
def test_quantize_matches_host_helpers(pkg, shape, bits):
    g = torch.Generator().manual_seed(shape[0] * 7 + shape[1] + bits)
    x = (torch.randn(shape, generator=g) * 0.3).bfloat16()
    x[0, 0] = 0.05      # exact ties of x / 0.1 after bf16 rounding are rare; force a few half-way cases
    x.view(-1)[::17] = 0.25
    got = pkg.quantize_int_cuda(x.cuda(), bits=bits, scale=0.1).cpu()
    codes = pkg.fake_quant_int(x, bits=bits, scale=0.1)
    want = pkg.pack_int4_k_major(codes) if bits == 4 else codes
    assert got.dtype == want.dtype and got.shape == want.shape
    assert torch.equal(got, want)
    np.testing.assert_array_equal(
        got.numpy(), oracle.pack_int4_k_major(oracle.fake_quant_int(x.float().numpy(), bits=bits, scale=0.1))
        if bits == 4 else oracle.fake_quant_int(x.float().numpy(), bits=bits, scale=0.1))


def test_quantize_saturates_and_handles_batches(pkg):
    x = torch.tensor([[-100.0, 100.0, 0.74, -0.85, 0.0, 3e38, -3e38, 0.049]], dtype=torch.bfloat16).repeat(2, 3, 1)
    got = pkg.quantize_int_cuda(x.cuda(), bits=4, scale=0.1).cpu()
    assert got.shape == (2, 3, 4)
    assert torch.equal(got, pkg.pack_int4_k_major(pkg.fake_quant_int(x, bits=4, scale=0.1)))


@pytest.mark.parametrize("rows,cols", [(64, 128), (7, 12), (1, 2), (513, 1408), (1000, 24)])
def test_token_repack_matches_oracle(pkg, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    packed = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8)
    got = pkg.repack_int4_tokens(packed.cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.repack_tokens(packed.numpy()))


@pytest.mark.parametrize("sizes,tile,align", [
    ([17, 31, 24], 32, 8), ([2, 0, 7], 4, 4), ([0, 0, 0], 64, 8), ([300, 0, 256, 7, 129, 512, 1, 255], 256, 8),
    ([5] * 1500, 128, 8), ([100000, 3, 0, 41], 128, 128),
])
def test_group_info_on_device_matches_host(pkg, sizes, tile, align):
    sizes_t = torch.tensor(sizes, dtype=torch.int64)
    want = oracle.calculate_group_info(sizes, tile, align_tile=align)
    info = pkg.calculate_group_info_on_device(sizes_t.cuda(), tile, total_rows=sum(sizes), align_tile=align)
    torch.cuda.synchronize()
    count = int(info.device_num_tasks.item())
    assert int(info.device_overflow.item()) == 0
    assert count == len(want["group_id"]) and count <= info.num_tasks
    for name in ("group_id", "block_start", "actual_start", "actual_end", "start_within_block", "actual_size"):
        got = getattr(info, name).cpu().numpy()
        np.testing.assert_array_equal(got[:count], np.asarray(want[name], dtype=np.int64), err_msg=name)
        assert not got[count:].any(), name          # padding entries are empty tasks
    host = pkg.calculate_group_info(sizes_t, tile, align_tile=align)
    assert host.num_tasks == count


def test_group_info_capacity_overflow_is_reported(pkg):
    sizes = torch.tensor([300, 300, 300], dtype=torch.int64).cuda()
    info = pkg.calculate_group_info_on_device(sizes, 128, total_rows=900, max_tasks=4)
    torch.cuda.synchronize()
    assert int(info.device_overflow.item()) == 1 and int(info.device_num_tasks.item()) == 4


def test_forward_reports_an_overflowed_task_list_and_clamps_task_bounds(pkg):
    """A task array that is too small leaves rows unwritten: the forward kernel says so through the status word
    (code 3, detail = tasks kept) instead of dropping tasks silently; rows of the tasks that fit are right."""
    from strix_halo_int4_gemms_b200 import native

    sizes = [300, 300, 300]
    data = make_ragged_fwd_inputs(m=900, n=256, k=256, group_sizes=sizes, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0), seed=5)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    info = pkg.calculate_group_info_on_device(dev["group_sizes"], 128, total_rows=900, max_tasks=4)
    assert info.tile == 128
    out = torch.full((900, 256), float("nan"), device="cuda", dtype=torch.bfloat16)
    native.reset_device_status(0)
    pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], group_info=info, out=out)
    torch.cuda.synchronize()
    status, (kept, _site, _) = native.device_status(0)
    assert status == 3 and kept == 4
    native.reset_device_status(0)
    want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]), layout="nn")
    got = as_f32(out)
    np.testing.assert_array_equal(got[:384], want[:384])        # group 0 (3 tasks) and the first task of group 1
    assert np.isnan(got[512:]).all()                             # the rest was never written
    # group sizes that claim more rows than the operand has: bounds are clamped on the device, nothing is written past row 900
    big = torch.tensor([300, 300, 400], dtype=torch.int64).cuda()
    info = pkg.calculate_group_info_on_device(big, 128, total_rows=1000)
    guard = torch.full((1024, 256), float("nan"), device="cuda", dtype=torch.bfloat16)
    pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], big, a_scale=dev["a_scale"], b_scale=dev["b_scale"], group_info=info, out=guard[:900])
    torch.cuda.synchronize()
    assert native.device_status(0)[0] == 0
    assert torch.isnan(guard[900:]).all() and not torch.isnan(guard[:900]).any()


@pytest.mark.parametrize("sub,block_m", [(0, 128), (0, 256), (128, 256), (32, 64)])
def test_forward_with_device_built_tasks(pkg, sub, block_m):
    """No host synchronisation between group_sizes and the output: tasks and their count stay on the GPU."""
    sizes = [300, 0, 256, 7, 129, 512, 1, 255]
    data = make_ragged_fwd_inputs(m=sum(sizes), n=768, k=512, group_sizes=sizes, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, sub), seed=31)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    cfg = pkg.RaggedDotConfig(block_m=block_m)
    info = pkg.calculate_group_info_on_device(dev["group_sizes"], block_m, total_rows=sum(sizes), align_tile=cfg.align_tile)
    out = pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"],
                              scale=scale_spec(pkg, sub), config=cfg, group_info=info)
    _status_clean()
    want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]),
                                 layout="nn", subchannel=sub)
    np.testing.assert_array_equal(as_f32(out), want)


def _flat_case(sizes, m, n, seed):
    g = torch.Generator().manual_seed(seed)
    total = sum(sizes)
    x = torch.randint(-8, 8, (total, m), generator=g, dtype=torch.int8)
    dy = torch.randint(-8, 8, (total, n), generator=g, dtype=torch.int8)
    sa = ((torch.rand(len(sizes), m, generator=g) + 0.5) * 0.05).bfloat16()
    sb = ((torch.rand(len(sizes), n, generator=g) + 0.5) * 0.05).bfloat16()
    return x, dy, sa, sb


@pytest.mark.parametrize("sizes,m,n", [
    ([17, 0, 300, 128, 255], 256, 512),        # odd starts, an empty group, a group longer than one K block
    ([1, 1, 1, 1], 128, 256),                  # single tokens, every second one on the high nibble
    ([513, 64], 2048, 1408),                   # the benchmark's tile grid with its column edge
    ([0, 0, 9], 128, 256),
    ([33, 18, 70], 48, 40),                    # pitches TMA cannot describe: CUDA-core kernel
])
def test_flat_backward_matches_oracle(pkg, sizes, m, n):
    x, dy, sa, sb = _flat_case(sizes, m, n, seed=len(sizes) * 1000 + m)
    lhs = pkg.repack_int4_tokens(pkg.pack_int4_k_major(x).cuda())
    rhs = pkg.repack_int4_tokens(pkg.pack_int4_k_major(dy).cuda())
    out = pkg.ragged_dot_int4_bwd_flat(lhs, rhs, torch.tensor(sizes, dtype=torch.int64).cuda(), a_scale=sa.cuda(), b_scale=sb.cuda())
    _status_clean()
    want = oracle.ragged_dot_bwd_flat(lhs.cpu().numpy(), rhs.cpu().numpy(), sizes, bf16_bits(sa), bf16_bits(sb))
    np.testing.assert_array_equal(out.cpu().numpy(), want)


def test_flat_backward_equals_padded_backward_on_the_gpu(pkg):
    """Same groups through the reference-shaped API (operands stacked per group, padded) and the flat entry."""
    sizes = [200, 0, 77, 128]
    m, n = 256, 256
    x, dy, sa, sb = _flat_case(sizes, m, n, seed=77)
    cap = 256
    lhs_pad = torch.zeros(len(sizes), cap // 2, m, dtype=torch.uint8)
    rhs_pad = torch.zeros(len(sizes), cap // 2, n, dtype=torch.uint8)
    start = 0
    for g, size in enumerate(sizes):
        xg = torch.zeros(cap, m, dtype=torch.int8)
        dg = torch.zeros(cap, n, dtype=torch.int8)
        xg[:size] = x[start:start + size]
        dg[:size] = dy[start:start + size]
        lhs_pad[g] = pkg.pack_int4_k_major(xg.t().contiguous()).t()
        rhs_pad[g] = pkg.pack_int4_k_major(dg.t().contiguous()).t()
        start += size
    sizes_t = torch.tensor(sizes, dtype=torch.int64).cuda()
    padded = pkg.ragged_dot_int4_bwd(lhs_pad.cuda(), rhs_pad.cuda(), sizes_t, a_scale=sa.cuda(), b_scale=sb.cuda(), layout=pkg.GemmLayout.TN)
    flat = pkg.ragged_dot_int4_bwd_flat(pkg.repack_int4_tokens(pkg.pack_int4_k_major(x).cuda()),
                                        pkg.repack_int4_tokens(pkg.pack_int4_k_major(dy).cuda()), sizes_t,
                                        a_scale=sa.cuda(), b_scale=sb.cuda())
    _status_clean()
    assert torch.equal(padded, flat)
