"""The BASELINE configurations at full size on a B200.

The oracle cannot redo a 4096^3 or 8192^3 product in seconds, so each configuration is checked by
(a) exact comparison with the oracle on a sample of rows / groups and (b) properties that do not
depend on size: a checksum of checksums over the int32 accumulators
(sum_ij C_ij == sum_k colsum(A)_k * rowsum(B)_k), linearity in A, and run-to-run bit equality.
Operands are generated on the GPU as random bytes (every byte is a valid pair of int4 codes)."""
import numpy as np
import pytest
import torch

from helpers import as_f32, assert_close_rms, bf16_bits
from oracle import reference_math as oracle

pytestmark = pytest.mark.gpu


def _scales(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return ((torch.rand(shape, generator=g) + 0.5) * 0.05).to(torch.bfloat16)


def _random_bytes(shape, seed, *, int8=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if int8:
        return torch.randint(-127, 128, shape, generator=g, device="cuda", dtype=torch.int8)
    return torch.randint(0, 256, shape, generator=g, device="cuda", dtype=torch.uint8)


def _launch(pkg, a, b, sa, sb, *, m, n, k, dtype="int4", sub=0, epilogue="none", out="bf16", order="reference", path=None):
    from strix_halo_int4_gemms_b200 import native
    from helpers import scale_spec

    out_dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "s32": torch.int32}[out]
    code = {"bf16": native.OUT_BF16, "f32": native.OUT_F32, "s32": native.OUT_S32}[out]
    c = torch.empty((m, n), device="cuda", dtype=out_dtype)
    variant = native.make_variant(dtype=pkg.OperandDType(dtype), layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, sub),
                                  epilogue=pkg.Epilogue(epilogue), out_dtype=code, path=native.PATH_TCGEN05 if path is None else path,
                                  accumulate_order=native.ACCUMULATE_REFERENCE if order == "reference" else native.ACCUMULATE_FUSED)
    native.launch_dense(variant, device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=a.data_ptr(), b_ptr=b.data_ptr(),
                        a_scale_ptr=sa.data_ptr(), b_scale_ptr=sb.data_ptr(), c_ptr=c.data_ptr(), m=m, n=n, k=k)
    torch.cuda.synchronize()
    assert native.device_status(0)[0] == 0
    return c


def _sample_rows(m):
    return torch.cat([torch.arange(0, 128), torch.arange(m // 2 - 64, m // 2 + 64), torch.arange(m - 128, m)])


def _checksum_of_checksums(a_codes_colsum, b_codes_rowsum):
    return int((a_codes_colsum.to(torch.int64) * b_codes_rowsum.to(torch.int64)).sum().item())


def _unpacked_sums(pkg, a, b):
    """Column sums of logical A [M, K] and row sums of logical B [K, N], computed on the GPU in int64."""
    a_codes = pkg.unpack_int4_on_device(a)                                    # [M, K]
    b_codes = pkg.unpack_int4_on_device(b.t().contiguous()).t()               # [K, N]
    return a_codes.to(torch.int64).sum(0), b_codes.to(torch.int64).sum(1)


def test_config2_int4_per_channel_4096_cubed(pkg):
    m = n = k = 4096
    a, b = _random_bytes((m, k // 2), 1), _random_bytes((k // 2, n), 2)
    sa, sb = _scales((m,), 3).cuda(), _scales((n,), 4).cuda()
    acc = _launch(pkg, a, b, sa, sb, m=m, n=n, k=k, out="s32")
    colsum, rowsum = _unpacked_sums(pkg, a, b)
    assert int(acc.to(torch.int64).sum().item()) == _checksum_of_checksums(colsum, rowsum)
    rows = _sample_rows(m)
    want_acc = oracle.int32_accumulators(a[rows.cuda()].cpu().numpy(), b.cpu().numpy(), int4=True)
    np.testing.assert_array_equal(acc[rows.cuda()].cpu().numpy(), want_acc)
    out = _launch(pkg, a, b, sa, sb, m=m, n=n, k=k)
    want = oracle.reference_mm(a[rows.cuda()].cpu().numpy(), b.cpu().numpy(), int4=True, a_scale_bits=bf16_bits(sa[rows.cuda()]), b_scale_bits=bf16_bits(sb))
    np.testing.assert_array_equal(as_f32(out[rows.cuda()]), want)
    assert torch.equal(out, _launch(pkg, a, b, sa, sb, m=m, n=n, k=k))  # deterministic


def test_config2_linearity_in_a(pkg):
    """acc(a1 + a2, b) == acc(a1, b) + acc(a2, b) with codes kept inside [-8, 7]."""
    m = n = k = 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    a1 = torch.randint(-4, 4, (m, k), generator=g, device="cuda", dtype=torch.int8)
    a2 = torch.randint(-4, 4, (m, k), generator=g, device="cuda", dtype=torch.int8)
    b = _random_bytes((k // 2, n), 6)
    ones_m, ones_n = torch.ones(m, dtype=torch.bfloat16, device="cuda"), torch.ones(n, dtype=torch.bfloat16, device="cuda")
    acc = lambda codes: _launch(pkg, pkg.pack_int4_k_major(codes), b, ones_m, ones_n, m=m, n=n, k=k, out="s32")
    assert torch.equal(acc(a1 + a2), acc(a1) + acc(a2))


def test_config3_int8_relu2_8192_cubed(pkg):
    m = n = k = 8192
    a, b = _random_bytes((m, k), 7, int8=True), _random_bytes((k, n), 8, int8=True)
    g = torch.Generator().manual_seed(9)
    sa = ((torch.rand(m, generator=g) + 0.5) * 0.01).to(torch.bfloat16).cuda()
    sb = ((torch.rand(n, generator=g) + 0.5) * 0.01).to(torch.bfloat16).cuda()
    acc = _launch(pkg, a, b, sa, sb, m=m, n=n, k=k, dtype="int8", out="s32")
    assert int(acc.to(torch.int64).sum().item()) == _checksum_of_checksums(a.to(torch.int64).sum(0), b.to(torch.int64).sum(1))
    del acc
    out = _launch(pkg, a, b, sa, sb, m=m, n=n, k=k, dtype="int8", epilogue="relu2")
    rows = _sample_rows(m)
    want = oracle.reference_mm(a[rows.cuda()].cpu().numpy(), b.cpu().numpy(), int4=False, a_scale_bits=bf16_bits(sa[rows.cuda()]),
                               b_scale_bits=bf16_bits(sb), epilogue="relu2")
    got = as_f32(out[rows.cuda()])
    assert_close_rms(got, want, what="config 3")
    np.testing.assert_array_equal(got, want)


def test_config4_int4_sc256_fused_swiglu(pkg):
    m, k, d = 4096, 4096, 14336
    a, b = _random_bytes((m, k // 2), 10), _random_bytes((k // 2, 2 * d), 11)
    sa, sb = _scales((m, k // 256), 12).cuda(), _scales((k // 256, 2 * d), 13).cuda()
    out = _launch(pkg, a, b, sa, sb, m=m, n=d, k=k, sub=256, epilogue="swiglu")
    assert tuple(out.shape) == (m, d)
    rows = torch.cat([torch.arange(0, 64), torch.arange(m - 64, m)])
    want = oracle.reference_mm(a[rows.cuda()].cpu().numpy(), b.cpu().numpy(), int4=True, a_scale_bits=bf16_bits(sa[rows.cuda()]),
                               b_scale_bits=bf16_bits(sb), subchannel=256, epilogue="swiglu")
    got = as_f32(out[rows.cuda()])
    assert_close_rms(got, want, what="config 4")
    assert np.mean(got == want) > 0.98  # only exp() differs between the two implementations
    # the plain product of the same operands is fully specified: bit-equal
    plain = _launch(pkg, a, b[:, :4096].contiguous(), sa, sb[:, :4096].contiguous(), m=m, n=4096, k=k, sub=256)
    want = oracle.reference_mm(a[rows.cuda()].cpu().numpy(), b[:, :4096].cpu().numpy(), int4=True, a_scale_bits=bf16_bits(sa[rows.cuda()]),
                               b_scale_bits=bf16_bits(sb[:, :4096].contiguous()), subchannel=256)
    np.testing.assert_array_equal(as_f32(plain[rows.cuda()]), want)
    # the library's default (fused) accumulation order against the reference order, EVERY element, on the GPU:
    # the bf16 outputs may differ by one unit in the last place where the fp32 sums straddle a rounding boundary
    fused = _launch(pkg, a, b, sa, sb, m=m, n=d, k=k, sub=256, epilogue="swiglu", order="fused")
    diff = (fused.float() - out.float()).abs()
    bound = 1e-2 * out.float().abs() + 1e-2 * out.float().pow(2).mean().sqrt()
    assert bool((diff <= bound).all())
    assert float((fused == out).float().mean()) > 0.95
    sampled = as_f32(fused[rows.cuda()])
    want_swiglu = oracle.reference_mm(a[rows.cuda()].cpu().numpy(), b.cpu().numpy(), int4=True, a_scale_bits=bf16_bits(sa[rows.cuda()]),
                                      b_scale_bits=bf16_bits(sb), subchannel=256, epilogue="swiglu")
    assert_close_rms(sampled, want_swiglu, what="config 4, fused order")


def test_config4_whole_output_against_the_cuda_core_kernel(pkg):
    """Every element of a config-4-shaped product (a 1024-row slice of M, all 14336 columns): the tensor-core kernel in
    the reference order against the CUDA-core kernel, which the small cases pin to the oracle.  Only exp() may differ."""
    from strix_halo_int4_gemms_b200 import native

    m, k, d = 1024, 4096, 14336
    a, b = _random_bytes((m, k // 2), 20), _random_bytes((k // 2, 2 * d), 21)
    sa, sb = _scales((m, k // 256), 22).cuda(), _scales((k // 256, 2 * d), 23).cuda()
    plain_tc = _launch(pkg, a, b, sa, sb, m=m, n=2 * d, k=k, sub=256)
    plain_cc = _launch(pkg, a, b, sa, sb, m=m, n=2 * d, k=k, sub=256, path=native.PATH_SIMT)
    assert torch.equal(plain_tc, plain_cc)                       # [up | gate] before the activation: bit for bit
    fused_tc = _launch(pkg, a, b, sa, sb, m=m, n=d, k=k, sub=256, epilogue="swiglu")
    fused_cc = _launch(pkg, a, b, sa, sb, m=m, n=d, k=k, sub=256, epilogue="swiglu", path=native.PATH_SIMT)
    assert float((fused_tc == fused_cc).float().mean()) > 0.999  # same instruction sequence on both; bf16 rounding hides the rest


def _config5_group_sizes():
    g = torch.Generator().manual_seed(0)
    probs = torch._sample_dirichlet(torch.full((64,), 0.5), generator=g)
    probs[torch.randperm(64, generator=g)[:3]] = 0
    draws = torch.multinomial(probs / probs.sum(), 32768, replacement=True, generator=g)
    return torch.bincount(draws, minlength=64)


def test_config5_ragged_forward(pkg):
    sizes = _config5_group_sizes()
    assert int(sizes.sum()) == 32768 and int((sizes == 0).sum()) >= 3
    rows, k, n, groups = 32768, 2048, 1408, 64
    lhs, rhs = _random_bytes((rows, k // 2), 20), _random_bytes((groups, k // 2, n), 21)
    sa, sb = _scales((rows,), 22).cuda(), _scales((groups, n), 23).cuda()
    out = pkg.ragged_dot_int4(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb)
    torch.cuda.synchronize()
    ends = torch.cumsum(sizes, 0)
    order = torch.argsort(sizes)
    nonempty = [int(g) for g in order if sizes[g] > 0]
    for g in (nonempty[0], nonempty[len(nonempty) // 2], nonempty[-1]):  # smallest, median, largest group
        lo, hi = int(ends[g] - sizes[g]), int(ends[g])
        want = oracle.reference_mm(lhs[lo:hi].cpu().numpy(), rhs[g].cpu().numpy(), int4=True,
                                   a_scale_bits=bf16_bits(sa[lo:hi]), b_scale_bits=bf16_bits(sb[g]))
        np.testing.assert_array_equal(as_f32(out[lo:hi]), want, err_msg=f"group {g}")
    # every row written exactly as the dense kernel would with that row's expert: spot check 4 boundary rows
    again = pkg.ragged_dot_int4(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb)
    assert torch.equal(out, again)


def test_config5_ragged_backward(pkg):
    sizes = _config5_group_sizes()
    groups, m, n = 64, 2048, 1408
    cap = int(sizes.max()) + int(sizes.max()) % 2
    cap += (-cap) % 32  # keep the packed pitch a multiple of 16 bytes
    lhs, rhs = _random_bytes((groups, cap // 2, m), 30), _random_bytes((groups, cap // 2, n), 31)
    sa, sb = _scales((groups, m), 32).cuda(), _scales((groups, n), 33).cuda()
    out = pkg.ragged_dot_int4_bwd(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb, layout=pkg.GemmLayout.TN)
    torch.cuda.synchronize()
    assert tuple(out.shape) == (groups, m, n) and out.dtype is torch.float32
    order = torch.argsort(sizes)
    nonempty = [int(g) for g in order if sizes[g] > 0]
    empty = [int(g) for g in order if sizes[g] == 0]
    assert float(out[empty].abs().max()) == 0.0
    for g in (nonempty[0], nonempty[len(nonempty) // 2], nonempty[-1]):
        want = oracle.ragged_dot_bwd(lhs[g:g + 1].cpu().numpy(), rhs[g:g + 1].cpu().numpy(), [int(sizes[g])],
                                     bf16_bits(sa[g:g + 1]), bf16_bits(sb[g:g + 1]), layout="tn")
        np.testing.assert_array_equal(out[g].cpu().numpy(), want[0], err_msg=f"group {g}")
    assert torch.equal(out, pkg.ragged_dot_int4_bwd(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb, layout=pkg.GemmLayout.TN))


def test_config5_forward_with_tasks_built_on_the_device(pkg):
    """Same launch with the task arrays and their count built and kept on the GPU: identical output."""
    sizes = _config5_group_sizes().cuda()
    rows, k, n, groups = 32768, 2048, 1408, 64
    lhs, rhs = _random_bytes((rows, k // 2), 20), _random_bytes((groups, k // 2, n), 21)
    sa, sb = _scales((rows,), 22).cuda(), _scales((groups, n), 23).cuda()
    want = pkg.ragged_dot_int4(lhs, rhs, sizes, a_scale=sa, b_scale=sb)
    cfg = pkg.RaggedDotConfig(block_m=256)
    info = pkg.calculate_group_info_on_device(sizes, cfg.block_m, total_rows=rows, align_tile=cfg.align_tile)
    got = pkg.ragged_dot_int4(lhs, rhs, sizes, a_scale=sa, b_scale=sb, config=cfg, group_info=info)
    torch.cuda.synchronize()
    assert int(info.device_overflow.item()) == 0
    assert torch.equal(got, want)


def test_config5_flat_backward_from_forward_format_operands(pkg):
    """x [32768, 2048] and dy [32768, 1408] in the forward packing -> token repack on the GPU -> flat backward;
    checked against the oracle on the smallest, the median and the largest group and against a second run."""
    sizes = _config5_group_sizes()
    tokens, groups, m, n = 32768, 64, 2048, 1408
    x, dy = _random_bytes((tokens, m // 2), 40), _random_bytes((tokens, n // 2), 41)
    sa, sb = _scales((groups, m), 42).cuda(), _scales((groups, n), 43).cuda()
    lhs, rhs = pkg.repack_int4_tokens(x), pkg.repack_int4_tokens(dy)
    assert tuple(lhs.shape) == (tokens // 2, m) and tuple(rhs.shape) == (tokens // 2, n)
    out = pkg.ragged_dot_int4_bwd_flat(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb)
    torch.cuda.synchronize()
    ends = torch.cumsum(sizes, 0)
    order = torch.argsort(sizes)
    nonempty = [int(g) for g in order if sizes[g] > 0]
    empty = [int(g) for g in order if sizes[g] == 0]
    assert float(out[empty].abs().max()) == 0.0
    for g in (nonempty[0], nonempty[len(nonempty) // 2], nonempty[-1]):
        lo, hi = int(ends[g] - sizes[g]), int(ends[g])
        xg = oracle.unpack_int4_k_major(x[lo:hi].cpu().numpy())      # [tokens of g, m]
        dg = oracle.unpack_int4_k_major(dy[lo:hi].cpu().numpy())     # [tokens of g, n]
        want = oracle.scaled_matmul(np.ascontiguousarray(xg.T), dg, oracle.bf16_bits_to_f32(bf16_bits(sa[g])),
                                    oracle.bf16_bits_to_f32(bf16_bits(sb[g])))
        np.testing.assert_array_equal(out[g].cpu().numpy(), want, err_msg=f"group {g}")
    assert torch.equal(out, pkg.ragged_dot_int4_bwd_flat(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb, static_scratch=True))


def test_config2_whole_output_against_the_cuda_core_kernel(pkg):
    """Every element of the 4096^3 int4 product: the tensor-core kernel (the pair form the defaults choose) against the
    CUDA-core kernel, which the small cases pin to the oracle bit for bit."""
    from strix_halo_int4_gemms_b200 import native

    m = n = k = 4096
    a, b = _random_bytes((m, k // 2), 40), _random_bytes((k // 2, n), 41)
    sa, sb = _scales((m,), 42).cuda(), _scales((n,), 43).cuda()
    tc = _launch(pkg, a, b, sa, sb, m=m, n=n, k=k)
    cc = _launch(pkg, a, b, sa, sb, m=m, n=n, k=k, path=native.PATH_SIMT)
    assert torch.equal(tc, cc)


def test_config5_forward_whole_output_against_the_cuda_core_kernel(pkg):
    """All 32768 x 1408 outputs of the grouped forward dot on the config-5 size vector, both kernels, bit for bit."""
    from strix_halo_int4_gemms_b200 import native

    sizes = _config5_group_sizes()
    rows, k, n, groups = 32768, 2048, 1408, 64
    lhs, rhs = _random_bytes((rows, k // 2), 50), _random_bytes((groups, k // 2, n), 51)
    sa, sb = _scales((rows,), 52).cuda(), _scales((groups, n), 53).cuda()
    config = pkg.RaggedDotConfig(block_m=256)     # the task height the public API picks for this shape
    info = pkg.calculate_group_info(sizes.cuda(), config.block_m, align_tile=config.align_tile)
    results = []
    for path in (native.PATH_TCGEN05, native.PATH_SIMT):
        out = torch.full((rows, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        native.launch_ragged_fwd_kernel(lhs, rhs, group_info=info, a_scale=sa, b_scale=sb, out=out, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL),
                                        config=config, layout=pkg.GemmLayout.NN, rows=rows, cols=n, k_packed=k // 2, scale_cols=1, path=path)
        torch.cuda.synchronize()
        assert native.device_status(0)[0] == 0
        results.append(out)
    assert torch.equal(pkg.ragged_dot_int4(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb), results[0])   # the default call
    assert not bool(torch.isnan(results[0]).any())   # every row belongs to a group: every element is written
    assert torch.equal(results[0], results[1])


def test_config5_backward_whole_output_against_the_cuda_core_kernel(pkg):
    """All 64 x 2048 x 1408 fp32 outputs of the grouped backward dot, both kernels, bit for bit (empty groups: zeros)."""
    from strix_halo_int4_gemms_b200 import native

    sizes = _config5_group_sizes()
    groups, m, n = 64, 2048, 1408
    cap = int(sizes.max())
    cap += (-cap) % 32
    lhs, rhs = _random_bytes((groups, cap // 2, m), 60), _random_bytes((groups, cap // 2, n), 61)
    sa, sb = _scales((groups, m), 62).cuda(), _scales((groups, n), 63).cuda()
    results = []
    for path in (native.PATH_TCGEN05, native.PATH_SIMT):
        out = torch.full((groups, m, n), float("nan"), device="cuda", dtype=torch.float32)
        native.launch_ragged_bwd_kernel(lhs, rhs, sizes.cuda(), a_scale=sa, b_scale=sb, out=out, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL),
                                        config=pkg.RaggedBwdDotConfig(), layout=pkg.GemmLayout.TN, rows=m, cols=n, k_packed=cap // 2,
                                        scale_cols=1, path=path)
        torch.cuda.synchronize()
        assert native.device_status(0)[0] == 0
        results.append(out)
    assert not bool(torch.isnan(results[0]).any())
    assert torch.equal(results[0], results[1])
