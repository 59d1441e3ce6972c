"""Seeded random shapes through both device kernels: the tensor-core kernel (whichever form the library
picks, and both forms forced) against the CUDA-core kernel of the same library, bit for bit.  The CUDA-core
kernel is pinned to the oracle by the other GPU tests; this file widens the set of shapes and variants far
beyond what the oracle could redo in the time a test may take."""
import random

import pytest
import torch

from helpers import abi_dense, dense_case

pytestmark = pytest.mark.gpu
AUTO, SIMT = 0, 2


def _cases(seed, count):
    rng = random.Random(seed)
    out = []
    for _ in range(count):
        dtype = rng.choice(["int4", "int8"])
        layout = rng.choice(["nn", "nn", "nt", "tn", "tt"])
        sub = rng.choice([0, 0, 32, 64, 128, 256])
        epilogue = rng.choice(["none", "none", "relu2", "swiglu"])
        if layout == "tt":            # TT has plain per-channel / subchannel kernels only on the tensor cores
            epilogue, sub = "none", rng.choice([0, 128]) if dtype == "int4" else 0
        # pitches must stay multiples of 16 bytes for TMA: M for transposed A, N (2N for SwiGLU) for row-major B
        m = rng.choice([16, 48, 128, 208, 256, 400, 512, 784, 1024])
        n = rng.choice([16, 64, 144, 256, 272, 512, 640, 1408]) if epilogue != "swiglu" else rng.choice([64, 128, 256, 448])
        k = rng.choice([32, 64, 160, 256, 416, 512, 1024, 2080])
        if sub and k % sub:           # the reference requires K to be a multiple of the K-group for its kernels
            k = max(sub, k // sub * sub)
        out.append((len(out), dtype, layout, sub, epilogue, m, n, k))
    return out


@pytest.mark.parametrize("case", _cases(20241125, 48), ids=lambda c: "-".join(str(x) for x in c))
def test_tensor_core_kernel_equals_cuda_core_kernel(pkg, case):
    index, dtype, layout, sub, epilogue, m, n, k = case
    data = dense_case(pkg, m=m, n=n, k=k, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue, seed=1000 + index)
    kw = dict(m=m, n=n, k=k, dtype=dtype, layout=layout, sub=sub, epilogue=epilogue)
    want = abi_dense(pkg, data, path=SIMT, **kw)
    # path AUTO: the tensor-core kernel wherever one is instantiated for the variant (the CUDA-core kernel again
    # otherwise); cta_group: the library's choice, single CTAs, CTA pairs (single where no pair kernel exists).
    # Both kernels use the same exp instruction, so SwiGLU is bit-equal here too.
    for cta_group in (0, 1, 2):
        got = abi_dense(pkg, data, path=AUTO, cta_group=cta_group, **kw)
        assert torch.equal(got, want), f"cta_group {cta_group}"


# ---------------------------------------------------------------------------------------------------------------
# grouped dots: the same comparison through the pointer-level launchers (path AUTO against the CUDA-core kernel)
# ---------------------------------------------------------------------------------------------------------------
def _group_sizes(rng, groups, mean):
    sizes = [max(0, int(rng.gauss(mean, mean))) for _ in range(groups)]
    for _ in range(rng.randint(0, 2)):
        sizes[rng.randrange(groups)] = 0          # empty groups
    if sum(sizes) == 0:
        sizes[0] = 1
    return sizes


def _ragged_cases(seed, count):
    rng = random.Random(seed)
    out = []
    for i in range(count):
        layout = rng.choice(["nn", "nn", "nt"])
        sub = rng.choice([0, 0, 32, 128, 256])
        block_m = rng.choice([32, 64, 128, 256, 256]) if (layout == "nn" and sub in (0, 128, 256)) else rng.choice([32, 64, 128])
        k = rng.choice([256, 512, 1024])
        n = rng.choice([64, 256, 400, 1408])
        sizes = _group_sizes(rng, rng.choice([2, 5, 9]), rng.choice([20, 150, 400]))
        out.append((i, layout, sub, block_m, k, n, tuple(sizes), rng.choice(["bf16", "f32"])))
    return out


@pytest.mark.parametrize("case", _ragged_cases(7, 24), ids=lambda c: f"{c[0]}-{c[1]}-sc{c[2]}-bm{c[3]}-k{c[4]}-n{c[5]}-{c[7]}")
def test_grouped_forward_tensor_core_equals_cuda_core(pkg, case):
    from helpers import scale_spec
    from strix_halo_int4_gemms_b200 import native
    from strix_halo_int4_gemms_b200.autotune import make_ragged_fwd_inputs

    index, layout, sub, block_m, k, n, sizes, out_name = case
    lay = getattr(pkg.GemmLayout, layout.upper())
    data = make_ragged_fwd_inputs(m=sum(sizes), n=n, k=k, group_sizes=list(sizes), layout=lay, scale=scale_spec(pkg, sub), seed=500 + index)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    cfg = pkg.RaggedDotConfig(block_m=block_m)
    info = pkg.calculate_group_info(dev["group_sizes"], cfg.block_m, align_tile=cfg.align_tile)
    out_dtype = torch.float32 if out_name == "f32" else torch.bfloat16
    outs = []
    for path in (native.PATH_AUTO, native.PATH_SIMT):
        out = torch.full((sum(sizes), n), float("nan"), device="cuda", dtype=out_dtype)
        native.launch_ragged_fwd_kernel(dev["lhs"], dev["rhs"], group_info=info, a_scale=dev["a_scale"], b_scale=dev["b_scale"], out=out,
                                        scale=scale_spec(pkg, sub), config=cfg, layout=lay, rows=sum(sizes), cols=n, k_packed=k // 2,
                                        scale_cols=(k // sub if sub else 1), path=path)
        outs.append(out)
    torch.cuda.synchronize()
    assert native.device_status(0)[0] == 0
    assert not torch.isnan(outs[0]).any()
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("seed", range(12))
def test_grouped_backward_tensor_core_equals_cuda_core_and_flat_equals_stacked(pkg, seed):
    from helpers import scale_spec
    from strix_halo_int4_gemms_b200 import native
    from strix_halo_int4_gemms_b200.autotune import make_ragged_bwd_inputs

    rng = random.Random(900 + seed)
    sub = rng.choice([0, 0, 128])
    m, n = rng.choice([128, 256, 400]), rng.choice([64, 256, 400])
    sizes = _group_sizes(rng, rng.choice([2, 4, 7]), rng.choice([30, 200, 500]))
    if sub:
        sizes = [s // sub * sub for s in sizes]   # K-groups must tile each group's reduction
        if sum(sizes) == 0:
            sizes[0] = sub
    cap = max(32, (max(sizes) + 31) // 32 * 32)
    data = make_ragged_bwd_inputs(m=m, n=n, k_capacity=cap, group_sizes=sizes, layout=pkg.GemmLayout.TN, scale=scale_spec(pkg, sub), seed=seed)
    dev = {name: data[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale")}
    sizes_t = torch.tensor(sizes, dtype=torch.int64).cuda()
    outs = []
    for path in (native.PATH_AUTO, native.PATH_SIMT):
        out = torch.full((len(sizes), m, n), float("nan"), device="cuda", dtype=torch.float32)
        native.launch_ragged_bwd_kernel(dev["lhs"], dev["rhs"], sizes_t, a_scale=dev["a_scale"], b_scale=dev["b_scale"], out=out,
                                        scale=scale_spec(pkg, sub), config=pkg.RaggedBwdDotConfig(), layout=pkg.GemmLayout.TN,
                                        rows=m, cols=n, k_packed=cap // 2, scale_cols=(cap // sub if sub else 1), path=path)
        outs.append(out)
    torch.cuda.synchronize()
    assert native.device_status(0)[0] == 0
    assert torch.equal(outs[0], outs[1])
    if sub == 0:
        # the same groups laid out flat: concatenate each group's valid token rows (TN: [cap/2, M] per group, two tokens per byte)
        lhs_codes = [pkg.unpack_int4_k_major(data["lhs"][g].t().contiguous())[:, :s].t() for g, s in enumerate(sizes)]   # [s, M] each
        rhs_codes = [pkg.unpack_int4_k_major(data["rhs"][g].t().contiguous())[:, :s].t() for g, s in enumerate(sizes)]   # [s, N] each
        x = torch.cat(lhs_codes, 0)
        dy = torch.cat(rhs_codes, 0)
        flat = pkg.ragged_dot_int4_bwd_flat(pkg.repack_int4_tokens(pkg.pack_int4_k_major(x).cuda()),
                                            pkg.repack_int4_tokens(pkg.pack_int4_k_major(dy).cuda()), sizes_t,
                                            a_scale=dev["a_scale"], b_scale=dev["b_scale"])
        torch.cuda.synchronize()
        assert torch.equal(flat, outs[0])
