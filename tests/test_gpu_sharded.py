"""The multi-GPU partitioning code on ONE device: every shard of a 2-, 4- and 8-way split is run in turn through
distributed.py and the library, and the pieces must reassemble to the unsharded result bit for bit."""
import numpy as np
import pytest
import torch

from helpers import scale_spec
from strix_halo_int4_gemms_b200 import distributed as shard
from strix_halo_int4_gemms_b200.autotune import make_ragged_bwd_inputs, make_ragged_fwd_inputs

pytestmark = pytest.mark.gpu


def _dense_problem(pkg, m, n, k, *, sub, swiglu, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    cols = 2 * n if swiglu else n
    a = torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.uint8)
    b = torch.randint(0, 256, (k // 2, cols), generator=g, device="cuda", dtype=torch.uint8)
    groups = k // sub if sub else 0
    sa = ((torch.rand((m, groups) if groups else (m,), device="cuda", generator=g) + 0.5) * 0.05).bfloat16()
    sb = ((torch.rand((groups, cols) if groups else (cols,), device="cuda", generator=g) + 0.5) * 0.05).bfloat16()
    return a, b, sa, sb


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("sub,swiglu,n", [(0, False, 1024), (256, True, 2048), (64, False, 3072)])   # every shard a multiple of 128 columns
def test_column_parallel_shards_reassemble(pkg, world, sub, swiglu, n):
    m, k = 512, 1024
    a, b, sa, sb = _dense_problem(pkg, m, n, k, sub=sub, swiglu=swiglu, seed=world)
    scale = scale_spec(pkg, sub)
    run = (lambda bb, ss: pkg.fused_swiglu_up_gate(a, bb, a_scale=sa, b_scale=ss, scale=scale)) if swiglu else \
          (lambda bb, ss: pkg.mm(a, bb, a_scale=sa, b_scale=ss, scale=scale))
    whole = run(b, sb)
    pieces = torch.full_like(whole, float("nan"))
    covered = 0
    for rank in range(world):
        b_r, s_r, (lo, hi) = shard.shard_dense_rhs(b, sb, layout=pkg.GemmLayout.NN, world_size=world, rank=rank, swiglu=swiglu)
        assert (lo, hi) == shard.column_block(n, world, rank)
        if hi > lo:
            pieces[:, lo:hi] = run(b_r, s_r)
        covered += hi - lo
    torch.cuda.synchronize()
    assert covered == n and torch.equal(pieces, whole)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_shards_reassemble(pkg, world):
    sizes = [300, 0, 256, 7, 129, 512, 1, 255, 64, 64, 0, 900, 33, 128, 2, 77]
    pc = scale_spec(pkg, 0)
    fwd = make_ragged_fwd_inputs(m=sum(sizes), n=512, k=512, group_sizes=sizes, layout=pkg.GemmLayout.NN, scale=pc, seed=3)
    dev = {name: fwd[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    whole = pkg.ragged_dot_int4(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"])
    plan = shard.assign_groups(sizes, world)
    assert sorted(g for groups in plan for g in groups) == list(range(len(sizes)))
    # LPT cannot do better than the largest group allows
    assert shard.load_imbalance(sizes, plan) <= max(1.35, max(sizes) / (sum(sizes) / world)) + 1e-9
    pieces = torch.full_like(whole, float("nan"))
    for groups in plan:
        part = shard.shard_ragged_fwd(dev["lhs"], dev["rhs"], dev["a_scale"], dev["b_scale"], dev["group_sizes"], groups)
        if part.lhs.shape[0] == 0:
            continue
        out = pkg.ragged_dot_int4(part.lhs, part.rhs, part.group_sizes.cuda(), a_scale=part.a_scale, b_scale=part.b_scale)
        pieces[part.row_index.cuda()] = out
    torch.cuda.synchronize()
    assert torch.equal(pieces, whole)

    bwd = make_ragged_bwd_inputs(m=256, n=512, k_capacity=928, group_sizes=sizes, layout=pkg.GemmLayout.TN, scale=pc, seed=4)
    dev = {name: bwd[name].cuda() for name in ("lhs", "rhs", "a_scale", "b_scale", "group_sizes")}
    whole = pkg.ragged_dot_int4_bwd(dev["lhs"], dev["rhs"], dev["group_sizes"], a_scale=dev["a_scale"], b_scale=dev["b_scale"], layout=pkg.GemmLayout.TN)
    pieces = torch.full_like(whole, float("nan"))
    for groups in plan:
        if not groups:
            continue
        lhs, rhs, sa, sb, gs = shard.shard_ragged_bwd(dev["lhs"], dev["rhs"], dev["a_scale"], dev["b_scale"], dev["group_sizes"], groups)
        pieces[torch.tensor(groups).cuda()] = pkg.ragged_dot_int4_bwd(lhs, rhs, gs, a_scale=sa, b_scale=sb, layout=pkg.GemmLayout.TN)
    torch.cuda.synchronize()
    assert torch.equal(pieces, whole)
