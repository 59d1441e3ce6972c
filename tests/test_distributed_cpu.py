"""Sharding logic of the multi-GPU path, run as 2 gloo ranks on CPU: column-parallel dense and SwiGLU,
expert-parallel grouped dots, and the optional all-gathers.  The per-rank GEMM is done by the CPU math
(the oracle / the API's reference mode), so what is under test is partitioning and reassembly."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import strix_halo_int4_gemms_b200 as pkg
        from strix_halo_int4_gemms_b200 import distributed as shard
        from helpers import bf16_bits, dense_case
        from oracle import reference_math as oracle

        # ---- dense, column-parallel (N = 80 -> blocks of 48 and 32) ----------------------------
        case = dense_case(pkg, m=24, n=80, k=64, seed=1)
        full = pkg.mm(case["a"], case["b"], a_scale=case["a_scale"], b_scale=case["b_scale"], use_reference=True)
        b_loc, sb_loc, (lo, hi) = shard.shard_dense_rhs(case["b"], case["b_scale"], layout=pkg.GemmLayout.NN, world_size=world, rank=rank)
        assert b_loc.is_contiguous() and tuple(b_loc.shape) == (32, hi - lo)
        local = pkg.mm(case["a"], b_loc, a_scale=case["a_scale"], b_scale=sb_loc, use_reference=True)
        assert torch.equal(local, full[:, lo:hi])
        ranges = [shard.column_block(80, world, r) for r in range(world)]
        gathered = shard.all_gather_columns(local.float(), ranges)
        assert torch.equal(gathered, full.float())

        # ---- fused SwiGLU: each rank owns [up_r | gate_r] -------------------------------------
        sc = pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 32)
        case = dense_case(pkg, m=16, n=64, k=64, sub=32, epilogue="swiglu", seed=2)
        full = pkg.fused_swiglu_up_gate(case["a"], case["b"], a_scale=case["a_scale"], b_scale=case["b_scale"], scale=sc, use_reference=True)
        b_loc, sb_loc, (lo, hi) = shard.shard_dense_rhs(case["b"], case["b_scale"], layout=pkg.GemmLayout.NN, world_size=world, rank=rank, swiglu=True)
        assert tuple(b_loc.shape) == (32, 2 * (hi - lo)) and tuple(sb_loc.shape) == (2, 2 * (hi - lo))
        local = pkg.fused_swiglu_up_gate(case["a"], b_loc, a_scale=case["a_scale"], b_scale=sb_loc, scale=sc, use_reference=True)
        assert torch.equal(local, full[:, lo:hi])

        # ---- grouped forward, expert-parallel with LPT assignment -------------------------------
        from strix_halo_int4_gemms_b200.autotune import make_ragged_bwd_inputs, make_ragged_fwd_inputs

        sizes = [40, 0, 7, 90, 13, 30]
        pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
        data = make_ragged_fwd_inputs(m=sum(sizes), n=24, k=64, group_sizes=sizes, layout=pkg.GemmLayout.NN, scale=pc, seed=3)
        want = oracle.ragged_dot_fwd(data["lhs"].numpy(), data["rhs"].numpy(), sizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]))
        plan = shard.assign_groups(sizes, world)
        assert sorted(g for groups in plan for g in groups) == list(range(len(sizes)))
        mine = shard.shard_ragged_fwd(data["lhs"], data["rhs"], data["a_scale"], data["b_scale"], data["group_sizes"], plan[rank])
        assert int(mine.group_sizes.sum()) == mine.lhs.shape[0] == mine.row_index.numel()
        local = oracle.ragged_dot_fwd(mine.lhs.numpy(), mine.rhs.numpy(), mine.group_sizes.tolist(), bf16_bits(mine.a_scale), bf16_bits(mine.b_scale))
        assert np.array_equal(local, want[mine.row_index.numpy()])
        every = [shard.shard_ragged_fwd(data["lhs"], data["rhs"], data["a_scale"], data["b_scale"], data["group_sizes"], groups).row_index for groups in plan]
        rebuilt = shard.all_gather_rows(torch.from_numpy(local), every, sum(sizes))
        assert np.array_equal(rebuilt.numpy(), want)

        # ---- grouped backward: disjoint [g] slabs ---------------------------------------------
        ksizes = [37, 0, 64, 5, 20, 48]
        data = make_ragged_bwd_inputs(m=8, n=16, k_capacity=64, group_sizes=ksizes, layout=pkg.GemmLayout.TN, scale=pc, seed=4)
        want = oracle.ragged_dot_bwd(data["lhs"].numpy(), data["rhs"].numpy(), ksizes, bf16_bits(data["a_scale"]), bf16_bits(data["b_scale"]), layout="tn")
        plan = shard.assign_groups(ksizes, world)
        lhs, rhs, sa, sb, gs = shard.shard_ragged_bwd(data["lhs"], data["rhs"], data["a_scale"], data["b_scale"], data["group_sizes"], plan[rank])
        local = oracle.ragged_dot_bwd(lhs.numpy(), rhs.numpy(), gs.tolist(), bf16_bits(sa), bf16_bits(sb), layout="tn")
        assert np.array_equal(local, want[plan[rank]])

        dist.barrier()
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_over_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["ok0", "ok1"]


def test_column_blocks_cover_every_column_once():
    from strix_halo_int4_gemms_b200.distributed import column_block

    for n, world in ((4096, 8), (1408, 8), (80, 2), (14336, 4), (100, 3), (16, 8)):
        edges = [column_block(n, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert all(lo % 16 == 0 for lo, _ in edges if lo < n)
    assert [column_block(4096, 8, r) for r in (0, 7)] == [(0, 512), (3584, 4096)]
    with pytest.raises(ValueError):
        column_block(64, 2, 2)


def test_lpt_assignment_balances_skewed_groups():
    from strix_halo_int4_gemms_b200.distributed import assign_groups, load_imbalance

    g = torch.Generator().manual_seed(0)
    probs = torch.distributions.Dirichlet(torch.full((64,), 0.5)).sample()
    probs[torch.randperm(64, generator=g)[:3]] = 0
    sizes = torch.multinomial(probs / probs.sum(), 32768, replacement=True, generator=g).bincount(minlength=64).tolist()
    for world in (1, 2, 4, 8):
        plan = assign_groups(sizes, world)
        assert sorted(x for groups in plan for x in groups) == list(range(64))
        worst_single = max(sizes) / (sum(sizes) / world)
        assert load_imbalance(sizes, plan) <= max(1.02, worst_single + 1e-9)
    contiguous = [list(range(r * 8, r * 8 + 8)) for r in range(8)]
    assert load_imbalance(sizes, assign_groups(sizes, 8)) <= load_imbalance(sizes, contiguous)


def test_lpt_assignment_with_a_cost_per_group_spreads_the_groups():
    """The backward dot pays for every group's output slab: with a cost per group no rank ends up with one huge group
    while another holds a dozen small ones."""
    from strix_halo_int4_gemms_b200.distributed import assign_groups

    sizes = [4330] + [100] * 31 + [0] * 8 + [900] * 24
    by_rows = assign_groups(sizes, 8)
    by_cost = assign_groups(sizes, 8, per_group_cost=1024)
    assert sorted(x for groups in by_cost for x in groups) == list(range(64))
    counts_rows = [len(groups) for groups in by_rows]
    counts_cost = [len(groups) for groups in by_cost]
    assert max(counts_cost) - min(counts_cost) < max(counts_rows) - min(counts_rows)
    assert max(counts_cost) <= 10
    with pytest.raises(ValueError):
        assign_groups(sizes, 8, per_group_cost=-1)
