"""The allocation-free entry point, b200_int4_gemms_launch_ragged_bwd_flat_static, against the entry
point it shadows (b200_int4_gemms_launch_ragged_bwd_flat, caller-provided workspace).

Collected last on purpose: the built-in scratch is shared by every call in the process, so this file
shows that it works after whatever ran before it as well as on its own, and that two calls in a row
(the second finding the first one's group starts still in the array) both give the right answer."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(pkg, sizes, m, n, seed):
    g = torch.Generator().manual_seed(seed)
    total = sum(sizes)
    x = torch.randint(-8, 8, (total, m), generator=g, dtype=torch.int8)
    dy = torch.randint(-8, 8, (total, n), generator=g, dtype=torch.int8)
    return dict(
        lhs=pkg.repack_int4_tokens(pkg.pack_int4_k_major(x).cuda()),
        rhs=pkg.repack_int4_tokens(pkg.pack_int4_k_major(dy).cuda()),
        sizes=torch.tensor(sizes, dtype=torch.int64).cuda(),
        sa=((torch.rand(len(sizes), m, generator=g) + 0.5) * 0.05).bfloat16().cuda(),
        sb=((torch.rand(len(sizes), n, generator=g) + 0.5) * 0.05).bfloat16().cuda(),
    )


def _run(pkg, c, *, static, out=None):
    return pkg.ragged_dot_int4_bwd_flat(c["lhs"], c["rhs"], c["sizes"], a_scale=c["sa"], b_scale=c["sb"], out=out,
                                        static_scratch=static)


def test_static_scratch_matches_workspace_entry_on_two_calls_in_a_row(pkg):
    from strix_halo_int4_gemms_b200 import native

    first = _case(pkg, [17, 0, 300, 128, 255, 4], 256, 512, seed=1)     # 6 groups, odd starts
    second = _case(pkg, [513, 64], 384, 256, seed=2)                    # fewer groups, other offsets
    want_first = _run(pkg, first, static=False)
    want_second = _run(pkg, second, static=False)
    got_first = _run(pkg, first, static=True)
    got_second = _run(pkg, second, static=True)      # the array still holds the first call's six starts
    got_first_again = _run(pkg, first, static=True)
    torch.cuda.synchronize()
    assert native.device_status(0)[0] == 0
    assert torch.equal(got_first, want_first)
    assert torch.equal(got_second, want_second)
    assert torch.equal(got_first_again, want_first)


def test_static_scratch_call_leaves_device_memory_alone(pkg):
    c = _case(pkg, [100, 28, 0, 129], 128, 256, seed=3)
    out = torch.empty((4, 128, 256), device="cuda", dtype=torch.float32)
    _run(pkg, c, static=True, out=out)               # first call on the device: one-time set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    _run(pkg, c, static=True, out=out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == torch_before
    assert free_after >= free_before        # nothing was taken from the device
    assert torch.equal(out, _run(pkg, c, static=False))


def test_static_scratch_refuses_more_groups_than_it_holds(pkg):
    from strix_halo_int4_gemms_b200 import native

    lib = native.load_dispatch_library()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    v = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.TN, scale=pc, epilogue=pkg.Epilogue.NONE,
                            out_dtype=native.OUT_F32)
    six = [ctypes.c_void_p(16)] * 6
    rc = lib.b200_int4_gemms_launch_ragged_bwd_flat_static(ctypes.byref(v), 0, 0, *six, 128, 256, 100000,
                                                           native.STATIC_SCRATCH_MAX_GROUPS + 1)
    assert rc == 1
    message = lib.b200_int4_gemms_last_error().decode()
    assert "at most 4096 groups" in message and "workspace" in message
    # the limit itself is accepted (4096 groups of one token each)
    groups = native.STATIC_SCRATCH_MAX_GROUPS
    c = _case(pkg, [1] * groups, 128, 256, seed=4)
    assert torch.equal(_run(pkg, c, static=True), _run(pkg, c, static=False))
