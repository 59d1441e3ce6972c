"""A bounded device wait that runs out: the kernel must return, say where it gave up, and leave the context usable.

Uses a TEST-ONLY build of the library (build.py: build_wait_test_library) in which the per-channel kernels' MMA warp
never signals "accumulator full" and every wait gives up after 5 ms instead of 2 s.  Nothing faults and nothing hangs:
the epilogue warps' wait (site 30) times out, raises the CTA's abort flag, every other role falls through at its next
wait, TMEM is freed, the kernel ends.  The shipped library is then used on the same context and must be correct."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import as_f32, dense_case, oracle_dense, scale_spec

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _build_module():
    spec = importlib.util.spec_from_file_location("b200_build", ROOT / "strix-halo-int4-gemms_b200" / "build.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("cta_group,m", [(1, 128), (2, 512)])   # one CTA per tile; CTA pairs (both CTAs of a pair give up)
def test_wait_runs_out_and_the_context_survives(pkg, cta_group, m):
    from strix_halo_int4_gemms_b200 import native

    test_lib = _build_module().build_wait_test_library()
    n, k = 512, 256
    case = dense_case(pkg, m=m, n=n, k=k, seed=11)
    dev = {name: case[name].cuda() for name in ("a", "b", "a_scale", "b_scale")}
    out = torch.zeros((m, n), device="cuda", dtype=torch.bfloat16)
    variant = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=scale_spec(pkg, 0),
                                  epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16, cta_group=cta_group, path=native.PATH_TCGEN05)
    launch = dict(device_index=0, stream_handle=torch.cuda.current_stream().cuda_stream, a_ptr=dev["a"].data_ptr(), b_ptr=dev["b"].data_ptr(),
                  a_scale_ptr=dev["a_scale"].data_ptr(), b_scale_ptr=dev["b_scale"].data_ptr(), c_ptr=out.data_ptr(), m=m, n=n, k=k)

    native.reset_device_status(0, library_path=test_lib)
    native.launch_dense(variant, library_path=test_lib, **launch)
    torch.cuda.synchronize()                                   # returns: the kernel gave up instead of spinning
    status, (block, site, _) = native.device_status(0, library_path=test_lib)
    assert status == 1 and site == 30 and block >= 0           # STATUS_WAIT_TIMEOUT at the epilogue's wait for the accumulator
    native.reset_device_status(0, library_path=test_lib)
    assert native.device_status(0, library_path=test_lib)[0] == 0

    # the same context, the shipped library: a normal launch is correct
    native.launch_dense(variant, **launch)
    torch.cuda.synchronize()
    assert native.device_status(0)[0] == 0
    np.testing.assert_array_equal(as_f32(out), oracle_dense(case))
