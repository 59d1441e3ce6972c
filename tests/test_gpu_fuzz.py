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
