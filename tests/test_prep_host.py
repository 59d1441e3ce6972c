"""Host-side checks of the formats either side of the GEMM path: the token repack and the flat backward
restatement of the oracle (pinned against the padded per-group form the reference API takes), and the
host mirror of the repack."""
import numpy as np
import pytest
import torch

from oracle import reference_math as oracle


def _codes(rng, shape):
    return rng.integers(-8, 8, size=shape, dtype=np.int8)


@pytest.mark.parametrize("tokens,features", [(1, 2), (7, 12), (8, 16), (33, 64)])
def test_repack_tokens_moves_every_code(tokens, features):
    rng = np.random.default_rng(tokens * 100 + features)
    codes = _codes(rng, (tokens, features))
    packed = oracle.pack_int4_k_major(codes)                       # [T, F/2]
    by_tokens = oracle.repack_tokens(packed)                       # [ceil(T/2), F]
    assert by_tokens.shape == ((tokens + 1) // 2, features) and by_tokens.dtype == np.uint8
    back = oracle.unpack_int4_k_major(np.ascontiguousarray(by_tokens.T)).T   # [2*ceil(T/2), F]
    np.testing.assert_array_equal(back[:tokens], codes)
    assert not back[tokens:].any()                                 # the odd last row is padded with zero codes


def test_host_repack_matches_oracle(pkg):
    rng = np.random.default_rng(5)
    packed = rng.integers(0, 256, size=(37, 24), dtype=np.uint8)
    got = pkg.repack_int4_tokens(torch.from_numpy(packed)).numpy()
    np.testing.assert_array_equal(got, oracle.repack_tokens(packed))


@pytest.mark.parametrize("sizes", [[5, 0, 8, 3], [1, 1, 1], [16, 16], [0, 7]])
def test_flat_backward_equals_padded_backward(sizes):
    """The flat form is the reference's per-group form with the padding removed: same numbers."""
    rng = np.random.default_rng(sum(sizes) + len(sizes))
    m, n, total = 12, 10, sum(sizes)
    x = _codes(rng, (total, m))
    dy = _codes(rng, (total, n))
    sa = oracle.f32_to_bf16_bits(rng.uniform(0.02, 0.08, size=(len(sizes), m)).astype(np.float32))
    sb = oracle.f32_to_bf16_bits(rng.uniform(0.02, 0.08, size=(len(sizes), n)).astype(np.float32))
    lhs_flat = oracle.repack_tokens(oracle.pack_int4_k_major(x))
    rhs_flat = oracle.repack_tokens(oracle.pack_int4_k_major(dy))
    got = oracle.ragged_dot_bwd_flat(lhs_flat, rhs_flat, sizes, sa, sb)

    # padded TN operands as the reference API wants them: [G, Kcap/2, M] and [G, Kcap/2, N]
    cap = max(2, (max(sizes) + 1) // 2 * 2)
    lhs_pad = np.zeros((len(sizes), cap // 2, m), dtype=np.uint8)
    rhs_pad = np.zeros((len(sizes), cap // 2, n), dtype=np.uint8)
    start = 0
    for g, size in enumerate(sizes):
        xg = np.zeros((cap, m), dtype=np.int8)
        dg = np.zeros((cap, n), dtype=np.int8)
        xg[:size] = x[start:start + size]
        dg[:size] = dy[start:start + size]
        lhs_pad[g] = oracle.pack_int4_k_major(np.ascontiguousarray(xg.T)).T
        rhs_pad[g] = oracle.pack_int4_k_major(np.ascontiguousarray(dg.T)).T
        start += size
    want = oracle.ragged_dot_bwd(lhs_pad, rhs_pad, sizes, sa, sb, layout="tn")
    np.testing.assert_array_equal(got, want)


def test_quantize_wrapper_validates_like_the_host_helper(pkg):
    x = torch.zeros(4, 4, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        pkg.quantize_int_cuda(x, bits=3, scale=0.1)
    with pytest.raises(TypeError, match="scale must be a positive"):
        pkg.quantize_int_cuda(x, bits=4, scale="0.1")
    with pytest.raises(ValueError, match="scale must be positive"):
        pkg.quantize_int_cuda(x, bits=4, scale=0.0)
    with pytest.raises(RuntimeError, match="CUDA bfloat16"):
        pkg.quantize_int_cuda(x, bits=4, scale=0.1)   # host tensor: there is no CPU path
