"""Operand-format helpers of the package against the oracle and the reference fixtures (CPU)."""
import numpy as np
import pytest
import torch

from oracle import reference_math as oracle


def test_fake_quant_int_rejects_bad_scale(pkg):
    x = torch.ones((2,), dtype=torch.bfloat16)
    for bad in (0.0, -0.1):
        with pytest.raises(ValueError, match="scale must be positive"):
            pkg.fake_quant_int(x, bits=4, scale=bad)
    with pytest.raises(TypeError, match="scalar"):
        pkg.fake_quant_int(x, bits=4, scale=torch.ones((2,)))
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        pkg.fake_quant_int(x, bits=5, scale=1.0)


def test_pack_unpack_known_vector(pkg):
    x = torch.tensor([[-8, -1, 0, 7], [3, -4, 5, -6]], dtype=torch.int8)
    packed = pkg.pack_int4_k_major(x)
    assert packed.dtype is torch.uint8 and packed.is_contiguous()
    assert packed.tolist() == [[0xF8, 0x70], [0xC3, 0xA5]]
    assert torch.equal(pkg.unpack_int4_k_major(packed), x)
    odd = pkg.pack_int4_k_major(torch.tensor([[1, -2, 3]], dtype=torch.int8))
    assert pkg.unpack_int4_k_major(odd).tolist() == [[1, -2, 3, 0]]


@pytest.mark.parametrize("name", ["even", "odd", "batched"])
def test_pack_matches_reference_fixture(pkg, golden, name):
    x = torch.from_numpy(golden[f"pack/{name}/x"])
    packed = pkg.pack_int4_k_major(x)
    np.testing.assert_array_equal(packed.numpy(), golden[f"pack/{name}/packed"])
    np.testing.assert_array_equal(pkg.unpack_int4_k_major(packed).numpy(), golden[f"pack/{name}/unpacked"])


def test_fake_quant_matches_reference_fixture(pkg, golden):
    from helpers import bits_to_bf16

    x = bits_to_bf16(golden["fake_quant/x_bits"])
    np.testing.assert_array_equal(pkg.fake_quant_int(x, bits=4, scale=0.1).numpy(), golden["fake_quant/q4_scale0p1"])
    np.testing.assert_array_equal(pkg.fake_quant_int(x, bits=8, scale=0.01).numpy(), golden["fake_quant/q8_scale0p01"])


def test_scale_packers(pkg):
    logical = torch.arange(2 * 3 * 4, dtype=torch.bfloat16).reshape(2, 3, 4)
    packed = pkg.pack_rhs_subchannel_scales(logical)
    assert tuple(packed.shape) == (2, 4, 3) and packed.is_contiguous()
    assert torch.equal(packed, logical.transpose(-2, -1))
    assert torch.equal(pkg.pack_ragged_rhs_subchannel_scales(logical), packed)
    with pytest.raises(ValueError, match="at least 2 dimensions"):
        pkg.pack_rhs_subchannel_scales(torch.ones(3))
    with pytest.raises(ValueError, match=r"\(G, N, scale_cols\)"):
        pkg.pack_ragged_rhs_subchannel_scales(torch.ones(3, 4))


def test_random_roundtrip_against_oracle(pkg):
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-8, 8, (7, 33), generator=g, dtype=torch.int8)
    packed = pkg.pack_int4_k_major(x)
    np.testing.assert_array_equal(packed.numpy(), oracle.pack_int4_k_major(x.numpy()))
    np.testing.assert_array_equal(pkg.unpack_int4_k_major(packed).numpy(), oracle.unpack_int4_k_major(packed.numpy()))
