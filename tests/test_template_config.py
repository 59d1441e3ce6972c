"""Launch-shape contract (CPU).  Modelled on the reference's tests/test_template_config.py and tests/test_native.py:97-128."""
import pytest

from strix_halo_int4_gemms_b200.template_config import (
    LaunchShape,
    is_tile_multiple_shape,
    plan_template,
    representative_generation_shape,
    tile_multiple_rejection_reasons,
)


def _kernel(pkg, **kw):
    base = dict(dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.NONE, m=128, n=256, k=256)
    base.update(kw)
    return pkg.default_registry.select(**base)


def test_accepts_multiples_and_names_each_violation(pkg):
    k = _kernel(pkg, split_k=2)
    assert is_tile_multiple_shape(k, LaunchShape(256, 512, 128))
    reasons = tile_multiple_rejection_reasons(k, LaunchShape(130, 300, 96))
    assert reasons == (
        "M=130 is not divisible by BLOCK_M=128",
        "N=300 is not divisible by BLOCK_N=256",
        "K=96 is not divisible by BLOCK_K*SPLIT_K=64",
    )
    with pytest.raises(ValueError, match=f"{k.kernel_id} requires tile-multiple shape: M=130"):
        LaunchShape(130, 256, 128).validate_for(k)
    assert tile_multiple_rejection_reasons(k, LaunchShape(0, 256, 128)) == ("M, N, and K must be positive; got (0, 256, 128)",)


def test_subchannel_needs_k_multiple_of_group(pkg):
    k = _kernel(pkg, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 256))
    assert "K=128 is not divisible by SUBCHANNEL=256" in tile_multiple_rejection_reasons(k, LaunchShape(128, 256, 128))
    assert representative_generation_shape(k) == LaunchShape(128, 256, 256)


def test_plan_template_flags(pkg):
    k = _kernel(pkg, m=128, n=128, epilogue=pkg.Epilogue.SWIGLU, scale=pkg.ScaleSpec(pkg.ScaleMode.SUBCHANNEL, 64))
    plan = plan_template(k, LaunchShape(128, 128, 128))
    assert plan.needs_packed_int4 and plan.needs_subchannel_loop and plan.needs_fused_swiglu_up_gate
    assert not plan.needs_per_channel_epilogue_scale and not plan.needs_relu2_activation
    assert plan.even_k and plan.split_k == 1
    with pytest.raises(ValueError, match="requires tile-multiple shape"):
        plan_template(k, LaunchShape(128, 130, 128))


def test_every_entry_accepts_its_representative_shape(pkg):
    for k in pkg.default_registry.all()[::37]:
        assert is_tile_multiple_shape(k, representative_generation_shape(k)), k.kernel_id
