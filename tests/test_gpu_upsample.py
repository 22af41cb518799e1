"""GPU tests of the convex field upsampling kernel (MatchStereo.upsample_field, models/match_stereo.py:73-84)
through the C ABI: against the reference's own outputs (golden files) and against the oracle."""
import pytest
import torch

from _cases import assert_close_sum_of_products, golden_upsample_names, load_golden_upsample

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_upsample_names())
def test_kernel_matches_reference_vectors(name):
    import matchattention_b200 as ma
    c = load_golden_upsample(name)
    out = ma.upsample_field(c["field"].cuda(), c["mask"].cuda(), c["factor"]).cpu()
    scale = float(c["field"].float().abs().max()) * c["factor"]
    assert_close_sum_of_products(out, c["out"], c["dtype"], scale, name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 48, 48, 2, 2), (1, 37, 131, 2, 4), (2, 96, 96, 2, 2), (1, 9, 300, 3, 8), (1, 5, 4, 8, 1)])
def test_kernel_matches_oracle(shape, dtype):
    import matchattention_b200 as ma
    import oracle
    B, H, W, D, f = shape
    g = torch.Generator().manual_seed(H * W + f)
    field = (torch.randn(B, H, W, D, generator=g) * 4).to(dtype)
    mask = (torch.randn(B, 9 * f * f, H, W, generator=g) * 2).to(dtype)
    ref = oracle.upsample_field(field, mask, f)
    out = ma.upsample_field(field.cuda(), mask.cuda(), f).cpu()
    assert_close_sum_of_products(out, ref, dtype, float(field.float().abs().max()) * f)
    if dtype != torch.float32:
        same = (out.view(torch.int16) == ref.view(torch.int16)).float().mean().item()
        assert same > 0.99, f"only {same:.3%} bit-identical to the oracle"


def test_constant_field_is_reproduced():
    """The weights are a convex combination: away from the zero-padded border a constant field comes
    back as factor * constant whatever the mask says."""
    import matchattention_b200 as ma
    B, H, W, D, f = 1, 12, 14, 2, 4
    field = torch.full((B, H, W, D), 1.5, device="cuda")
    mask = torch.randn(B, 9 * f * f, H, W, device="cuda")
    out = ma.upsample_field(field, mask, f)
    inner = out[:, f:-f, f:-f]
    assert torch.allclose(inner, torch.full_like(inner, 1.5 * f), atol=1e-5)


def test_bad_arguments_raise():
    import matchattention_b200 as ma
    field = torch.zeros(1, 4, 4, 2, device="cuda")
    with pytest.raises(ValueError):
        ma.upsample_field(field, torch.zeros(1, 36, 4, 5, device="cuda"), 2)
    with pytest.raises(RuntimeError):
        ma.upsample_field(field, torch.zeros(1, 81, 4, 4, device="cuda"), 3)        # factor 3 is not built
    with pytest.raises(RuntimeError):
        ma.upsample_field(field.cpu(), torch.zeros(1, 36, 4, 4), 2)
