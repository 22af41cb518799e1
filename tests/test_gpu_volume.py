"""GPU tests of the stereo cost-volume kernel (GlobalCorrelation, models/cost_volume.py:26-51) through the
C ABI: against volumes returned by the reference module (golden files) and against the oracle."""
import pytest
import torch

from _cases import assert_close, golden_volume_names, load_golden_volume

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_volume_names())
def test_kernel_matches_reference_vectors(name):
    import matchattention_b200 as ma
    c = load_golden_volume(name)
    vol = ma.stereo_volume(c["correlation"].cuda()).cpu()
    assert_close(vol, c["volume"], c["dtype"], name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 48, 48), (2, 17, 33), (1, 3, 120), (1, 5, 1), (2, 68, 120)])
def test_kernel_matches_oracle(shape, dtype):
    import matchattention_b200 as ma
    import oracle
    B, H, W = shape
    g = torch.Generator().manual_seed(H + W)
    corr = (torch.randn(B, H, W, W, generator=g) * 3).to(dtype)
    ref = oracle.stereo_volume(corr)
    vol = ma.stereo_volume(corr.cuda()).cpu()
    assert_close(vol, ref, dtype)
    if dtype != torch.float32:
        same = (vol.view(torch.int16) == ref.view(torch.int16)).float().mean().item()
        assert same > 0.99, f"only {same:.3%} bit-identical to the oracle"


def test_too_wide_rows_are_refused():
    import matchattention_b200 as ma
    with pytest.raises(RuntimeError):
        ma.stereo_volume(torch.zeros(1, 2, 200, 200, device="cuda"))
