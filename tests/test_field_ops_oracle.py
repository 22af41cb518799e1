"""CPU tests: the C restatements of consistency_mask and local_disparity_estimator against vectors
produced by running the reference's own functions (tests/golden/make_golden.py).

Both functions end in a discrete decision (a threshold, an arg max).  The tests gate the continuous
quantity behind it (the field difference; the result where the arg max is not a tie) and the discrete
output wherever the continuous one is not within its own error of the decision boundary."""
import pytest
import torch

import oracle
from _cases import golden_names_with_prefix, load_golden_arrays, ulp16

# The sampler inside consistency_mask: PyTorch's CPU build evaluates it in the tensor type, its CUDA
# build in float32 from the same 16-bit normalised coordinate.  The oracle restates the CUDA build (the
# model runs there); against the CPU-made vectors the 16-bit difference is therefore only bounded by
# the coordinate's rounding (a 16-bit ulp at +-1 times half the map width, times the field's slope).
# Observed: 3e-3 (float16) and 3e-2 (bfloat16) of the largest difference; the bounds below are relative to it.
DIFF_REL_TOL = {torch.float32: 1e-6, torch.float16: 6e-3, torch.bfloat16: 5e-2}


@pytest.mark.parametrize("name", golden_names_with_prefix("consistency_"))
def test_consistency_mask_oracle_matches_reference_vectors(name):
    c = load_golden_arrays(name)
    mask, diff = oracle.consistency_mask(c["field"], c["threshold"])
    err = (diff.float() - c["diff"].float()).abs()
    tol = DIFF_REL_TOL[c["dtype"]] * max(1.0, float(c["diff"].float().abs().max()))
    assert err.max() <= tol, f"{name}: field difference off by {err.max():.4g} (allowed {tol:.4g})"
    decided = (c["diff"].float() - c["threshold"]).abs() > tol
    assert decided.float().mean() > 0.7
    assert torch.equal(mask[decided], c["mask"][decided]), f"{name}: mask differs away from the threshold"


@pytest.mark.parametrize("name", golden_names_with_prefix("disparity_"))
def test_local_disparity_oracle_matches_reference_vectors(name):
    c = load_golden_arrays(name)
    dt = c["dtype"]
    flow, blur, centre = oracle.local_disparity(c["volume"])
    assert (flow[..., 1] == 0).all()
    if dt == torch.float32:
        assert (blur - c["blur_max"]).abs().max() <= 1e-6
    else:
        assert ((blur.float() - c["blur_max"].float()).abs() <= ulp16(c["blur_max"].float(), dt)).all()
    clear = c["gap"] > (1e-6 if dt == torch.float32 else 0.0)          # the arg max is not a tie
    assert clear.float().mean() > 0.5
    err = (flow[..., 0].float() - c["flow"][..., 0].float()).abs()[clear]
    allowed = 1e-4 * c["flow"][..., 0].float().abs().clamp_min(1.0)[clear] if dt == torch.float32 else \
        ulp16(c["flow"][..., 0].float(), dt)[clear]
    assert (err <= allowed).all(), f"{name}: disparity off by {err.max():.4g}"


def test_local_disparity_of_a_peaked_volume():
    """One symmetric peak per pixel, away from the ends: the estimate is the peak's index, signed by view."""
    B, D, H, W = 2, 16, 3, 4
    idx = torch.randint(3, D - 3, (B, H, W), generator=torch.Generator().manual_seed(1))
    vol = torch.full((B, D, H, W), 1e-4)
    for off, val in ((0, 0.5), (-1, 0.15), (1, 0.15), (-2, 0.05), (2, 0.05)):      # 0.05 < 1/D: dropped again
        vol.scatter_(1, (idx + off)[:, None], val)
    flow, _, centre = oracle.local_disparity(vol)
    assert torch.equal(centre, idx.int())
    sign = torch.tensor([-1.0, 1.0]).view(2, 1, 1)
    assert torch.allclose(flow[..., 0], sign * idx.float(), atol=1e-4)


def test_consistency_mask_of_consistent_fields():
    """Opposite constant fields of the two views are consistent everywhere the sample stays inside the map."""
    H, W = 6, 9
    field = torch.zeros(2, H, W, 2)
    field[0, ..., 0], field[1, ..., 0] = -2.0, 2.0
    mask, diff = oracle.consistency_mask(field)
    assert (diff[0, :, 2:] == 0).all() and (mask[0, :, 2:] == 1).all()
    assert (diff[0, :, :2] == 2).all() and (mask[0, :, :2] == 0).all()      # sampled outside: zero padding


@pytest.mark.parametrize("name", golden_names_with_prefix("flowinit_"))
def test_flow_init_oracle_matches_reference_vectors(name):
    """GlobalCorrelation's flow branch + local_flow_estimator: probabilities within one 16-bit ulp (1e-6 in
    float32), the pooled maximum likewise, the flow wherever the arg max is not a tie."""
    c = load_golden_arrays(name)
    dt, H, W = c["dtype"], c["H"], c["W"]
    flow, prob, blur, centre = oracle.flow_init(c["correlation"], H, W)
    if dt == torch.float32:
        assert (prob - c["prob"]).abs().max() <= 1e-6 and (blur - c["blur_max"]).abs().max() <= 1e-6
    else:
        assert ((prob.float() - c["prob"].float()).abs() <= ulp16(c["prob"].float(), dt)).all()
        assert ((blur.float() - c["blur_max"].float()).abs() <= ulp16(c["blur_max"].float(), dt)).all()
    clear = (c["gap"] > (1e-6 if dt == torch.float32 else 0.0)).view(-1, H, W)
    assert clear.float().mean() > 0.5
    err = (flow.float() - c["flow"].float()).abs()[clear]
    ref = c["flow"].float()[clear]
    allowed = 1e-4 * ref.abs().clamp_min(1.0) if dt == torch.float32 else 2 * ulp16(ref.abs().clamp_min(1.0), dt)
    assert (err <= allowed).all(), f"{name}: flow off by {err.max():.4g}"
