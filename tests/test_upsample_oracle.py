"""CPU test: the C restatement of the convex field upsampling (MatchStereo.upsample_field,
models/match_stereo.py:73-84) against vectors produced by running the reference."""
import pytest
import torch

import oracle
from _cases import assert_close_sum_of_products, golden_upsample_names, load_golden_upsample


@pytest.mark.parametrize("name", golden_upsample_names())
def test_upsample_oracle_matches_reference_vectors(name):
    c = load_golden_upsample(name)
    out = oracle.upsample_field(c["field"], c["mask"], c["factor"])
    assert out.shape == c["out"].shape
    scale = float(c["field"].float().abs().max()) * c["factor"]
    assert_close_sum_of_products(out, c["out"], c["dtype"], scale, name)
