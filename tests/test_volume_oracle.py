"""CPU test: the C restatement of the stereo cost-volume construction (GlobalCorrelation,
models/cost_volume.py:26-51) against volumes returned by the reference module itself."""
import pytest

import oracle
from _cases import assert_close, golden_volume_names, load_golden_volume


@pytest.mark.parametrize("name", golden_volume_names())
def test_volume_oracle_matches_reference_vectors(name):
    c = load_golden_volume(name)
    vol = oracle.stereo_volume(c["correlation"])
    assert vol.shape == c["volume"].shape
    assert_close(vol, c["volume"], c["dtype"], name)     # probabilities <= 1: the operator's tolerances apply
