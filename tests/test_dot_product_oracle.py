"""CPU tests of the dot-product scoring.  The reference has this scoring only in its native kernel
(models/src/match_former_fused_forward.cu:222-251) and no PyTorch form of it: PARITY IS UNPINNED.  The vectors
were made by the reference's own functions with the one scoring line swapped (tests/golden/make_golden.py,
dot_product_cases)."""
import pytest
import torch

import oracle
from oracle import matchattn_numpy
from _cases import assert_close, golden_names_with_prefix, load_golden


@pytest.mark.parametrize("name", golden_names_with_prefix("dot_"))
def test_c_oracle_matches_the_restated_vectors(name):
    c = load_golden(name)
    out, attn = oracle.forward(c["max_offset"], c["q"], c["k"], c["v"], c["H"], c["W"], c["r"], c["scale"],
                               attn_type="dot_product")
    assert_close(attn, c["attn"], c["dtype"], name + " attn")
    assert_close(out, c["out"], c["dtype"], name + " out")
    if c["dtype"] != torch.float32:
        for got, ref in ((out, c["out"]), (attn, c["attn"])):
            differing = (got.view(torch.int16) != ref.view(torch.int16)).float().mean().item()
            assert differing < 5e-3, f"{name}: {differing:.2%} of elements differ"


def test_scoring_functions_differ_and_unknown_is_refused():
    c = load_golden(golden_names_with_prefix("dot_")[0])
    args = (c["max_offset"], c["q"], c["k"], c["v"], c["H"], c["W"], c["r"], c["scale"])
    l1 = oracle.forward(*args)[1]
    dot = oracle.forward(*args, attn_type="dot_product")[1]
    assert not torch.equal(l1, dot)
    with pytest.raises(KeyError):
        oracle.forward(*args, attn_type="l2_norm")


@pytest.mark.parametrize("name", [n for n in golden_names_with_prefix("dot_") if not n.endswith("bf16")])
def test_numpy_restatement_matches_the_restated_vectors(name):
    """The second, independent restatement (numpy; no bfloat16 there)."""
    c = load_golden(name)
    out, attn = matchattn_numpy.forward(c["max_offset"].numpy(), c["q"].numpy(), c["k"].numpy(), c["v"].numpy(),
                                        c["H"], c["W"], c["r"], c["scale"], attn_type="dot_product")
    assert_close(torch.from_numpy(attn), c["attn"], c["dtype"], name + " attn")
    assert_close(torch.from_numpy(out), c["out"], c["dtype"], name + " out")
