"""GPU tests of the dot-product scoring (general kernel).  The reference has this scoring only as an unused
native kernel (models/src/match_former_fused_forward.cu:222-251): PARITY IS UNPINNED; the vectors restate it
(tests/golden/make_golden.py, dot_product_cases) and the CPU oracle is pinned to them."""
import pytest
import torch

import oracle
from _cases import assert_close, golden_names_with_prefix, load_golden, make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_names_with_prefix("dot_"))
def test_kernel_matches_the_restated_vectors(name):
    import matchattention_b200 as ma
    c = load_golden(name)
    dev = [c[key].cuda() for key in ("max_offset", "q", "k", "v")]
    out, attn = ma.match_attention(*dev, c["H"], c["W"], c["r"], c["scale"], attn_type="dot_product")
    assert_close(attn.cpu(), c["attn"], c["dtype"], name + " attn")
    assert_close(out.cpu(), c["out"], c["dtype"], name + " out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_kernel_matches_oracle_on_a_model_shape(dtype):
    import matchattention_b200 as ma
    B, H, W, h, hd, r = 2, 48, 64, 8, 16, 1
    mo, q, k, v = make_inputs(71, B, H, W, h, hd, r, dtype, kind="flow", spread=6.0, per_head=True, border_frac=0.1)
    q, k = (q * 0.5).to(dtype), (k * 0.5).to(dtype)
    ref_out, ref_attn = oracle.forward(mo, q, k, v, H, W, r, hd ** -0.5, attn_type="dot_product")
    out, attn = ma.match_attention(mo.cuda(), q.cuda(), k.cuda(), v.cuda(), H, W, r, hd ** -0.5, attn_type="dot_product")
    assert_close(attn.cpu(), ref_attn, dtype, "attn")
    assert_close(out.cpu(), ref_out, dtype, "out")
    band_out, band_attn = ma.match_attention(mo.cuda()[:, 8 * W:20 * W].contiguous(), q.cuda()[:, 8 * W:20 * W].contiguous(),
                                             k.cuda(), v.cuda(), H, W, r, hd ** -0.5, attn_type="dot_product",
                                             q_row_begin=8, q_row_end=20)
    assert torch.equal(band_out, out[:, 8 * W:20 * W]) and torch.equal(band_attn, attn[:, 8 * W:20 * W])


def test_tuned_variants_refuse_the_dot_product():
    import matchattention_b200 as ma
    B, H, W, h, hd, r = 1, 16, 16, 8, 16, 1
    mo, q, k, v = (t.cuda() for t in make_inputs(72, B, H, W, h, hd, r, torch.float16, kind="flow", spread=2.0))
    with pytest.raises(RuntimeError):
        ma.match_attention(mo, q, k, v, H, W, r, 0.25, attn_type="dot_product", strategy=ma.ops.STRATEGY_STAGED)
    with pytest.raises(NotImplementedError):
        ma.match_attention(mo, q, k, v, H, W, r, 0.25, attn_type="l2_norm")
