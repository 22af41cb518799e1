"""GPU tests of the operator with the caller's glue folded in (clamp of the centres, gate,
concatenated output layout) against the same steps done separately: the caller's clamp as the
reference writes it, the oracle, and the gate / cat in PyTorch on the CPU."""
import pytest
import torch

from _cases import assert_close, clamp_like_caller, make_inputs

pytestmark = pytest.mark.gpu

CASES = [
    # B, H, W, h, hd, r
    (2, 30, 36, 8, 16, 1),
    (2, 24, 20, 4, 40, 2),
    (1, 17, 19, 4, 32, 1),
    (1, 16, 18, 3, 12, 1),     # any-shape kernel
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
def test_cross_core_equals_clamp_op_gate_cat(case, dtype):
    import oracle
    import matchattention_b200 as ma
    B, H, W, h, hd, r = case
    raw, q, k, v = make_inputs(80 + hd, B, H, W, h, hd, r, dtype, kind="raw")       # centres far outside too
    g = torch.Generator().manual_seed(5)
    gate = torch.sigmoid(torch.randn(B, H * W, h * hd, generator=g)).to(dtype)
    scale = hd ** -0.5
    mo = clamp_like_caller(raw, H, W, r)
    ref_out, ref_attn = oracle.forward(mo, q, k, v, H, W, r, scale)
    expect = torch.cat((gate * ref_out, ref_attn.view(B, H * W, -1)), dim=-1)
    got = ma.cross_attention_core(raw.cuda(), q.cuda(), k.cuda(), v.cuda(), gate.cuda(), H, W, r, scale).cpu()
    assert got.shape == expect.shape
    assert_close(got, expect, dtype, "gated concat", ties=hd > 16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_self_core_equals_clamp_op(dtype):
    import oracle
    import matchattention_b200 as ma
    B, H, W, h, hd, r = 2, 26, 22, 4, 16, 2
    raw, q, k, v = make_inputs(90, B, H, W, h, hd, r, dtype, kind="raw")
    mo = clamp_like_caller(raw, H, W, r)
    ref_out, _ = oracle.forward(mo, q, k, v, H, W, r, 0.25)
    got = ma.self_attention_core(raw.cuda(), q.cuda(), k.cuda(), v.cuda(), H, W, r, 0.25).cpu()
    assert_close(got, ref_out, dtype, "self core")


def test_fused_clamp_equals_separate_clamp_bitwise():
    import matchattention_b200 as ma
    B, H, W, h, hd, r = 1, 40, 44, 8, 16, 1
    raw, q, k, v = (t.cuda() for t in make_inputs(91, B, H, W, h, hd, r, torch.float16, kind="raw"))
    mo = clamp_like_caller(raw.cpu(), H, W, r).cuda()
    sep_out, sep_attn = ma.match_attention(mo, q, k, v, H, W, r, 0.25)
    fused = ma.cross_attention_core(raw, q, k, v, None, H, W, r, 0.25)
    assert torch.equal(fused[..., :h * hd], sep_out)
    assert torch.equal(fused[..., h * hd:], sep_attn.view(B, H * W, -1))


@pytest.mark.parametrize("case", [(4, 20, 22, 8, 16, 1), (2, 16, 18, 4, 40, 2), (2, 12, 14, 3, 12, 1)])
def test_batch_swap_folded_into_the_kernel(case):
    """kv_shift = B/2 reads the other view's keys / values: bit-identical to rolling K and V first."""
    import matchattention_b200 as ma
    B, H, W, h, hd, r = case
    raw, q, k, v = (t.cuda() for t in make_inputs(92, B, H, W, h, hd, r, torch.float16, kind="raw"))
    gate = torch.rand_like(q)
    want = ma.cross_attention_core(raw, q, k.roll(B // 2, 0).contiguous(), v.roll(B // 2, 0).contiguous(), gate, H, W,
                                   r, hd ** -0.5)
    got = ma.cross_attention_core(raw, q, k, v, gate, H, W, r, hd ** -0.5, kv_shift=B // 2)
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):
        ma.cross_attention_core(raw, q, k, v, gate, H, W, r, hd ** -0.5, kv_shift=B)
