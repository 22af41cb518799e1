"""GPU parity tests: the CUDA kernels, called through the C ABI, against the
golden vectors (outputs of the reference itself) and against the CPU oracle on
seeded inputs.  Tolerances: float32 1e-4 relative, float16 2e-3 absolute
(bfloat16: 8x the float16 bound, for its 3 fewer significand bits)."""
import pytest
import torch

from _cases import (assert_close, excess, golden_names, golden_sampled_names, load_golden, load_golden_sampled,
                    make_inputs)

pytestmark = pytest.mark.gpu


def _ma():
    import matchattention_b200
    return matchattention_b200


def _oracle():
    import oracle
    return oracle


def run_kernel(c_or_inputs, H, W, r, scale, **kw):
    mo, q, k, v = (t.cuda() for t in c_or_inputs)
    out, attn = _ma().match_attention(mo, q, k, v, H, W, r, scale, **kw)
    torch.cuda.synchronize()
    return out.cpu(), (attn.cpu() if attn is not None else None)


@pytest.mark.parametrize("force_generic", [False, True])
@pytest.mark.parametrize("name", golden_names())
def test_kernel_matches_reference_vectors(name, force_generic):
    c = load_golden(name)
    out, attn = run_kernel((c["max_offset"], c["q"], c["k"], c["v"]), c["H"], c["W"], c["r"], c["scale"],
                           force_generic=force_generic)
    assert_close(attn, c["attn"], c["dtype"], name + " attn")
    assert_close(out, c["out"], c["dtype"], name + " out")


@pytest.mark.parametrize("name", golden_sampled_names())
def test_kernel_matches_reference_at_full_size(name):
    """The CPU-runnable configuration (104x208 tokens) at full size against the reference's own outputs
    at every 26th query."""
    c = load_golden_sampled(name)
    out, attn = run_kernel(c["inputs"], c["H"], c["W"], c["r"], c["scale"])
    assert_close(attn[:, c["index"]], c["attn"], c["dtype"], name + " attn")
    assert_close(out[:, c["index"]], c["out"], c["dtype"], name + " out")


SHAPES = [
    # B, H, W, h, hd, r, kind
    (1, 104, 208, 8, 16, 1, "cross"),     # the CPU-runnable config, disparity-like offsets
    (1, 104, 208, 8, 16, 1, "self"),      # ... and its per-head small-offset variant
    (2, 48, 48, 4, 40, 2, "self"),        # model stage shapes: tiny 1/32 (hd 40, r 2)
    (2, 37, 53, 4, 32, 2, "flow"),        # 1/16, odd map sizes
    (2, 40, 56, 4, 16, 1, "flow"),        # 1/8
    (2, 64, 72, 4, 8, 1, "flow"),         # 1/4
    (1, 33, 47, 4, 64, 1, "flow"),        # small / base variants: wide heads
    (1, 24, 31, 4, 80, 2, "raw"),
    (1, 20, 22, 4, 128, 1, "raw"),
    (1, 19, 23, 3, 24, 1, "raw"),         # three heads, 3 chunks per head
    (2, 17, 18, 1, 48, 2, "raw"),
    (1, 16, 16, 2, 256, 1, "flow"),
    (1, 12, 14, 5, 12, 1, "raw"),         # hd not a multiple of 8: any-shape kernel
    (1, 14, 12, 2, 16, 3, "raw"),         # r = 3: any-shape kernel
    (1, 9, 11, 2, 8, 0, "raw"),           # r = 0
    (1, 4, 4, 2, 16, 1, "raw"),           # smallest map that fits the window
    (1, 6, 6, 2, 16, 2, "raw"),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_kernel_matches_oracle(shape, dtype):
    B, H, W, h, hd, r, kind = shape
    inputs = make_inputs(100 + H + hd, B, H, W, h, hd, r, dtype, kind=kind, spread=min(24.0, W / 3), per_head=True,
                         border_frac=0.2)
    scale = hd ** -0.5
    ref_out, ref_attn = _oracle().forward(*inputs, H, W, r, scale)
    out, attn = run_kernel(inputs, H, W, r, scale)
    ties = hd > 16          # see _cases.py: rounding ties of wide-head score sums
    assert_close(attn, ref_attn, dtype, "attn", ties=ties)
    assert_close(out, ref_out, dtype, "out", ties=ties)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("per_head", [False, True])
def test_headline_config_full_size(dtype, per_head):
    """B=4, 384x384 tokens, 8 heads x 16, 3x3 sub-windows, flow-like offsets of up to 24 tokens, 10 % of the
    queries left unclamped at the borders: every element against the oracle."""
    B, H, W, h, hd, r = 4, 384, 384, 8, 16, 1
    inputs = make_inputs(7, B, H, W, h, hd, r, dtype, kind="flow", spread=24.0, border_frac=0.1, per_head=per_head)
    ref_out, ref_attn = _oracle().forward(*inputs, H, W, r, 0.25)
    out, attn = run_kernel(inputs, H, W, r, 0.25)
    assert_close(attn, ref_attn, dtype, "attn")
    assert_close(out, ref_out, dtype, "out")
    if dtype != torch.float32:
        # rounding points are the reference's: almost every element is bit-identical
        same = (out.view(torch.int16) == ref_out.view(torch.int16)).float().mean().item()
        assert same > 0.99, f"only {same:.4%} of out is bit-identical to the oracle"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_row_band_equals_slice_of_full(dtype):
    B, H, W, h, hd, r = 2, 45, 38, 4, 32, 2
    mo, q, k, v = make_inputs(9, B, H, W, h, hd, r, dtype, kind="flow", spread=6.0)
    full_out, full_attn = run_kernel((mo, q, k, v), H, W, r, 0.2)
    for r0, r1 in ((0, 7), (7, 30), (30, 45)):
        sl = slice(r0 * W, r1 * W)
        out, attn = run_kernel((mo[:, sl].contiguous(), q[:, sl].contiguous(), k, v), H, W, r, 0.2,
                               q_row_begin=r0, q_row_end=r1)
        assert torch.equal(out, full_out[:, sl]) and torch.equal(attn, full_attn[:, sl])


def test_variants_agree_bitwise_in_float16():
    """Tile width, lanes per head and skipping attn_out do not change a single bit."""
    B, H, W, h, hd, r = 1, 40, 44, 4, 32, 1
    inputs = make_inputs(10, B, H, W, h, hd, r, torch.float16, kind="flow", spread=5.0)
    base_out, base_attn = run_kernel(inputs, H, W, r, 0.3)
    for kw in (dict(tile_w=1), dict(tile_w=4), dict(tile_w=64), dict(chunks_per_lane=1), dict(chunks_per_lane=2),
               dict(chunks_per_lane=4)):
        out, attn = run_kernel(inputs, H, W, r, 0.3, **kw)
        assert torch.equal(attn, base_attn), kw
        assert (out.float() - base_out.float()).abs().max() <= 2e-3, kw
    out, attn = run_kernel(inputs, H, W, r, 0.3, need_attn=False)
    assert attn is None and torch.equal(out, base_out)


@pytest.mark.parametrize("r", [1, 2])
@pytest.mark.parametrize("h,hd", [(1, 8), (3, 8), (5, 16), (6, 8), (7, 24), (3, 40)])
def test_launch_geometry_of_small_maps(h, hd, r):
    """Small launches run in narrower blocks, and a query's lanes need not divide a warp: whatever tile the
    library picks, the result is the one of one-query-wide tiles, bit for bit, and matches the oracle."""
    for H, W in ((7, 9), (13, 6), (21, 33)):
        inputs = make_inputs(300 + 7 * h + H, 2, H, W, h, hd, r, torch.float16, kind="flow", spread=3.0, border_frac=0.2,
                             per_head=True)
        out, attn = run_kernel(inputs, H, W, r, hd ** -0.5)
        out1, attn1 = run_kernel(inputs, H, W, r, hd ** -0.5, tile_w=1)
        assert torch.equal(out, out1) and torch.equal(attn, attn1), (H, W)
        ref_out, ref_attn = _oracle().forward(*inputs, H, W, r, hd ** -0.5)
        assert_close(attn, ref_attn, torch.float16, f"attn {H}x{W}", ties=hd > 16)
        assert_close(out, ref_out, torch.float16, f"out {H}x{W}", ties=hd > 16)


def test_properties_at_full_size():
    """Size-independent checks on the headline shape: weights sum to one, identical offsets across heads give
    the same result as a per-head run, and shifting the whole problem by one token shifts the result."""
    B, H, W, h, hd, r = 2, 384, 384, 8, 16, 1
    mo, q, k, v = (t.cuda() for t in make_inputs(11, B, H, W, h, hd, r, torch.float32, kind="flow", border_frac=0.0))
    mo = (mo * 64).round() / 64          # so that x + 1 below is exact and the fractions do not change
    ma = _ma()
    out, attn = ma.match_attention(mo, q, k, v, H, W, r, 0.25)
    assert (attn.sum(-1) - 1).abs().max().item() < 1e-5
    assert out.abs().max() <= v.abs().max() * (1 + 1e-5)
    # translation by one token along x: roll q, k, v and the offsets together (interior rows/cols only)
    roll = lambda t: t.view(B, H, W, -1).roll(1, dims=2).reshape(t.shape)
    mo2 = roll(mo).clone()
    mo2[..., 0] += 1
    out2, attn2 = ma.match_attention(mo2.contiguous(), roll(q).contiguous(), roll(k).contiguous(),
                                     roll(v).contiguous(), H, W, r, 0.25)
    inner = torch.zeros(B, H, W, dtype=torch.bool, device="cuda")
    inner[:, :, 1:] = True
    x_ok = (mo[..., 0] >= r + 1) & (mo[..., 0] < W - r - 3)
    inner = inner.view(B, -1) & roll(x_ok.all(-1).view(B, -1, 1).float()).view(B, -1).bool()
    d = (roll(out) - out2).abs().view(B, H * W, -1)[inner]
    assert d.max().item() < 1e-5


def test_integral_centres_give_plain_window_softmax():
    B, H, W, h, hd, r = 1, 30, 28, 4, 16, 1
    mo, q, k, v = make_inputs(12, B, H, W, h, hd, r, torch.float32, kind="self")
    mo = torch.floor(mo)
    out, attn = run_kernel((mo, q, k, v), H, W, r, 0.25)
    a = attn.view(B, H * W, h, 4, 4)
    assert a[..., 3, :].abs().max() == 0 and a[..., :, 3].abs().max() == 0
    ref_out, ref_attn = _oracle().forward(mo, q, k, v, H, W, r, 0.25)
    assert_close(out, ref_out, torch.float32)


def test_nan_and_huge_centres_do_not_fault():
    B, H, W, h, hd, r = 1, 16, 16, 2, 16, 1
    mo, q, k, v = make_inputs(13, B, H, W, h, hd, r, torch.float32, kind="self")
    mo[0, 0, 0, 0] = float("nan")
    mo[0, 1, 0, 0] = 1e30
    mo[0, 2, 1, 1] = -1e30
    mo[0, 3, 1, 0] = float("inf")
    out, attn = run_kernel((mo, q, k, v), H, W, r, 0.25)
    ref_out, ref_attn = _oracle().forward(mo, q, k, v, H, W, r, 0.25)
    finite = torch.isfinite(ref_out)
    assert torch.equal(torch.isfinite(out), finite)
    assert (out[finite] - ref_out[finite]).abs().max() < 1e-4
