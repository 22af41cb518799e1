"""GPU tests of the binned path (queries sorted by target tile, K/V tiles in shared
memory, scratch from the caller) through the C ABI: against the oracle, against the
direct kernel, with per-head centres (device-side fallback) and with row bands."""
import pytest
import torch

from _cases import assert_close, make_inputs

pytestmark = pytest.mark.gpu

BINNED = 2
CASES = [
    # B, H, W, h, hd, kind, spread, per_head
    (1, 40, 44, 8, 16, "flow", 6.0, False),
    (2, 33, 29, 4, 32, "raw", 6.0, False),      # centres far outside the map: everything lands in border bins
    (1, 30, 31, 3, 8, "flow", 5.0, False),
    (2, 37, 41, 4, 40, "flow", 12.0, False),
    (1, 20, 21, 5, 24, "raw", 5.0, False),
    (1, 4, 4, 2, 16, "raw", 2.0, False),        # a single bin, smaller than the staged region
    (2, 96, 128, 8, 16, "flow", 24.0, False),
    (1, 64, 64, 4, 16, "cross", 16.0, False),
]


def _run(inputs, H, W, hd, **kw):
    import matchattention_b200 as ma
    mo, q, k, v = (t.cuda() for t in inputs)
    out, attn = ma.match_attention(mo, q, k, v, H, W, 1, hd ** -0.5, **kw)
    torch.cuda.synchronize()
    return out.cpu(), (attn.cpu() if attn is not None else None)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
def test_binned_matches_oracle_and_direct(case, dtype):
    import oracle
    B, H, W, h, hd, kind, spread, per_head = case
    inputs = make_inputs(50 + H + hd, B, H, W, h, hd, 1, dtype, kind=kind, spread=spread, border_frac=0.2,
                         per_head=per_head)
    ref_out, ref_attn = oracle.forward(*inputs, H, W, 1, hd ** -0.5)
    out, attn = _run(inputs, H, W, hd, strategy=BINNED)
    ties = hd > 16
    assert_close(attn, ref_attn, dtype, "attn", ties=ties)
    assert_close(out, ref_out, dtype, "out", ties=ties)
    d_out, d_attn = _run(inputs, H, W, hd, strategy=1)
    assert torch.equal(attn, d_attn)
    assert_close(out, d_out, dtype, "binned vs direct", ties=ties)


def test_per_head_centres_fall_back_on_the_device():
    """Heads that look at different places cannot share a tile: the sorting pass notices and the
    direct kernel, launched in the same call, does the work.  The result must be the direct one."""
    B, H, W, h, hd = 1, 48, 40, 8, 16
    inputs = make_inputs(61, B, H, W, h, hd, 1, torch.float16, kind="flow", spread=8.0, per_head=True)
    out, attn = _run(inputs, H, W, hd, strategy=BINNED)
    d_out, d_attn = _run(inputs, H, W, hd, strategy=1)
    assert torch.equal(out, d_out) and torch.equal(attn, d_attn)


def test_binned_row_band_and_skipped_attn():
    B, H, W, h, hd = 2, 45, 38, 4, 32
    mo, q, k, v = make_inputs(62, B, H, W, h, hd, 1, torch.float16, kind="flow", spread=6.0)
    full_out, full_attn = _run((mo, q, k, v), H, W, hd, strategy=BINNED)
    r0, r1 = 7, 30
    sl = slice(r0 * W, r1 * W)
    out, attn = _run((mo[:, sl].contiguous(), q[:, sl].contiguous(), k, v), H, W, hd, strategy=BINNED,
                     q_row_begin=r0, q_row_end=r1)
    assert torch.equal(out, full_out[:, sl]) and torch.equal(attn, full_attn[:, sl])
    out2, none = _run((mo, q, k, v), H, W, hd, strategy=BINNED, need_attn=False)
    assert none is None and torch.equal(out2, full_out)


def test_binned_rejects_what_it_does_not_cover():
    import matchattention_b200 as ma
    B, H, W, h, hd = 1, 16, 16, 2, 16
    mo, q, k, v = (t.cuda() for t in make_inputs(63, B, H, W, h, hd, 1, torch.float32, kind="self"))
    with pytest.raises(RuntimeError):          # float32 has no binned path
        ma.match_attention(mo, q, k, v, H, W, 1, 0.25, strategy=BINNED)
    mo, q, k, v = (t.cuda() for t in make_inputs(63, B, H, W, h, hd, 2, torch.float16, kind="self"))
    with pytest.raises(RuntimeError):          # r = 2 neither
        ma.match_attention(mo, q, k, v, H, W, 2, 0.25, strategy=BINNED)
    small = torch.empty(16, dtype=torch.uint8, device="cuda")
    mo, q, k, v = (t.cuda() for t in make_inputs(63, B, H, W, h, hd, 1, torch.float16, kind="self"))
    with pytest.raises(RuntimeError):          # scratch too small
        ma.match_attention(mo, q, k, v, H, W, 1, 0.25, strategy=BINNED, workspace=small)
    assert ma.workspace_bytes(B, H, W, h, hd, 1, torch.float16) > 0
    assert ma.workspace_bytes(B, H, W, h, hd, 1, torch.float32) == 0


SORTED, SORTED_MMA = 3, 4


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("knobs", [dict(strategy=SORTED), dict(strategy=SORTED_MMA), dict(variant=2), dict(variant=3)],
                         ids=["sorted-scalar", "sorted-matrix", "matrix-4-items", "matrix-2-items"])
@pytest.mark.parametrize("case", CASES + [(1, 40, 44, 8, 16, "flow", 6.0, True), (2, 30, 28, 4, 32, "self", 3.0, True)])
def test_opt_in_kernels_match_oracle_and_direct(case, knobs, dtype):
    """The other ways of running the same operator -- queries walked in sorted order, float32 sums on
    the matrix instructions (four or two items per lane) -- against the oracle and the default kernel."""
    import oracle
    B, H, W, h, hd, kind, spread, per_head = case
    inputs = make_inputs(50 + H + hd, B, H, W, h, hd, 1, dtype, kind=kind, spread=spread, border_frac=0.2,
                         per_head=per_head)
    ref_out, ref_attn = oracle.forward(*inputs, H, W, 1, hd ** -0.5)
    out, attn = _run(inputs, H, W, hd, **knobs)
    ties = hd > 16
    assert_close(attn, ref_attn, dtype, "attn", ties=ties)
    assert_close(out, ref_out, dtype, "out", ties=ties)
    d_out, d_attn = _run(inputs, H, W, hd, strategy=1)
    assert_close(attn, d_attn, dtype, "attn vs direct", ties=ties)
    assert_close(out, d_out, dtype, "out vs direct", ties=ties)


def test_matrix_kernel_row_band():
    B, H, W, h, hd = 2, 45, 38, 4, 16
    mo, q, k, v = make_inputs(64, B, H, W, h, hd, 1, torch.float16, kind="flow", spread=6.0)
    full_out, full_attn = _run((mo, q, k, v), H, W, hd, variant=3)
    r0, r1 = 7, 30
    sl = slice(r0 * W, r1 * W)
    out, attn = _run((mo[:, sl].contiguous(), q[:, sl].contiguous(), k, v), H, W, hd, variant=3,
                     q_row_begin=r0, q_row_end=r1)
    assert torch.equal(out, full_out[:, sl]) and torch.equal(attn, full_attn[:, sl])
