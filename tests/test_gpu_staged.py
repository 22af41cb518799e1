"""GPU tests of the staged path (strategy 5: per tile of queries the K / V region its windows fall into
is copied to shared memory by the tensor memory accelerator, completion on an mbarrier; tiles whose windows
spread too far are served by global loads in the same launch) through the C ABI: against the oracle and
against the direct kernel, with smooth centres (tiles staged), random centres (every tile falls back),
centres outside the map, odd map sizes, row bands and the head counts / widths the path covers."""
import pytest
import torch

from _cases import assert_close, make_inputs

pytestmark = pytest.mark.gpu
STAGED = 5            # persistent form: producer warp + 24 consumer warps, one block per SM
STAGED_BLOCKS = 6     # one block per tile
STRATEGIES = [STAGED, STAGED_BLOCKS]

CASES = [
    # B, H, W, h, hd, kind, spread, per_head
    (2, 48, 64, 8, 16, "self", 3.0, True),        # self attention: one centre per head, small offsets
    (1, 40, 44, 8, 16, "flow", 2.0, False),       # smooth shared centres, odd tile edges
    (2, 33, 29, 8, 16, "flow", 20.0, False),      # random centres: no tile fits, all served by global loads
    (1, 37, 41, 4, 16, "self", 3.0, True),
    (1, 30, 31, 2, 8, "self", 2.0, True),
    (2, 20, 21, 16, 8, "flow", 1.5, False),
    (1, 19, 50, 1, 16, "self", 3.0, True),
    (1, 24, 31, 8, 8, "raw", 2.0, False),         # centres far outside the map: border clamping inside a region
    (1, 4, 4, 8, 16, "raw", 2.0, False),          # smallest map
    (1, 96, 128, 8, 16, "cross", 16.0, False),    # disparity-like: some tiles fit, some do not
]


def _run(inputs, H, W, hd, **kw):
    import matchattention_b200 as ma
    mo, q, k, v = (t.cuda() for t in inputs)
    out, attn = ma.match_attention(mo, q, k, v, H, W, 1, hd ** -0.5, **kw)
    torch.cuda.synchronize()
    return out.cpu(), (attn.cpu() if attn is not None else None)


@pytest.mark.parametrize("strategy", STRATEGIES, ids=["persistent", "blocks"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
def test_staged_matches_oracle_and_direct(case, dtype, strategy):
    import oracle
    B, H, W, h, hd, kind, spread, per_head = case
    inputs = make_inputs(70 + H + hd, B, H, W, h, hd, 1, dtype, kind=kind, spread=spread, border_frac=0.05,
                         per_head=per_head)
    ref_out, ref_attn = oracle.forward(*inputs, H, W, 1, hd ** -0.5)
    out, attn = _run(inputs, H, W, hd, strategy=strategy)
    assert_close(attn, ref_attn, dtype, "attn")
    assert_close(out, ref_out, dtype, "out")
    d_out, d_attn = _run(inputs, H, W, hd, strategy=1)
    assert_close(attn, d_attn, dtype, "attn vs direct")
    assert_close(out, d_out, dtype, "out vs direct")
    same = (out.view(torch.int16) == d_out.view(torch.int16)).float().mean().item()
    assert same > 0.999, f"only {same:.4%} of out is bit-identical to the direct kernel"


@pytest.mark.parametrize("strategy,tile_h", [(STAGED, 6), (STAGED_BLOCKS, 8)], ids=["persistent", "blocks"])
def test_staged_tiles_are_really_staged(strategy, tile_h):
    """The 64-bit status word in the workspace counts the tiles that fell back to global loads: none for
    smooth centres away from the borders, all of them for centres spread over tens of tokens; its top bit (a
    wait that ran out) stays clear."""
    import matchattention_b200 as ma
    B, H, W, h, hd = 1, 64, 64, 8, 16
    tiles = (W // 16) * ((H + tile_h - 1) // tile_h)
    for spread, border, expect in ((2.0, 0.0, 0), (30.0, 0.0, tiles)):
        inputs = make_inputs(81, B, H, W, h, hd, 1, torch.float16, kind="flow", spread=spread, border_frac=border)
        mo, q, k, v = (t.cuda() for t in inputs)
        ws = torch.full((8,), 0xff, dtype=torch.uint8, device="cuda")
        ma.match_attention(mo, q, k, v, H, W, 1, 0.25, strategy=strategy, workspace=ws)
        torch.cuda.synchronize()
        count = int(ws.view(torch.int64).item())
        assert count == expect, f"spread {spread}: status {count}, expected {expect} of {tiles} tiles falling back"


@pytest.mark.parametrize("strategy", STRATEGIES, ids=["persistent", "blocks"])
def test_staged_row_band_and_skipped_attn(strategy):
    B, H, W, h, hd = 2, 45, 38, 8, 16
    mo, q, k, v = make_inputs(82, B, H, W, h, hd, 1, torch.float16, kind="self", spread=3.0, per_head=True)
    full_out, full_attn = _run((mo, q, k, v), H, W, hd, strategy=strategy)
    r0, r1 = 7, 30
    sl = slice(r0 * W, r1 * W)
    out, attn = _run((mo[:, sl].contiguous(), q[:, sl].contiguous(), k, v), H, W, hd, strategy=strategy,
                     q_row_begin=r0, q_row_end=r1)
    assert torch.equal(out, full_out[:, sl]) and torch.equal(attn, full_attn[:, sl])
    out2, none = _run((mo, q, k, v), H, W, hd, strategy=strategy, need_attn=False)
    assert none is None and torch.equal(out2, full_out)


def test_staged_rejects_what_it_does_not_cover():
    import matchattention_b200 as ma
    for h, hd, r, dtype in ((8, 16, 1, torch.float32), (4, 32, 1, torch.float16), (8, 16, 2, torch.float16),
                            (3, 16, 1, torch.float16)):
        mo, q, k, v = (t.cuda() for t in make_inputs(83, 1, 16, 16, h, hd, r, dtype, kind="self"))
        for strategy in STRATEGIES:
            with pytest.raises(RuntimeError):
                ma.match_attention(mo, q, k, v, 16, 16, r, 0.25, strategy=strategy)
