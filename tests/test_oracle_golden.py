"""CPU tests: the oracle (C and numpy restatements) against the golden vectors
that were produced by running the reference's own Python functions."""
import numpy as np
import pytest
import torch

import oracle
from oracle import matchattn_numpy
from _cases import (assert_close, excess, golden_names, golden_sampled_names, load_golden, load_golden_sampled,
                    make_inputs)


@pytest.mark.parametrize("name", golden_names())
def test_c_oracle_matches_reference_vectors(name):
    c = load_golden(name)
    out, attn = oracle.forward(c["max_offset"], c["q"], c["k"], c["v"], c["H"], c["W"], c["r"], c["scale"])
    assert_close(attn, c["attn"], c["dtype"], name + " attn")
    assert_close(out, c["out"], c["dtype"], name + " out")


@pytest.mark.parametrize("name", golden_sampled_names())
def test_c_oracle_matches_reference_at_full_size(name):
    """The CPU-runnable configuration (104x208 tokens) at full size against the reference's outputs at
    every 26th query."""
    c = load_golden_sampled(name)
    out, attn = oracle.forward(*c["inputs"], c["H"], c["W"], c["r"], c["scale"])
    assert_close(attn[:, c["index"]], c["attn"], c["dtype"], name + " attn")
    assert_close(out[:, c["index"]], c["out"], c["dtype"], name + " out")


@pytest.mark.parametrize("name", golden_names("*_f16") + golden_names("*_bf16"))
def test_c_oracle_16bit_is_nearly_bit_exact(name):
    """The rounding points are those of eager PyTorch: apart from last-bit effects of exp and of
    summation order, the 16-bit oracle output equals the reference's bit for bit."""
    c = load_golden(name)
    out, attn = oracle.forward(c["max_offset"], c["q"], c["k"], c["v"], c["H"], c["W"], c["r"], c["scale"])
    for got, ref in ((out, c["out"]), (attn, c["attn"])):
        differing = (got.view(torch.int16) != ref.view(torch.int16)).float().mean().item()
        assert differing < 5e-3, f"{name}: {differing:.2%} of elements differ"


@pytest.mark.parametrize("name", golden_names("*_f32") + golden_names("*_f16"))
def test_numpy_restatement_matches_reference_vectors(name):
    c = load_golden(name)
    out, attn = matchattn_numpy.forward(c["max_offset"].numpy(), c["q"].numpy(), c["k"].numpy(), c["v"].numpy(),
                                        c["H"], c["W"], c["r"], c["scale"])
    assert_close(torch.from_numpy(attn), c["attn"], c["dtype"], name + " attn")
    assert_close(torch.from_numpy(out), c["out"], c["dtype"], name + " out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("r", [1, 2])
def test_c_and_numpy_agree_on_fresh_inputs(dtype, r):
    mo, q, k, v = make_inputs(5 + r, 2, 9, 11, 3, 16, r, dtype, kind="flow", spread=4.0, border_frac=0.3,
                              per_head=True)
    out_c, attn_c = oracle.forward(mo, q, k, v, 9, 11, r, 0.25)
    out_n, attn_n = matchattn_numpy.forward(mo.numpy(), q.numpy(), k.numpy(), v.numpy(), 9, 11, r, 0.25)
    assert_close(torch.from_numpy(attn_n), attn_c, dtype, "attn")
    assert_close(torch.from_numpy(out_n), out_c, dtype, "out")


def test_attention_rows_sum_to_one():
    mo, q, k, v = make_inputs(3, 1, 12, 14, 4, 8, 2, torch.float32, kind="raw")
    _, attn = oracle.forward(mo, q, k, v, 12, 14, 2, 0.35)
    assert torch.allclose(attn.sum(-1), torch.ones(1, 12 * 14, 4), atol=1e-5)


def test_integral_centre_is_plain_window_softmax():
    """With an integral centre only the nw sub-window has weight: the result is an ordinary softmax
    over the (2r+1)^2 window centred there."""
    H, W, h, hd, r = 8, 9, 2, 8, 1
    mo, q, k, v = make_inputs(4, 1, H, W, h, hd, r, torch.float32, kind="self")
    mo = torch.floor(mo)
    out, attn = oracle.forward(mo, q, k, v, H, W, r, 0.5)
    side = 2 * r + 2
    a = attn.view(1, H * W, h, side, side)
    assert a[..., -1, :].abs().max() == 0 and a[..., :, -1].abs().max() == 0
    n, hh = 31, 1
    x0, y0 = int(mo[0, n, hh, 0]), int(mo[0, n, hh, 1])
    qv = q[0, n, hh * hd:(hh + 1) * hd]
    sc, vals = [], []
    for j in range(-r, r + 1):
        for i in range(-r, r + 1):
            tok = (y0 + j) * W + x0 + i
            sc.append(-(qv - k[0, tok, hh * hd:(hh + 1) * hd]).abs().sum() * 0.5)
            vals.append(v[0, tok, hh * hd:(hh + 1) * hd])
    p = torch.softmax(torch.stack(sc), 0)
    expect = (p[:, None] * torch.stack(vals)).sum(0)
    assert torch.allclose(out[0, n, hh * hd:(hh + 1) * hd], expect, atol=1e-5)


def test_row_band_equals_slice_of_full():
    H, W, h, hd, r = 10, 8, 2, 8, 1
    mo, q, k, v = make_inputs(6, 2, H, W, h, hd, r, torch.float16, kind="flow", spread=3.0)
    out, attn = oracle.forward(mo, q, k, v, H, W, r, 0.3)
    r0, r1 = 3, 7
    sl = slice(r0 * W, r1 * W)
    out_b, attn_b = oracle.forward(mo[:, sl].contiguous(), q[:, sl].contiguous(), k, v, H, W, r, 0.3,
                                   q_row_begin=r0, q_row_end=r1)
    assert torch.equal(out_b, out[:, sl]) and torch.equal(attn_b, attn[:, sl])


def test_oracle_rejects_bad_arguments():
    mo, q, k, v = make_inputs(1, 1, 6, 6, 1, 8, 1, torch.float32, kind="self")
    with pytest.raises(RuntimeError):
        oracle.forward(mo[:, :18].contiguous(), q[:, :18].contiguous(), k[:, :18].contiguous(),
                       v[:, :18].contiguous(), 3, 6, 1, 1.0)   # 2r+2 > H
