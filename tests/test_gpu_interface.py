"""GPU tests of the reference-facing interface: the 12-argument in-place call,
the opaque custom op, the MF_FusedForwardOps module, the drop-in module name,
streams, CUDA graphs and error reporting."""
import importlib
import sys

import pytest
import torch

from _cases import assert_close, make_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def case():
    import oracle
    B, H, W, h, hd, r = 2, 30, 36, 4, 16, 1
    inputs = make_inputs(21, B, H, W, h, hd, r, torch.float16, kind="flow", spread=5.0)
    ref = oracle.forward(*inputs, H, W, r, 0.25)
    return dict(H=H, W=W, h=h, r=r, M=16, scale=0.25, cpu=inputs, gpu=tuple(t.cuda() for t in inputs), ref=ref)


def test_module_has_reference_signature(case):
    from matchattention_b200 import MF_FusedForwardOps
    mo, q, k, v = case["gpu"]
    out, attn = MF_FusedForwardOps()(mo, q, k, v, case["H"], case["W"], [case["r"]] * 2, case["M"],
                                     attn_type="l1_norm", scale=case["scale"])
    assert out.shape == q.shape and attn.shape == (*q.shape[:2], case["h"], case["M"])
    assert_close(out, case["ref"][0], torch.float16)
    assert_close(attn, case["ref"][1], torch.float16)


def test_dropin_module_name(case):
    import matchattention_b200
    matchattention_b200.install_dropin()
    mod = importlib.import_module("match_attention")
    mo, q, k, v = case["gpu"]
    out = torch.full_like(q, float("nan"))
    attn = torch.full((*q.shape[:2], case["h"], case["M"]), float("nan"), dtype=q.dtype, device=q.device)
    ret = mod.fused_forward(mo, q, k, v, out, attn, case["H"], case["W"], [1, 1], 16, "l1_norm", case["scale"])
    assert ret is None
    assert_close(out, case["ref"][0], torch.float16)
    assert_close(attn, case["ref"][1], torch.float16)
    sys.modules.pop("match_attention", None)


def test_custom_op_is_registered_and_opaque(case):
    import matchattention_b200  # noqa: F401
    mo, q, k, v = case["gpu"]
    out, attn = torch.empty_like(q), q.new_empty(*q.shape[:2], case["h"], 16)
    torch.ops.matchattn_b200.fused_forward_ops(mo, q, k, v, out, attn, case["H"], case["W"], [1, 1], 16, "l1_norm",
                                               case["scale"])
    assert_close(out, case["ref"][0], torch.float16)
    torch.library.opcheck(torch.ops.matchattn_b200.fused_forward_ops.default,
                          (mo, q, k, v, out, attn, case["H"], case["W"], [1, 1], 16, "l1_norm", case["scale"]),
                          test_utils=("test_schema", "test_faketensor"))


def test_side_stream_and_cuda_graph(case):
    from matchattention_b200 import match_attention
    mo, q, k, v = case["gpu"]
    out, attn = torch.empty_like(q), q.new_empty(*q.shape[:2], case["h"], 16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            match_attention(mo, q, k, v, case["H"], case["W"], 1, case["scale"], out=out, attn_out=attn)
        graph = torch.cuda.CUDAGraph()
        out.zero_()
        with torch.cuda.graph(graph, stream=side):
            match_attention(mo, q, k, v, case["H"], case["W"], 1, case["scale"], out=out, attn_out=attn)
        out.zero_()
        graph.replay()
    side.synchronize()
    assert_close(out, case["ref"][0], torch.float16)


def test_bad_arguments_raise_and_leave_the_device_usable(case):
    from matchattention_b200 import match_attention, launch, fused_forward
    mo, q, k, v = case["gpu"]
    H, W = case["H"], case["W"]
    with pytest.raises(RuntimeError):      # CPU tensors: there is no CPU path
        match_attention(*case["cpu"], H, W, 1, 0.25)
    with pytest.raises(ValueError):        # wrong map size
        match_attention(mo, q, k, v, H + 1, W, 1, 0.25)
    with pytest.raises(ValueError):        # non-contiguous input
        match_attention(mo, q.transpose(0, 1).contiguous().transpose(0, 1), k, v, H, W, 1, 0.25)
    with pytest.raises(TypeError):         # mixed dtypes
        match_attention(mo.float(), q, k, v, H, W, 1, 0.25)
    with pytest.raises(NotImplementedError):   # a scoring function that does not exist
        launch(mo, q, k, v, torch.empty_like(q), None, H, W, (1, 1), "l2_norm", 1.0)
    with pytest.raises(RuntimeError):      # rx != ry is rejected by the library
        launch(mo, q, k, v, torch.empty_like(q), None, H, W, (1, 2), "l1_norm", 1.0)
    with pytest.raises(ValueError):        # attn_num inconsistent with win_r
        fused_forward(mo, q, k, v, torch.empty_like(q), q.new_empty(*q.shape[:2], 4, 36), H, W, [1, 1], 36,
                      "l1_norm", 1.0)
    small = make_inputs(3, 1, 3, 8, 2, 8, 1, torch.float16, kind="raw")
    with pytest.raises(RuntimeError):      # window does not fit a 3-row map
        match_attention(*(t.cuda() for t in small), 3, 8, 1, 0.25)
    out, _ = match_attention(mo, q, k, v, H, W, 1, 0.25)
    torch.cuda.synchronize()
    assert_close(out, case["ref"][0], torch.float16)


def test_checked_entry_point_finds_no_stray_index():
    """matchattn_fused_forward_checked: the same results as the plain call, and not one index outside its
    array, on the inputs most likely to produce one: centres far outside the map, NaN, infinities, the
    smallest map that fits the window, odd sizes, the any-shape kernel."""
    import matchattention_b200 as ma
    from _cases import make_inputs
    for B, H, W, h, hd, r, dtype in ((2, 33, 29, 8, 16, 1, torch.float16), (1, 4, 4, 2, 16, 1, torch.float32),
                                     (1, 17, 19, 4, 40, 2, torch.bfloat16), (1, 12, 14, 5, 12, 1, torch.float16)):
        mo, q, k, v = (t.cuda() for t in make_inputs(91, B, H, W, h, hd, r, dtype, kind="raw"))
        mo[0, 0, 0, 0] = float("nan")
        mo[0, 1, 0, 1] = float("inf")
        mo[0, 2, :, :] = -60000.0
        out, attn = torch.empty_like(q), q.new_empty(B, H * W, h, (2 * r + 2) ** 2)
        violations, first = ma.ops.launch_checked(mo, q, k, v, out, attn, H, W, r, hd ** -0.5)
        assert (violations, first) == (0, 0)
        want_out, want_attn = ma.match_attention(mo, q, k, v, H, W, r, hd ** -0.5)
        torch.cuda.synchronize()
        same = lambda a, b: torch.equal(torch.nan_to_num(a.float(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
        assert same(out, want_out) and same(attn, want_attn)
