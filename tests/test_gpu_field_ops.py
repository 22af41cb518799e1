"""GPU tests of the consistency-mask and local-disparity kernels through the library: against the C
oracle on the golden inputs and on larger seeded inputs, and -- where the reference's Python code is
present -- against the reference's own functions run on the same GPU (the strictest check: same
PyTorch build, same arithmetic)."""
import pytest
import torch

from _cases import golden_names_with_prefix, load_golden_arrays, ulp16

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _ma():
    import matchattention_b200
    return matchattention_b200


def _close16(got, ref, dt, ulps=1.0):
    g, r = got.float().cpu(), ref.float().cpu()
    if dt == torch.float32:
        return bool(((g - r).abs() <= 1e-4 * r.abs().clamp_min(1.0)).all())
    return bool(((g - r).abs() <= ulps * ulp16(r, dt)).all())


@pytest.mark.parametrize("name", golden_names_with_prefix("consistency_"))
def test_consistency_mask_kernel_matches_oracle(name):
    import oracle
    c = load_golden_arrays(name)
    want_mask, want_diff = oracle.consistency_mask(c["field"], c["threshold"])
    mask, diff = _ma().consistency_mask(c["field"].cuda(), c["threshold"], return_diff=True)
    torch.cuda.synchronize()
    assert _close16(diff, want_diff, c["dtype"]), name
    decided = (want_diff.float() - c["threshold"]).abs() > 2 * ulp16(want_diff.float(), torch.float16)
    assert torch.equal(mask.cpu()[decided], want_mask[decided])


@pytest.mark.parametrize("dtype", DTYPES)
def test_consistency_mask_kernel_on_a_large_field(dtype):
    import oracle
    g = torch.Generator().manual_seed(5)
    field = (torch.randn(2, 96, 128, 2, generator=g) * 3).to(dtype)
    want_mask, want_diff = oracle.consistency_mask(field)
    mask, diff = _ma().consistency_mask(field.cuda(), return_diff=True)
    assert _close16(diff, want_diff, dtype)
    decided = (want_diff.float() - 2).abs() > 2 * ulp16(want_diff.float(), torch.float16)
    assert torch.equal(mask.cpu()[decided], want_mask[decided])
    assert torch.equal(_ma().consistency_mask(field.cuda()), mask)


@pytest.mark.parametrize("name", golden_names_with_prefix("disparity_"))
def test_local_disparity_kernel_matches_oracle(name):
    import oracle
    c = load_golden_arrays(name)
    dt = c["dtype"]
    want_flow, want_blur, want_centre = oracle.local_disparity(c["volume"])
    flow, blur, centre = _ma().local_disparity_estimator(c["volume"].cuda(), return_debug=True)
    torch.cuda.synchronize()
    assert _close16(blur, want_blur, dt)
    clear = c["gap"] > (1e-6 if dt == torch.float32 else 0.0)
    assert torch.equal(centre.cpu()[clear], want_centre[clear])
    assert _close16(flow.cpu()[clear], want_flow[clear], dt)
    assert (flow[..., 1] == 0).all()


def _reference():
    from oracle import ref_loader
    if not ref_loader.available():
        pytest.skip("the reference's Python code is not present (oracle/make_ref.py places it under oracle/_ref/)")
    return ref_loader.import_reference()


@pytest.mark.parametrize("dtype", DTYPES)
def test_consistency_mask_kernel_matches_reference_on_the_gpu(dtype):
    _, blocks = _reference()
    g = torch.Generator().manual_seed(6)
    field = (torch.randn(2, 96, 128, 2, generator=g) * 3).to(dtype).cuda()
    want = blocks.MatchAttentionLayer.consistency_mask(None, field)
    mask, diff = _ma().consistency_mask(field, return_diff=True)
    decided = (diff.float() - 2).abs() > 2 * ulp16(diff.float().cpu(), torch.float16).cuda()
    assert decided.float().mean() > 0.95
    assert torch.equal(mask[decided], want[decided])
    mismatch = (mask != want).float().mean().item()
    assert mismatch < 2e-3, f"{mismatch:.2e} of the mask differs from the reference"


@pytest.mark.parametrize("dtype", DTYPES)
def test_local_disparity_kernel_matches_reference_on_the_gpu(dtype):
    _reference()
    from models.cost_volume import local_disparity_estimator
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(7)
    B, D, H, W = 2, 48, 48, 48
    vol = torch.softmax(torch.randn(B, D, H, W, generator=g) * 2.0, dim=1).to(dtype).cuda()
    want = local_disparity_estimator(vol.clone())
    flow = _ma().local_disparity_estimator(vol)
    blur = F.avg_pool1d(vol.permute(0, 2, 3, 1).reshape(B, -1, D), kernel_size=5, stride=1, padding=2).float()
    top2 = blur.topk(2, dim=-1).values
    clear = ((top2[..., 0] - top2[..., 1]) > (1e-6 if dtype == torch.float32 else 0.0)).view(B, H, W)
    assert clear.float().mean() > 0.5
    assert _close16(flow[..., 0][clear], want[..., 0][clear], dtype)
    assert (flow[..., 1] == 0).all()


@pytest.mark.parametrize("name", golden_names_with_prefix("flowinit_"))
def test_flow_init_kernels_match_oracle(name):
    import oracle
    c = load_golden_arrays(name)
    dt, H, W = c["dtype"], c["H"], c["W"]
    want_flow, want_prob, want_blur, want_centre = oracle.flow_init(c["correlation"], H, W)
    flow, prob, blur, centre = _ma().flow_init(c["correlation"].cuda(), H, W, return_debug=True)
    torch.cuda.synchronize()
    assert _close16(prob, want_prob, dt) and _close16(blur, want_blur, dt)
    clear = c["gap"] > (1e-6 if dt == torch.float32 else 0.0)
    assert torch.equal(centre.cpu()[clear], want_centre[clear])
    assert _close16(flow.cpu().view(-1, H * W, 2)[clear], want_flow.view(-1, H * W, 2)[clear], dt, ulps=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,W", [(12, 16), (9, 37)])
def test_flow_init_kernels_match_reference_on_the_gpu(dtype, H, W):
    """The reference's GlobalCorrelation.forward(stereo=False) on the same GPU against the kernels, fed with
    the correlation the module itself computes."""
    _reference()
    from models.cost_volume import GlobalCorrelation
    import torch.nn.functional as F
    torch.manual_seed(11)
    B, C = 1, 32
    mod = GlobalCorrelation(C).eval().cuda().to(dtype)
    x = (torch.randn(2 * B, H, W, C) * 8).cuda().to(dtype)
    with torch.inference_mode():
        xn = mod.norm(x)
        ref, tgt = xn.chunk(2, dim=0)
        corr = torch.matmul(mod.q(ref).view(B, -1, C), mod.k(tgt).view(B, -1, C).transpose(-2, -1)) * mod.scale
        want_flow, want_prob = mod(x, stereo=False)
        blur = F.avg_pool2d(want_prob.view(2 * B, H * W, H * W), kernel_size=5, stride=1, padding=2).float()
    flow, prob = _ma().flow_init(corr, H, W)
    assert _close16(prob, want_prob, dtype)
    top2 = blur.topk(2, dim=-1).values
    clear = ((top2[..., 0] - top2[..., 1]) > (1e-6 if dtype == torch.float32 else 0.0)).view(2 * B, H, W)
    assert clear.float().mean() > 0.5
    assert _close16(flow[clear], want_flow[clear], dtype, ulps=2.0)
