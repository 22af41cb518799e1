"""Backward of the operator.

CPU: the plain-loop restatement of the gradient formulas (oracle/matchattn_backward.py) against the gradients
autograd gives over the reference's own functions (tests/golden/backward_*.npz).
GPU: the CUDA backward, through the autograd function and the reference-compatible module, against the same
vectors, and against autograd over the reference's functions run on the same GPU (float32 and float16)."""
import pytest
import torch

from _cases import golden_names_with_prefix, load_golden_arrays, make_inputs


def _rel(got, ref):
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("name", golden_names_with_prefix("backward_"))
def test_backward_restatement_matches_reference_autograd(name):
    from oracle import matchattn_backward
    c = load_golden_arrays(name)
    got = matchattn_backward.backward(c["max_offset"], c["q"], c["k"], c["v"], c["g_out"], c["g_attn"], c["H"], c["W"],
                                      c["r"], c["scale"])
    for g, key in zip(got, ("d_max_offset", "d_q", "d_k", "d_v")):
        assert _rel(g, c[key]) < 1e-5, key


@pytest.mark.gpu
@pytest.mark.parametrize("name", golden_names_with_prefix("backward_"))
def test_backward_kernel_matches_reference_autograd_vectors(name):
    import matchattention_b200 as ma
    c = load_golden_arrays(name)
    leaves = [c[n].cuda().requires_grad_(True) for n in ("max_offset", "q", "k", "v")]
    out, attn = ma.match_attention_autograd(*leaves, c["H"], c["W"], c["r"], c["scale"])
    ((out * c["g_out"].cuda()).sum() + (attn * c["g_attn"].cuda()).sum()).backward()
    for leaf, key in zip(leaves, ("d_max_offset", "d_q", "d_k", "d_v")):
        assert _rel(leaf.grad, c[key]) < 1e-4, key


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 2e-2)], ids=["f32", "f16"])
@pytest.mark.parametrize("need_attn_grad", [True, False])
def test_backward_kernel_matches_reference_autograd_on_the_gpu(dtype, tol, need_attn_grad):
    """Through MF_FusedForwardOps (the reference's module interface) on a model-like shape; in float16 the
    reference's autograd rounds every intermediate to 16 bits while the kernel works in float32, hence the
    looser bound there."""
    from oracle import ref_loader
    if not ref_loader.available():
        pytest.skip("the reference's Python code is not present (oracle/make_ref.py places it under oracle/_ref/)")
    impl, _ = ref_loader.import_reference()
    import matchattention_b200 as ma
    B, H, W, h, hd, r = 2, 24, 31, 4, 16, 1
    inputs = make_inputs(55, B, H, W, h, hd, r, dtype, kind="flow", spread=5.0, border_frac=0.1, per_head=True)
    g = torch.Generator().manual_seed(56)
    g_out = torch.randn(inputs[1].shape, generator=g).to(dtype).cuda()
    g_attn = torch.randn(B, H * W, h, 16, generator=g).to(dtype).cuda()

    def run(fn):
        leaves = [t.cuda().requires_grad_(True) for t in inputs]
        out, attn = fn(*leaves)
        loss = (out.float() * g_out.float()).sum()
        if need_attn_grad:
            loss = loss + (attn.float() * g_attn.float()).sum()
        loss.backward()
        return [t.grad for t in leaves]

    want = run(lambda mo, q, k, v: ref_loader.reference_op(impl, mo, q, k, v, H, W, h, r, hd ** -0.5))
    module = ma.MF_FusedForwardOps()
    got = run(lambda mo, q, k, v: module(mo, q, k, v, H, W, [r, r], 16, attn_type="l1_norm", scale=hd ** -0.5))
    for gg, ww, key in zip(got, want, ("d_max_offset", "d_q", "d_k", "d_v")):
        assert _rel(gg, ww) < tol, key


@pytest.mark.gpu
def test_inference_path_is_untouched_by_autograd_support():
    import matchattention_b200 as ma
    mo, q, k, v = (t.cuda() for t in make_inputs(57, 1, 12, 13, 2, 16, 1, torch.float16, kind="self"))
    with torch.no_grad():
        out, attn = ma.MF_FusedForwardOps()(mo, q.requires_grad_(True), k, v, 12, 13, [1, 1], 16, scale=0.25)
    assert not out.requires_grad and out.grad_fn is None


@pytest.mark.gpu
@pytest.mark.parametrize("h,hd,r", [(3, 12, 1), (2, 8, 3), (2, 24, 2), (8, 16, 1)],
                         ids=["scalar-hd12", "scalar-r3", "vector-hd24-r2", "vector-hd16-r1"])
def test_backward_kernels_match_the_restatement(h, hd, r):
    """Both CUDA kernels (one element at a time for any head width and radius; eight channels at a time
    for head widths that are multiples of 8 and r <= 2) against the float64 plain-loop restatement."""
    import matchattention_b200 as ma
    from oracle import matchattn_backward
    B, H, W = 1, 9, 10
    mo, q, k, v = make_inputs(57, B, H, W, h, hd, r, torch.float32, kind="flow", spread=3.0, border_frac=0.2,
                              per_head=True)
    gen = torch.Generator().manual_seed(58)
    g_out = torch.randn(q.shape, generator=gen)
    g_attn = torch.randn(B, H * W, h, (2 * r + 2) ** 2, generator=gen)
    want = matchattn_backward.backward(mo, q, k, v, g_out, g_attn, H, W, r, hd ** -0.5)
    leaves = [t.cuda().requires_grad_(True) for t in (mo, q, k, v)]
    out, attn = ma.match_attention_autograd(*leaves, H, W, r, hd ** -0.5)
    ((out * g_out.cuda()).sum() + (attn * g_attn.cuda()).sum()).backward()
    for leaf, ref, key in zip(leaves, want, ("d_max_offset", "d_q", "d_k", "d_v")):
        assert _rel(leaf.grad, ref) < 1e-4, key
