"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE.

Usage (only where the reference checkout exists; it is imported, not copied):

    python tests/golden/make_golden.py [--ref /path/to/MatchAttention]

Each .npz holds seeded inputs and the outputs of the reference's own functions
(models/mat_pytorch_impl.py, driven exactly as models/attention_blocks.py:79-91
drives them) on those inputs.  bfloat16 arrays are stored as their int16 bit
patterns (numpy has no bfloat16); the key ``dtype`` says how to read them.

The files are derived artefacts: the tests compare the CPU oracle and the CUDA
kernels with them, so that parity is checked even where the reference is not
installed.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.ref_loader import import_reference, install_timm_shim, reference_op  # noqa: E402,F401


def reference_clamp(blocks, max_offset, H, W, r):
    fake_self = types.SimpleNamespace(win_r=[r, r])
    return blocks.MatchAttention.clamp_max_offset(fake_self, max_offset, H, W)


def grid_xy(B, H, W, h):
    ys, xs = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
    g = torch.stack((xs, ys), dim=-1).view(1, H * W, 1, 2)
    return g.repeat(B, 1, h, 1)


def to_np(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def save_case(name, dtype, H, W, h, r, scale, mo, q, k, v, out, attn, note):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(
        path, dtype=str(dtype).replace("torch.", ""), H=H, W=W, h=h, r=r, scale=np.float64(scale),
        max_offset=to_np(mo), q=to_np(q), k=to_np(k), v=to_np(v), out=to_np(out), attn=to_np(attn), note=note)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def synthetic_cases(impl, blocks):
    specs = [
        # name, seed, B, H, W, h, hd, r, kind
        ("raw_r1", 11, 2, 6, 7, 2, 8, 1, "raw"),
        ("raw_r2", 12, 1, 7, 9, 3, 8, 2, "raw"),
        ("cross_r1", 13, 1, 13, 26, 8, 16, 1, "cross"),
        ("self_r1", 14, 1, 13, 26, 8, 16, 1, "self"),
        ("model_r2_hd40", 15, 2, 8, 10, 4, 40, 2, "self"),
        ("model_r1_hd32", 16, 2, 9, 12, 4, 32, 1, "cross"),
    ]
    for name, seed, B, H, W, h, hd, r, kind in specs:
        gen = torch.Generator().manual_seed(seed)
        N, C = H * W, h * hd
        q32, k32, v32 = (torch.randn(B, N, C, generator=gen) for _ in range(3))
        grid = grid_xy(B, H, W, h)
        if kind == "raw":          # centres anywhere, also outside the map; never clamped
            rel = torch.empty(B, N, h, 2).uniform_(-1.0, 1.0, generator=gen)
            rel = rel * torch.tensor([W * 0.75, H * 0.75])
            mo32 = grid + rel
            integral = torch.rand(B, N, h, 1, generator=gen) < 0.15   # some exactly integral centres
            mo32 = torch.where(integral, torch.round(mo32), mo32)
        elif kind == "cross":      # disparity-like, the same for every head (attention_blocks.py:162)
            rel_x = torch.empty(B, N, 1, 1).uniform_(-16.0, 0.0, generator=gen).repeat(1, 1, h, 1)
            mo32 = grid + torch.cat((rel_x, torch.zeros_like(rel_x)), dim=-1)
        else:                      # per-head small offsets
            mo32 = grid + torch.empty(B, N, h, 2).uniform_(-3.0, 3.0, generator=gen)
        scale = hd ** -0.5
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            mo = mo32.to(dtype)
            if kind != "raw":
                mo = reference_clamp(blocks, mo, H, W, r)
            q, k, v = q32.to(dtype), k32.to(dtype), v32.to(dtype)
            out, attn = reference_op(impl, mo, q, k, v, H, W, h, r, scale)
            tag = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[dtype]
            save_case(f"{name}_{tag}", dtype, H, W, h, r, scale, mo, q, k, v, out, attn,
                      f"seed {seed}, kind {kind}, reference mat_pytorch_impl on CPU")


def wide_head_cases(impl, blocks):
    """Head widths of the small and base model variants (64, 80, 128) and beyond, where the float32 sum
    of a score is no longer exact: small maps, float32 / float16 / bfloat16."""
    sys.path.insert(0, os.path.dirname(HERE))
    from _cases import make_inputs
    specs = [
        # name, seed, B, H, W, h, hd, r, kind
        ("wide_hd64_r1", 51, 1, 11, 13, 4, 64, 1, "flow"),
        ("wide_hd80_r2", 52, 1, 9, 10, 4, 80, 2, "raw"),
        ("wide_hd128_r1", 53, 1, 8, 9, 2, 128, 1, "raw"),
        ("wide_hd256_r1", 54, 1, 6, 7, 2, 256, 1, "flow"),
    ]
    for name, seed, B, H, W, h, hd, r, kind in specs:
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            mo, q, k, v = make_inputs(seed, B, H, W, h, hd, r, dtype, kind=kind, spread=W / 3, per_head=True,
                                      border_frac=0.2)
            scale = hd ** -0.5
            out, attn = reference_op(impl, mo, q, k, v, H, W, h, r, scale)
            tag = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[dtype]
            save_case(f"{name}_{tag}", dtype, H, W, h, r, scale, mo, q, k, v, out, attn,
                      f"_cases.make_inputs(seed {seed}, kind {kind}, spread W/3, per_head, border_frac 0.2), "
                      "reference mat_pytorch_impl on CPU")


def sampled_full_size_cases(impl):
    """The CPU-runnable configuration at full size (B=1, 104x208 tokens, 8 heads x 16, r=1; cross and self
    offsets; float32 and float16).  Inputs are regenerated from the seed by tests/_cases.make_inputs (a
    SHA-256 of their bytes is stored to catch a generator that changed); of the reference's outputs every
    26th query is stored, which keeps a file below a megabyte."""
    import hashlib
    sys.path.insert(0, os.path.dirname(HERE))
    from _cases import make_inputs
    B, H, W, h, hd, r, stride = 1, 104, 208, 8, 16, 1, 26
    for kind, seed, spread in (("cross", 61, 16.0), ("self", 62, 3.0)):
        for dtype in (torch.float32, torch.float16):
            mo, q, k, v = make_inputs(seed, B, H, W, h, hd, r, dtype, kind=kind, spread=spread, border_frac=0.0,
                                      per_head=(kind == "self"))
            out, attn = reference_op(impl, mo, q, k, v, H, W, h, r, hd ** -0.5)
            digest = hashlib.sha256(b"".join(to_np(t).tobytes() for t in (mo, q, k, v))).hexdigest()
            idx = torch.arange(0, H * W, stride)
            tag = {torch.float32: "f32", torch.float16: "f16"}[dtype]
            path = os.path.join(HERE, f"sampled_config0_{kind}_{tag}.npz")
            np.savez_compressed(path, dtype=str(dtype).replace("torch.", ""), B=B, H=H, W=W, h=h, hd=hd, r=r,
                                seed=seed, kind=kind, spread=spread, scale=np.float64(hd ** -0.5),
                                inputs_sha256=digest, query_index=idx.numpy(), out=to_np(out[:, idx]),
                                attn=to_np(attn[:, idx]),
                                note="reference mat_pytorch_impl on CPU at full size; every 26th query stored")
            print(f"sampled_config0_{kind}_{tag}: {os.path.getsize(path) / 1024:.0f} KiB")


def model_cases(ref_root, impl):
    """Inputs captured from MatchAttention calls inside a MatchStereo-tiny forward
    (random-init weights, seeded noise images), one self and one cross call per
    stage; batch item 0 only, cast to float16; expected = reference op in float16."""
    from models.match_stereo import MatchStereo
    from models.attention_blocks import MatchAttention
    torch.manual_seed(21)
    args = types.SimpleNamespace(variant="tiny", mat_impl="pytorch")
    model = MatchStereo(args).eval()
    captured = []

    def hook(mod, inputs):
        x, max_offset = inputs[0], inputs[1]
        B, H, W, _ = x.shape
        N = H * W
        xx = x.view(B, N, -1)
        if mod.cross:
            a, b = xx.chunk(2, dim=0)
            ref, tgt = torch.cat((a, b), 0), torch.cat((b, a), 0)
        else:
            if mod.noc_embed:
                xx = torch.cat((xx, inputs[2].view(B, N, -1)), dim=-1)
            ref, tgt = xx, xx
        q, k, v = mod.q(ref), mod.k(tgt), mod.v(tgt)
        mo = mod.clamp_max_offset(max_offset, H, W)
        captured.append(dict(cross=mod.cross, H=H, W=W, h=mod.num_head, r=mod.win_r[0], scale=mod.scale,
                             mo=mo.detach(), q=q.detach(), k=k.detach(), v=v.detach()))

    for m in model.modules():
        if isinstance(m, MatchAttention):
            m.register_forward_pre_hook(hook)
    img0 = torch.rand(1, 3, 192, 192) * 255
    img1 = torch.roll(img0, shifts=-5, dims=-1) + torch.randn(1, 3, 192, 192) * 2
    with torch.inference_mode():
        model(img0, img1, stereo=True)
    print(f"captured {len(captured)} MatchAttention calls")
    seen = set()
    for idx, c in enumerate(captured):
        key = (c["H"], c["cross"])
        if key in seen:
            continue
        # take the LAST layer of each stage instead of the first: fields have moved by then
        last = max(i for i, d in enumerate(captured) if (d["H"], d["cross"]) == key)
        c = captured[last]
        seen.add(key)
        sl = slice(0, 1)
        mo, q, k, v = (c[n][sl].to(torch.float16).contiguous() for n in ("mo", "q", "k", "v"))
        out, attn = reference_op(impl, mo, q, k, v, c["H"], c["W"], c["h"], c["r"], c["scale"])
        kind = "cross" if c["cross"] else "self"
        save_case(f"stereo_tiny_{c['H']}x{c['W']}_{kind}_f16", torch.float16, c["H"], c["W"], c["h"], c["r"],
                  c["scale"], mo, q, k, v, out, attn,
                  f"call {last} of a MatchStereo-tiny forward at 192x192, torch seed 21, batch item 0, cast to f16")


def upsample_cases(ref_root):
    """MatchStereo.upsample_field (models/match_stereo.py:73-84) on seeded inputs, factors 2 and 4."""
    from models.match_stereo import MatchStereo
    for name, seed, B, H, W, D, factor in (("upsample_f2", 31, 2, 7, 9, 2, 2), ("upsample_f4", 32, 1, 6, 5, 2, 4),
                                           ("upsample_f2_d8", 33, 1, 5, 6, 8, 2)):
        gen = torch.Generator().manual_seed(seed)
        field32 = torch.randn(B, H, W, D, generator=gen) * 3
        mask32 = torch.randn(B, 9 * factor * factor, H, W, generator=gen) * 2
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            field, mask = field32.to(dtype), mask32.to(dtype)
            out = MatchStereo.upsample_field(None, field, mask, factor)
            tag = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[dtype]
            path = os.path.join(HERE, f"{name}_{tag}.npz")
            np.savez_compressed(path, dtype=str(dtype).replace("torch.", ""), factor=factor, field=to_np(field),
                                mask=to_np(mask), out=to_np(out),
                                note=f"seed {seed}, MatchStereo.upsample_field of the reference on CPU")
            print(f"{name}_{tag}: {os.path.getsize(path) / 1024:.0f} KiB")


def volume_cases(ref_root):
    """GlobalCorrelation.forward, stereo branch (models/cost_volume.py:17-55): the correlation the module
    computes from its input (lines 18-24, recomputed here with the module's own layers) and the cost volume
    it returns (lines 26-51: masking, diagonal shifts, softmax over disparity, out-of-view fill)."""
    from models.cost_volume import GlobalCorrelation
    for name, seed, B, H, W, C in (("volume_w12", 41, 1, 5, 12, 16), ("volume_w20", 42, 2, 3, 20, 8)):
        torch.manual_seed(seed)
        mod = GlobalCorrelation(C).eval()
        x32 = torch.randn(2 * B, H, W, C) * 2
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            m = mod.to(dtype)
            x = x32.to(dtype)
            with torch.inference_mode():
                xn = m.norm(x)
                ref, tgt = xn.chunk(2, dim=0)
                corr = torch.matmul(m.q(ref), m.k(tgt).transpose(-2, -1)) * m.scale
                _, volume = m(x, stereo=True)
            tag = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[dtype]
            path = os.path.join(HERE, f"{name}_{tag}.npz")
            np.savez_compressed(path, dtype=str(dtype).replace("torch.", ""), correlation=to_np(corr.contiguous()),
                                volume=to_np(volume.contiguous()),
                                note=f"seed {seed}, GlobalCorrelation(dim={C}) of the reference on CPU, stereo=True")
            print(f"{name}_{tag}: {os.path.getsize(path) / 1024:.0f} KiB")


def field_op_cases(ref_root, blocks):
    """MatchAttentionLayer.consistency_mask (models/attention_blocks.py:130-138) and
    local_disparity_estimator (models/cost_volume.py:123-178) on seeded inputs.  Besides the reference's
    outputs the files hold the continuous quantity behind each discrete decision (the thresholded
    field difference; the gap between the best and the second-best blurred probability), so that a test
    can gate the decision only where it is not a tie."""
    from models.cost_volume import local_disparity_estimator
    from utils.utils import bilinear_sample_by_offset, init_coords
    import torch.nn.functional as F
    tags = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}
    for name, seed, B, H, W, amp in (("consistency_a", 71, 2, 11, 14, 2.5), ("consistency_b", 72, 4, 9, 23, 6.0)):
        gen = torch.Generator().manual_seed(seed)
        field32 = torch.randn(B, H, W, 2, generator=gen) * amp
        for dtype in tags:
            field = field32.to(dtype)
            mask = blocks.MatchAttentionLayer.consistency_mask(None, field)
            # the quantity the reference thresholds (same statements, models/attention_blocks.py:131-136)
            offset = field + init_coords(field)
            a, b = field.chunk(2, dim=0)
            tgt = torch.cat((b, a), dim=0)
            warped = bilinear_sample_by_offset(tgt.permute(0, 3, 1, 2).contiguous(), offset).permute(0, 2, 3, 1)
            diff = torch.abs(field + warped).sum(dim=-1, keepdim=True)
            path = os.path.join(HERE, f"{name}_{tags[dtype]}.npz")
            np.savez_compressed(path, dtype=str(dtype).replace("torch.", ""), field=to_np(field), mask=to_np(mask),
                                diff=to_np(diff.contiguous()), threshold=2.0,
                                note=f"seed {seed}, MatchAttentionLayer.consistency_mask of the reference on CPU")
            print(f"{name}_{tags[dtype]}: {os.path.getsize(path) / 1024:.0f} KiB")
    for name, seed, B, D, H, W, sharp in (("disparity_a", 81, 2, 24, 7, 24, 3.0), ("disparity_b", 82, 4, 40, 5, 40, 1.0)):
        gen = torch.Generator().manual_seed(seed)
        vol32 = torch.softmax(torch.randn(B, D, H, W, generator=gen) * sharp, dim=1)
        for dtype in tags:
            vol = vol32.to(dtype)
            flow = local_disparity_estimator(vol.clone())
            blur = F.avg_pool1d(vol.permute(0, 2, 3, 1).reshape(B, -1, D), kernel_size=5, stride=1, padding=2)
            top2 = blur.float().topk(2, dim=-1).values
            path = os.path.join(HERE, f"{name}_{tags[dtype]}.npz")
            np.savez_compressed(path, dtype=str(dtype).replace("torch.", ""), volume=to_np(vol), flow=to_np(flow),
                                blur_max=to_np(blur.max(-1).values.view(B, H, W).contiguous()),
                                gap=(top2[..., 0] - top2[..., 1]).view(B, H, W).numpy(),
                                note=f"seed {seed}, local_disparity_estimator of the reference on CPU")
            print(f"{name}_{tags[dtype]}: {os.path.getsize(path) / 1024:.0f} KiB")


def flow_init_cases(ref_root):
    """GlobalCorrelation.forward with stereo=False (models/cost_volume.py:56-69, local_flow_estimator :71-121):
    the scaled correlation the module computes (recomputed here with its own layers) and what it returns."""
    from models.cost_volume import GlobalCorrelation
    import torch.nn.functional as F
    tags = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}
    for name, seed, B, H, W, C, gain in (("flowinit_a", 91, 1, 6, 7, 16, 6.0), ("flowinit_b", 92, 2, 5, 9, 8, 12.0)):
        torch.manual_seed(seed)
        mod = GlobalCorrelation(C).eval()
        x32 = torch.randn(2 * B, H, W, C) * gain
        for dtype in tags:
            m, x = mod.to(dtype), x32.to(dtype)
            with torch.inference_mode():
                xn = m.norm(x)
                ref, tgt = xn.chunk(2, dim=0)
                corr = torch.matmul(m.q(ref).view(B, -1, C), m.k(tgt).view(B, -1, C).transpose(-2, -1)) * m.scale
                flow, prob = m(x, stereo=False)
                blur = F.avg_pool2d(prob.view(2 * B, H * W, H * W), kernel_size=5, stride=1, padding=2)
            top2 = blur.float().topk(2, dim=-1).values
            path = os.path.join(HERE, f"{name}_{tags[dtype]}.npz")
            np.savez_compressed(path, dtype=str(dtype).replace("torch.", ""), H=H, W=W,
                                correlation=to_np(corr.contiguous()), flow=to_np(flow.contiguous()),
                                prob=to_np(prob.contiguous()), blur_max=to_np(blur.max(-1).values.contiguous()),
                                gap=(top2[..., 0] - top2[..., 1]).numpy(),
                                note=f"seed {seed}, GlobalCorrelation(dim={C}) of the reference on CPU, stereo=False")
            print(f"{name}_{tags[dtype]}: {os.path.getsize(path) / 1024:.0f} KiB")


def backward_cases(impl):
    """Gradients that autograd gives for the reference's 'pytorch' path (float32, CPU): of
    sum(out * g_out) + sum(attn * g_attn) with seeded g_out, g_attn, with respect to q, k, v and max_offset."""
    sys.path.insert(0, os.path.dirname(HERE))
    from _cases import make_inputs
    for name, seed, B, H, W, h, hd, r, kind in (("backward_r1", 101, 1, 9, 11, 2, 8, 1, "flow"),
                                                ("backward_r2", 102, 2, 7, 8, 3, 16, 2, "self")):
        mo, q, k, v = make_inputs(seed, B, H, W, h, hd, r, torch.float32, kind=kind, spread=3.0, border_frac=0.2,
                                  per_head=True)
        gen = torch.Generator().manual_seed(seed + 1)
        g_out = torch.randn(q.shape, generator=gen)
        g_attn = torch.randn(B, H * W, h, (2 * r + 2) ** 2, generator=gen)
        leaves = [t.clone().requires_grad_(True) for t in (mo, q, k, v)]
        out, attn = reference_op(impl, *leaves, H, W, h, r, hd ** -0.5)
        ((out * g_out).sum() + (attn * g_attn).sum()).backward()
        path = os.path.join(HERE, name + "_f32.npz")
        np.savez_compressed(path, dtype="float32", H=H, W=W, h=h, r=r, scale=np.float64(hd ** -0.5),
                            max_offset=mo.numpy(), q=q.numpy(), k=k.numpy(), v=v.numpy(), g_out=g_out.numpy(),
                            g_attn=g_attn.numpy(), d_max_offset=leaves[0].grad.numpy(), d_q=leaves[1].grad.numpy(),
                            d_k=leaves[2].grad.numpy(), d_v=leaves[3].grad.numpy(),
                            note=f"seed {seed}, autograd over the reference's mat_pytorch_impl on CPU")
        print(f"{name}_f32: {os.path.getsize(path) / 1024:.0f} KiB")


def dot_product_cases(impl):
    """Dot-product scoring.  The reference has it only in its native kernel
    (models/src/match_former_fused_forward.cu:222-251), with no PyTorch counterpart, so PARITY IS UNPINNED
    for this scoring: the vectors come from the reference's own functions with the one scoring line
    (models/mat_pytorch_impl.py:74) swapped for the product form, on the keys gathered with the indices the
    reference's compute_match_attention returns."""
    sys.path.insert(0, os.path.dirname(HERE))
    from _cases import make_inputs
    for name, seed, B, H, W, h, hd, r, kind in (("dot_r1", 111, 2, 9, 11, 4, 16, 1, "flow"),
                                                ("dot_r2", 112, 1, 8, 9, 2, 24, 2, "raw")):
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            mo, q, k, v = make_inputs(seed, B, H, W, h, hd, r, dtype, kind=kind, spread=3.0, border_frac=0.2,
                                      per_head=True)
            # unit-scale scores, so that the 16-bit softmax is not saturated
            q, k = (q * 0.5).to(dtype), (k * 0.5).to(dtype)
            scale = hd ** -0.5
            N, M = H * W, (2 * r + 2) ** 2
            qh, kh, vh = (t.view(B, N, h, hd) for t in (q, k, v))
            m_id = torch.floor(mo).to(torch.int32)
            wgt = impl.compute_bilinear_weights(mo)
            _, idx = impl.compute_match_attention(qh, kh, m_id, [r, r], H, W)
            k_sampled = torch.gather(kh.unsqueeze(3).expand(-1, -1, -1, M, -1), dim=1, index=idx)
            score = (qh.unsqueeze(3) * k_sampled).sum(dim=-1)
            attn = impl.compute_bilinear_softmax(score * scale, wgt, [r, r])
            out = impl.attention_aggregate(vh, attn, idx, [r, r])
            tag = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[dtype]
            save_case(f"{name}_{tag}", dtype, H, W, h, r, scale, mo, q, k, v, out, attn,
                      f"seed {seed}, kind {kind}; dot-product scoring restated (parity unpinned), the rest is the "
                      "reference's mat_pytorch_impl on CPU")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("MATCHATTN_REF"), required="MATCHATTN_REF" not in os.environ,
                    help="checkout of the reference project (or set MATCHATTN_REF)")
    ap.add_argument("--skip-model", action="store_true")
    ap.add_argument("--only-upsample", action="store_true", help="regenerate only the upsample_field vectors")
    ap.add_argument("--only-new", action="store_true", help="only the wide-head and sampled full-size operator vectors")
    ap.add_argument("--only-field-ops", action="store_true", help="only the consistency-mask and disparity vectors")
    ap.add_argument("--only-dot", action="store_true", help="only the dot-product scoring vectors")
    a = ap.parse_args()
    impl, blocks = import_reference(a.ref)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    if a.only_dot:
        dot_product_cases(impl)
        return
    if a.only_field_ops:
        field_op_cases(a.ref, blocks)
        flow_init_cases(a.ref)
        backward_cases(impl)
        return
    if a.only_new:
        wide_head_cases(impl, blocks)
        sampled_full_size_cases(impl)
        return
    if not a.only_upsample:   # (the flag also regenerates the cost-volume vectors)
        synthetic_cases(impl, blocks)
        wide_head_cases(impl, blocks)
        sampled_full_size_cases(impl)
        if not a.skip_model:
            model_cases(a.ref, impl)
    upsample_cases(a.ref)
    volume_cases(a.ref)
    field_op_cases(a.ref, blocks)
    flow_init_cases(a.ref)
    backward_cases(impl)
    dot_product_cases(impl)


if __name__ == "__main__":
    main()
