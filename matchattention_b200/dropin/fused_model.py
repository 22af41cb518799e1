"""Run an already-built reference model on the fused kernels of this library.

``install_dropin()`` alone swaps the operator behind ``--mat_impl cuda`` and
changes nothing else.  :func:`patch_reference_model` goes one step further for
callers who want the steps either side of the operator fused as well.  It
rebinds methods on the model INSTANCE (no reference file is edited, no reference
module is imported here: modules are recognised by their class names):

* ``MatchAttention.forward`` (models/attention_blocks.py:61-101): the q/k/v/g
  and output projections stay ``nn.Linear``; clamp, operator, gate and the
  ``cat((g*x, attn))`` layout become one kernel (``cross_attention_core``); the
  self branch never writes the attention weights it discards
  (``self_attention_core``);
* ``MatchStereo.upsample_field`` (models/match_stereo.py:73-84) -> ``upsample_field``;
* ``GlobalCorrelation.forward``, stereo branch (models/cost_volume.py:17-55):
  the masks, the two loops over the disparities, the softmax and the
  out-of-view fill -> ``stereo_volume``, the estimator after it
  (models/cost_volume.py:123-178) -> ``local_disparity_estimator``; the flow
  branch (:56-69 with local_flow_estimator :71-121) -> ``flow_init``; the matmul
  before them stays cuBLAS;
* ``MatchAttentionLayer.consistency_mask`` (models/attention_blocks.py:130-138)
  -> ``consistency_mask``.

:func:`unpatch_reference_model` removes the instance attributes again.
"""
from __future__ import annotations

import types

import torch

from .. import ops


def _kernels(traceable: bool):
    """The six fused steps: plain functions (eager) or their opaque custom-op forms (torch.compile)."""
    if traceable:
        return types.SimpleNamespace(
            cross=ops.cross_attention_core_op, self_=ops.self_attention_core_op, upsample=ops.upsample_field_op,
            volume=ops.stereo_volume_op, mask=ops.consistency_mask_op, disparity=ops.local_disparity_op,
            flow_init=ops.flow_init_op)
    return types.SimpleNamespace(
        cross=ops.cross_attention_core, self_=ops.self_attention_core, upsample=ops.upsample_field,
        volume=ops.stereo_volume, mask=ops.consistency_mask, disparity=ops.local_disparity_estimator,
        flow_init=ops.flow_init)


def _make_attention_forward(kn):
    def forward(self, x, max_offset, noc_mask=None):
        B, H, W, _ = x.shape
        N = H * W
        r = self.win_r[0]
        x = x.view(B, N, -1)
        if self.cross:
            # keys/values of a view come from the other view: project the batch as it is, the kernel
            # reads item (b + B/2) mod B (no copy of K and V)
            q, g, k, v = self.q(x), self.g(x), self.k(x), self.v(x)
            y = kn.cross(max_offset, q, k, v, g, H, W, r, self.scale, True, B // 2)
        else:
            if self.noc_embed:
                x = torch.cat((x, noc_mask.view(B, N, -1)), dim=-1)
            q, k, v = self.q(x), self.k(x), self.v(x)
            y = kn.self_(max_offset, q, k, v, H, W, r, self.scale, True)
        return self.proj_drop(self.proj(y)).view(B, H, W, -1)
    return forward


def _make_upsample_field(kn):
    def upsample_field(self, field, mask, factor):
        return kn.upsample(field, mask, factor)
    return upsample_field


def _make_consistency_mask(kn):
    def consistency_mask(self, field, A=2):
        return kn.mask(field, float(A))
    return consistency_mask


def _make_correlation_forward(kn, reference_forward):
    def forward(self, x, stereo=True):
        B2, H, W, C = x.shape
        if (stereo and W > ops.STEREO_VOLUME_MAX_W) or (not stereo and (H < 5 or W < 5)):
            return reference_forward(x, stereo=stereo)
        x = self.norm(x)
        ref, tgt = x.chunk(2, dim=0)
        ref, tgt = self.q(ref), self.k(tgt)
        if stereo:
            correlation = torch.matmul(ref, tgt.transpose(-2, -1)) * self.scale
            volume = kn.volume(correlation)
            return kn.disparity(volume), volume
        correlation = torch.matmul(ref.reshape(B2 // 2, H * W, C), tgt.reshape(B2 // 2, H * W, C).transpose(-2, -1)) * self.scale
        flow, prob = kn.flow_init(correlation, H, W)
        return flow, prob
    return forward


def patch_reference_model(model, *, attention: bool = True, upsample: bool = True, volume: bool = True,
                          consistency: bool = True, traceable: bool = False):
    """Rebind the listed steps of a reference ``MatchStereo`` instance to this library's kernels.
    ``traceable=True`` goes through the opaque custom-op forms so that ``torch.compile`` can trace the
    model around them."""
    kn = _kernels(traceable)
    unpatch_reference_model(model)
    for m in model.modules():
        name = type(m).__name__
        if attention and name == "MatchAttention":
            if any(p > 0 for p in (m.attn_drop.p, m.proj_drop.p)) and m.training:
                continue                                   # dropout on the attention weights: keep the reference path
            m.forward = types.MethodType(_make_attention_forward(kn), m)
        elif upsample and name == "MatchStereo":
            m.upsample_field = types.MethodType(_make_upsample_field(kn), m)
        elif consistency and name == "MatchAttentionLayer":
            m.consistency_mask = types.MethodType(_make_consistency_mask(kn), m)
        elif volume and name == "GlobalCorrelation":
            m.forward = types.MethodType(_make_correlation_forward(kn, m.forward), m)
    return model


def unpatch_reference_model(model):
    for m in model.modules():
        for attr in ("forward", "upsample_field", "consistency_mask"):
            if attr in m.__dict__:
                del m.__dict__[attr]
    return model
