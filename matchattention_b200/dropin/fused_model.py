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
  out-of-view fill -> ``stereo_volume``; the matmul before and the local
  disparity estimator after stay the reference's;
* ``MatchAttentionLayer.consistency_mask`` (models/attention_blocks.py:130-138)
  -> ``consistency_mask``.

:func:`unpatch_reference_model` removes the instance attributes again.
"""
from __future__ import annotations

import types

import torch

from .. import ops


def _attention_forward(self, x, max_offset, noc_mask=None):
    B, H, W, _ = x.shape
    N = H * W
    r = self.win_r[0]
    x = x.view(B, N, -1)
    if self.cross:
        # keys/values of a view come from the other view: project once, swap the batch halves after
        q, g = self.q(x), self.g(x)
        k, v = self.k(x).roll(B // 2, 0), self.v(x).roll(B // 2, 0)
        y = ops.cross_attention_core(max_offset, q, k, v, g, H, W, r, self.scale, clamp=True)
    else:
        if self.noc_embed:
            x = torch.cat((x, noc_mask.view(B, N, -1)), dim=-1)
        q, k, v = self.q(x), self.k(x), self.v(x)
        y = ops.self_attention_core(max_offset, q, k, v, H, W, r, self.scale, clamp=True)
    return self.proj_drop(self.proj(y)).view(B, H, W, -1)


def _upsample_field(self, field, mask, factor):
    return ops.upsample_field(field, mask, factor)


def _consistency_mask(self, field, A=2):
    return ops.consistency_mask(field, float(A))


def _make_correlation_forward(reference_forward, local_disparity_estimator):
    def forward(self, x, stereo=True):
        if not stereo or x.shape[2] > ops.STEREO_VOLUME_MAX_W:
            return reference_forward(x, stereo=stereo)
        x = self.norm(x)
        ref, tgt = x.chunk(2, dim=0)
        correlation = torch.matmul(self.q(ref), self.k(tgt).transpose(-2, -1)) * self.scale
        volume = ops.stereo_volume(correlation)
        return local_disparity_estimator(volume), volume
    return forward


def patch_reference_model(model, *, attention: bool = True, upsample: bool = True, volume: bool = True,
                          consistency: bool = True):
    """Rebind the listed steps of a reference ``MatchStereo`` instance to this library's kernels."""
    import sys
    for m in model.modules():
        name = type(m).__name__
        if attention and name == "MatchAttention":
            if any(p > 0 for p in (m.attn_drop.p, m.proj_drop.p)) and m.training:
                continue                                   # dropout on the attention weights: keep the reference path
            m.forward = types.MethodType(_attention_forward, m)
        elif upsample and name == "MatchStereo":
            m.upsample_field = types.MethodType(_upsample_field, m)
        elif consistency and name == "MatchAttentionLayer" and hasattr(ops, "consistency_mask"):
            m.consistency_mask = types.MethodType(_consistency_mask, m)
        elif volume and name == "GlobalCorrelation":
            estimator = getattr(sys.modules[type(m).__module__], "local_disparity_estimator")
            m.forward = types.MethodType(_make_correlation_forward(m.forward, estimator), m)
    return model


def unpatch_reference_model(model):
    for m in model.modules():
        for attr in ("forward", "upsample_field", "consistency_mask"):
            if attr in m.__dict__:
                del m.__dict__[attr]
    return model
