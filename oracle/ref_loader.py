"""Import the reference's own Python code (TEST INFRASTRUCTURE ONLY).

The reference is looked for in this order: an explicit path, $MATCHATTN_REF,
the unmodified copy that oracle/make_ref.py placed under oracle/_ref/.  Nothing
in the shipped package imports this module.

The reference imports four helpers from ``timm``, which is not installed
anywhere this project runs; :func:`install_timm_shim` provides exactly those
four names (DropPath is never instantiated at drop_path = 0).
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_COPY = os.path.join(HERE, "_ref")


def install_timm_shim() -> None:
    if "timm" in sys.modules:
        return
    import torch
    import torch.nn as nn

    class DropPath(nn.Module):
        def __init__(self, p=0.0):
            super().__init__()

        def forward(self, x):
            return x

    def to_2tuple(x):
        return tuple(x) if isinstance(x, (tuple, list)) else (x, x)

    def register_model(fn):
        return fn

    pkgs = {n: types.ModuleType(n) for n in (
        "timm", "timm.models", "timm.models.layers", "timm.models.layers.helpers", "timm.models.registry")}
    pkgs["timm.models.layers"].DropPath = DropPath
    pkgs["timm.models.layers"].trunc_normal_ = torch.nn.init.trunc_normal_
    pkgs["timm.models.layers.helpers"].to_2tuple = to_2tuple
    pkgs["timm.models.registry"].register_model = register_model
    pkgs["timm"].models = pkgs["timm.models"]
    pkgs["timm.models"].layers = pkgs["timm.models.layers"]
    pkgs["timm.models"].registry = pkgs["timm.models.registry"]
    pkgs["timm.models.layers"].helpers = pkgs["timm.models.layers.helpers"]
    sys.modules.update(pkgs)


def _copy_is_intact() -> bool:
    manifest = os.path.join(REF_COPY, "MANIFEST.json")
    if not os.path.exists(manifest):
        return False
    with open(manifest) as f:
        files = json.load(f).get("files", {})
    for rel, digest in files.items():
        path = os.path.join(REF_COPY, rel)
        if not os.path.exists(path):
            return False
        with open(path, "rb") as g:
            if hashlib.sha256(g.read()).hexdigest() != digest:
                return False
    return bool(files)


def reference_root(explicit: str | None = None) -> str | None:
    """Directory holding the reference's ``models`` and ``utils`` packages, or None."""
    for cand in (explicit, os.environ.get("MATCHATTN_REF")):
        if cand and os.path.isfile(os.path.join(cand, "models", "mat_pytorch_impl.py")):
            return cand
    return REF_COPY if _copy_is_intact() else None


def available() -> bool:
    return reference_root() is not None


def import_reference(explicit: str | None = None):
    """Returns the reference modules (mat_pytorch_impl, attention_blocks); raises if none is found."""
    root = reference_root(explicit)
    if root is None:
        raise ImportError("the reference's Python code is not available: run oracle/make_ref.py where a checkout "
                          "exists (it places an unmodified copy under oracle/_ref/)")
    install_timm_shim()
    if root not in sys.path:
        sys.path.insert(0, root)
    import models.mat_pytorch_impl as impl
    import models.attention_blocks as blocks
    return impl, blocks


def reference_op(impl, max_offset, q, k, v, H, W, h, r, scale):
    """The 'pytorch' branch of MatchAttention.forward (models/attention_blocks.py:82-91, no dropout),
    calling the reference's own five functions."""
    import torch
    B, N, _ = q.shape
    win_r = [r, r]
    m_id = torch.floor(max_offset).to(torch.int32)
    wgt = impl.compute_bilinear_weights(max_offset)
    attn, idx = impl.compute_match_attention(q.view(B, N, h, -1), k.view(B, N, h, -1), m_id, win_r, H, W)
    attn = attn * scale
    attn = impl.compute_bilinear_softmax(attn, wgt, win_r)
    out = impl.attention_aggregate(v.view(B, N, h, -1), attn, idx, win_r)
    return out, attn
