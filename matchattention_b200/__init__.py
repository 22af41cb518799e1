"""B200-native MatchAttention operator (hand-written CUDA for sm_100a behind a C ABI).

Public surface:

* ``MF_FusedForwardOps`` / ``fused_forward`` / ``fused_forward_ops`` -- the
  reference's operator interface for this path;
* ``match_attention`` -- functional form with the row-band and skip-attn options;
* ``cross_attention_core`` / ``self_attention_core`` -- the operator with the caller's
  clamp, gate and concatenation folded in;
* ``install_dropin()`` -- makes ``import match_attention`` resolve to this
  implementation so that the unmodified reference model runs on it with
  ``--mat_impl cuda``.

The first use of any of these loads matchattention_b200/lib/libmatchattn_b200.so
and raises if it has not been built (``python -m matchattention_b200.build``);
there is no CPU or PyTorch fallback.  (The load is deferred to first use only so
that the build module itself can be run from a tree without the library.)
"""
import importlib

_OPS = ("MF_FusedForwardOps", "describe_dispatch", "fused_forward", "fused_forward_ops", "launch",
        "match_attention", "workspace_bytes", "cross_attention_core", "self_attention_core", "launch_glue",
        "upsample_field", "stereo_volume", "consistency_mask", "local_disparity_estimator", "flow_init", "match_attention_autograd")
__all__ = list(_OPS) + ["install_dropin", "abi_version"]


def __getattr__(name):
    if name in _OPS:
        return getattr(importlib.import_module(".ops", __name__), name)
    if name in ("ops", "_lib", "band", "build"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def abi_version() -> int:
    from . import _lib
    return int(_lib.lib.matchattn_version())


def install_dropin() -> None:
    """Register this implementation under the module name ``match_attention``, the
    name the reference imports (models/match_former_ops.py:29)."""
    import sys
    from .dropin import match_attention as shim
    sys.modules["match_attention"] = shim
