"""B200-native MatchAttention operator (hand-written CUDA for sm_100a behind a C ABI).

Public surface:

* ``MF_FusedForwardOps`` / ``fused_forward`` / ``fused_forward_ops`` -- the
  reference's operator interface for this path;
* ``match_attention`` -- functional form with the row-band and skip-attn options;
* ``install_dropin()`` -- makes ``import match_attention`` resolve to this
  implementation so that the unmodified reference model runs on it with
  ``--mat_impl cuda``.

Importing the package loads matchattention_b200/lib/libmatchattn_b200.so and
fails if it has not been built (``python -m matchattention_b200.build``).
"""
from . import _lib
from .ops import (MF_FusedForwardOps, describe_dispatch, fused_forward, fused_forward_ops, launch,
                  match_attention)

__all__ = ["MF_FusedForwardOps", "fused_forward", "fused_forward_ops", "match_attention", "launch",
           "describe_dispatch", "install_dropin", "abi_version"]


def abi_version() -> int:
    return int(_lib.lib.matchattn_version())


def install_dropin() -> None:
    """Register this implementation under the module name ``match_attention``, the
    name the reference imports (models/match_former_ops.py:29)."""
    import sys
    from .dropin import match_attention as shim
    sys.modules["match_attention"] = shim
