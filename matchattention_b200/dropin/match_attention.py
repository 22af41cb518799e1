"""Stand-in for the reference's compiled extension module ``match_attention``.

The reference calls ``match_attention.fused_forward(max_offset, q, k, v, output,
attn_out, H, W, win_r, attn_num, attn_type, scale)`` (models/match_former_ops.py:29-33;
the pybind definition is models/src/match_former_cuda.cpp:41-44).  Putting this
directory on ``sys.path`` (or calling ``matchattention_b200.install_dropin()``)
makes that import resolve here, so the unmodified reference model runs on the
B200 kernel when started with ``--mat_impl cuda``.
"""
from matchattention_b200.ops import fused_forward  # noqa: F401

__all__ = ["fused_forward"]
