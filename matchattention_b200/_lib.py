"""ctypes binding of libmatchattn_b200.so (the C ABI in include/matchattn.h).

The library is loaded from matchattention_b200/lib/.  There is no fallback: if
it is missing, importing this module raises, and so does every op.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libmatchattn_b200.so")

# every symbol include/matchattn.h declares
EXPORTS = ("matchattn_fused_forward", "matchattn_fused_forward_ex", "matchattn_fused_forward_ws",
           "matchattn_fused_forward_static", "matchattn_fused_forward_glue", "matchattn_fused_forward_checked",
           "matchattn_fused_backward", "matchattn_upsample_field",
           "matchattn_stereo_volume", "matchattn_consistency_mask", "matchattn_local_disparity",
           "matchattn_flow_init", "matchattn_flow_init_scratch_bytes", "matchattn_copy_blocks",
           "matchattn_workspace_bytes", "matchattn_describe_dispatch", "matchattn_version", "matchattn_strerror")

F32, F16, BF16 = 0, 1, 2
L1_NORM = 0
DOT_PRODUCT = 1
ATTN_TYPE_CODE = {"l1_norm": L1_NORM, "dot_product": DOT_PRODUCT}

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA library first with "
            "`python -m matchattention_b200.build` (needs nvcc); there is no CPU or PyTorch fallback")
    lib = ctypes.CDLL(LIB_PATH)
    base = [_vp] * 6 + [_i] * 9 + [_f, _i, _i, _vp]
    lib.matchattn_fused_forward.restype = _i
    lib.matchattn_fused_forward.argtypes = base
    lib.matchattn_fused_forward_ex.restype = _i
    lib.matchattn_fused_forward_ex.argtypes = base + [_i, _i, _i, _i]
    lib.matchattn_fused_forward_ws.restype = _i
    lib.matchattn_fused_forward_ws.argtypes = base + [_vp, ctypes.c_size_t, _i]
    lib.matchattn_fused_forward_static.restype = _i
    lib.matchattn_fused_forward_static.argtypes = base
    lib.matchattn_fused_forward_checked.restype = _i
    lib.matchattn_fused_forward_checked.argtypes = [_vp] * 6 + [_i] * 9 + [_f, _i, _i, _vp, _vp]
    lib.matchattn_fused_backward.restype = _i
    lib.matchattn_fused_backward.argtypes = [_vp] * 10 + [_i] * 9 + [_f, _i, _i, _vp]
    lib.matchattn_fused_forward_glue.restype = _i
    lib.matchattn_fused_forward_glue.argtypes = [_vp] * 7 + [_i] * 9 + [_f, _i, _i, _i, ctypes.c_longlong,
                                                 ctypes.c_longlong, _i, _vp]
    lib.matchattn_upsample_field.restype = _i
    lib.matchattn_upsample_field.argtypes = [_vp] * 3 + [_i] * 6 + [_vp]
    lib.matchattn_stereo_volume.restype = _i
    lib.matchattn_stereo_volume.argtypes = [_vp, _vp, _i, _i, _i, _i, _vp]
    lib.matchattn_consistency_mask.restype = _i
    lib.matchattn_consistency_mask.argtypes = [_vp, _vp, _vp, _i, _i, _i, _f, _i, _vp]
    lib.matchattn_local_disparity.restype = _i
    lib.matchattn_local_disparity.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]
    lib.matchattn_flow_init_scratch_bytes.restype = ctypes.c_size_t
    lib.matchattn_flow_init_scratch_bytes.argtypes = [_i, _i, _i]
    lib.matchattn_flow_init.restype = _i
    lib.matchattn_flow_init.argtypes = [_vp] * 6 + [ctypes.c_size_t, _i, _i, _i, _i, _vp]
    lib.matchattn_workspace_bytes.restype = ctypes.c_size_t
    lib.matchattn_workspace_bytes.argtypes = [_i] * 9
    lib.matchattn_describe_dispatch.restype = ctypes.c_char_p
    lib.matchattn_describe_dispatch.argtypes = [_i] * 5
    lib.matchattn_copy_blocks.restype = _i
    lib.matchattn_copy_blocks.argtypes = [ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(ctypes.c_size_t), _i, _i, _vp]
    lib.matchattn_version.restype = _i
    lib.matchattn_version.argtypes = []
    lib.matchattn_strerror.restype = ctypes.c_char_p
    lib.matchattn_strerror.argtypes = [_i]
    return lib


lib = _load()


def strerror(status: int) -> str:
    return lib.matchattn_strerror(int(status)).decode()


def check(status: int) -> None:
    if status != 0:
        raise RuntimeError(f"matchattn_b200: {strerror(status)} (status {status})")
