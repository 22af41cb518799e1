"""CPU tests of the boundary: the shared library loads, exports every symbol the
header declares, validates arguments before touching a device, and the Python
host layer refuses CPU tensors.  No kernel is launched here."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "matchattn.h")).read()
    return sorted(set(re.findall(r"MATCHATTN_API\s+[\w\s\*]+?\b(matchattn_\w+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    from matchattention_b200 import _lib
    assert declared_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol():
    from matchattention_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert _lib.lib.matchattn_version() >= 100
    assert _lib.strerror(0) == "ok"


def test_arguments_are_rejected_on_the_host():
    """Every one of these returns before any CUDA call, so they run without a GPU."""
    from matchattention_b200 import _lib
    f = _lib.lib.matchattn_fused_forward
    p = ctypes.c_void_p(4096)   # never dereferenced

    def call(mo=p, q=p, k=p, v=p, out=p, attn=p, B=1, H=8, W=8, h=2, hd=16, rx=1, ry=1, dtype=1, attn_type=0,
             scale=1.0, r0=0, r1=8):
        return f(mo, q, k, v, out, attn, B, H, W, h, hd, rx, ry, dtype, attn_type, scale, r0, r1, None)

    assert call(q=None) == 1
    assert call(B=0) == 2 and call(r0=5, r1=5) == 2 and call(r1=9) == 2
    assert call(H=3, r1=3) == 3
    assert call(dtype=7) == 4
    assert call(attn_type=2) == 5
    assert call(rx=1, ry=2) == 6 and call(rx=5, ry=5, H=32, W=32, r1=32) == 6
    assert call(q=ctypes.c_void_p(4097)) == 7
    assert call(B=70000) == 8
    for code in (1, 2, 3, 4, 5, 6, 7, 8):
        assert _lib.strerror(code) not in ("ok", "unknown status")


def test_block_copy_arguments_are_checked_on_the_host():
    """matchattn_copy_blocks: an empty list is fine, a negative count or a missing array or pointer is
    refused before any CUDA call."""
    from matchattention_b200 import _lib
    f = _lib.lib.matchattn_copy_blocks
    none = ctypes.POINTER(ctypes.c_void_p)()
    assert f(none, none, ctypes.POINTER(ctypes.c_size_t)(), 0, 0, None) == 0
    assert f(none, none, ctypes.POINTER(ctypes.c_size_t)(), -1, 0, None) == 1
    assert f(none, none, ctypes.POINTER(ctypes.c_size_t)(), 2, 1, None) == 1
    dst, src = (ctypes.c_void_p * 2)(4096, None), (ctypes.c_void_p * 2)(8192, 8192)
    sizes = (ctypes.c_size_t * 2)(0, 64)              # the first block is empty and skipped, the second lacks a target
    assert f(dst, src, sizes, 2, 0, None) == 1


def test_dispatch_table():
    from matchattention_b200 import describe_dispatch
    assert describe_dispatch(8, 16, 1, torch.float16) == "fast cpl=2 lph=1"
    assert describe_dispatch(8, 16, 1, torch.float16, aligned32=False) == "generic"
    assert describe_dispatch(4, 8, 1, torch.float16, aligned32=False) == "fast cpl=1 lph=1"
    assert describe_dispatch(4, 40, 2, torch.bfloat16) == "fast cpl=5 lph=1"
    assert describe_dispatch(4, 128, 1, torch.float32) == "fast cpl=4 lph=4"
    assert describe_dispatch(4, 12, 1, torch.float32) == "generic"
    assert describe_dispatch(4, 16, 3, torch.float32) == "generic"


def test_cpu_tensors_are_refused():
    from matchattention_b200 import match_attention
    t = torch.zeros(1, 64, 16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        match_attention(torch.zeros(1, 64, 2, 2), t, t, t, 8, 8, 1, 1.0)
