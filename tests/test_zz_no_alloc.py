"""GPU test of matchattn_fused_forward_static, the entry point for callers that may not
allocate device memory (its scratch is a fixed area inside the library).  Called through
the C ABI with ctypes; the result is compared with the plain matchattn_fused_forward on
the same inputs, for two calls in a row with different inputs (the second call finds the
first call's leftovers in the shared scratch area and must not be disturbed by them).

The file name sorts last on purpose: a run that stops at the first failure has then
already been through every other test."""
import ctypes

import pytest
import torch

from _cases import assert_close, make_inputs

pytestmark = pytest.mark.gpu

F16 = 1


def _lib():
    from matchattention_b200 import _lib as binding
    return binding


def _call(fn, mo, q, k, v, out, attn, B, H, W, h, hd, *extra):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(mo.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), attn.data_ptr(),
              B, H, W, h, hd, 1, 1, F16, 0, float(hd ** -0.5), 0, H, stream, *extra)


def test_static_scratch_entry_matches_the_plain_entry_twice_in_a_row():
    binding = _lib()
    lib = binding.lib
    rounds = [
        # B, H, W, h, hd, seed, spread : the second call is smaller than the first, so most of the
        # scratch still holds the first call's histogram, cursors and sorted records
        (2, 96, 80, 8, 16, 71, 20.0),
        (1, 40, 52, 4, 32, 72, 6.0),
    ]
    for B, H, W, h, hd, seed, spread in rounds:
        mo, q, k, v = (t.cuda() for t in make_inputs(seed, B, H, W, h, hd, 1, torch.float16, kind="flow",
                                                     spread=spread, border_frac=0.15))
        want_out, want_attn = torch.empty_like(q), q.new_empty(B, H * W, h, 16)
        got_out = torch.full_like(q, float("nan"))
        got_attn = torch.full((B, H * W, h, 16), float("nan"), dtype=q.dtype, device=q.device)
        binding.check(_call(lib.matchattn_fused_forward, mo, q, k, v, want_out, want_attn, B, H, W, h, hd))
        binding.check(_call(lib.matchattn_fused_forward_static, mo, q, k, v, got_out, got_attn, B, H, W, h, hd))
        torch.cuda.synchronize()
        ties = hd > 16
        assert_close(got_attn, want_attn, torch.float16, "attn", ties=ties)
        assert_close(got_out, want_out, torch.float16, "out", ties=ties)


def test_static_scratch_entry_refuses_what_does_not_fit():
    """Sizes are checked before anything is launched, so the buffers can be tiny."""
    binding = _lib()
    lib = binding.lib
    tiny = torch.zeros(64, dtype=torch.float16, device="cuda")
    B, H, W, h, hd = 8, 384, 384, 8, 16            # needs about 14 MB of scratch, the area holds 8 MiB
    assert lib.matchattn_workspace_bytes(B, H, W, h, hd, 1, F16, 0, H) > (8 << 20)
    rc = _call(lib.matchattn_fused_forward_static, tiny, tiny, tiny, tiny, tiny, tiny, B, H, W, h, hd)
    assert rc == 10 and "scratch" in binding.strerror(rc)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.matchattn_fused_forward_static(tiny.data_ptr(), tiny.data_ptr(), tiny.data_ptr(), tiny.data_ptr(),
                                            tiny.data_ptr(), tiny.data_ptr(), 1, 16, 16, 2, 16, 1, 1, 0, 0, 1.0, 0, 16,
                                            stream)     # float32: the binned path does not cover it
    assert rc == 9
    torch.cuda.synchronize()
