"""One process driving two GPUs: the kernels that opt in to large dynamic shared memory (the binned
path behind matchattn_fused_forward_ws / _static, the stereo cost volume) must work on the second
device too -- that opt-in is a per-device attribute of a kernel.  Skipped below two GPUs."""
import pytest
import torch

from _cases import assert_close, make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_large_shared_memory_kernels_on_a_second_device():
    import matchattention_b200 as ma
    from matchattention_b200 import _lib as binding
    B, H, W, h, hd = 1, 40, 44, 8, 16
    inputs = make_inputs(91, B, H, W, h, hd, 1, torch.float16, kind="flow", spread=6.0)
    corr = (torch.randn(1, 6, 120, 120) * 3).half()          # W = 120: 116 KB of shared memory
    results = []
    for index in (0, 1):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            mo, q, k, v = (t.to(dev) for t in inputs)
            direct = ma.match_attention(mo, q, k, v, H, W, 1, hd ** -0.5, strategy=1)
            binned = ma.match_attention(mo, q, k, v, H, W, 1, hd ** -0.5, strategy=2)
            out, attn = torch.empty_like(q), q.new_empty(B, H * W, h, 16)
            binding.check(binding.lib.matchattn_fused_forward_static(
                mo.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), attn.data_ptr(),
                B, H, W, h, hd, 1, 1, 1, 0, float(hd ** -0.5), 0, H, torch.cuda.current_stream().cuda_stream))
            vol = ma.stereo_volume(corr.to(dev))
            torch.cuda.synchronize()
            assert torch.equal(binned[1], direct[1]) and torch.equal(attn, direct[1])
            assert_close(binned[0], direct[0], torch.float16, f"binned vs direct on cuda:{index}")
            assert_close(out, direct[0], torch.float16, f"static vs direct on cuda:{index}")
            results.append((direct[0].cpu(), vol.cpu()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
