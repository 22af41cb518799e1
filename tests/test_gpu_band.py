"""GPU test of the row-band path over NCCL and over peer copies: needs at least two GPUs (skipped otherwise).
Each rank is its own process on its own GPU; the result on rank 0 must equal the
single-GPU result bit for bit and match the oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from _cases import make_inputs
        from matchattention_b200 import match_attention
        from matchattention_b200.band import band_match_attention
        B, H, W, h, hd, r = 2, 61, 40, 4, 32, 1
        args = (None, None, None, None)
        if rank == 0:
            args = tuple(t.to(dev) for t in make_inputs(41, B, H, W, h, hd, r, torch.float16, kind="flow", spread=9.0))
        out, attn = band_match_attention(*args, B, H, W, h, hd, r, 0.2, torch.float16, dev)
        torch.cuda.synchronize()
        if rank == 0:
            one_out, one_attn = match_attention(*args, H, W, r, 0.2)
            results.put((bool(torch.equal(out, one_out)), bool(torch.equal(attn, one_attn))))
        dist.barrier()
        # the resident forms: every rank regenerates the same seeded inputs, keeps its own rows of K / V in
        # full-size buffers poisoned elsewhere, exchanges all rows (all-gather) or halo rows only
        from matchattention_b200.band import band_match_attention_resident, band_rows
        H2 = 64                                                   # divisible by 2 and 4: the in-place all-gather path
        mo, q, k, v = (t.to(dev) for t in make_inputs(43, B, H2, W, h, hd, r, torch.float16, kind="flow", spread=3.0,
                                                      border_frac=0.0))
        one_out, one_attn = match_attention(mo, q, k, v, H2, W, r, 0.2)
        r0, r1 = band_rows(H2, world, rank)
        sl = slice(r0 * W, r1 * W)
        ok = True
        for max_dy in (None, 4.0):
            kv = [torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
            kv[0][:, sl], kv[1][:, sl] = k[:, sl], v[:, sl]
            ob, ab = band_match_attention_resident(mo[:, sl].contiguous(), q[:, sl].contiguous(), kv[0], kv[1], H2, W, r,
                                                   0.2, max_abs_dy=max_dy)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(ob, one_out[:, sl])) and bool(torch.equal(ab, one_attn[:, sl]))
        # the same halo rows pulled out of the neighbours' memory by peer copies (buffers mapped into every
        # process), twice (the copy plan is reused), with and without the attention weights
        from matchattention_b200.band import PeerBuffers
        peers = PeerBuffers(B, H2 * W, h * hd, torch.float16, dev)
        for t, src in zip(peers.local, (k, v)):
            t.fill_(float("nan"))
            t[:, sl] = src[:, sl]
        torch.cuda.synchronize()
        dist.barrier()
        for need_attn, by_kernel in ((True, False), (False, True), (True, None)):
            peers.copy_by_kernel = by_kernel        # copy engines / copy kernel with plain peer loads
            ob, ab = band_match_attention_resident(mo[:, sl].contiguous(), q[:, sl].contiguous(), *peers.local, H2, W, r,
                                                   0.2, max_abs_dy=4.0, peers=peers, need_attn=need_attn)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(ob, one_out[:, sl])) and (ab is None or bool(torch.equal(ab, one_attn[:, sl])))
            ok = ok and (ab is None) == (not need_attn)
        # the producers write new rows and the call follows at once on the same stream: the first meeting
        # of the ranks must order every rank's writes before the neighbours' pulls
        for step in range(3):
            k2, v2 = k * (step + 2), v + (step + 1)
            want_out, want_attn = match_attention(mo, q, k2, v2, H2, W, r, 0.2)
            peers.local[0][:, sl], peers.local[1][:, sl] = k2[:, sl], v2[:, sl]
            ob, ab = band_match_attention_resident(mo[:, sl].contiguous(), q[:, sl].contiguous(), *peers.local, H2, W, r,
                                                   0.2, max_abs_dy=4.0, peers=peers)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(ob, want_out[:, sl])) and bool(torch.equal(ab, want_attn[:, sl]))
        results.put(("resident", rank, ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_band_split_over_nccl_equals_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29600 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(rank, world, port, results)) for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    got = [results.get(timeout=5) for _ in range(world + 1)]
    assert (True, True) in got
    assert sorted(g[1] for g in got if g[0] == "resident") == list(range(world))
    assert all(g[2] for g in got if g[0] == "resident")
