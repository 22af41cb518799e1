"""CPU tests of the row-band multi-GPU path: world_size 2 and 3 over gloo.  The band
computation is injected (the CPU oracle), so what is tested is the partition, the
broadcast of K/V, the movement of the band inputs and the reassembly of the outputs."""
import math
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_band_rows_partition():
    from matchattention_b200.band import band_rows
    for H in (1, 2, 7, 96, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            bands = [band_rows(H, world, p) for p in range(world)]
            assert bands[0][0] == 0 and bands[-1][1] == H
            assert all(bands[i][1] == bands[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in bands]
            assert max(sizes) - min(sizes) <= 1


def test_halo_rows_cover_the_window():
    from matchattention_b200.band import halo_rows
    assert halo_rows(100, 0, 50, 1, 0.0) == (0, 54)
    assert halo_rows(100, 50, 100, 2, 3.5) == (44, 100)
    H, r = 64, 1
    for r0, r1, dy in ((10, 20, 2.0), (0, 64, 5.0), (30, 31, 0.4)):
        h0, h1 = halo_rows(H, r0, r1, r, dy)
        lowest = max(0, math.floor(r0 - dy) - r)              # floor(y) - r for the most upward centre
        highest = min(H - 1, math.floor(r1 - 1 + dy) + r + 1)    # floor(y) + r + 1 for the most downward one
        assert h0 <= lowest and h1 > highest


def test_interior_rows_are_exactly_the_rows_that_need_no_halo():
    from matchattention_b200.band import band_rows, halo_rows, interior_rows
    for H in (16, 64, 100, 1024):
        for world in (1, 2, 3, 4, 8):
            for r in (0, 1, 2):
                for dy in (0.0, 0.4, 3.0, 33.0, 200.0):
                    for rank in range(world):
                        r0, r1 = band_rows(H, world, rank)
                        i0, i1 = interior_rows(H, r0, r1, r, dy)
                        assert r0 <= i0 <= i1 <= r1
                        for y in range(r0, r1):
                            g0, g1 = halo_rows(H, y, y + 1, r, dy)
                            assert (i0 <= y < i1) == (g0 >= r0 and g1 <= r1), (H, world, r, dy, rank, y)


def test_halo_copy_plan_moves_exactly_the_reachable_rows():
    """The copy plan of the peer path (pointers and sizes handed to matchattn_copy_blocks), run here with
    host tensors standing in for the mapped buffers of every rank and memmove for the device copies:
    afterwards a rank holds its own rows and its halo rows of every tensor and item, and nothing else."""
    import ctypes
    import types
    from matchattention_b200.band import _halo_copy_plan, band_rows, halo_rows
    B, H, W, C, r = 2, 40, 3, 4, 1
    for world, dy in ((2, 3.0), (4, 2.0), (5, 0.4), (3, 30.0)):
        truth = [torch.arange(B * H * W * C, dtype=torch.float32).view(B, H * W, C) + 1000 * t for t in range(2)]
        buffers = []                                  # buffers[rank][tensor]: own rows valid, the rest NaN
        for rank in range(world):
            r0, r1 = band_rows(H, world, rank)
            mine = [torch.full_like(t, float("nan")) for t in truth]
            for m, t in zip(mine, truth):
                m[:, r0 * W:r1 * W] = t[:, r0 * W:r1 * W]
            buffers.append(mine)
        for rank in range(world):
            fake = types.SimpleNamespace(shape=(B, H * W, C), local=buffers[rank], _plans={},
                                         remote=lambda index, p: buffers[p][index])
            dst, src, nbytes, count, total = _halo_copy_plan(fake, H, W, r, world, rank, dy)
            for i in range(count):
                ctypes.memmove(dst[i], src[i], nbytes[i])
            assert total == sum(nbytes[i] for i in range(count))
        for rank in range(world):
            r0, r1 = band_rows(H, world, rank)
            g0, g1 = halo_rows(H, r0, r1, r, dy)
            for m, t in zip(buffers[rank], truth):
                rows = m.view(B, H, W * C)
                valid = ~torch.isnan(rows).any(dim=2)                       # [B, H]
                want = torch.zeros(H, dtype=torch.bool)
                want[g0:g1] = True
                assert bool((valid == want).all()), (world, dy, rank)
                assert torch.equal(m[:, g0 * W:g1 * W], t[:, g0 * W:g1 * W])


def _worker(rank, world, port, H, W, results, max_abs_dy=None):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from _cases import make_inputs
        from matchattention_b200.band import band_match_attention
        B, h, hd, r = 2, 2, 8, 1
        mo, q, k, v = make_inputs(31, B, H, W, h, hd, r, torch.float16, kind="flow", spread=4.0,
                                  border_frac=0.1 if max_abs_dy is None else 0.0)

        def op(mo_b, q_b, kk, vv, H_, W_, r_, scale, r0, r1, need_attn):
            return oracle.forward(mo_b, q_b, kk, vv, H_, W_, r_, scale, q_row_begin=r0, q_row_end=r1, nthreads=1,
                                  want_attn=need_attn)

        args = (mo, q, k, v) if rank == 0 else (None, None, None, None)
        kv = None
        if max_abs_dy is not None and rank != 0:
            # poison the receive buffers: rows outside the halo must never be read
            kv = [torch.full((B, H * W, h * hd), float("nan"), dtype=torch.float16) for _ in range(2)]
        out, attn = band_match_attention(*args, B, H, W, h, hd, r, 0.3, torch.float16, torch.device("cpu"), op=op,
                                         kv_buffers=kv, max_abs_dy=max_abs_dy)
        if rank == 0:
            ref_out, ref_attn = oracle.forward(mo, q, k, v, H, W, r, 0.3, nthreads=1)
            results.put((bool(torch.equal(out, ref_out)), bool(torch.equal(attn, ref_attn))))
        else:
            assert out is None and attn is None
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H", [(2, 10), (3, 10), (5, 4)])
def test_band_split_reassembles_the_full_result(world, H):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + (os.getpid() + world * 7 + H) % 2000
    procs = [ctx.Process(target=_worker, args=(rank, world, port, H, 8, results)) for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert results.get(timeout=5) == (True, True)


def test_band_split_with_halo_exchange():
    """Offsets of at most 4 rows (the generator's spread): only the reachable K/V rows travel, the
    rest of the receive buffers is NaN, and the result still equals the full one bit for bit."""
    world, H = 3, 30
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + (os.getpid() + 977) % 2000
    procs = [ctx.Process(target=_worker, args=(rank, world, port, H, 8, results, 4.0)) for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert results.get(timeout=5) == (True, True)


# ---- the resident form: every rank holds its own rows of q / max_offset / K / V -------------------------

def _resident_worker(rank, world, port, H, W, results, max_abs_dy, in_place):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from _cases import make_inputs
        from matchattention_b200.band import band_match_attention_resident, band_rows
        B, h, hd, r = 2, 2, 8, 1
        mo, q, k, v = make_inputs(33, B, H, W, h, hd, r, torch.float16, kind="flow", spread=4.0,
                                  border_frac=0.1 if max_abs_dy is None else 0.0)       # same on every rank (seeded)
        r0, r1 = band_rows(H, world, rank)
        sl = slice(r0 * W, r1 * W)

        def op(mo_b, q_b, kk, vv, H_, W_, r_, scale, a, b, need_attn):
            return oracle.forward(mo_b, q_b, kk, vv, H_, W_, r_, scale, q_row_begin=a, q_row_end=b, nthreads=1,
                                  want_attn=need_attn)

        kv = [torch.full((B, H * W, h * hd), float("nan"), dtype=torch.float16) for _ in range(2)]
        if in_place:      # resident layout: the rank's own rows already sit in the full-size buffers
            kv[0][:, sl], kv[1][:, sl] = k[:, sl], v[:, sl]
            kin, vin = kv
        else:
            kin, vin = k[:, sl].contiguous(), v[:, sl].contiguous()
        out, attn = band_match_attention_resident(mo[:, sl].contiguous(), q[:, sl].contiguous(), kin, vin, H, W, r, 0.3,
                                                  op=op, kv_full=kv, max_abs_dy=max_abs_dy)
        ref_out, ref_attn = oracle.forward(mo, q, k, v, H, W, r, 0.3, nthreads=1)
        ok = r1 == r0 or (bool(torch.equal(out, ref_out[:, sl])) and bool(torch.equal(attn, ref_attn[:, sl])))
        if max_abs_dy is None:
            ok = ok and bool(torch.equal(kv[0], k)) and bool(torch.equal(kv[1], v))
        results.put(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("in_place", [False, True], ids=["bands", "resident"])
@pytest.mark.parametrize("world,H,dy", [(2, 10, None), (3, 10, None), (3, 30, 4.0), (4, 16, None)])
def test_resident_bands_equal_the_full_result(world, H, dy, in_place):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + (os.getpid() + 31 * world + H + 500 * in_place) % 2000
    procs = [ctx.Process(target=_resident_worker, args=(rank, world, port, H, 8, results, dy, in_place))
             for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(results.get(timeout=5) for _ in range(world))


# ---- failure paths, all on the host: nothing here faults, traps or hangs a device ------------------------

def _failure_worker(rank, world, port, scenario, results):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=6))
    from matchattention_b200.band import BandArgumentError, band_check
    verdict = "no error"
    try:
        if scenario == "rank_raises":
            # rank 1 fails while preparing its inputs: it reports the error instead of vanishing
            err = ValueError("could not load my band") if rank == 1 else None
            band_check(2, 16, 8, 2, 8, 1, torch.float16, error=err)
        elif scenario == "shape_mismatch":
            band_check(2, 16 if rank == 0 else 18, 8, 2, 8, 1, torch.float16)
        elif scenario == "rank_absent":
            if rank == 1:
                results.put((rank, "left"))
                return                            # never joins the handshake (the process exits between steps)
            band_check(2, 16, 8, 2, 8, 1, torch.float16)
    except BandArgumentError as exc:
        verdict = "BandArgumentError: " + str(exc)
    except Exception as exc:                      # the process group's timeout or the peer's closed connection
        verdict = "transport error: " + type(exc).__name__
    results.put((rank, verdict))
    try:
        dist.destroy_process_group()
    except Exception:
        pass


@pytest.mark.parametrize("scenario", ["rank_raises", "shape_mismatch", "rank_absent"])
def test_band_failures_are_detected_on_the_host(scenario):
    import time
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + (os.getpid() + 611 + len(scenario)) % 2000
    procs = [ctx.Process(target=_failure_worker, args=(rank, world, port, scenario, results)) for rank in range(world)]
    t0 = time.time()
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode is not None, "a rank hung instead of failing"
    got = dict(results.get(timeout=5) for _ in range(world))
    assert time.time() - t0 < 60
    if scenario == "rank_raises":
        assert all(v.startswith("BandArgumentError") and "could not load my band" in v for v in got.values()), got
    elif scenario == "shape_mismatch":
        assert all(v.startswith("BandArgumentError") and "disagree" in v for v in got.values()), got
    else:
        assert got[1] == "left" and got[0].startswith("transport error"), got
