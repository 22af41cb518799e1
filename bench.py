"""Benchmark of the MatchAttention operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the fused operator over one batch of synthetic input.
The default workload is the headline configuration: B=4 items of a 384x384
token map (a 1536x1536 pair at 1/4 resolution), C=128 as 8 heads x 16, 3x3
sub-windows (r=1), float16, flow-like offsets uniform in +-24 tokens shared by
the heads, 10 % of the queries left unclamped next to a border.  With N GPUs
every rank processes its own batch (independent pairs, no collective): weak
scaling.  Rank 0 prints ONE JSON line: the device-resident throughput (`value`,
sustained over at least 0.3 s) with its roofline, the other configuration shapes
(`shapes`), the end-to-end throughput from pinned host buffers (`e2e`, with a
copy-only leg), the reference's own PyTorch path timed on the host cores
(`cpu_baseline`), at one GPU the reference's MatchStereo-T forward with this
library's kernels (`model`, ms per pair), and with several GPUs the row-band
split of one very large pair (`band`).

`--impl reference` times the reference's own CPU implementation of the path (the
unmodified copy under oracle/_ref/, else the C restatement) on the host cores,
on a bounded sample of the same workload.  `--mode` selects the other
measurements (model, model_pairs, model_ops, band, upsample, volume, backward).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch  # noqa: E402

WORKLOADS = {
    # name: B, H, W, h, hd, r, dtype, kind, spread (tokens), border_frac, per_head
    "op_384x384_b4_h8x16_r1_f16_flow": (4, 384, 384, 8, 16, 1, torch.float16, "flow", 24.0, 0.1, False),
    "op_384x384_b4_h8x16_r1_f32_flow": (4, 384, 384, 8, 16, 1, torch.float32, "flow", 24.0, 0.1, False),
    "op_384x384_b4_h8x16_r1_bf16_flow": (4, 384, 384, 8, 16, 1, torch.bfloat16, "flow", 24.0, 0.1, False),
    "op_384x384_b4_h8x16_r1_f16_flow_perhead": (4, 384, 384, 8, 16, 1, torch.float16, "flow", 24.0, 0.1, True),
    "op_384x384_b4_h8x16_r1_f16_smooth": (4, 384, 384, 8, 16, 1, torch.float16, "self", 3.0, 0.0, True),
    "op_384x384_b1_h8x16_r1_f16_flow": (1, 384, 384, 8, 16, 1, torch.float16, "flow", 24.0, 0.1, False),
    "op_384x384_b1_h8x16_r1_f16_smooth": (1, 384, 384, 8, 16, 1, torch.float16, "flow", 3.0, 0.0, False),
    "op_384x384_b1_h8x16_r1_f16_flow_perhead": (1, 384, 384, 8, 16, 1, torch.float16, "flow", 24.0, 0.1, True),
    "op_96x96_b2_h4x32_r2_f16_self": (2, 96, 96, 4, 32, 2, torch.float16, "self", 3.0, 0.0, True),      # 1/16 stage of MatchStereo-T
    "op_48x48_b2_h4x40_r2_f16_self": (2, 48, 48, 4, 40, 2, torch.float16, "self", 3.0, 0.0, True),      # 1/32 stage
    "op_104x208_b1_h8x16_r1_f32_cross": (1, 104, 208, 8, 16, 1, torch.float32, "cross", 16.0, 0.0, False),
}
DEFAULT_WORKLOAD = "op_384x384_b4_h8x16_r1_f16_flow"
DTYPE_NAME = {torch.float16: "f16", torch.float32: "f32", torch.bfloat16: "bf16"}
FALLBACK_HBM_GBS = 6650.0
MIN_REGION_S = 0.3


def algorithmic_bytes_per_query(h, hd, r, esize, with_attn=True):
    """q + k + v + out once each, the offsets, and attn_out: s*(4C + 2h + h*M)."""
    C, M = h * hd, (2 * r + 2) ** 2
    return esize * (4 * C + 2 * h + (h * M if with_attn else 0))


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, MEASURED_PEAKS.json absent)"


def ncu_traffic_per_launch(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's kernel, from the table kept
    beside the ncu summaries (profiles/ncu_traffic.json names the capture each figure comes from); None for
    a workload that was never captured."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            entry = json.load(f).get(workload)
        return float(entry["dram_bytes_per_launch"]) if entry else None
    except Exception:
        return None


class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML (read-only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index, period=0.02):
        self.samples, self.period, self._stop = [], period, threading.Event()
        self.max_mhz, self.ok = None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(index).uuid
            try:
                self.dev = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                mhz = self.nv.nvmlDeviceGetClockInfo(self.dev, self.nv.NVML_CLOCK_SM)
                try:
                    mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.dev)
                except Exception:
                    mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                self.samples.append((time.perf_counter(), mhz, mask))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.ok:
            self.thread.start()

    def stop(self):
        self._stop.set()
        if self.ok:
            self.thread.join(timeout=1.0)

    def summary(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        window = "timed region"
        if len(inside) < 3:
            inside, window = self.samples, "whole run (timed region shorter than 3 samples)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "window": "no samples"}
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside), "window": window}


def bind_to_gpu_cpus(index):
    """Restrict this process to the CPUs NVML reports as local to GPU `index` (a read-only query), so that
    its threads and the pinned buffers they first touch sit on the GPU's NUMA node.  Returns a short
    description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = torch.cuda.get_device_properties(index).uuid
        try:
            handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return "NVML's CPU set for the GPU does not intersect this process's: left unbound"
        os.sched_setaffinity(0, allowed)
        return f"bound to {len(allowed)} CPUs local to the GPU ({min(allowed)}-{max(allowed)})"
    except Exception as exc:
        return f"left unbound ({type(exc).__name__})"


def make_workload(name, seed):
    from _cases import make_inputs
    B, H, W, h, hd, r, dtype, kind, spread, border, per_head = WORKLOADS[name]
    mo, q, k, v = make_inputs(seed, B, H, W, h, hd, r, dtype, kind=kind, spread=spread, border_frac=border,
                              per_head=per_head)
    return dict(B=B, H=H, W=W, h=h, hd=hd, r=r, dtype=dtype, scale=hd ** -0.5, inputs=(mo, q, k, v))


def time_cpu_port(wl, budget_s=8.0, nthreads=0):
    """The oracle port (C restatement) on the host cores over one batch item of the workload, repeated."""
    import oracle
    mo, q, k, v = (t[:1].contiguous() for t in wl["inputs"])
    H, W, r = wl["H"], wl["W"], wl["r"]
    oracle.forward(mo, q, k, v, H, W, r, wl["scale"], nthreads=nthreads)      # warm-up (builds tables)
    reps, t_total = 0, 0.0
    while reps < 3 or (t_total < budget_s and reps < 50):
        t0 = time.perf_counter()
        oracle.forward(mo, q, k, v, H, W, r, wl["scale"], nthreads=nthreads)
        t_total += time.perf_counter() - t0
        reps += 1
    cores = nthreads if nthreads > 0 else oracle.max_threads()
    return H * W * reps / t_total, cores, reps, t_total


def reference_cpu_step(wl):
    """A callable running the reference's own PyTorch path (models/mat_pytorch_impl.py, driven as
    models/attention_blocks.py:82-91 drives it) on the host cores over one batch item of the workload, in
    float32 (PyTorch's CPU kernels for 16-bit types are not what anybody would time), with every host
    thread PyTorch can use.  None when the reference's code is not present."""
    from oracle import ref_loader
    if not ref_loader.available():
        return None, 0
    impl, _ = ref_loader.import_reference()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    mo, q, k, v = (t[:1].float().contiguous() for t in wl["inputs"])
    H, W, h, r, scale = wl["H"], wl["W"], wl["h"], wl["r"], wl["scale"]

    def step():
        with torch.inference_mode():
            return ref_loader.reference_op(impl, mo, q, k, v, H, W, h, r, scale)
    return step, torch.get_num_threads()


def time_cpu_reference(wl, budget_s=12.0):
    step, cores = reference_cpu_step(wl)
    if step is None:
        return None
    step()
    reps, t_total = 0, 0.0
    while reps < 2 or (t_total < budget_s and reps < 20):
        t0 = time.perf_counter()
        step()
        t_total += time.perf_counter() - t0
        reps += 1
    return wl["H"] * wl["W"] * reps / t_total, cores, reps, t_total


def run_reference_arm(args, rank):
    """The reference's CPU implementation of the path on the host cores: its own PyTorch code when the
    unmodified copy under oracle/_ref/ is present, else the C restatement (kind says which)."""
    if rank != 0:
        return
    wl = make_workload(args.workload, 1234)
    H, W, r = wl["H"], wl["W"], wl["r"]
    step, cores = reference_cpu_step(wl)
    kind = "reference"
    what = "models/mat_pytorch_impl.py of the reference (unmodified), float32, torch CPU threads = cores"
    if step is None:
        import oracle
        mo, q, k, v = (t[:1].contiguous() for t in wl["inputs"])
        cores, kind = oracle.max_threads(), "port"
        what = f"C restatement of the reference algorithm, {DTYPE_NAME[wl['dtype']]} rounding points emulated"

        def step():
            return oracle.forward(mo, q, k, v, H, W, r, wl["scale"])
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    value = H * W * steps / dt
    sample = f"one batch item ({H * W} queries) of the workload per step, {steps} steps; {what}"
    line = {"impl": "reference", "metric": "matchattention_queries_per_s", "value": value, "unit": "queries/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt / steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE_NAME[wl["dtype"]],
            "data": "synthetic", "config": config_dict(args.workload, wl),
            "cpu_baseline": {"value": value, "unit": "queries/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def measure_band(rank, world, dev, dist, steps=10, warmup=3):
    """One very large pair split by query row bands (strong scaling): 1024x1024 tokens (a 4096x4096 pair at
    1/4 resolution), B=2 views, 4 heads x 32, float16, smooth flow of at most 32 tokens.  Three ways of getting
    K/V to the ranks, each timed on the device (max over ranks) against the same call on one GPU:
      source_broadcast    rank 0 owns everything: NCCL broadcast of K and V, band inputs scattered, band
                          outputs gathered every step (the form the specification of this mode names)
      resident_allgather  every rank holds its own rows of q/max_offset/K/V and keeps its rows of the outputs:
                          K/V rows all-gathered every step
      resident_halo       same, but only the rows a band can reach (|dy| <= 33 rows) move between neighbours
                          (NCCL send / receive)
      resident_halo_peer  same rows, pulled out of the neighbours' memory over NVLink (the ranks' K/V buffers
                          mapped into every process; no NCCL on the data path): `_copy_engines` by one
                          cudaMemcpyAsync per block, `_copy_kernel` by a copy kernel with plain peer loads,
                          no suffix: the library chooses between the two by the size of the band's interior
    Returns the dict that goes into the JSON line (on rank 0; None elsewhere)."""
    import matchattention_b200 as ma
    from matchattention_b200.band import (PeerBuffers, band_match_attention, band_match_attention_resident, band_rows,
                                          halo_rows)
    B, H, W, h, hd, r, dtype = 2, 1024, 1024, 4, 32, 1, torch.float16
    N, C, M = H * W, h * hd, 16
    scale = hd ** -0.5
    # the same seeded tensors on every rank (generated on the device), so that any rank can slice its band
    g = torch.Generator(device=dev).manual_seed(99)
    q, k, v = (torch.randn(B, N, C, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(3))
    ys, xs = torch.meshgrid(torch.arange(H, device=dev, dtype=torch.float32),
                            torch.arange(W, device=dev, dtype=torch.float32), indexing="ij")
    coarse = (torch.rand(B, 2, 9, 9, generator=g, device=dev) * 2 - 1) * 32.0
    flow = torch.nn.functional.interpolate(coarse, size=(H, W), mode="bilinear", align_corners=True)
    mo = torch.stack((xs + flow[:, 0], ys + flow[:, 1]), dim=-1).view(B, N, 1, 2).expand(B, N, h, 2)
    mo = torch.cat((mo[..., :1].clamp(r, W - 1 - r - 1e-3), mo[..., 1:].clamp(r, H - 1 - r - 1e-3)), -1).to(dtype).contiguous()
    del ys, xs, flow, coarse
    r0, r1 = band_rows(H, world, rank)
    sl = slice(r0 * W, r1 * W)
    bands = [t[:, sl].contiguous() for t in (mo, q)]
    # resident layout: full-size K/V buffers in which only this rank's own rows are valid on entry
    kv_full = [torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
    kv_full[0][:, sl], kv_full[1][:, sl] = k[:, sl], v[:, sl]
    out_band, attn_band = torch.empty_like(bands[1]), q.new_empty(B, (r1 - r0) * W, h, M)
    max_dy = 33.0

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n=steps):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    full_out, full_attn = torch.empty_like(q), q.new_empty(B, N, h, M)
    one_gpu = timed(lambda: ma.match_attention(mo, q, k, v, H, W, r, scale, out=full_out, attn_out=full_attn))
    res = {"workload": "op_1024x1024_b2_h4x32_r1_f16_rowband", "one_gpu_ms": one_gpu, "n_gpus": world,
           "kv_bytes": 2 * B * N * C * 2, "variants": {}}
    if world > 1:
        src_args = (mo, q, k, v) if rank == 0 else (None, None, None, None)
        kv_recv = [k, v] if rank == 0 else kv_full
        esz = 2
        variants = {
            "source_broadcast": (lambda: band_match_attention(*src_args, B, H, W, h, hd, r, scale, dtype, dev,
                                                              kv_buffers=kv_recv),
                                 2 * B * N * C * esz),
            "resident_allgather": (lambda: band_match_attention_resident(*bands, *kv_full, H, W, r, scale,
                                                                         out=out_band, attn_out=attn_band),
                                   2 * B * (N - (r1 - r0) * W) * C * esz),
            "resident_halo": (lambda: band_match_attention_resident(*bands, *kv_full, H, W, r, scale,
                                                                    out=out_band, attn_out=attn_band, max_abs_dy=max_dy),
                              2 * B * ((lambda hr: (hr[1] - hr[0]) - (r1 - r0))(halo_rows(H, r0, r1, r, max_dy))) * W * C * esz),
        }
        halo_bytes = variants["resident_halo"][1]
        peers, peer_note = None, None
        try:        # collective: every rank tries, and all of them drop the variant if one could not map
            peers = PeerBuffers(B, N, C, dtype, dev)
            for t, src in zip(peers.local, (k, v)):
                t.fill_(float("nan"))
                t[:, sl] = src[:, sl]
        except Exception as exc:
            peer_note = "peer mapping unavailable: " + str(exc).splitlines()[0][:200]
        ok_all = torch.tensor([int(peers is not None)], device=dev)
        dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
        if bool(ok_all.item()):
            res["peer_buffers_multicast_bound"] = peers.multicast_bound
            def peer_call(by_kernel):
                def call():
                    peers.copy_by_kernel = by_kernel
                    return band_match_attention_resident(*bands, *peers.local, H, W, r, scale, out=out_band,
                                                         attn_out=attn_band, max_abs_dy=max_dy, peers=peers)
                return call
            variants["resident_halo_peer_copy_engines"] = (peer_call(False), halo_bytes)
            variants["resident_halo_peer_copy_kernel"] = (peer_call(True), halo_bytes)
            variants["resident_halo_peer"] = (peer_call(None), halo_bytes)        # the library's own choice
        else:
            res["resident_halo_peer_note"] = peer_note or "peer mapping unavailable on another rank"
            peers = None
        for name, (fn, recv_bytes) in variants.items():
            ms = timed(fn)
            res["variants"][name] = {"ms": ms, "speedup_vs_one_gpu": one_gpu / ms,
                                     "kv_bytes_received_per_rank": recv_bytes,
                                     "kv_receive_GBps_if_exchange_were_all": recv_bytes / ms / 1e6}
        # the resident forms must reproduce the one-GPU result on the band
        for t, src in zip(kv_full, (k, v)):        # back to "only my rows are valid" before the check
            t.fill_(float("nan"))
            t[:, sl] = src[:, sl]
        band_match_attention_resident(*bands, *kv_full, H, W, r, scale, out=out_band, attn_out=attn_band,
                                      max_abs_dy=max_dy)
        same = torch.equal(out_band, full_out[:, sl]) and torch.equal(attn_band, full_attn[:, sl])
        if peers is not None:
            out_band.zero_()
            attn_band.zero_()
            band_match_attention_resident(*bands, *peers.local, H, W, r, scale, out=out_band, attn_out=attn_band,
                                          max_abs_dy=max_dy, peers=peers)
            same = same and torch.equal(out_band, full_out[:, sl]) and torch.equal(attn_band, full_attn[:, sl])
        ok = torch.tensor([int(same)], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        res["bands_bit_identical_to_one_gpu"] = bool(ok.item())
        best = min(res["variants"].items(), key=lambda kv_: kv_[1]["ms"])
        res["best"] = {"variant": best[0], "ms": best[1]["ms"], "speedup_vs_one_gpu": best[1]["speedup_vs_one_gpu"]}
    return res if rank == 0 else None


def run_band_mode(args, rank, local_rank, world):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = measure_band(rank, world, dev, dist, steps=max(3, min(args.steps, 20)), warmup=max(3, min(args.warmup, 5)))
    if rank == 0:
        ms = res["best"]["ms"] if world > 1 else res["one_gpu_ms"]
        line = {"metric": "matchattention_queries_per_s", "value": 2 * 1024 * 1024 / (ms * 1e-3), "unit": "queries/s",
                "n_gpus": world, "steps": max(3, min(args.steps, 20)), "warmup": max(3, min(args.warmup, 5)),
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic", "config": {"workload": res["workload"], "mode": "row bands"}, "band": res,
                "gpu_launches": max(3, min(args.steps, 20))}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_model_ops_mode(args):
    """The 52 MatchAttention calls of one MatchStereo-T forward at 1536x1536 (both view directions, B=2,
    4 heads): per stage the token map, channel count, window radius and number of layers of the
    reference model; self-attention calls use small per-head offsets and skip attn_out, cross-attention
    calls use one smooth disparity-like offset per query.  Timed eagerly and as one CUDA graph."""
    import matchattention_b200 as ma
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.float16
    stages = [(48, 160, 2, 8), (96, 128, 2, 8), (192, 64, 1, 8), (384, 32, 1, 2)]      # side, C, r, layers
    B, h = 2, 4
    g = torch.Generator(device=dev).manual_seed(7)
    calls, alg_bytes = [], 0
    for side, C, r, layers in stages:
        N, hd, M = side * side, C // h, (2 * r + 2) ** 2
        q, k, v = (torch.randn(B, N, C, generator=g, device=dev).to(dtype) for _ in range(3))
        ys, xs = torch.meshgrid(torch.arange(side, device=dev, dtype=torch.float32),
                                torch.arange(side, device=dev, dtype=torch.float32), indexing="ij")
        grid = torch.stack((xs, ys), -1).view(1, N, 1, 2)
        coarse = torch.rand(B, 1, 7, 7, generator=g, device=dev) * (-side / 8.0)          # disparity up to 1/8 of the width
        disp = torch.nn.functional.interpolate(coarse, size=(side, side), mode="bilinear", align_corners=True)
        cross = grid + torch.cat((disp.view(B, N, 1, 1), torch.zeros(B, N, 1, 1, device=dev)), -1)
        cross = cross.expand(B, N, h, 2)
        selfo = grid + (torch.rand(B, N, h, 2, generator=g, device=dev) * 2 - 1)
        def clamp(mo):
            return torch.cat((mo[..., :1].clamp(r, side - 1 - r - 1e-3), mo[..., 1:].clamp(r, side - 1 - r - 1e-3)),
                             -1).to(dtype).contiguous()
        cross, selfo = clamp(cross), clamp(selfo)
        out, attn = torch.empty_like(q), q.new_empty(B, N, h, M)
        for _ in range(layers):
            calls.append((selfo, q, k, v, out, None, side, r, hd))
            calls.append((cross, q, k, v, out, attn, side, r, hd))
            alg_bytes += 2 * B * N * (4 * C + 2 * h) + 2 * B * N * (4 * C + 2 * h + h * M)

    def knobs_of(r):     # --variant / --chunks-per-lane apply to the r = 2 calls (kernel experiments)
        return dict(variant=args.variant, chunks_per_lane=args.chunks_per_lane) if r == 2 else {}

    def forward_ops():
        for mo, q, k, v, out, attn, side, r, hd in calls:
            ma.launch(mo, q, k, v, out, attn, side, side, (r, r), "l1_norm", hd ** -0.5, **knobs_of(r))

    def timed(fn, n):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    n = max(5, min(args.steps, 100))
    eager_ms = timed(forward_ops, n)
    # one call of each distinct kind on its own (the layers of a stage repeat it)
    per_call = []
    for idx in sorted({(c[6], c[5] is None): i for i, c in enumerate(calls)}.values()):
        mo, q, k, v, out, attn, side, r, hd = calls[idx]
        def twenty():
            for _ in range(20):
                ma.launch(mo, q, k, v, out, attn, side, side, (r, r), "l1_norm", hd ** -0.5, **knobs_of(r))
        # as a CUDA graph of 20 launches: the small calls take less device time than a launch takes the host
        g20, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(st):
            twenty()
            with torch.cuda.graph(g20, stream=st):
                twenty()
        torch.cuda.synchronize()
        us = 1e3 * timed(g20.replay, 20) / 20
        per_call.append({"side": side, "r": r, "hd": hd, "kind": "self" if attn is None else "cross", "us": round(us, 2)})
    graph = torch.cuda.CUDAGraph()
    side_stream = torch.cuda.Stream()
    with torch.cuda.stream(side_stream):
        forward_ops()
        with torch.cuda.graph(graph, stream=side_stream):
            forward_ops()
    torch.cuda.synchronize()
    graph_ms = timed(graph.replay, n)
    line = {"metric": "matchstereo_t_1536_op_sequence_ms_per_pair", "value": graph_ms, "unit": "ms", "n_gpus": 1,
            "steps": n, "warmup": max(3, args.warmup), "ms_per_step": graph_ms, "higher_is_better": False,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "52 MatchAttention calls of MatchStereo-T at 1536x1536 (B=2, h=4)",
                       "stages_side_C_r_layers": stages, "eager_ms": eager_ms, "cuda_graph_ms": graph_ms,
                       "algorithmic_bytes": alg_bytes, "algorithmic_GBps_graph": alg_bytes / graph_ms / 1e6,
                       "per_call_us_in_a_graph_of_20": per_call},
            "gpu_launches": 52 * n}
    print(json.dumps(line), flush=True)


def measure_model(args, compile_ours, compile_reference, steps=None):
    """The reference's own MatchStereo forward on the GPU with its operator swapped (BASELINE.json configs[2]:
    MatchStereo-T, random-init weights, float16, a 1536x1536 synthetic stereo pair; ms per pair).

    The model is the unmodified reference code (the copy oracle/make_ref.py places under oracle/_ref/): it is
    the harness around the operator, not the thing built here.  Arms, all on the same GPU, same weights, same
    pair, each timed with the reference's protocol (models run_img.py:100-112: warm-up, then the mean of the
    timed forwards between two CUDA events):
      pytorch        mat_impl='pytorch' (the reference's five torch functions), eager
      dropin         mat_impl='cuda' with this library behind the module name match_attention, eager
      fused          dropin + the steps around the operator on this library's kernels (dropin/fused_model.py)
      fused_graph    the fused forward captured once as a CUDA graph and replayed
      fused_compiled / fused_compiled_graph / pytorch_compiled   (--model-compile) the same under torch.compile,
                     which is how the reference's own driver runs the model
    plus the 52 operator calls of the forward, with the inputs the model really gave them, replayed alone as
    one CUDA graph (the operator's share of the forward)."""
    import types
    from oracle import ref_loader
    metric = f"matchstereo_{args.model_variant}_{args.model_size[0]}x{args.model_size[1]}_ms_per_pair"
    if not ref_loader.available():
        return {"metric": metric, "unavailable": "the reference's Python code is not present under "
                "oracle/_ref/ (oracle/make_ref.py places it where a checkout exists)"}
    import matchattention_b200 as ma
    from matchattention_b200.dropin.fused_model import patch_reference_model
    from _cases import make_stereo_pair
    ref_loader.import_reference()
    from models.match_stereo import MatchStereo
    from models.match_former_ops import MF_FusedForwardOps
    ma.install_dropin()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.backends.cudnn.benchmark = True
    dtype = {"f16": torch.float16, "f32": torch.float32, "bf16": torch.bfloat16}[args.model_dtype]
    Hi, Wi = args.model_size
    stereo = not args.model_flow
    left, right = make_stereo_pair(11, Hi, Wi, args.model_max_disp)
    left, right = left.to(dev, dtype), right.to(dev, dtype)

    def build(mat_impl):
        torch.manual_seed(21)
        m = MatchStereo(types.SimpleNamespace(variant=args.model_variant, mat_impl=mat_impl))
        return m.eval().to(dev).to(dtype)

    n = max(5, min(steps if steps is not None else args.steps, 50))
    warm = max(5, min(args.warmup, 10))

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1.0))

    sampler = ClockSampler(0)
    sampler.start()
    t_wall0 = time.perf_counter()
    arms, parity, notes = {}, {}, {}
    with torch.inference_mode():
        ref_model = build("pytorch")
        want = ref_model(left, right, stereo=stereo)
        arms["pytorch"] = timed(lambda: ref_model(left, right, stereo=stereo))
        del ref_model
        torch.cuda.empty_cache()

        model = build("cuda")
        # the operator calls of one forward, with their real inputs
        calls = []

        def grab(mod, a, kw, out):
            calls.append((a[0], a[1], a[2], a[3], a[4], a[5], a[6][0], kw["scale"]))
        hooks = [m.register_forward_hook(grab, with_kwargs=True) for m in model.modules()
                 if isinstance(m, MF_FusedForwardOps)]
        got = model(left, right, stereo=stereo)
        for hk in hooks:
            hk.remove()
        parity["dropin_field_up_rel"] = rel(got["field_up"], want["field_up"])
        arms["dropin"] = timed(lambda: model(left, right, stereo=stereo))

        outs = [(torch.empty_like(c[1]), c[1].new_empty(c[1].size(0), c[1].size(1), c[0].size(2), (2 * c[6] + 2) ** 2))
                for c in calls]

        def ops_only():
            for (mo, q, k, v, H, W, r, scale), (o, a) in zip(calls, outs):
                ma.launch(mo, q, k, v, o, a, H, W, (r, r), "l1_norm", scale)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            ops_only()
            gops = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gops, stream=side):
                ops_only()
        torch.cuda.synchronize()
        op_ms = timed(gops.replay)
        n_calls = len(calls)
        alg = sum(c[1].element_size() * (4 * c[1].numel() + c[0].numel() + o[1].numel()) for c, o in zip(calls, outs))
        del calls, outs, gops

        patch_reference_model(model)
        got = model(left, right, stereo=stereo)
        parity["fused_field_up_rel"] = rel(got["field_up"], want["field_up"])
        arms["fused"] = timed(lambda: model(left, right, stereo=stereo))

        static = {}
        try:
            with torch.cuda.stream(side):
                for _ in range(3):
                    model(left, right, stereo=stereo)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    static["out"] = model(left, right, stereo=stereo)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            parity["fused_graph_field_up_rel"] = rel(static["out"]["field_up"], want["field_up"])
            arms["fused_graph"] = timed(graph.replay)
        except Exception as exc:          # a step of the model that cannot be captured
            notes["fused_graph"] = "not captured: " + str(exc).splitlines()[0][:200]
            torch.cuda.synchronize()
        compiled_field = None
        if compile_ours or compile_reference:
            torch.backends.cuda.matmul.allow_tf32 = True
        if compile_ours:
            # torch.compile around the opaque ops, as the reference's own driver compiles its model
            # (run_img.py:55-58: default mode, dynamic=False, TF32 matmuls allowed)
            torch.backends.cuda.matmul.allow_tf32 = True
            try:
                patch_reference_model(model, traceable=True)
                cmodel = torch.compile(model, dynamic=False)
                t0 = time.perf_counter()
                got = cmodel(left, right, stereo=stereo)
                torch.cuda.synchronize()
                notes["fused_compiled_compile_s"] = round(time.perf_counter() - t0, 1)
                parity["fused_compiled_field_up_rel"] = rel(got["field_up"], want["field_up"])
                compiled_field = got["field_up"].clone()
                arms["fused_compiled"] = timed(lambda: cmodel(left, right, stereo=stereo))
                try:
                    with torch.cuda.stream(side):
                        for _ in range(3):
                            cmodel(left, right, stereo=stereo)
                        cgraph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(cgraph, stream=side):
                            static["cout"] = cmodel(left, right, stereo=stereo)
                    torch.cuda.synchronize()
                    arms["fused_compiled_graph"] = timed(cgraph.replay)
                    parity["fused_compiled_graph_field_up_rel"] = rel(static["cout"]["field_up"], want["field_up"])
                except Exception as exc:
                    notes["fused_compiled_graph"] = "not captured: " + str(exc).splitlines()[0][:200]
                    torch.cuda.synchronize()
            except Exception as exc:
                notes["fused_compiled"] = "failed: " + str(exc).splitlines()[0][:300]
        if compile_reference:
            try:
                del model
                torch.cuda.empty_cache()
                ref_model = build("pytorch")
                cref = torch.compile(ref_model, dynamic=False)
                t0 = time.perf_counter()
                want_compiled = cref(left, right, stereo=stereo)
                torch.cuda.synchronize()
                notes["pytorch_compiled_compile_s"] = round(time.perf_counter() - t0, 1)
                # compilation itself changes the rounding (TF32 matmuls, float32 intermediates inside fused
                # kernels): the reference's compiled model against its own eager run, and ours against it
                parity["pytorch_compiled_vs_pytorch_eager_field_up_rel"] = rel(want_compiled["field_up"], want["field_up"])
                if compiled_field is not None:
                    parity["fused_compiled_vs_pytorch_compiled_field_up_rel"] = rel(compiled_field, want_compiled["field_up"])
                arms["pytorch_compiled"] = timed(lambda: cref(left, right, stereo=stereo))
            except Exception as exc:
                notes["pytorch_compiled"] = "failed: " + str(exc).splitlines()[0][:300]
    sampler.stop()
    best = min((v, k) for k, v in arms.items() if not k.startswith("pytorch"))
    line = {"metric": metric, "value": best[0], "unit": "ms", "n_gpus": 1, "steps": n, "warmup": warm,
            "ms_per_step": best[0], "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": args.model_dtype, "data": "synthetic",
            "config": {"workload": f"MatchStereo-{args.model_variant} forward, {Hi}x{Wi} pair, "
                                   f"{'stereo' if stereo else 'flow'}, random-init weights (seed 21), batch of 2 views",
                       "arm_reported": best[1], "arms_ms_per_pair": arms, "notes": notes,
                       "field_up_rel_diff_vs_pytorch_branch": parity,
                       "operator_calls": n_calls, "operator_calls_alone_graph_ms": op_ms,
                       "operator_algorithmic_bytes": alg, "operator_algorithmic_GBps": alg / op_ms / 1e6,
                       "target_ms": 5.0},
            "clocks": sampler.summary(t_wall0, time.perf_counter()),
            "gpu_launches": n_calls * n}
    return line


def run_model_pairs_mode(args, rank, local_rank, world):
    """BASELINE.json configs[3]: a fixed batch of image pairs (8 by default) through the reference's model
    with this library's kernels, the pairs dealt out to the GPUs (one process per GPU, weights replicated,
    no collective on the data path: a barrier brackets the timed region).  A step is the whole batch; with N
    GPUs each rank runs its share of the pairs one after the other (strong scaling over the fixed batch).
    Arm: the fused forward captured once as a CUDA graph and replayed, inputs copied into the graph's input
    buffers from device-resident images (`value`) or from pinned host memory with the up-sampled field read
    back to the host (`e2e`).  Rank 0 prints one JSON line with pairs per second over all GPUs."""
    import types
    from oracle import ref_loader
    Hi, Wi = args.model_size
    metric = f"match{'flow' if args.model_flow else 'stereo'}_{args.model_variant}_{Hi}x{Wi}_pairs_per_s"
    if not ref_loader.available():
        if rank == 0:
            print(json.dumps({"metric": metric, "unavailable": "the reference's Python code is not present under "
                              "oracle/_ref/ (oracle/make_ref.py places it where a checkout exists)"}), flush=True)
        return
    import matchattention_b200 as ma
    from matchattention_b200.dropin.fused_model import patch_reference_model
    from _cases import make_stereo_pair
    ref_loader.import_reference()
    from models.match_stereo import MatchStereo
    ma.install_dropin()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    torch.backends.cudnn.benchmark = True
    dtype = {"f16": torch.float16, "f32": torch.float32, "bf16": torch.bfloat16}[args.model_dtype]
    stereo = not args.model_flow
    total = args.model_pairs
    if total % world != 0:
        raise SystemExit(f"--model-pairs {total} does not divide over {world} GPUs")
    mine = [i for i in range(total) if i % world == rank]
    host = [tuple(t.to(dtype).pin_memory() for t in make_stereo_pair(100 + i, Hi, Wi, args.model_max_disp)) for i in mine]
    resident = [(a.to(dev), b.to(dev)) for a, b in host]
    torch.manual_seed(21)
    model = MatchStereo(types.SimpleNamespace(variant=args.model_variant, mat_impl="cuda")).eval().to(dev).to(dtype)
    patch_reference_model(model)
    s_left, s_right = torch.empty_like(resident[0][0]), torch.empty_like(resident[0][1])
    s_left.copy_(resident[0][0]); s_right.copy_(resident[0][1])
    side = torch.cuda.Stream()
    with torch.inference_mode():
        with torch.cuda.stream(side):
            for _ in range(3):
                model(s_left, s_right, stereo=stereo)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out = model(s_left, s_right, stereo=stereo)
    torch.cuda.synchronize()
    field = out["field_up"]
    field_host = torch.empty(field.shape, dtype=field.dtype).pin_memory()

    def step_resident():
        for a, b in resident:
            s_left.copy_(a, non_blocking=True)
            s_right.copy_(b, non_blocking=True)
            graph.replay()

    def step_host():
        for a, b in host:
            s_left.copy_(a, non_blocking=True)
            s_right.copy_(b, non_blocking=True)
            graph.replay()
            field_host.copy_(field, non_blocking=True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step, k):
        for _ in range(max(1, min(args.warmup, 3))):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            step()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / k

    k = max(2, min(args.steps, 5))
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0 = time.perf_counter()
    with torch.inference_mode():
        ms_res = timed(step_resident, k)
        t1 = time.perf_counter()
        ms_host = timed(step_host, k)
    sampler.stop()
    if rank == 0:
        h2d = sum(a.numel() * a.element_size() + b.numel() * b.element_size() for a, b in host)
        d2h = field.numel() * field.element_size() * len(host)
        print(json.dumps({
            "metric": metric, "value": total / ms_res * 1e3, "unit": "pairs/s", "n_gpus": world, "steps": k,
            "warmup": max(1, min(args.warmup, 3)), "ms_per_step": ms_res, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": args.model_dtype, "data": "synthetic",
            "config": {"workload": f"Match{'Flow' if args.model_flow else 'Stereo'}-{args.model_variant} forward, batch of "
                                   f"{total} pairs of {Hi}x{Wi}, dealt out over {world} GPU(s), random-init weights (seed 21)",
                       "pairs_per_rank": len(mine), "ms_per_pair_per_gpu": ms_res / len(mine),
                       "arm": "fused steps, one CUDA graph per forward"},
            "e2e": {"value": total / ms_host * 1e3, "unit": "pairs/s", "ms_per_step": ms_host,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "bytes per rank; images from pinned host memory, up-sampled field read back"},
            "clocks": sampler.summary(t0, t1)}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_model_mode(args):
    print(json.dumps(measure_model(args, args.model_compile, args.model_compile)), flush=True)


def run_upsample_mode(args):
    """The convex upsampling of the field that follows the last MatchAttention block of MatchStereo at
    1536x1536: field [2, 384, 384, 2] x 4, mask [2, 144, 384, 384], float16."""
    import matchattention_b200 as ma
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, H, W, D, f, dtype = 2, 384, 384, 2, 4, torch.float16
    g = torch.Generator(device=dev).manual_seed(3)
    field = (torch.randn(B, H, W, D, generator=g, device=dev) * 4).to(dtype)
    mask = (torch.randn(B, 9 * f * f, H, W, generator=g, device=dev) * 2).to(dtype)
    n = max(20, args.steps)
    for _ in range(max(3, args.warmup)):
        out = ma.upsample_field(field, mask, f)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        out = ma.upsample_field(field, mask, f)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    nbytes = (field.numel() + mask.numel() + out.numel()) * 2
    peak, kind = measured_peak()
    print(json.dumps({"metric": "upsample_field_ms", "value": ms, "unit": "ms", "n_gpus": 1, "steps": n,
                      "higher_is_better": False, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "upsample_field 2x384x384x2 by 4", "bytes": nbytes,
                                 "note": "working set 106 MB fits the 126 MB L2: repeated calls are served from L2"},
                      "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peak, "unit": "GB/s",
                                   "frac": nbytes / ms / 1e6 / peak, "peak_kind": kind}}), flush=True)


def run_volume_mode(args):
    """The stereo cost volume of GlobalCorrelation at 1/32 of 1536x1536 (48x48 tokens) and of 2176x3840
    (68x120 tokens), float16: one kernel instead of the reference's loops over the disparities."""
    import matchattention_b200 as ma
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows = []
    for B, H, W in ((1, 48, 48), (1, 68, 120)):
        corr = (torch.randn(B, H, W, W, device=dev) * 3).half()
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(side):
            ma.stereo_volume(corr)
            with torch.cuda.graph(graph, stream=side):
                for _ in range(10):
                    vol = ma.stereo_volume(corr)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            graph.replay()
        e0.record()
        for _ in range(20):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        rows.append({"B": B, "H": H, "W": W, "us_per_call": e0.elapsed_time(e1) / 200 * 1000,
                     "bytes": (corr.numel() + vol.numel()) * 2})
    print(json.dumps({"metric": "stereo_volume_us", "value": rows[0]["us_per_call"], "unit": "us", "n_gpus": 1,
                      "higher_is_better": False, "dtype": "f16", "data": "synthetic", "config": {"shapes": rows}}), flush=True)


def run_backward_mode(args):
    """Training step of the operator alone: forward + backward through autograd on one batch item of the
    chosen workload (gradients of both outputs given), the backward kernel by itself, and, where the
    reference's code is present, autograd over the reference's 'pytorch' path on the same GPU (its native
    path has no backward).  One JSON line; the value is the forward + backward time."""
    import matchattention_b200 as ma
    from matchattention_b200 import _lib
    from matchattention_b200.ops import _DTYPE_CODE
    from oracle import ref_loader
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    wl = make_workload(args.workload, seed=1234)
    B, H, W, h, hd, r, scale = 1, wl["H"], wl["W"], wl["h"], wl["hd"], wl["r"], wl["scale"]
    mo, q, k, v = (t[:1].contiguous().to(dev) for t in wl["inputs"])
    g = torch.Generator(device=dev).manual_seed(5)
    g_out = torch.randn(q.shape, generator=g, device=dev).to(q.dtype)
    g_attn = torch.randn(B, H * W, h, (2 * r + 2) ** 2, generator=g, device=dev).to(q.dtype)
    d_q, d_mo = torch.empty_like(q), torch.empty_like(mo)
    d_k, d_v = (torch.zeros(k.shape, dtype=torch.float32, device=dev) for _ in range(2))
    stream = torch.cuda.current_stream().cuda_stream

    def kernel_only():
        _lib.check(_lib.lib.matchattn_fused_backward(
            mo.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), g_out.data_ptr(), g_attn.data_ptr(), d_q.data_ptr(),
            d_k.data_ptr(), d_v.data_ptr(), d_mo.data_ptr(), B, H, W, h, hd, r, r, _DTYPE_CODE[q.dtype], _lib.L1_NORM,
            float(scale), 0, H, stream))

    def autograd_step(op):
        def step():
            leaves = [t.detach().requires_grad_(True) for t in (mo, q, k, v)]
            out, attn = op(*leaves)
            torch.autograd.backward([out, attn], [g_out, g_attn])
        return step

    def timed(fn, n):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    n = max(10, min(args.steps, 50))
    ours = timed(autograd_step(lambda a, b, c, d: ma.match_attention_autograd(a, b, c, d, H, W, r, scale)), n)
    kern = timed(kernel_only, n)
    fwd = timed(lambda: ma.match_attention(mo, q, k, v, H, W, r, scale), n)
    ref = None
    if ref_loader.available():
        impl, _ = ref_loader.import_reference()
        ref = timed(autograd_step(lambda a, b, c, d: ref_loader.reference_op(impl, a, b, c, d, H, W, h, r, scale)), 5)
    print(json.dumps({"metric": "matchattention_forward_backward_ms", "value": ours, "unit": "ms", "n_gpus": 1, "steps": n,
                      "higher_is_better": False, "dtype": str(q.dtype)[6:], "data": "synthetic",
                      "config": {"workload": args.workload + " (one batch item)", "queries": H * W},
                      "backward_kernel_ms": kern, "forward_kernel_ms": fwd,
                      "reference_pytorch_autograd_ms": ref,
                      "gpu_launches": 2 * n + n + n}), flush=True)


SHAPE_WORKLOADS = ("op_384x384_b4_h8x16_r1_f32_flow", "op_384x384_b4_h8x16_r1_bf16_flow",
                   "op_384x384_b4_h8x16_r1_f16_flow_perhead", "op_384x384_b4_h8x16_r1_f16_smooth",
                   "op_104x208_b1_h8x16_r1_f32_cross", "op_96x96_b2_h4x32_r2_f16_self", "op_48x48_b2_h4x40_r2_f16_self")


def time_shape(name, dev, peak, seed=4321, region_s=0.1):
    """One other configuration shape, timed on the device the same way as the headline (a CUDA graph of the
    launches, replayed until the region lasts `region_s`); returns the entry for the line's `shapes` list."""
    import matchattention_b200 as ma
    wl = make_workload(name, seed)
    B, H, W, h, hd, r, dtype = (wl[n] for n in ("B", "H", "W", "h", "hd", "r", "dtype"))
    mo, q, k, v = (t.to(dev) for t in wl["inputs"])
    out, attn = torch.empty_like(q), q.new_empty(B, H * W, h, (2 * r + 2) ** 2)
    per_graph = 20

    def launches():
        for _ in range(per_graph):
            ma.launch(mo, q, k, v, out, attn, H, W, (r, r), "l1_norm", wl["scale"])
    graph, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=dev)
    with torch.cuda.stream(cap):
        launches()
        with torch.cuda.graph(graph, stream=cap):
            launches()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    reps = max(3, min(5000, int(region_s * 1e3 / max(e0.elapsed_time(e1), 1e-3)) + 1))
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (reps * per_graph)
    esize = 2 if dtype != torch.float32 else 4
    nbytes = algorithmic_bytes_per_query(h, hd, r, esize) * B * H * W
    achieved = nbytes / (ms * 1e-3) / 1e9
    return {"workload": name, "ms": ms, "queries_per_s": B * H * W / (ms * 1e-3), "achieved_GBps": achieved,
            "frac": achieved / peak, "dispatch": ma.describe_dispatch(h, hd, r, dtype),
            "algorithmic_MB": nbytes / 1e6, "launches_timed": reps * per_graph,
            "l2": "exceeds L2" if nbytes > 126e6 else "fits L2 (resident between launches, as between the layers of the model)"}


def config_dict(name, wl):
    step_mb = wl["B"] * wl["H"] * wl["W"] * algorithmic_bytes_per_query(wl["h"], wl["hd"], wl["r"],
                                                                        torch.empty(0, dtype=wl["dtype"]).element_size()) / 1e6
    l2 = "inputs+outputs of one step exceed the 126 MB L2; no flush between steps" if step_mb > 126 else \
         f"inputs+outputs of one step ({step_mb:.0f} MB) fit the 126 MB L2 and stay resident between steps, as they " \
         "do between the layers of the model; not a bandwidth measurement"
    return {"workload": name, "B_per_gpu": wl["B"], "token_map": [wl["H"], wl["W"]], "heads": wl["h"],
            "head_dim": wl["hd"], "win_r": wl["r"], "window_taps": (2 * wl["r"] + 2) ** 2, "l2": l2}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU-baseline leg (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-shapes", action="store_true", help="skip the timing of the other configuration shapes")
    ap.add_argument("--no-model", action="store_true", help="skip the MatchStereo-T forward leg of the default line")
    ap.add_argument("--mode", choices=["pairs", "band", "model", "model_ops", "upsample", "volume", "backward", "model_pairs"], default="pairs",
                    help="pairs: every GPU its own batch (default); band: one large pair split by query row bands; "
                         "model_ops: the 52 operator calls of one MatchStereo-T forward at 1536x1536")
    ap.add_argument("--no-band", action="store_true", help="with more than one GPU: skip the row-band measurement")
    ap.add_argument("--model-variant", default="tiny", choices=["tiny", "small", "base"])
    ap.add_argument("--model-size", type=int, nargs=2, default=[1536, 1536], metavar=("H", "W"))
    ap.add_argument("--model-dtype", default="f16", choices=["f16", "bf16", "f32"])
    ap.add_argument("--model-max-disp", type=int, default=192)
    ap.add_argument("--model-pairs", type=int, default=8, help="model_pairs mode: size of the batch dealt out to the GPUs")
    ap.add_argument("--model-flow", action="store_true", help="model mode: optical-flow forward (stereo=False)")
    ap.add_argument("--model-compile", action="store_true",
                    help="model mode: also time the model under torch.compile (minutes of compilation)")
    ap.add_argument("--tile-w", type=int, default=0)
    ap.add_argument("--chunks-per-lane", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true", help="time K plain launches instead of one graph of K launches")
    ap.add_argument("--variant", type=int, default=0, help="0 auto, 1 scalar kernel, 2/3 matrix-instruction kernels")
    ap.add_argument("--strategy", type=int, default=0, help="0 auto, 1 direct kernel, 2 binned path")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import matchattention_b200 as ma   # raises if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    if args.mode == "band":
        run_band_mode(args, rank, local_rank, world)
        return
    if args.mode == "model_ops":
        run_model_ops_mode(args)
        return
    if args.mode == "model":
        run_model_mode(args)
        return
    if args.mode == "model_pairs":
        run_model_pairs_mode(args, rank, local_rank, world)
        return
    if args.mode == "upsample":
        run_upsample_mode(args)
        return
    if args.mode == "volume":
        run_volume_mode(args)
        return
    if args.mode == "backward":
        run_backward_mode(args)
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    binding = bind_to_gpu_cpus(local_rank)      # before any pinned allocation: first touch decides the NUMA node
    wl = make_workload(args.workload, 1234 + rank)
    B, H, W, h, hd, r, dtype = (wl[n] for n in ("B", "H", "W", "h", "hd", "r", "dtype"))
    M = (2 * r + 2) ** 2
    host = [t.pin_memory() for t in wl["inputs"]]
    mo, q, k, v = (t.to(dev) for t in host)
    out = torch.empty_like(q)
    attn = q.new_empty(B, H * W, h, M)
    knobs = dict(tile_w=args.tile_w, chunks_per_lane=args.chunks_per_lane, variant=args.variant,
                 strategy=args.strategy)

    def step():
        ma.launch(mo, q, k, v, out, attn, H, W, (r, r), "l1_norm", wl["scale"], **knobs)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    # ---- device-resident timing: exactly K steps between two events on the launching stream.
    # The K launches are replayed as one CUDA graph so that the small workloads, whose kernel takes
    # less device time than a launch takes the host, are timed on the device too (--no-graph: plain launches).
    for _ in range(args.warmup):
        step()
    barrier()
    run_steps = None
    if not args.no_graph:
        graph, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=dev)
        with torch.cuda.stream(cap):
            step()
            with torch.cuda.graph(graph, stream=cap):
                for _ in range(args.steps):
                    step()
        run_steps = graph.replay
        barrier()
    # The K-step region is repeated until it lasts MIN_REGION_S on the device (the kernel takes a fraction of
    # a millisecond, K of them are too short a sample for the clock record); the per-step time is the mean.
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def k_steps():
        if run_steps is not None:
            run_steps()
        else:
            for _ in range(args.steps):
                step()

    ev0.record()
    k_steps()
    ev1.record()
    barrier()
    once_ms = max(ev0.elapsed_time(ev1), 1e-3)
    reps = max(1, min(2000, int(MIN_REGION_S * 1e3 / once_ms) + 1))
    if dist is not None:
        t = torch.tensor([reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        reps = int(t.item())
    t_wall0 = time.perf_counter()
    ev0.record()
    for _ in range(reps):
        k_steps()
    ev1.record()
    barrier()
    t_wall1 = time.perf_counter()
    ms_total = ev0.elapsed_time(ev1)
    if dist is not None:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / (args.steps * reps)
    queries_per_step = B * H * W * world
    value = queries_per_step / (ms_per_step * 1e-3)

    # ---- end to end: pinned host inputs -> device, kernel, outputs -> pinned host, every step
    e2e = None
    if not args.no_e2e:
        host_out = torch.empty(out.shape, dtype=dtype).pin_memory()
        host_attn = torch.empty(attn.shape, dtype=dtype).pin_memory()
        d_in = [torch.empty_like(t, device=dev) for t in host]
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = host_out.numel() * host_out.element_size() + host_attn.numel() * host_attn.element_size()

        # Batch items are independent, so the step is pipelined item by item over a few streams:
        # the host->device copy of item i+1, the kernel of item i and the device->host copy of
        # item i-1 overlap (the two copy directions use separate DMA engines).
        lanes = [torch.cuda.Stream(device=dev) for _ in range(min(3, B))]
        fork, joins = torch.cuda.Event(), [torch.cuda.Event() for _ in lanes]

        def e2e_step(with_kernel=True, with_attn=True):
            main = torch.cuda.current_stream()
            fork.record(main)
            for i in range(B):
                st = lanes[i % len(lanes)]
                if i < len(lanes):
                    st.wait_event(fork)
                with torch.cuda.stream(st):
                    for d, s in zip(d_in, host):
                        d[i:i + 1].copy_(s[i:i + 1], non_blocking=True)
                    if with_kernel:
                        ma.launch(d_in[0][i:i + 1], d_in[1][i:i + 1], d_in[2][i:i + 1], d_in[3][i:i + 1], out[i:i + 1],
                                  attn[i:i + 1] if with_attn else None, H, W, (r, r), "l1_norm", wl["scale"], **knobs)
                    host_out[i:i + 1].copy_(out[i:i + 1], non_blocking=True)
                    if with_attn:
                        host_attn[i:i + 1].copy_(attn[i:i + 1], non_blocking=True)
            for st, ev in zip(lanes, joins):
                ev.record(st)
                main.wait_event(ev)

        e2e_steps = max(3, min(args.steps, 20))

        def timed_e2e(**kw):
            for _ in range(3):
                e2e_step(**kw)
            barrier()
            ev0.record()
            for _ in range(e2e_steps):
                e2e_step(**kw)
            ev1.record()
            barrier()
            ms = ev0.elapsed_time(ev1)
            if dist is not None:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms / e2e_steps

        ms_e2e = timed_e2e()
        ms_copy = timed_e2e(with_kernel=False)            # the same copies without the kernel: the host link's ceiling
        ms_self = timed_e2e(with_attn=False)              # what a self-attention caller needs back: out only
        d2h_out = host_out.numel() * host_out.element_size()
        e2e = {"value": queries_per_step / (ms_e2e * 1e-3), "unit": "queries/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "ms_per_step": ms_e2e, "kernel_launches_per_step": B,
               "h2d_GBps_per_gpu": h2d / ms_e2e / 1e6, "d2h_GBps_per_gpu": d2h / ms_e2e / 1e6,
               "copy_only": {"ms_per_step": ms_copy, "queries_per_s": queries_per_step / (ms_copy * 1e-3),
                             "h2d_GBps_per_gpu": h2d / ms_copy / 1e6, "d2h_GBps_per_gpu": d2h / ms_copy / 1e6,
                             "note": "the same host<->device copies with no kernel between them"},
               "without_attn_out": {"ms_per_step": ms_self, "queries_per_s": queries_per_step / (ms_self * 1e-3),
                                    "d2h_bytes_per_step": d2h_out,
                                    "note": "attention weights neither written nor copied back (self-attention callers)"},
               "host_binding": binding,
               "pipeline": f"{B} batch items over {len(lanes)} streams, pinned host buffers"}
    band = None
    if world > 1 and not args.no_band and args.workload == DEFAULT_WORKLOAD:
        del host_out, host_attn, d_in
        torch.cuda.empty_cache()
        band = measure_band(rank, world, dev, dist)
    shapes = None
    if rank == 0 and not args.no_shapes and args.workload == DEFAULT_WORKLOAD:
        peak_gbs, _ = measured_peak()
        shapes = [time_shape(name, dev, peak_gbs) for name in SHAPE_WORKLOADS]
    model = None
    if world == 1 and not args.no_model and args.workload == DEFAULT_WORKLOAD:
        # the other half of the metric: the reference's MatchStereo-T forward at 1536x1536 with the operator
        # swapped, ms per pair (see measure_model; the reference's own compiled arm only with --model-compile)
        try:
            full = measure_model(args, compile_ours=True, compile_reference=args.model_compile, steps=10)
            cfg = full.get("config", {})
            model = {"metric": full["metric"], "unit": "ms", "value": full.get("value"),
                     "arm_reported": cfg.get("arm_reported"), "arms_ms_per_pair": cfg.get("arms_ms_per_pair"),
                     "notes": cfg.get("notes"), "field_up_rel_diff": cfg.get("field_up_rel_diff_vs_pytorch_branch"),
                     "operator_calls_alone_graph_ms": cfg.get("operator_calls_alone_graph_ms"),
                     "target_ms": 5.0, "workload": cfg.get("workload"), "unavailable": full.get("unavailable")}
        except Exception as exc:
            model = {"error": str(exc).splitlines()[0][:300] if str(exc) else type(exc).__name__}
    if sampler:
        sampler.stop()

    if rank == 0:
        esize = 2 if dtype != torch.float32 else 4
        bpq = algorithmic_bytes_per_query(h, hd, r, esize)
        peak, peak_kind = measured_peak()
        achieved = bpq * B * H * W / (ms_per_step * 1e-3) / 1e9     # one launch = one rank's batch
        line = {
            "metric": "matchattention_queries_per_s", "value": value, "unit": "queries/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE_NAME[dtype], "data": "synthetic",
            "config": config_dict(args.workload, wl),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": ncu_traffic_per_launch(args.workload), "peak_kind": peak_kind,
                         "algorithmic_bytes_per_query": bpq, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "frac_first_k_steps": bpq * B * H * W / (once_ms / args.steps * 1e-3) / 1e9 / peak,
                         "kernel": ma.describe_dispatch(h, hd, r, dtype)},
            "clocks": sampler.summary(t_wall0, t_wall1) if sampler else None,
            "timed_region": {"k_step_repeats": reps, "seconds": ms_total * 1e-3,
                             "first_k_steps_ms_per_step": once_ms / args.steps,
                             "note": "value and ms_per_step are the mean over the whole region; first_k_steps is the "
                                     "K steps timed once beforehand (a burst of a few milliseconds, before the "
                                     "power cap lowers the SM clock; see clocks)"},
            "gpu_launches": args.steps * reps,      # the device-resident timed region: one kernel per step
        }
        if band is not None:
            line["band"] = band          # one huge pair split by query row bands over the same GPUs (strong scaling)
        if model is not None:
            line["model"] = model        # MatchStereo-T ms per pair: the reference's model around this library's kernels
        if shapes is not None:
            line["shapes"] = shapes      # the other configuration shapes, same run, same clock record
        if e2e is not None:
            line["e2e"] = e2e
        if not args.no_cpu_baseline:
            cpu_qps, cores, reps, secs = time_cpu_port(wl)
            port = {"value": cpu_qps, "unit": "queries/s", "cores": cores, "kind": "port",
                    "sample": f"one batch item ({H * W} queries) of the workload, {reps} repetitions in {secs:.1f} s, "
                              f"C restatement of the reference algorithm with its {DTYPE_NAME[dtype]} rounding points"}
            ref = time_cpu_reference(wl)
            if ref is not None:
                line["cpu_baseline"] = {
                    "value": ref[0], "unit": "queries/s", "cores": ref[1], "kind": "reference",
                    "sample": f"one batch item ({H * W} queries) of the workload, {ref[2]} repetitions in {ref[3]:.1f} s, "
                              "models/mat_pytorch_impl.py of the reference (unmodified) in float32 on the host cores"}
                line["cpu_port"] = port
            else:
                line["cpu_baseline"] = port
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
