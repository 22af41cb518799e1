"""Row-band split of one MatchAttention call across the GPUs of a box.

A single very large pair does not need a batch to shard: the queries are
independent, so rank p takes the query rows [r0, r1) of the token map and runs
the fused kernel on that band alone (the C ABI's q_row_begin / q_row_end).  A
window can reach any key row, so every rank needs the whole K and V: they are
replicated with a broadcast (NCCL over NVLink on GPUs) into each rank's own
memory, and the kernel then reads them with ordinary loads.  The band inputs
(q, max_offset) travel to their rank and the band outputs come back to the
source rank with point-to-point copies.

The reference has no multi-GPU code; this is the partition its operator admits.
One process per GPU; `torch.distributed` must be initialised by the caller.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def band_rows(H: int, world: int, rank: int, r: int = 0) -> Tuple[int, int]:
    """Rows [r0, r1) of rank `rank`: H split as evenly as possible, the first H % world ranks
    one row longer.  A rank may get an empty band when H < world."""
    base, extra = divmod(H, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def halo_rows(H: int, r0: int, r1: int, r: int, max_abs_dy: float) -> Tuple[int, int]:
    """Key/value rows a band [r0, r1) can touch when no sampling centre lies more than
    `max_abs_dy` rows away from its own query row: the window adds r rows above and r + 1 below
    (floor + 2r + 2 taps), one more row covers the rounding of the bound."""
    reach = int(max_abs_dy) + 1
    return max(0, r0 - reach - r), min(H, r1 + reach + r + 2)


def _default_op(mo, q, k, v, H, W, r, scale, r0, r1, need_attn):
    from .ops import match_attention
    return match_attention(mo, q, k, v, H, W, r, scale, need_attn=need_attn, q_row_begin=r0, q_row_end=r1)


def _p2p(ops: List) -> None:
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


def band_match_attention(max_offset: Optional[torch.Tensor], q: Optional[torch.Tensor], k: Optional[torch.Tensor],
                         v: Optional[torch.Tensor], B: int, H: int, W: int, h: int, hd: int, r: int, scale: float,
                         dtype: torch.dtype, device: torch.device, *, src: int = 0, group=None,
                         need_attn: bool = True, op: Optional[Callable] = None, kv_buffers=None,
                         max_abs_dy: Optional[float] = None):
    """Run one MatchAttention call split by query row bands over the ranks of `group`.

    On rank `src` pass the full tensors (max_offset [B,H*W,h,2], q/k/v [B,H*W,C]); on the other
    ranks pass None.  Returns (out, attn) holding the full result on `src` and (None, None)
    elsewhere.  `op` replaces the band computation (tests run the CPU oracle through it);
    `kv_buffers` lets a caller reuse the (k, v) receive buffers between calls.

    K and V are replicated with a broadcast.  If the caller can bound how far a sampling centre
    lies from its query row (`max_abs_dy`, in rows; e.g. the flow magnitude limit of the model),
    each rank instead receives only the rows its band can reach (halo_rows) by point-to-point
    copies into its full-size buffer; rows outside stay untouched and are never read.  The bound
    is the caller's promise: a centre beyond it reads stale rows.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    op = op or _default_op
    C, N, M = h * hd, H * W, (2 * r + 2) ** 2
    r0, r1 = band_rows(H, world, rank)
    rows = r1 - r0

    # K and V: broadcast into this rank's own buffers
    if rank == src:
        kk, vv = k.contiguous(), v.contiguous()
    elif kv_buffers is not None:
        kk, vv = kv_buffers
    else:
        kk = torch.empty((B, N, C), dtype=dtype, device=device)
        vv = torch.empty((B, N, C), dtype=dtype, device=device)
    src_global = dist.get_global_rank(group, src) if group is not None else src

    def peer(p):
        return dist.get_global_rank(group, p) if group is not None else p

    if max_abs_dy is None:
        dist.broadcast(kk, src=src_global, group=group)
        dist.broadcast(vv, src=src_global, group=group)
    elif rank == src:
        ops, keep = [], []
        for p in range(world):
            p0, p1 = band_rows(H, world, p)
            if p == src or p1 == p0:
                continue
            h0, h1 = halo_rows(H, p0, p1, r, max_abs_dy)
            for t in (kk, vv):
                part = t[:, h0 * W:h1 * W].contiguous()
                keep.append(part)
                ops.append(dist.P2POp(dist.isend, part, peer(p), group))
        _p2p(ops)
    elif rows > 0:
        h0, h1 = halo_rows(H, r0, r1, r, max_abs_dy)
        parts = [torch.empty((B, (h1 - h0) * W, C), dtype=dtype, device=device) for _ in range(2)]
        _p2p([dist.P2POp(dist.irecv, t, peer(src), group) for t in parts])
        kk[:, h0 * W:h1 * W] = parts[0]
        vv[:, h0 * W:h1 * W] = parts[1]

    # band inputs: src slices and sends, the others receive
    if rank == src:
        ops, keep = [], []
        for p in range(world):
            p0, p1 = band_rows(H, world, p)
            if p == src or p1 == p0:
                continue
            qb = q[:, p0 * W:p1 * W].contiguous()
            mb = max_offset[:, p0 * W:p1 * W].contiguous()
            keep += [qb, mb]
            ops += [dist.P2POp(dist.isend, qb, peer(p), group), dist.P2POp(dist.isend, mb, peer(p), group)]
        _p2p(ops)
        q_band = q[:, r0 * W:r1 * W].contiguous()
        mo_band = max_offset[:, r0 * W:r1 * W].contiguous()
    elif rows > 0:
        q_band = torch.empty((B, rows * W, C), dtype=dtype, device=device)
        mo_band = torch.empty((B, rows * W, h, 2), dtype=dtype, device=device)
        _p2p([dist.P2POp(dist.irecv, q_band, peer(src), group), dist.P2POp(dist.irecv, mo_band, peer(src), group)])

    out_band = attn_band = None
    if rows > 0:
        out_band, attn_band = op(mo_band, q_band, kk, vv, H, W, r, scale, r0, r1, need_attn)

    # band outputs back to src
    if rank != src:
        if rows > 0:
            ops = [dist.P2POp(dist.isend, out_band, peer(src), group)]
            if need_attn:
                ops.append(dist.P2POp(dist.isend, attn_band, peer(src), group))
            _p2p(ops)
        return None, None
    out = torch.empty((B, N, C), dtype=dtype, device=device)
    attn = torch.empty((B, N, h, M), dtype=dtype, device=device) if need_attn else None
    ops, recv = [], []
    for p in range(world):
        p0, p1 = band_rows(H, world, p)
        if p1 == p0:
            continue
        if p == src:
            out[:, p0 * W:p1 * W] = out_band
            if need_attn:
                attn[:, p0 * W:p1 * W] = attn_band
            continue
        ob = torch.empty((B, (p1 - p0) * W, C), dtype=dtype, device=device)
        ops.append(dist.P2POp(dist.irecv, ob, peer(p), group))
        ab = None
        if need_attn:
            ab = torch.empty((B, (p1 - p0) * W, h, M), dtype=dtype, device=device)
            ops.append(dist.P2POp(dist.irecv, ab, peer(p), group))
        recv.append((p0, p1, ob, ab))
    _p2p(ops)
    for p0, p1, ob, ab in recv:
        out[:, p0 * W:p1 * W] = ob
        if need_attn:
            attn[:, p0 * W:p1 * W] = ab
    return out, attn
