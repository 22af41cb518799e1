"""Row-band split of one MatchAttention call across the GPUs of a box.

A single very large pair does not need a batch to shard: the queries are
independent, so rank p takes the query rows [r0, r1) of the token map and runs
the fused kernel on that band alone (the C ABI's q_row_begin / q_row_end).  A
window can reach any key row, so every rank needs the whole K and V: they are
replicated with a broadcast (NCCL over NVLink on GPUs) into each rank's own
memory, and the kernel then reads them with ordinary loads.  The band inputs
(q, max_offset) travel to their rank and the band outputs come back to the
source rank with point-to-point copies.

Two forms:

* :func:`band_match_attention` -- one rank owns q/k/v/max_offset (the form the specification of
  this mode names): K and V are broadcast from it, the band inputs travel to their rank and the
  band outputs come back.  Everything that moves leaves or enters the owner's links, so this form
  cannot be faster than the owner computing alone (measured; see the benchmark's ``band`` object).
* :func:`band_match_attention_resident` -- every rank already holds ITS rows of q, max_offset, K and
  V (the state of a pipeline whose producers are band-parallel too) and keeps its rows of the
  outputs.  K/V rows are exchanged with an all-gather, or, when the caller can bound how far a
  centre lies from its query row, only the halo rows move between neighbouring ranks: through NCCL
  send / receive, or -- with :class:`PeerBuffers`, full-size K / V buffers that every rank maps into its
  own address space -- pulled straight out of the neighbours' memory over NVLink by peer copies.

:func:`band_check` is the CPU-side handshake to run before either form when the ranks' arguments
come from different code paths: it fails on every rank if one rank reports an error or the
arguments differ, and -- given a process group with a short timeout -- when a rank never arrives.

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


def interior_rows(H: int, r0: int, r1: int, r: int, max_abs_dy: float) -> Tuple[int, int]:
    """Query rows [i0, i1) of the band [r0, r1) whose windows stay inside the band's own key/value rows
    under the same bound as halo_rows (their halo needs no other rank); i0 == i1 when there are none."""
    reach = int(max_abs_dy) + 1
    i0 = r0 if r0 == 0 else r0 + reach + r
    i1 = r1 if r1 == H else r1 - (reach + r + 2)
    i0, i1 = min(max(i0, r0), r1), min(max(i1, r0), r1)
    return (i0, i1) if i1 > i0 else (r0, r0)


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


class BandArgumentError(RuntimeError):
    """Raised on every rank by :func:`band_check` when the ranks disagree or one of them failed."""


def band_check(B: int, H: int, W: int, h: int, hd: int, r: int, dtype: torch.dtype, *, group=None,
               error: Optional[BaseException] = None) -> None:
    """Host-side handshake before a band call (no device work, nothing enqueued on a stream).

    Every rank contributes the arguments it is about to use and, if its own preparation failed, the
    error (pass the exception instead of raising it, so that the rank still takes part).  If any
    rank reports an error or the arguments differ, EVERY rank raises BandArgumentError before any
    collective on device data starts.  A rank that died or never calls makes the others' gather fail
    once the process group's timeout expires: create the group with a short timeout
    (``dist.new_group(timeout=...)`` / ``init_process_group(timeout=...)``) to bound that wait.
    """
    world = dist.get_world_size(group)
    mine = {"args": (B, H, W, h, hd, r, str(dtype)), "error": None if error is None else f"{type(error).__name__}: {error}"}
    everyone = [None] * world
    dist.all_gather_object(everyone, mine, group=group)
    failed = [(p, e["error"]) for p, e in enumerate(everyone) if e["error"] is not None]
    if failed:
        raise BandArgumentError("rank(s) failed before the band call: " + "; ".join(f"rank {p}: {e}" for p, e in failed))
    if any(e["args"] != everyone[0]["args"] for e in everyone):
        raise BandArgumentError("ranks disagree on the band call's arguments: "
                                + "; ".join(f"rank {p}: {e['args']}" for p, e in enumerate(everyone)))


def _exchange_rows(fulls: List[torch.Tensor], H: int, W: int, r: int, world: int, rank: int, group,
                   max_abs_dy: Optional[float], peer) -> None:
    """Complete the [B, H*W, C] buffers `fulls` in place.  On entry each holds this rank's own rows
    [r0, r1); on return it also holds every other rank's rows (all-gather) or, with `max_abs_dy`, the
    rows this rank's band can reach (halo rows from the neighbouring ranks).  Rows move straight between
    the buffers, item by item (an item's rows are contiguous): no staging copies."""
    if world == 1:
        return
    B = fulls[0].size(0)
    r0, r1 = band_rows(H, world, rank)
    if max_abs_dy is None and H % world == 0 and fulls[0].is_cuda:
        for full in fulls:                         # in-place all-gather: the input is the output's own slice
            for b in range(B):
                dist.all_gather_into_tensor(full[b], full[b, r0 * W:r1 * W], group=group)
        return
    ops = []
    for p in range(world):
        if p == rank:
            continue
        p0, p1 = band_rows(H, world, p)
        if max_abs_dy is None:
            need_me, need_p = (r0, r1), (p0, p1)   # uneven bands (or a CPU group): every band to every rank
        else:
            h0, h1 = halo_rows(H, p0, p1, r, max_abs_dy)
            need_me = (max(h0, r0), min(h1, r1))   # rows of mine that p can reach
            g0, g1 = halo_rows(H, r0, r1, r, max_abs_dy)
            need_p = (max(g0, p0), min(g1, p1))    # rows of p that I can reach
        for full in fulls:
            for b in range(B):
                if need_me[1] > need_me[0]:
                    ops.append(dist.P2POp(dist.isend, full[b, need_me[0] * W:need_me[1] * W], peer(p), group))
                if need_p[1] > need_p[0]:
                    ops.append(dist.P2POp(dist.irecv, full[b, need_p[0] * W:need_p[1] * W], peer(p), group))
    _p2p(ops)


class PeerBuffers:
    """Full-size key / value buffers [B, H*W, C] of every rank, each mapped into every process of the group
    (CUDA peer access over NVLink / NVSwitch through torch's symmetric memory; plain loads and copies, no
    multicast object is created).  Construct it once, collectively, on every rank; a rank's producer writes
    its own rows into ``local[0]`` (K) and ``local[1]`` (V) and passes them as k and v to
    :func:`band_match_attention_resident` together with ``peers=this``."""

    def __init__(self, B: int, N: int, C: int, dtype: torch.dtype, device: torch.device, group=None, count: int = 2):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # peer copies only
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.shape, self.dtype = (B, N, C), dtype
        self.local, self._handles = [], []
        for _ in range(count):
            t = symm.empty(B, N, C, dtype=dtype, device=device)
            self._handles.append(symm.rendezvous(t, self.group))
            self.local.append(t)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        # The pulls and the meetings run beside the band's kernels, which fill every SM: on streams of
        # ordinary priority the one-block all-reduce of a meeting is dispatched only after the blocks of
        # a kernel launched before it (measured: 0.3 ms per meeting at 2 GPUs).  Hence a high-priority
        # stream here and, when the group is the whole job, an NCCL communicator of its own for the
        # meetings whose internal stream has high priority too.
        self.stream = torch.cuda.Stream(device=device, priority=-1)
        self._meet_group = self.group
        if self.group is dist.group.WORLD and dist.get_backend(self.group) == "nccl":
            try:
                options = dist.ProcessGroupNCCL.Options()
                options.is_high_priority_stream = True
                self._meet_group = dist.new_group(backend="nccl", pg_options=options)
            except Exception:
                self._meet_group = self.group
        self._plans = {}
        # Halo rows by the copy engines (False: the SMs stay with the interior rows) or by a copy kernel with
        # plain peer loads (True).  None chooses per call: the kernel when the band's interior is smaller
        # than its edges (measured at 8 GPUs, 56 interior rows of 128: 0.32 against 0.36 ms), the copy
        # engines otherwise (2 GPUs, 440 of 512: 0.68 against 0.69 ms).
        self.copy_by_kernel = None

    @property
    def multicast_bound(self) -> bool:
        """True if the mapping also created an NVLink multicast address (not used by this module; it is
        asked not to through TORCH_SYMM_MEM_DISABLE_MULTICAST)."""
        return any(int(getattr(hdl, "multicast_ptr", 0) or 0) != 0 for hdl in self._handles)

    def remote(self, index: int, rank: int) -> torch.Tensor:
        """Rank `rank`'s buffer number `index`, as a tensor of this process."""
        return self._handles[index].get_buffer(rank, self.shape, self.dtype)

    def meet(self) -> None:
        """Stream-ordered meeting of the ranks (a one-word all-reduce): when it has run on this rank's
        stream, everything every rank had enqueued before its own call has run."""
        dist.all_reduce(self._flag, group=self._meet_group)


def _halo_copy_plan(peers: PeerBuffers, H: int, W: int, r: int, world: int, rank: int, max_abs_dy: float):
    """The device-to-device copies that bring the rows this rank's band can reach out of the neighbouring
    ranks' buffers into its own: one per tensor, item and neighbour (the rows of an item are contiguous).
    Built once per geometry (the mapped buffers do not move) as the argument arrays of
    matchattn_copy_blocks; returns (dst, src, nbytes, count, total_bytes)."""
    import ctypes
    key = (H, W, r, world, rank, float(max_abs_dy))
    plan = peers._plans.get(key)
    if plan is None:
        r0, r1 = band_rows(H, world, rank)
        g0, g1 = halo_rows(H, r0, r1, r, max_abs_dy)
        B, N, C = peers.shape
        esz = peers.local[0].element_size()
        dst, src, nbytes = [], [], []
        for p in range(world):
            if p == rank:
                continue
            p0, p1 = band_rows(H, world, p)
            lo, hi = max(g0, p0), min(g1, p1)
            if hi <= lo:
                continue
            for index, mine in enumerate(peers.local):
                theirs = peers.remote(index, p)
                for b in range(B):
                    off = (b * N + lo * W) * C * esz
                    dst.append(mine.data_ptr() + off)
                    src.append(theirs.data_ptr() + off)
                    nbytes.append((hi - lo) * W * C * esz)
        n = len(dst)
        plan = ((ctypes.c_void_p * n)(*dst), (ctypes.c_void_p * n)(*src), (ctypes.c_size_t * n)(*nbytes), n, sum(nbytes))
        peers._plans[key] = plan
    return plan


def _pull_halo_rows(peers: PeerBuffers, H: int, W: int, r: int, world: int, rank: int, max_abs_dy: float,
                    pulled_event: Optional[torch.cuda.Event] = None) -> int:
    """Pull the halo rows on the current stream, between two meetings of the ranks: the first says every
    rank's own rows are in place, the second that every pull is done (producers may write their rows
    again).  `pulled_event` is recorded between this rank's copies and the second meeting.  Returns the
    number of bytes pulled."""
    from . import _lib
    dst, src, nbytes, count, total = _halo_copy_plan(peers, H, W, r, world, rank, max_abs_dy)
    by_kernel = peers.copy_by_kernel
    if by_kernel is None:
        r0, r1 = band_rows(H, world, rank)
        i0, i1 = interior_rows(H, r0, r1, r, max_abs_dy)
        by_kernel = 2 * (i1 - i0) < (r1 - r0)
    peers.meet()
    with torch.cuda.device(peers.local[0].device):
        _lib.check(_lib.lib.matchattn_copy_blocks(dst, src, nbytes, count, int(bool(by_kernel)),
                                                  torch.cuda.current_stream().cuda_stream))
    if pulled_event is not None:
        pulled_event.record()
    peers.meet()
    return total


def _peer_band_call(peers: PeerBuffers, mo_band, q_band, H, W, r, scale, world, rank, max_abs_dy, need_attn, out, attn_out):
    """The band with its halo pulled by peer copies on a second stream while the interior rows (whose windows
    stay inside the band's own rows) are computed; the edge rows follow the copies.  Launches are per
    item and per part (an item's rows of a part are contiguous), straight through the C ABI."""
    from . import _lib
    from .ops import _DTYPE_CODE
    B, Nq, C = q_band.shape
    h = mo_band.size(2)
    r0, r1 = band_rows(H, world, rank)
    k, v = peers.local
    M = (2 * r + 2) ** 2
    if out is None:
        out = torch.empty_like(q_band)
    if need_attn and attn_out is None:
        attn_out = q_band.new_empty(B, Nq, h, M)
    for name, t, shape in (("max_offset", mo_band, (B, Nq, h, 2)), ("q", q_band, (B, Nq, C)), ("out", out, (B, Nq, C)),
                           ("attn_out", attn_out if need_attn else None, (B, Nq, h, M))):
        if t is None:
            continue
        if (tuple(t.shape) != shape or t.dtype != k.dtype or t.device != k.device or not t.is_contiguous()):
            raise ValueError(f"{name}: expected a contiguous {shape} tensor of the buffers' dtype on their device")
    if Nq != (r1 - r0) * W or C % h != 0 or tuple(k.shape) != (B, H * W, C):
        raise ValueError("band tensors do not match the geometry of the peer buffers")
    esz, code = q_band.element_size(), _DTYPE_CODE[q_band.dtype]
    main = torch.cuda.current_stream(q_band.device)
    pulled = torch.cuda.Event()
    peers.stream.wait_stream(main)                  # this rank's producer has written its rows
    with torch.cuda.stream(peers.stream):
        _pull_halo_rows(peers, H, W, r, world, rank, max_abs_dy, pulled)

    fwd, stream_ptr = _lib.lib.matchattn_fused_forward, main.cuda_stream
    mo_p, q_p, k_p, v_p, out_p = (t.data_ptr() for t in (mo_band, q_band, k, v, out))
    attn_p = attn_out.data_ptr() if need_attn else None

    def part(a, b):
        if b <= a:
            return
        for i in range(B):
            first = i * Nq + (a - r0) * W                        # first query of the part within the band tensors
            _lib.check(fwd(mo_p + first * h * 2 * esz, q_p + first * C * esz, k_p + i * H * W * C * esz,
                           v_p + i * H * W * C * esz, out_p + first * C * esz,
                           attn_p + first * h * M * esz if need_attn else None,
                           1, H, W, h, C // h, r, r, code, _lib.L1_NORM, float(scale), a, b, stream_ptr))

    i0, i1 = interior_rows(H, r0, r1, r, max_abs_dy)
    with torch.cuda.device(q_band.device):
        part(i0, i1)
        main.wait_event(pulled)
        part(r0, i0)
        part(i1, r1)
    main.wait_stream(peers.stream)                  # the second meeting: nobody still reads this rank's rows
    return out, (attn_out if need_attn else None)


def band_match_attention_resident(mo_band: torch.Tensor, q_band: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                  H: int, W: int, r: int, scale: float, *, group=None, need_attn: bool = True,
                                  op: Optional[Callable] = None, kv_full=None, max_abs_dy: Optional[float] = None,
                                  out=None, attn_out=None, peers: Optional["PeerBuffers"] = None):
    """One MatchAttention call over row bands that already live on their ranks.

    Every rank passes ITS rows [r0, r1) = band_rows(H, world, rank) of max_offset [B,rows*W,h,2] and of
    q [B,rows*W,C], and gets back its rows of (out, attn).  Keys and values come in one of two layouts:

    * resident (no copies): `k` and `v` are full-size [B,H*W,C] buffers in which this rank's producer
      has written its own rows in place; the other rows are scratch that this call fills;
    * bands: `k` and `v` are [B,rows*W,C]; they are first copied into `kv_full` (a pair of full-size
      buffers, allocated when None and reusable between calls).

    The missing rows arrive by an all-gather of the bands or -- with `max_abs_dy`, the caller's bound in
    rows on |centre_y - query row| -- only the halo rows each band can reach travel between neighbouring
    ranks; rows outside stay untouched and are never read.  The kernel follows on the rank's own stream.
    With `peers` (and `max_abs_dy`), k and v must be ``peers.local`` and the halo rows are pulled out of
    the neighbours' memory by peer copies instead of NCCL send / receive.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    op = op or _default_op
    B, _, C = q_band.shape
    r0, r1 = band_rows(H, world, rank)
    if k.size(1) == H * W and (world == 1 or r1 - r0 != H):
        fulls = [k, v]                              # resident layout
    else:
        if kv_full is None:
            kv_full = [torch.empty((B, H * W, C), dtype=q_band.dtype, device=q_band.device) for _ in range(2)]
        fulls = list(kv_full)
        fulls[0][:, r0 * W:r1 * W] = k
        fulls[1][:, r0 * W:r1 * W] = v

    def peer(p):
        return dist.get_global_rank(group, p) if group is not None else p

    if peers is not None and world > 1:
        if max_abs_dy is None or k is not peers.local[0] or v is not peers.local[1]:
            raise ValueError("peers: pass max_abs_dy, and peers.local[0] / peers.local[1] as k / v")
        if op is _default_op and r1 > r0:
            return _peer_band_call(peers, mo_band, q_band, H, W, r, scale, world, rank, max_abs_dy, need_attn,
                                   out, attn_out)
        _pull_halo_rows(peers, H, W, r, world, rank, max_abs_dy)
    else:
        _exchange_rows(fulls, H, W, r, world, rank, group, max_abs_dy, peer)
    if r1 == r0:
        return None, None
    if op is _default_op:
        from .ops import match_attention
        return match_attention(mo_band, q_band, fulls[0], fulls[1], H, W, r, scale, need_attn=need_attn,
                               q_row_begin=r0, q_row_end=r1, out=out, attn_out=attn_out)
    return op(mo_band, q_band, fulls[0], fulls[1], H, W, r, scale, r0, r1, need_attn)
