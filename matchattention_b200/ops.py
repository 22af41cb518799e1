"""Host side of the B200 MatchAttention operator.

Mirrors the reference's operator interface for this path
(models/match_former_ops.py and the native module it imports):

* :func:`fused_forward` -- same 12 positional arguments and in-place contract
  as ``match_attention.fused_forward`` (models/src/match_former_cuda.cpp:24-44);
* ``torch.ops.matchattn_b200.fused_forward_ops`` -- opaque custom op with a fake
  kernel, the counterpart of ``match_attention::fused_forward_ops``
  (models/match_former_ops.py:6-62);
* :class:`MF_FusedForwardOps` -- module with the reference's ``forward``
  signature and return values (models/match_former_ops.py:65-121).

Differences, all on the safe side: arguments are validated (shape, dtype,
device, contiguity) and violations raise; the launch goes to PyTorch's current
stream; nothing is allocated or synchronised inside the call; outputs need not
be zero-filled.  Inputs must be CUDA tensors: there is no CPU path.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn as nn

import os

from . import _lib

# MATCHATTN_B200_NVTX=1 wraps every operator launch in an NVTX range named after its shape, so that a
# profiler's NVTX filter can pick the operator out of a model's timeline (off by default: two extra calls)
_NVTX = os.environ.get("MATCHATTN_B200_NVTX", "0") not in ("", "0")

_DTYPE_CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _window_radius(win_r) -> Tuple[int, int]:
    if isinstance(win_r, int):
        return win_r, win_r
    if len(win_r) != 2:
        raise ValueError(f"win_r must have two entries, got {win_r!r}")
    return int(win_r[0]), int(win_r[1])


def _check_tensors(max_offset, q, k, v, output, attn_out, H, W, rows, attn_num):
    if not q.is_cuda:
        raise RuntimeError("matchattn_b200 runs on CUDA tensors only (no CPU fallback); got device " + str(q.device))
    if q.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {q.dtype}: float32, float16 or bfloat16")
    if q.dim() != 3 or max_offset.dim() != 4 or max_offset.size(-1) != 2:
        raise ValueError("expected q [B,N,C] and max_offset [B,N,h,2]")
    B, Nq, C = q.shape
    h = max_offset.size(2)
    if C % h != 0:
        raise ValueError(f"C={C} is not a multiple of the head count h={h}")
    if Nq != rows * W:
        raise ValueError(f"q has {Nq} queries per item, expected rows*W = {rows}*{W}")
    expect = {"max_offset": (max_offset, (B, Nq, h, 2)), "k": (k, (B, H * W, C)), "v": (v, (B, H * W, C)),
              "output": (output, (B, Nq, C))}
    if attn_out is not None:
        expect["attn_out"] = (attn_out, (B, Nq, h, attn_num))
    expect["q"] = (q, (B, Nq, C))
    for name, (t, shape) in expect.items():
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
        if t.dtype != q.dtype:
            raise TypeError(f"{name} has dtype {t.dtype}, expected {q.dtype}")
        if t.device != q.device:
            raise RuntimeError(f"{name} is on {t.device}, expected {q.device}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    return B, h, C // h


STRATEGY_AUTO, STRATEGY_DIRECT, STRATEGY_BINNED = 0, 1, 2
STRATEGY_STAGED = 5
STRATEGY_STAGED_BLOCKS = 6

# scratch for the binned path, one buffer per (device, stream): calls on one stream are ordered, so
# they can share it; calls on different streams may overlap on the device and must not
_workspaces = {}


def workspace_bytes(B: int, H: int, W: int, h: int, hd: int, r: int, dtype: torch.dtype, q_row_begin: int = 0,
                    q_row_end: Optional[int] = None) -> int:
    """Scratch bytes the binned path needs for these sizes (0: it does not apply)."""
    return int(_lib.lib.matchattn_workspace_bytes(B, H, W, h, hd, r, _DTYPE_CODE[dtype], q_row_begin,
                                                  H if q_row_end is None else q_row_end))


def _workspace(device: torch.device, stream_id: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream_id)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def launch(max_offset, q, k, v, output, attn_out, H: int, W: int, win_r, attn_type: str = "l1_norm",
           scale: float = 1.0, q_row_begin: int = 0, q_row_end: Optional[int] = None, *,
           tile_w: int = 0, force_generic: bool = False, chunks_per_lane: int = 0, variant: int = 0,
           strategy: int = STRATEGY_AUTO, workspace: Optional[torch.Tensor] = None) -> None:
    """Validate, then enqueue the operator on the current stream of q's device.

    ``attn_out`` may be None (the attention weights are then not written).  With
    a row band, the query-side tensors hold rows [q_row_begin, q_row_end) only.
    ``strategy``: 0 lets the library choose (currently the direct kernel), 1 forces
    the direct kernel, 2 the binned path (queries sorted by target tile, K/V tiles
    staged in shared memory; 16-bit types, r = 1, head width <= 40), 5 the staged path (per tile of
    queries the K/V region its windows fall into is copied to shared memory by the tensor memory
    accelerator; tiles whose windows spread too far use global loads; 16-bit types, r = 1, head width 8 or
    16, at most 16 heads).  The binned path needs scratch
    memory: ``workspace`` (a uint8 CUDA tensor) or, when strategy >= 2 is asked for without one, a
    buffer this module allocates once per (device, stream) and keeps; strategy 0 and 1 allocate
    nothing.  The tuning knobs (tile_w, force_generic, chunks_per_lane, variant) belong to the
    direct kernels and imply strategy 1.
    """
    rx, ry = _window_radius(win_r)
    if q_row_end is None:
        q_row_end = H
    if attn_type not in _lib.ATTN_TYPE_CODE:
        raise NotImplementedError(f"attn_type {attn_type!r}: 'l1_norm' and 'dot_product' exist")
    attn_num = (2 * rx + 2) * (2 * ry + 2)
    B, h, hd = _check_tensors(max_offset, q, k, v, output, attn_out, H, W, q_row_end - q_row_begin, attn_num)
    knobs = tile_w or force_generic or chunks_per_lane or variant
    if knobs and strategy == STRATEGY_BINNED:
        raise ValueError("the direct-kernel knobs cannot be combined with strategy=2")
    if _NVTX:
        torch.cuda.nvtx.range_push(f"matchattn_b200 B{B} {H}x{W} h{h}x{hd} r{rx} {str(q.dtype)[6:]}")
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        args = (max_offset.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(),
                attn_out.data_ptr() if attn_out is not None else None,
                B, H, W, h, hd, rx, ry, _DTYPE_CODE[q.dtype], _lib.ATTN_TYPE_CODE[attn_type], float(scale),
                q_row_begin, q_row_end, stream)
        if knobs or strategy == STRATEGY_DIRECT:
            status = _lib.lib.matchattn_fused_forward_ex(*args, int(tile_w), int(bool(force_generic)),
                                                         int(chunks_per_lane), int(variant))
        elif strategy == STRATEGY_AUTO and workspace is None:
            # the library's own choice needs no scratch: nothing is looked up or allocated here
            status = _lib.lib.matchattn_fused_forward(*args)
        elif strategy in (STRATEGY_STAGED, STRATEGY_STAGED_BLOCKS):
            # needs no scratch; an 8-byte workspace, if given, receives the number of tiles that were
            # served by global loads because their windows did not fit the staged region
            ws_ptr, ws_len = (workspace.data_ptr(), workspace.numel()) if workspace is not None else (None, 0)
            status = _lib.lib.matchattn_fused_forward_ws(*args, ws_ptr, ws_len, int(strategy))
        else:
            need = workspace_bytes(B, H, W, h, hd, rx, q.dtype, q_row_begin, q_row_end) if rx == ry else 0
            ws_ptr, ws_len = None, 0
            if need:
                if workspace is None:
                    workspace = _workspace(q.device, stream, need)
                if workspace.device != q.device or workspace.dtype != torch.uint8 or not workspace.is_contiguous():
                    raise ValueError("workspace must be a contiguous uint8 tensor on q's device")
                ws_ptr, ws_len = workspace.data_ptr(), workspace.numel()
            status = _lib.lib.matchattn_fused_forward_ws(*args, ws_ptr, ws_len, int(strategy))
    if _NVTX:
        torch.cuda.nvtx.range_pop()
    _lib.check(status)


def launch_checked(max_offset, q, k, v, output, attn_out, H: int, W: int, r: int, scale: float):
    """The operator through matchattn_fused_forward_checked: every index is checked on the device.
    Returns (violations, first_offender) after synchronising; both 0 for a healthy kernel."""
    attn_num = (2 * r + 2) ** 2
    B, h, hd = _check_tensors(max_offset, q, k, v, output, attn_out, H, W, H, attn_num)
    status_words = torch.empty(2, dtype=torch.int64, device=q.device)
    with torch.cuda.device(q.device):
        status = _lib.lib.matchattn_fused_forward_checked(
            max_offset.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(),
            attn_out.data_ptr() if attn_out is not None else None, B, H, W, h, hd, r, r, _DTYPE_CODE[q.dtype],
            _lib.L1_NORM, float(scale), 0, H, status_words.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(status)
    words = status_words.cpu()
    return int(words[0]), int(words[1])


def fused_forward(max_offset, q, k, v, output, attn_out, H, W, win_r, attn_num, attn_type, scale) -> None:
    """Drop-in for ``match_attention.fused_forward`` (same 12 positional arguments,
    writes ``output`` and ``attn_out`` in place, returns None)."""
    rx, ry = _window_radius(win_r)
    if attn_num != (2 * rx + 2) * (2 * ry + 2):
        raise ValueError(f"attn_num={attn_num} does not match win_r={list(win_r)}")
    launch(max_offset, q, k, v, output, attn_out, int(H), int(W), (rx, ry), attn_type, float(scale))


@torch.library.custom_op("matchattn_b200::fused_forward_ops", mutates_args={"output", "attn_out"})
def fused_forward_ops(max_offset: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      output: torch.Tensor, attn_out: torch.Tensor, H: int, W: int, win_r: List[int],
                      attn_num: int, attn_type: str, scale: float) -> None:
    fused_forward(max_offset, q, k, v, output, attn_out, H, W, win_r, attn_num, attn_type, scale)


@fused_forward_ops.register_fake
def _(max_offset, q, k, v, output, attn_out, H, W, win_r, attn_num, attn_type, scale):
    B, N, C = q.shape
    h = max_offset.size(2)
    torch._check(output.shape == (B, N, C), lambda: f"output shape {output.shape}, expected {(B, N, C)}")
    torch._check(attn_out.shape == (B, N, h, attn_num),
                 lambda: f"attn_out shape {attn_out.shape}, expected {(B, N, h, attn_num)}")
    torch._check(output.dtype == q.dtype and attn_out.dtype == q.dtype, lambda: "output dtypes must equal q's")
    torch._check(output.device == q.device and attn_out.device == q.device, lambda: "outputs must be on q's device")
    return None


class MF_FusedForwardOps(nn.Module):
    """Same call and return values as the reference module of this name
    (models/match_former_ops.py:65-121); outputs are allocated uninitialised
    because the kernel overwrites every element.  Unlike the reference's module it can be trained through:
    when an input requires a gradient the call goes through match_attention_autograd."""

    def forward(self, max_offset: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, H: int, W: int,
                win_r: List[int], attn_num: int, attn_type: str = "l1_norm",
                scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
        if torch.is_grad_enabled() and any(t.requires_grad for t in (max_offset, q, k, v)):
            rx, ry = _window_radius(win_r)
            if attn_type != "l1_norm" or rx != ry:
                raise NotImplementedError("training needs attn_type 'l1_norm' and a square window")
            return match_attention_autograd(max_offset, q, k, v, int(H), int(W), rx, scale)
        B, N, _ = q.shape
        h = max_offset.size(2)
        output = torch.empty_like(v)
        attn_out = q.new_empty([B, N, h, attn_num])
        fused_forward_ops(max_offset, q, k, v, output, attn_out, H, W, list(win_r), attn_num, attn_type, scale)
        return output, attn_out


def match_attention(max_offset, q, k, v, H: int, W: int, r: int, scale: float, *, need_attn: bool = True,
                    q_row_begin: int = 0, q_row_end: Optional[int] = None, out=None, attn_out=None,
                    attn_type: str = "l1_norm", **knobs):
    """Functional form: allocates (or reuses) the outputs and returns (out, attn or None)."""
    B, Nq, _ = q.shape
    h = max_offset.size(2)
    if out is None:
        out = torch.empty_like(q)
    if need_attn and attn_out is None:
        attn_out = q.new_empty([B, Nq, h, (2 * r + 2) ** 2])
    launch(max_offset, q, k, v, out, attn_out if need_attn else None, H, W, (r, r), attn_type, scale,
           q_row_begin, q_row_end, **knobs)
    return out, (attn_out if need_attn else None)


def describe_dispatch(h: int, hd: int, r: int, dtype: torch.dtype, aligned32: bool = True) -> Optional[str]:
    res = _lib.lib.matchattn_describe_dispatch(h, hd, r, _DTYPE_CODE[dtype], int(aligned32))
    return res.decode() if res is not None else None


# ---- training: the operator as an autograd function ------------------------------------------------

class _MatchAttentionFn(torch.autograd.Function):
    """Forward = the fused kernel; backward = matchattn_fused_backward.  Nothing but the inputs is saved:
    the backward kernel recomputes scores and softmaxes."""

    @staticmethod
    def forward(ctx, max_offset, q, k, v, H, W, r, scale):
        out = torch.empty_like(q)
        attn = q.new_empty(q.size(0), q.size(1), max_offset.size(2), (2 * r + 2) ** 2)
        launch(max_offset, q, k, v, out, attn, H, W, (r, r), "l1_norm", scale)
        ctx.save_for_backward(max_offset, q, k, v)
        ctx.geometry = (H, W, r, scale)
        return out, attn

    @staticmethod
    def backward(ctx, d_out, d_attn):
        max_offset, q, k, v = ctx.saved_tensors
        H, W, r, scale = ctx.geometry
        B, Nq, C = q.shape
        h = max_offset.size(2)
        d_q = torch.empty_like(q)
        d_mo = torch.empty_like(max_offset) if ctx.needs_input_grad[0] else None
        d_k = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        d_v = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
        d_out = d_out.contiguous()
        d_attn = d_attn.contiguous() if d_attn is not None else None
        with torch.cuda.device(q.device):
            status = _lib.lib.matchattn_fused_backward(
                max_offset.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), d_out.data_ptr(),
                d_attn.data_ptr() if d_attn is not None else None, d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(),
                d_mo.data_ptr() if d_mo is not None else None, B, H, W, h, C // h, r, r, _DTYPE_CODE[q.dtype],
                _lib.L1_NORM, float(scale), 0, H, torch.cuda.current_stream().cuda_stream)
        _lib.check(status)
        return d_mo, d_q, d_k.to(k.dtype), d_v.to(v.dtype), None, None, None, None


def match_attention_autograd(max_offset, q, k, v, H: int, W: int, r: int, scale: float):
    """The operator for training: (out, attn) with gradients to q, k, v and max_offset, as autograd gives them
    for the reference's 'pytorch' path (its native path has no backward).  Contiguous CUDA tensors."""
    return _MatchAttentionFn.apply(max_offset.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), H, W, r,
                                   float(scale))


# ---- the caller's glue folded into the kernel ------------------------------------------------

def launch_glue(max_offset, q, k, v, gate, out_base, attn_base, H: int, W: int, r: int, scale: float, *,
                clamp: bool, out_stride: int = 0, attn_stride: int = 0, kv_shift: int = 0) -> None:
    """Enqueue the direct kernel with clamp / gate / strided outputs (see matchattn_fused_forward_glue)."""
    B, Nq, C = q.shape
    h = max_offset.size(2)
    M = (2 * r + 2) ** 2
    for name, t in (("max_offset", max_offset), ("q", q), ("k", k), ("v", v), ("gate", gate)):
        if t is None:
            continue
        if not t.is_cuda or t.dtype != q.dtype or t.device != q.device or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor of q's dtype on q's device")
    if tuple(max_offset.shape) != (B, Nq, h, 2) or tuple(k.shape) != (B, H * W, C) or tuple(v.shape) != (B, H * W, C) \
            or Nq != H * W or (gate is not None and tuple(gate.shape) != (B, Nq, C)):
        raise ValueError("shape mismatch")
    with torch.cuda.device(q.device):
        status = _lib.lib.matchattn_fused_forward_glue(
            max_offset.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
            gate.data_ptr() if gate is not None else None, out_base, attn_base,
            B, H, W, h, C // h, r, r, _DTYPE_CODE[q.dtype], _lib.L1_NORM, float(scale), 0, H,
            int(bool(clamp)), int(out_stride), int(attn_stride), int(kv_shift),
            torch.cuda.current_stream().cuda_stream)
    _lib.check(status)


def cross_attention_core(max_offset, q, k, v, gate, H: int, W: int, r: int, scale: float, clamp: bool = True,
                         kv_shift: int = 0):
    """What MatchAttention.forward does between its q/k/v/g projections and its output projection in
    the cross branch (models/attention_blocks.py:79-98), in one kernel: clamp the centres, run the
    operator, multiply by the gate and lay the result out as cat((g * x, attn), -1).

    ``kv_shift`` folds the branch's batch swap in as well: item b attends to the keys / values of item
    (b + kv_shift) mod B, so with B // 2 the caller passes K and V of the un-swapped batch.

    Returns a [B, N, C + h*(2r+2)^2] tensor ready for ``proj``."""
    B, N, C = q.shape
    h = max_offset.size(2)
    M = (2 * r + 2) ** 2
    width = C + h * M
    buf = q.new_empty(B, N, width)
    launch_glue(max_offset, q, k, v, gate, buf.data_ptr(), buf.data_ptr() + C * buf.element_size(), H, W, r, scale,
                clamp=clamp, out_stride=width, attn_stride=width, kv_shift=kv_shift)
    return buf


def self_attention_core(max_offset, q, k, v, H: int, W: int, r: int, scale: float, clamp: bool = True):
    """The self branch (models/attention_blocks.py:79-93,99): clamp + operator; the attention weights,
    which that branch discards, are never written.  Returns out [B, N, C]."""
    out = torch.empty_like(q)
    launch_glue(max_offset, q, k, v, None, out.data_ptr(), None, H, W, r, scale, clamp=clamp)
    return out


def upsample_field(field: torch.Tensor, mask: torch.Tensor, factor: int) -> torch.Tensor:
    """Convex upsampling of a field, same arguments and result as ``MatchStereo.upsample_field``
    (models/match_stereo.py:73-84): field [B,H,W,D], mask [B,9*f*f,H,W] -> [B,f*H,f*W,D], one kernel."""
    if not field.is_cuda:
        raise RuntimeError("matchattn_b200 runs on CUDA tensors only (no CPU fallback); got device " + str(field.device))
    if field.dtype not in _DTYPE_CODE or mask.dtype != field.dtype or mask.device != field.device:
        raise TypeError("field and mask must share a supported dtype (float32, float16, bfloat16) and device")
    if field.dim() != 4 or mask.dim() != 4:
        raise ValueError("expected field [B,H,W,D] and mask [B,9*f*f,H,W]")
    B, H, W, D = field.shape
    if tuple(mask.shape) != (B, 9 * factor * factor, H, W):
        raise ValueError(f"mask has shape {tuple(mask.shape)}, expected {(B, 9 * factor * factor, H, W)}")
    field, mask = field.contiguous(), mask.contiguous()
    out = field.new_empty(B, H * factor, W * factor, D)
    with torch.cuda.device(field.device):
        status = _lib.lib.matchattn_upsample_field(field.data_ptr(), mask.data_ptr(), out.data_ptr(), B, H, W, D,
                                                   int(factor), _DTYPE_CODE[field.dtype],
                                                   torch.cuda.current_stream().cuda_stream)
    _lib.check(status)
    return out


STEREO_VOLUME_MAX_W = 159      # the row's W x W slice must fit the kernel's shared memory


def stereo_volume(correlation: torch.Tensor) -> torch.Tensor:
    """The cost volume GlobalCorrelation builds from its row-wise correlation in the stereo branch
    (models/cost_volume.py:26-51): correlation [B,H,W,W] -> volume [2B,W,H,W] (softmaxed over the
    disparity axis, out-of-view columns filled), one kernel instead of the loops over disparities."""
    if not correlation.is_cuda:
        raise RuntimeError("matchattn_b200 runs on CUDA tensors only (no CPU fallback); got device "
                           + str(correlation.device))
    if correlation.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {correlation.dtype}")
    if correlation.dim() != 4 or correlation.size(2) != correlation.size(3):
        raise ValueError("expected correlation [B,H,W,W]")
    corr = correlation.contiguous()
    B, H, W, _ = corr.shape
    vol = corr.new_empty(2 * B, W, H, W)
    with torch.cuda.device(corr.device):
        status = _lib.lib.matchattn_stereo_volume(corr.data_ptr(), vol.data_ptr(), B, H, W, _DTYPE_CODE[corr.dtype],
                                                  torch.cuda.current_stream().cuda_stream)
    _lib.check(status)
    return vol


def consistency_mask(field: torch.Tensor, threshold: float = 2.0, return_diff: bool = False):
    """Same argument and result as ``MatchAttentionLayer.consistency_mask(field, A)``
    (models/attention_blocks.py:130-138): field [B,H,W,2] (two views stacked on the batch) ->
    noc_mask [B,H,W,1], one kernel.  ``return_diff`` also returns the thresholded quantity."""
    if not field.is_cuda:
        raise RuntimeError("matchattn_b200 runs on CUDA tensors only (no CPU fallback); got device " + str(field.device))
    if field.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {field.dtype}")
    if field.dim() != 4 or field.size(-1) != 2 or field.size(0) % 2:
        raise ValueError("expected field [B,H,W,2] with an even batch (two views)")
    field = field.contiguous()
    B, H, W, _ = field.shape
    mask = field.new_empty(B, H, W, 1)
    diff = field.new_empty(B, H, W, 1) if return_diff else None
    with torch.cuda.device(field.device):
        status = _lib.lib.matchattn_consistency_mask(field.data_ptr(), mask.data_ptr(),
                                                     diff.data_ptr() if return_diff else None, B, H, W,
                                                     float(threshold), _DTYPE_CODE[field.dtype],
                                                     torch.cuda.current_stream().cuda_stream)
    _lib.check(status)
    return (mask, diff) if return_diff else mask


def local_disparity_estimator(volume: torch.Tensor, return_debug: bool = False):
    """Same argument and result as ``local_disparity_estimator(cv)`` (models/cost_volume.py:123-167, with
    disp_to_flow :169-178): cost volume [B,D,H,W] -> field [B,H,W,2], one kernel.  ``return_debug``
    also returns the blurred maximum [B,H,W] and the window centre [B,H,W] (int32)."""
    if not volume.is_cuda:
        raise RuntimeError("matchattn_b200 runs on CUDA tensors only (no CPU fallback); got device " + str(volume.device))
    if volume.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {volume.dtype}")
    if volume.dim() != 4 or volume.size(0) % 2 or volume.size(1) < 5:
        raise ValueError("expected volume [B,D,H,W] with an even batch (two views) and D >= 5")
    vol = volume.contiguous()
    B, D, H, W = vol.shape
    flow = vol.new_empty(B, H, W, 2)
    blur = vol.new_empty(B, H, W) if return_debug else None
    centre = torch.empty(B, H, W, dtype=torch.int32, device=vol.device) if return_debug else None
    with torch.cuda.device(vol.device):
        status = _lib.lib.matchattn_local_disparity(vol.data_ptr(), flow.data_ptr(),
                                                    blur.data_ptr() if return_debug else None,
                                                    centre.data_ptr() if return_debug else None, B, D, H, W,
                                                    _DTYPE_CODE[vol.dtype], torch.cuda.current_stream().cuda_stream)
    _lib.check(status)
    return (flow, blur, centre) if return_debug else flow


def flow_init(correlation: torch.Tensor, H: int, W: int, return_debug: bool = False):
    """What GlobalCorrelation.forward does after its matmul when ``stereo=False`` (models/cost_volume.py:61-69,
    with local_flow_estimator :71-121): correlation [B,N,N] (N = H*W) -> (flow [2B,H,W,2], prob [2B,H,W,N]).
    ``return_debug`` adds the pooled maximum [2B,N] and the clamped window centre [2B,N] (int32)."""
    if not correlation.is_cuda:
        raise RuntimeError("matchattn_b200 runs on CUDA tensors only (no CPU fallback); got device "
                           + str(correlation.device))
    if correlation.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {correlation.dtype}")
    if correlation.dim() != 3 or correlation.size(1) != H * W or correlation.size(2) != H * W:
        raise ValueError("expected correlation [B, H*W, H*W]")
    corr = correlation.contiguous()
    B, N, _ = corr.shape
    prob = corr.new_empty(2 * B, H, W, N)
    flow = corr.new_empty(2 * B, H, W, 2)
    blur = corr.new_empty(2 * B, N) if return_debug else None
    centre = torch.empty(2 * B, N, dtype=torch.int32, device=corr.device) if return_debug else None
    nbytes = int(_lib.lib.matchattn_flow_init_scratch_bytes(B, H, W))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=corr.device)
    with torch.cuda.device(corr.device):
        status = _lib.lib.matchattn_flow_init(corr.data_ptr(), prob.data_ptr(), flow.data_ptr(),
                                              blur.data_ptr() if return_debug else None,
                                              centre.data_ptr() if return_debug else None, scratch.data_ptr(), nbytes,
                                              B, H, W, _DTYPE_CODE[corr.dtype], torch.cuda.current_stream().cuda_stream)
    _lib.check(status)
    return (flow, prob, blur, centre) if return_debug else (flow, prob)


# ---- the fused steps as opaque custom ops ------------------------------------------------------
# torch.compile cannot trace a ctypes call.  These wrappers give the compiler the same thing the
# reference gives it for its own extension (models/match_former_ops.py:6-62): an opaque op with a fake
# kernel that only states shapes and dtypes.  Eager callers should keep using the plain functions
# above (one Python dispatch less per call).

@torch.library.custom_op("matchattn_b200::cross_attention_core_op", mutates_args=())
def cross_attention_core_op(max_offset: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                            gate: torch.Tensor, H: int, W: int, r: int, scale: float, clamp: bool,
                            kv_shift: int) -> torch.Tensor:
    return cross_attention_core(max_offset.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(),
                                gate.contiguous(), H, W, r, scale, clamp, kv_shift)


@cross_attention_core_op.register_fake
def _(max_offset, q, k, v, gate, H, W, r, scale, clamp, kv_shift):
    B, N, C = q.shape
    return q.new_empty(B, N, C + max_offset.size(2) * (2 * r + 2) ** 2)


@torch.library.custom_op("matchattn_b200::self_attention_core_op", mutates_args=())
def self_attention_core_op(max_offset: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           H: int, W: int, r: int, scale: float, clamp: bool) -> torch.Tensor:
    return self_attention_core(max_offset.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), H, W, r,
                               scale, clamp)


@self_attention_core_op.register_fake
def _(max_offset, q, k, v, H, W, r, scale, clamp):
    return torch.empty_like(q, memory_format=torch.contiguous_format)


@torch.library.custom_op("matchattn_b200::upsample_field_op", mutates_args=())
def upsample_field_op(field: torch.Tensor, mask: torch.Tensor, factor: int) -> torch.Tensor:
    return upsample_field(field, mask, factor)


@upsample_field_op.register_fake
def _(field, mask, factor):
    B, H, W, D = field.shape
    return field.new_empty(B, H * factor, W * factor, D)


@torch.library.custom_op("matchattn_b200::stereo_volume_op", mutates_args=())
def stereo_volume_op(correlation: torch.Tensor) -> torch.Tensor:
    return stereo_volume(correlation)


@stereo_volume_op.register_fake
def _(correlation):
    B, H, W, _ = correlation.shape
    return correlation.new_empty(2 * B, W, H, W)


@torch.library.custom_op("matchattn_b200::consistency_mask_op", mutates_args=())
def consistency_mask_op(field: torch.Tensor, threshold: float) -> torch.Tensor:
    return consistency_mask(field, threshold)


@consistency_mask_op.register_fake
def _(field, threshold):
    B, H, W, _ = field.shape
    return field.new_empty(B, H, W, 1)


@torch.library.custom_op("matchattn_b200::local_disparity_op", mutates_args=())
def local_disparity_op(volume: torch.Tensor) -> torch.Tensor:
    return local_disparity_estimator(volume)


@local_disparity_op.register_fake
def _(volume):
    B, D, H, W = volume.shape
    return volume.new_empty(B, H, W, 2)


@torch.library.custom_op("matchattn_b200::flow_init_op", mutates_args=())
def flow_init_op(correlation: torch.Tensor, H: int, W: int) -> List[torch.Tensor]:
    return list(flow_init(correlation, H, W))


@flow_init_op.register_fake
def _(correlation, H, W):
    B, N, _ = correlation.shape
    return [correlation.new_empty(2 * B, H, W, 2), correlation.new_empty(2 * B, H, W, N)]
