"""numpy restatement of the MatchAttention operator.  TEST INFRASTRUCTURE ONLY.

Second, independent statement of the algorithm of the reference's 'pytorch'
path (models/mat_pytorch_impl.py:3-178, driven as in
models/attention_blocks.py:82-91).  It walks the window one tap at a time, so
it never builds the [B, N, h, M, hd] gathered copy of K and V that the
reference materialises.  Meant for small cases: it cross-checks the C oracle.

Arrays are float32 or float16.  numpy evaluates a float16 operation in float32
and rounds the result to float16, which is also what eager PyTorch does on
CPU, so the float16 path here rounds in the same places as the reference.
Reductions that the reference accumulates in float32 (the channel sum of the
L1 score, the softmax, the tap sum of the output) are accumulated in float32
here and rounded once.
"""
from __future__ import annotations

import numpy as np


def bilinear_weights(max_offset: np.ndarray) -> np.ndarray:
    """[..., 2] (x, y) -> [..., 4] weights nw, ne, sw, se (mat_pytorch_impl.py:3-27)."""
    dt = max_offset.dtype
    one = dt.type(1)
    frac = max_offset - np.floor(max_offset)
    fx, fy = frac[..., 0], frac[..., 1]
    gx, gy = one - fx, one - fy
    return np.stack([gx * gy, fx * gy, gx * fy, fx * fy], axis=-1).astype(dt)


def forward(max_offset, q, k, v, H: int, W: int, r: int, scale: float, attn_type: str = "l1_norm"):
    """max_offset [B,Nq,h,2], q [B,Nq,C], k/v [B,H*W,C] -> (out [B,Nq,C], attn [B,Nq,h,M])."""
    dt = q.dtype
    assert dt in (np.float32, np.float16)
    B, Nq, C = q.shape
    h = max_offset.shape[2]
    hd = C // h
    side, sub = 2 * r + 2, 2 * r + 1
    M = side * side

    wgt = bilinear_weights(max_offset)                          # [B,Nq,h,4]
    origin = np.floor(max_offset).astype(np.int64)              # attention_blocks.py:82
    x0, y0 = origin[..., 0], origin[..., 1]                     # [B,Nq,h]

    qh = q.reshape(B, Nq, h, hd)
    kh = k.reshape(B, H * W, h, hd)
    vh = v.reshape(B, H * W, h, hd)
    bidx = np.arange(B)[:, None, None]
    hidx = np.arange(h)[None, None, :]

    # scores: one tap per pass (mat_pytorch_impl.py:45-74), then * scale
    tok = np.empty((M, B, Nq, h), dtype=np.int64)
    score = np.empty((B, Nq, h, M), dtype=dt)
    for j in range(side):
        ty = np.clip(y0 - r + j, 0, H - 1)
        for i in range(side):
            tx = np.clip(x0 - r + i, 0, W - 1)
            m = j * side + i
            tok[m] = ty * W + tx
            ktap = kh[bidx, tok[m], hidx]                       # [B,Nq,h,hd]
            if attn_type == "dot_product":      # restated native-only scoring (parity unpinned): products rounded to dt
                score[..., m] = (qh * ktap).astype(dt).sum(axis=-1, dtype=np.float32).astype(dt)
            else:
                l1 = np.abs(qh - ktap).sum(axis=-1, dtype=np.float32).astype(dt)
                score[..., m] = -l1
    score = (score.astype(np.float32) * np.float32(scale)).astype(dt)

    # BilinearSoftmax (mat_pytorch_impl.py:78-165)
    grid = score.reshape(B, Nq, h, side, side)
    attn = np.zeros((B, Nq, h, side, side), dtype=dt)
    for t in range(4):
        oy, ox = t >> 1, t & 1
        win = grid[..., oy:oy + sub, ox:ox + sub].reshape(B, Nq, h, sub * sub).astype(np.float32)
        e = np.exp(win - win.max(axis=-1, keepdims=True))
        p = (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(dt)
        contrib = (wgt[..., t:t + 1] * p).astype(dt).reshape(B, Nq, h, sub, sub)
        attn[..., oy:oy + sub, ox:ox + sub] += contrib
    attn = attn.reshape(B, Nq, h, M)

    # weighted sum of the value taps (mat_pytorch_impl.py:167-178)
    acc = np.zeros((B, Nq, h, hd), dtype=np.float32)
    for m in range(M):
        vtap = vh[bidx, tok[m], hidx]
        acc += (attn[..., m:m + 1] * vtap).astype(dt).astype(np.float32)
    out = acc.astype(dt).reshape(B, Nq, C)
    return out, attn
