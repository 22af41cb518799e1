"""CPU restatement of the MatchAttention backward.  TEST INFRASTRUCTURE ONLY.

The formulas the CUDA backward kernel implements, written with plain loops in float64 (small cases only).
Pinned by tests/golden/backward_*.npz: the gradients autograd gives over the reference's own 'pytorch' path
(models/mat_pytorch_impl.py:3-178 driven as models/attention_blocks.py:82-91 drives it).
"""
from __future__ import annotations

import math

import numpy as np


def backward(max_offset, q, k, v, g_out, g_attn, H: int, W: int, r: int, scale: float):
    """max_offset [B,N,h,2], q/k/v/g_out [B,N,C], g_attn [B,N,h,M] -> (d_max_offset, d_q, d_k, d_v)."""
    mo, q, k, v, g_out, g_attn = (np.asarray(a, dtype=np.float64) for a in (max_offset, q, k, v, g_out, g_attn))
    B, N, C = q.shape
    h = mo.shape[2]
    hd = C // h
    side, sub = 2 * r + 2, 2 * r + 1
    M = side * side
    d_mo, d_q, d_k, d_v = np.zeros_like(mo), np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    for b in range(B):
        for n in range(N):
            for hh in range(h):
                x, y = mo[b, n, hh]
                xf, yf = math.floor(x), math.floor(y)
                dx, dy = x - xf, y - yf
                w = [(1 - dx) * (1 - dy), dx * (1 - dy), (1 - dx) * dy, dx * dy]
                ch = slice(hh * hd, (hh + 1) * hd)
                tok = [min(max(yf - r + j, 0), H - 1) * W + min(max(xf - r + i, 0), W - 1)
                       for j in range(side) for i in range(side)]
                qv = q[b, n, ch]
                s = np.array([-scale * np.abs(qv - k[b, t, ch]).sum() for t in tok])
                da = np.array([g_out[b, n, ch] @ v[b, t, ch] for t in tok]) + g_attn[b, n, hh]
                a, ds, dw = np.zeros(M), np.zeros(M), np.zeros(4)
                for t in range(4):
                    oy, ox = t >> 1, t & 1
                    idx = [(j + oy) * side + i + ox for j in range(sub) for i in range(sub)]
                    e = np.exp(s[idx] - s[idx].max())
                    p = e / e.sum()
                    a[idx] += w[t] * p
                    pda = p @ da[idx]
                    dw[t] = pda
                    ds[idx] += w[t] * p * (da[idx] - pda)
                d_mo[b, n, hh, 0] = (1 - dy) * (dw[1] - dw[0]) + dy * (dw[3] - dw[2])
                d_mo[b, n, hh, 1] = (1 - dx) * (dw[2] - dw[0]) + dx * (dw[3] - dw[1])
                for m, t in enumerate(tok):
                    sg = np.sign(qv - k[b, t, ch])
                    d_q[b, n, ch] -= scale * ds[m] * sg
                    d_k[b, t, ch] += scale * ds[m] * sg
                    d_v[b, t, ch] += a[m] * g_out[b, n, ch]
    return d_mo, d_q, d_k, d_v
