// Backward of the MatchAttention operator.
//
// The reference's native path has no backward (models/match_former_ops.py registers none; the attn_sum
// buffer "for backward" of models/src/match_former_fused_forward.cu:409,495 is never read); only its 'pytorch'
// path can be trained, through autograd over the five functions of models/mat_pytorch_impl.py.  This kernel
// computes what that autograd computes: gradients with respect to q, k, v and max_offset, given the
// gradients of both outputs (out and attn_out: the cross branch feeds the attention weights to its output
// projection, models/attention_blocks.py:95-98).
//
//   s_m   = -scale * sum_c |q_c - k_mc|                         scores of the (2r+2)^2 taps
//   p_t   = softmax of s over sub-window t (t = nw, ne, sw, se)  a_m = sum_t w_t p_tm,  out_c = sum_m a_m v_mc
//   da_m  = sum_c dout_c v_mc + dattn_m                          dv_mc += a_m dout_c
//   ds_m  = sum_t w_t p_tm (da_m - sum_m' p_tm' da_m')           dw_t   = sum_m p_tm da_m
//   dq_c  = -scale sum_m ds_m sign(q_c - k_mc)                   dk_mc += scale ds_m sign(q_c - k_mc)
//   d(max_offset) follows from dw through w = [(1-dx)(1-dy), dx(1-dy), (1-dx)dy, dx dy] (floor has no gradient)
//
// One thread per (query, head); the forward quantities are recomputed (nothing is saved by the forward);
// all arithmetic in float32 whatever the tensor type; dk and dv are float32 arrays [B, H*W, C] that the
// caller has zeroed, filled with atomic adds (several queries look at the same token).  Two kernels: one
// element at a time for any head width and radius, and eight channels at a time with four-float vector
// reductions for head widths that are multiples of 8 and r <= 2 (every model shape).
#include "../../include/matchattn.h"

#include <stdint.h>

#include "matchattn_kernels.cuh"

namespace matchattn {
namespace {

struct BwdParams {
    const void *mo, *q, *k, *v, *dout, *dattn;   // dattn may be null
    void *dq, *dmo;                               // tensor type; dmo may be null
    float *dk, *dv;                               // float32, pre-zeroed
    int B, H, W, h, hd, C, r, rows, Nq, N;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(128) backward_kernel(const BwdParams p)
{
    const int64_t per_item = static_cast<int64_t>(p.Nq) * p.h;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= per_item) return;
    const int b = blockIdx.y;
    const int head = static_cast<int>(t % p.h);
    const int64_t bq = static_cast<int64_t>(b) * p.Nq + t / p.h;
    const int r = p.r, side = 2 * r + 2, sub = 2 * r + 1, M = side * side;

    const T *mo = static_cast<const T *>(p.mo) + (bq * p.h + head) * 2;
    const float x = load_one<T>(mo), y = load_one<T>(mo + 1);
    const float xf = floorf(x), yf = floorf(y);
    const float dx = x - xf, dy = y - yf;
    const float wgt[4] = {(1.f - dx) * (1.f - dy), dx * (1.f - dy), (1.f - dx) * dy, dx * dy};
    const int x0 = window_origin(xf, r, p.W) - r, y0 = window_origin(yf, r, p.H) - r;

    const int64_t qoff = bq * p.C + head * p.hd;
    const T *qp = static_cast<const T *>(p.q) + qoff;
    const T *gop = static_cast<const T *>(p.dout) + qoff;
    const int64_t kv_base = static_cast<int64_t>(b) * p.N * p.C + head * p.hd;
    const T *kb = static_cast<const T *>(p.k) + kv_base;
    const T *vb = static_cast<const T *>(p.v) + kv_base;

    // forward: scores, sub-window softmaxes, attention weights; da from dout.v (+ dattn)
    float s[kMaxTaps], a[kMaxTaps], da[kMaxTaps];
    int tok[kMaxTaps];
    for (int j = 0; j < side; ++j) {
        const int ty = min(max(y0 + j, 0), p.H - 1);
        for (int i = 0; i < side; ++i) {
            const int tx = min(max(x0 + i, 0), p.W - 1);
            const int m = j * side + i;
            tok[m] = ty * p.W + tx;
            const T *kp = kb + static_cast<int64_t>(tok[m]) * p.C;
            const T *vp = vb + static_cast<int64_t>(tok[m]) * p.C;
            float l1 = 0.f, dot = 0.f;
            for (int c = 0; c < p.hd; ++c) {
                l1 += fabsf(load_one<T>(qp + c) - load_one<T>(kp + c));
                dot = fmaf(load_one<T>(gop + c), load_one<T>(vp + c), dot);
            }
            s[m] = -l1 * p.scale;
            a[m] = 0.f;
            da[m] = dot;
        }
    }
    if (p.dattn != nullptr) {
        const T *gap = static_cast<const T *>(p.dattn) + (bq * p.h + head) * M;
        for (int m = 0; m < M; ++m) da[m] += load_one<T>(gap + m);
    }
    float ds[kMaxTaps], dw[4];
    for (int m = 0; m < M; ++m) ds[m] = 0.f;
    for (int tq = 0; tq < 4; ++tq) {
        const int oy = tq >> 1, ox = tq & 1;
        float mx = -INFINITY;
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) mx = fmaxf(mx, s[(j + oy) * side + i + ox]);
        float den = 0.f;
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) den += expf(s[(j + oy) * side + i + ox] - mx);
        const float inv = 1.f / den;
        float pda = 0.f;                                   // sum_m p_tm da_m
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) {
                const int m = (j + oy) * side + i + ox;
                const float pr = expf(s[m] - mx) * inv;
                a[m] += wgt[tq] * pr;
                pda = fmaf(pr, da[m], pda);
            }
        dw[tq] = pda;
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) {
                const int m = (j + oy) * side + i + ox;
                const float pr = expf(s[m] - mx) * inv;
                ds[m] = fmaf(wgt[tq] * pr, da[m] - pda, ds[m]);
            }
    }

    // gradient of the sampling centre through the bilinear weights
    if (p.dmo != nullptr) {
        T *gmo = static_cast<T *>(p.dmo) + (bq * p.h + head) * 2;
        store_one<T>(gmo, (1.f - dy) * (dw[1] - dw[0]) + dy * (dw[3] - dw[2]));
        store_one<T>(gmo + 1, (1.f - dx) * (dw[2] - dw[0]) + dx * (dw[3] - dw[1]));
    }

    // dq, and the scatter into dk / dv
    T *gq = static_cast<T *>(p.dq) + qoff;
    for (int c = 0; c < p.hd; ++c) {
        const float qc = load_one<T>(qp + c), go = load_one<T>(gop + c);
        float acc = 0.f;
        for (int m = 0; m < M; ++m) {
            const int64_t off = static_cast<int64_t>(tok[m]) * p.C + c;
            const float d = qc - load_one<T>(kb + off);
            const float sg = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
            const float g = p.scale * ds[m] * sg;
            acc -= g;
            if (g != 0.f) atomicAdd(p.dk + kv_base + off, g);
            const float gv = a[m] * go;
            if (gv != 0.f) atomicAdd(p.dv + kv_base + off, gv);
        }
        store_one<T>(gq + c, acc);
    }
}


// ---- the same computation for head widths that are multiples of 8 and r = 1 or 2 -----------------------
// Eight channels at a time through 16- or 32-byte loads, the window in registers (R is a template
// argument), and the scatter into dk / dv as four-float vector reductions (red.global.add.v4.f32 through
// atomicAdd(float4 *), a quarter of the scalar kernel's atomic instructions).

template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&f)[8])
{
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half *p, float (&f)[8])
{
    const uint4 u = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&f)[8])
{
    const uint4 u = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T>
__device__ __forceinline__ void store8(T *p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<float>(float *p, const float (&f)[8])
{
    reinterpret_cast<float4 *>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half *p, const float (&f)[8])
{
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&t);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16 *p, const float (&f)[8])
{
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&t);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// (measured: the kernel is bound by the rate of the reductions into dk / dv, L2 throughput 62 % at 18 %
// occupancy; four blocks per SM instead of three change nothing at r = 1 and gain 25 % at r = 2)
template <typename T, int R>
__global__ void __launch_bounds__(128, R == 2 ? 4 : 3) backward_vec_kernel(const BwdParams p)
{
    constexpr int SIDE = 2 * R + 2, SUB = 2 * R + 1, M = SIDE * SIDE;
    const int64_t per_item = static_cast<int64_t>(p.Nq) * p.h;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= per_item) return;
    const int b = blockIdx.y;
    const int head = static_cast<int>(t % p.h);
    const int64_t bq = static_cast<int64_t>(b) * p.Nq + t / p.h;

    const T *mo = static_cast<const T *>(p.mo) + (bq * p.h + head) * 2;
    const float x = load_one<T>(mo), y = load_one<T>(mo + 1);
    const float xf = floorf(x), yf = floorf(y);
    const float dx = x - xf, dy = y - yf;
    const float wgt[4] = {(1.f - dx) * (1.f - dy), dx * (1.f - dy), (1.f - dx) * dy, dx * dy};
    const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
    int col[SIDE], row[SIDE];                      // element offsets of the window's columns and rows
#pragma unroll
    for (int i = 0; i < SIDE; ++i) {
        col[i] = min(max(x0 + i, 0), p.W - 1) * p.C;
        row[i] = min(max(y0 + i, 0), p.H - 1) * p.W * p.C;
    }

    const int64_t qoff = bq * p.C + head * p.hd;
    const T *qp = static_cast<const T *>(p.q) + qoff;
    const T *gop = static_cast<const T *>(p.dout) + qoff;
    const int64_t kv_base = static_cast<int64_t>(b) * p.N * p.C + head * p.hd;
    const T *kb = static_cast<const T *>(p.k) + kv_base;
    const T *vb = static_cast<const T *>(p.v) + kv_base;
    const int chunks = p.hd >> 3;

    float s[M], da[M];
#pragma unroll
    for (int m = 0; m < M; ++m) s[m] = da[m] = 0.f;
    for (int ch = 0; ch < chunks; ++ch) {
        float qv[8], gv[8];
        load8<T>(qp + 8 * ch, qv);
        load8<T>(gop + 8 * ch, gv);
#pragma unroll
        for (int j = 0; j < SIDE; ++j)
#pragma unroll
            for (int i = 0; i < SIDE; ++i) {
                float kv[8], vv[8];
                load8<T>(kb + row[j] + col[i] + 8 * ch, kv);
                load8<T>(vb + row[j] + col[i] + 8 * ch, vv);
                float l1 = 0.f, dot = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    l1 += fabsf(qv[c] - kv[c]);
                    dot = fmaf(gv[c], vv[c], dot);
                }
                s[j * SIDE + i] += l1;
                da[j * SIDE + i] += dot;
            }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) s[m] = -s[m] * p.scale;
    if (p.dattn != nullptr) {
        const T *gap = static_cast<const T *>(p.dattn) + (bq * p.h + head) * M;
#pragma unroll
        for (int m = 0; m < M; ++m) da[m] += load_one<T>(gap + m);
    }
    float a[M], ds[M], dw[4];
#pragma unroll
    for (int m = 0; m < M; ++m) a[m] = ds[m] = 0.f;
#pragma unroll
    for (int tq = 0; tq < 4; ++tq) {
        const int oy = tq >> 1, ox = tq & 1;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < SUB; ++j)
#pragma unroll
            for (int i = 0; i < SUB; ++i) mx = fmaxf(mx, s[(j + oy) * SIDE + i + ox]);
        float pr[SUB * SUB], den = 0.f;
#pragma unroll
        for (int j = 0; j < SUB; ++j)
#pragma unroll
            for (int i = 0; i < SUB; ++i) {
                pr[j * SUB + i] = expf(s[(j + oy) * SIDE + i + ox] - mx);
                den += pr[j * SUB + i];
            }
        const float inv = 1.f / den;
        float pda = 0.f;
#pragma unroll
        for (int j = 0; j < SUB; ++j)
#pragma unroll
            for (int i = 0; i < SUB; ++i) {
                pr[j * SUB + i] *= inv;
                pda = fmaf(pr[j * SUB + i], da[(j + oy) * SIDE + i + ox], pda);
            }
        dw[tq] = pda;
#pragma unroll
        for (int j = 0; j < SUB; ++j)
#pragma unroll
            for (int i = 0; i < SUB; ++i) {
                const int m = (j + oy) * SIDE + i + ox;
                const float wp = wgt[tq] * pr[j * SUB + i];
                a[m] += wp;
                ds[m] = fmaf(wp, da[m] - pda, ds[m]);
            }
    }
    if (p.dmo != nullptr) {
        T *gmo = static_cast<T *>(p.dmo) + (bq * p.h + head) * 2;
        store_one<T>(gmo, (1.f - dy) * (dw[1] - dw[0]) + dy * (dw[3] - dw[2]));
        store_one<T>(gmo + 1, (1.f - dx) * (dw[2] - dw[0]) + dx * (dw[3] - dw[1]));
    }
#pragma unroll
    for (int m = 0; m < M; ++m) ds[m] *= p.scale;

    T *gq = static_cast<T *>(p.dq) + qoff;
    float *dkb = p.dk + kv_base, *dvb = p.dv + kv_base;
    for (int ch = 0; ch < chunks; ++ch) {
        float qv[8], gv[8], acc[8];
        load8<T>(qp + 8 * ch, qv);
        load8<T>(gop + 8 * ch, gv);
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.f;
#pragma unroll
        for (int j = 0; j < SIDE; ++j)
#pragma unroll
            for (int i = 0; i < SIDE; ++i) {
                const int m = j * SIDE + i;
                const int off = row[j] + col[i] + 8 * ch;
                float kv[8], gk[8];
                load8<T>(kb + off, kv);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float d = qv[c] - kv[c];
                    gk[c] = d > 0.f ? ds[m] : (d < 0.f ? -ds[m] : 0.f);
                    acc[c] -= gk[c];
                }
                if (ds[m] != 0.f) {
                    atomicAdd(reinterpret_cast<float4 *>(dkb + off), make_float4(gk[0], gk[1], gk[2], gk[3]));
                    atomicAdd(reinterpret_cast<float4 *>(dkb + off) + 1, make_float4(gk[4], gk[5], gk[6], gk[7]));
                }
                if (a[m] != 0.f) {
                    atomicAdd(reinterpret_cast<float4 *>(dvb + off),
                              make_float4(a[m] * gv[0], a[m] * gv[1], a[m] * gv[2], a[m] * gv[3]));
                    atomicAdd(reinterpret_cast<float4 *>(dvb + off) + 1,
                              make_float4(a[m] * gv[4], a[m] * gv[5], a[m] * gv[6], a[m] * gv[7]));
                }
            }
        store8<T>(gq + 8 * ch, acc);
    }
}

template <typename T>
void launch_backward(const BwdParams &p, bool vec, dim3 grid, cudaStream_t stream)
{
    if (vec && p.r == 1) backward_vec_kernel<T, 1><<<grid, 128, 0, stream>>>(p);
    else if (vec && p.r == 2) backward_vec_kernel<T, 2><<<grid, 128, 0, stream>>>(p);
    else backward_kernel<T><<<grid, 128, 0, stream>>>(p);
}

}  // namespace
}  // namespace matchattn

extern "C" int matchattn_fused_backward(const void *max_offset, const void *q, const void *k, const void *v,
                                        const void *d_out, const void *d_attn, void *d_q, float *d_k, float *d_v,
                                        void *d_max_offset, int B, int H, int W, int h, int hd, int rx, int ry, int dtype,
                                        int attn_type, float scale, int q_row_begin, int q_row_end, void *cuda_stream)
{
    using namespace matchattn;
    if (!max_offset || !q || !k || !v || !d_out || !d_q || !d_k || !d_v) return MATCHATTN_ERR_NULL;
    if (dtype != MATCHATTN_F32 && dtype != MATCHATTN_F16 && dtype != MATCHATTN_BF16) return MATCHATTN_ERR_DTYPE;
    if (attn_type != MATCHATTN_L1_NORM) return MATCHATTN_ERR_ATTN_TYPE;
    if (B <= 0 || H <= 0 || W <= 0 || h <= 0 || hd <= 0) return MATCHATTN_ERR_SHAPE;
    if (q_row_begin < 0 || q_row_end > H || q_row_begin >= q_row_end) return MATCHATTN_ERR_SHAPE;
    if (rx != ry || rx < 0 || rx > MATCHATTN_MAX_R) return MATCHATTN_ERR_WINDOW;
    if (2 * rx + 2 > W || 2 * ry + 2 > H) return MATCHATTN_ERR_WINDOW_FIT;
    const long long C = 1LL * h * hd, N = 1LL * H * W, Nq = 1LL * (q_row_end - q_row_begin) * W;
    if (C > 65536 || N * C >= 2147483647LL || Nq * h >= 2147483647LL || B > 65535) return MATCHATTN_ERR_TOO_LARGE;
    BwdParams p{};
    p.mo = max_offset; p.q = q; p.k = k; p.v = v; p.dout = d_out; p.dattn = d_attn;
    p.dq = d_q; p.dmo = d_max_offset; p.dk = d_k; p.dv = d_v;
    p.B = B; p.H = H; p.W = W; p.h = h; p.hd = hd; p.C = static_cast<int>(C); p.r = rx;
    p.rows = q_row_end - q_row_begin; p.Nq = static_cast<int>(Nq); p.N = static_cast<int>(N);
    p.scale = scale;
    const long long per_item = Nq * h;
    const dim3 grid(static_cast<unsigned>((per_item + 127) / 128), B);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    // the vector kernel: head width a multiple of 8, r = 1 or 2, 16-byte aligned rows everywhere
    const auto al16 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    const bool vec = hd % 8 == 0 && (rx == 1 || rx == 2) && al16(q) && al16(k) && al16(v) && al16(d_out) && al16(d_q) &&
                     al16(d_k) && al16(d_v);
    switch (dtype) {
    case MATCHATTN_F32: launch_backward<float>(p, vec, grid, stream); break;
    case MATCHATTN_F16: launch_backward<__half>(p, vec, grid, stream); break;
    default: launch_backward<__nv_bfloat16>(p, vec, grid, stream); break;
    }
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}
