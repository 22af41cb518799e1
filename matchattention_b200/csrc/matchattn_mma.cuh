// MatchAttention forward for 16-bit types with the float32 accumulations done by
// warp-level matrix instructions.
//
// The arithmetic of the operator is element-wise (|q-k| per channel, a*v per
// channel and tap) followed by short float32 sums (over the channels of a head,
// over the taps of a window).  The element-wise part has to stay on the float16
// lanes because each result must round to 16 bits on its own; the sums do not:
// a sum of float16 values accumulated in float32 is exactly what
// mma.sync.m16n8k16 (f16/bf16 inputs, f32 accumulators) computes when the other
// operand is a constant 0/1 matrix.  So the 16->32-bit conversions and float32
// adds of the scalar kernel (two thirds of its instructions) become matrix
// instructions whose A fragments are the registers the lanes already hold.
//
// Layout.  A warp owns 128 "items" (an item = one head of one query, hd <= 40
// channels) arranged as 16 rows x 8 columns.  Lane (g = lane/4, t = lane%4) owns
// the four items (row g | g+8, column t | t+4), which is the ownership pattern
// of both the A fragment (rows g, g+8; k-slots 2t, 2t+1, 2t+8, 2t+9) and the
// accumulator fragment (rows g, g+8; columns 2t, 2t+1) of m16n8k16:
//   scores:  A = |q-k| registers of the column-t items, B1[k][n] = [n == 2*((k%8)/2)]
//            routes every lane's k-slots to accumulator column 2t; the column-(t+4)
//            items use B2 (column 2t+1).  After NW/2 + NW/2 instructions the four
//            accumulators of a lane are the L1 sums of its four items for one tap.
//   values:  A = a*v registers of two taps (k-slots 2t.. from tap m, 2t+8.. from tap
//            m+1), B[k][n] = [k%8 == n] adds the two taps into the accumulator of the
//            same channel pair.
// The two column halves are processed one after the other (scores, then values) so that a
// lane never holds more than two items' worth of taps and accumulators: 128 registers,
// two blocks of 256 threads per SM.
//
// Order of the queries.  Either the map is walked in 16 x 8 tiles, or -- when the caller
// supplies scratch -- in the order produced by the sorting passes of matchattn_binned.cuh
// (queries that look at the same tile of K/V are neighbours).  In both cases the taps are
// plain global loads; what makes them cheap is that neighbouring warps of a block ask for the
// same few kilobytes, which then come from L1.
#pragma once

#include "matchattn_kernels.cuh"

namespace matchattn {

template <typename T>
struct Mma;

template <>
struct Mma<__half> {
    static constexpr uint32_t kOneLo = 0x00003C00u, kOneHi = 0x3C000000u;
    static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
    {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t absdiff2(uint32_t q, uint32_t k)
    {
        const __half2 d = __hsub2(*reinterpret_cast<const __half2 *>(&q), *reinterpret_cast<const __half2 *>(&k));
        return *reinterpret_cast<const uint32_t *>(&d) & 0x7fff7fffu;
    }
    static __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t v)
    {
        const __half2 p = __hmul2_rn(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&v));
        return *reinterpret_cast<const uint32_t *>(&p);
    }
};

template <>
struct Mma<__nv_bfloat16> {
    static constexpr uint32_t kOneLo = 0x00003F80u, kOneHi = 0x3F800000u;
    static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
    {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t absdiff2(uint32_t q, uint32_t k)
    {
        const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&q),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&k));
        return *reinterpret_cast<const uint32_t *>(&d) & 0x7fff7fffu;
    }
    static __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t v)
    {
        const __nv_bfloat162 p = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162 *>(&a),
                                            *reinterpret_cast<const __nv_bfloat162 *>(&v));
        return *reinterpret_cast<const uint32_t *>(&p);
    }
};

// both halves of a register <- its low (or high) 16 bits
__device__ __forceinline__ uint32_t dup_lo(uint32_t x) { return __byte_perm(x, x, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t x) { return __byte_perm(x, x, 0x3232); }

// Geometry of this kernel: a warp takes a chunk of 128 consecutive items, a block 8 chunks.
constexpr int kMmaChunk = 128;
constexpr int kMmaItemsPerBlock = (kThreads / 32) * kMmaChunk;
constexpr int kMmaTileW = 16, kMmaTileH = 8;     // unsorted order walks the map in 16 x 8 query tiles

// fast exp for the softmax of this kernel: 2^(x*log2e) with the product and the subtraction of the
// maximum fused in one FMA.  Against expf it changes the share of attention weights that differ
// from the reference in their last bit from 7.7e-5 to 8.4e-5 (measured on the headline shape).
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// BilinearSoftmax for R = 1 from scores kept as 16-bit pairs.  `sc[m]` holds tap m of two items,
// `hi` says which of the two.  Writes the blended weights as pairs of taps.  Same rounding points
// as bilinear_softmax<T, 1>; the exponentials use ex2_approx.
template <typename T>
__device__ __forceinline__ void bilinear_softmax_r1_packed(const uint32_t (&sc)[16], const int hi, const uint32_t (&wgt)[2],
                                                           uint32_t (&aw)[8])
{
    constexpr float kLog2e = 1.4426950408889634f;
    float s[16];
#pragma unroll
    for (int m = 0; m < 16; ++m) s[m] = DT<T>::unpack(sc[m], hi);
    float top[4], bot[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float mid = fmaxf(s[4 + i], s[8 + i]);
        top[i] = fmaxf(s[i], mid);
        bot[i] = fmaxf(mid, s[12 + i]);
    }
    const float mt = fmaxf(top[1], top[2]), mb = fmaxf(bot[1], bot[2]);
    const float sub_max[4] = {fmaxf(top[0], mt), fmaxf(mt, top[3]), fmaxf(bot[0], mb), fmaxf(mb, bot[3])};
    const float gmax = fmaxf(fmaxf(sub_max[0], sub_max[1]), fmaxf(sub_max[2], sub_max[3]));
    const float gmin = fminf(fminf(sub_max[0], sub_max[1]), fminf(sub_max[2], sub_max[3]));
#pragma unroll
    for (int w = 0; w < 8; ++w) aw[w] = 0u;
    const float w4[4] = {DT<T>::unpack(wgt[0], 0), DT<T>::unpack(wgt[0], 1), DT<T>::unpack(wgt[1], 0),
                         DT<T>::unpack(wgt[1], 1)};
    if (gmax - gmin < 60.f) {
        const float shift = -gmax * kLog2e;
        float e[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) e[m] = ex2_approx(fmaf(s[m], kLog2e, shift));
        float ct[4], cb[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float mid = e[4 + i] + e[8 + i];
            ct[i] = e[i] + mid;
            cb[i] = mid + e[12 + i];
        }
        const float st = ct[1] + ct[2], sb = cb[1] + cb[2];
        const float den[4] = {ct[0] + st, st + ct[3], cb[0] + sb, sb + cb[3]};
#pragma unroll
        for (int t = 0; t < 4; ++t)
            blend_subwindow<T, 1>(aw, t, w4[t], softmax_rcp(den[t]), [&](int m) { return e[m]; });
    } else {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int oy = t >> 1, ox = t & 1;
            const float mx = sub_max[t];
            float den = 0.f;
#pragma unroll
            for (int j = 0; j < 3; ++j)
#pragma unroll
                for (int i = 0; i < 3; ++i) den += softmax_exp(s[(j + oy) * 4 + i + ox] - mx);
            blend_subwindow<T, 1>(aw, t, w4[t], softmax_rcp(den), [&](int m) { return softmax_exp(s[m] - mx); });
        }
    }
}

// SAMEQ: the head count is a multiple of 8 and all heads of a query share one sampling centre
// (checked by the sorting pass), so the two column halves of a row are two heads of the SAME
// query; a lane then handles 2 queries x 2 heads and keeps one window per query.
// POW2: scale is a power of two, so the scaled score is an exact 16-bit multiply.
// NCH: column halves in use.  2 = a lane owns four items (128 per warp); 1 = only the first column
// half, two items per lane (64 per warp): half the registers, no spills, more warps in flight.
template <typename T, int CPL, bool SAMEQ, bool POW2, int NCH>
__global__ void __launch_bounds__(kThreads, 2) fused_forward_mma_kernel(const Params p)
{
    static_assert(NCH == 2 || !SAMEQ, "sharing a window between column halves needs both of them");
    constexpr int R = 1, SIDE = 4, M = 16;
    constexpr int NW = CPL * 4;                 // 32-bit words per item and tap
    constexpr int SLICE_BYTES = CPL * 16;       // bytes of one head in a token row
    constexpr int NQ = SAMEQ ? 2 : 4;           // distinct windows per lane

    if (p.guard != nullptr && ((*p.guard != 0u) != (p.guard_run_if != 0))) return;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ones = Mma<T>::kOneLo | Mma<T>::kOneHi;
    const uint32_t b_sum = (g == 2 * t) ? ones : 0u;                      // k-slots of lane t -> accumulator column 2t
    const uint32_t b_id = (g == 2 * t) ? Mma<T>::kOneLo : ((g == 2 * t + 1) ? Mma<T>::kOneHi : 0u);
    const int RB = p.C * 2;                                               // bytes of a token row
    const int total_q = p.B * p.Nq;            // the host keeps B*Nq*h below 2^31

    // ---- the lane's four items (i4 = 2*rowhalf + colhalf) and their windows
    const int item0 = (blockIdx.x * (kThreads / 32) + warp) * (64 * NCH);
    bool valid[4];
    uint32_t qoff[4];                          // byte offset of the item's slice in q (and out)
    uint32_t aoff[4];                          // element offset of the item's weights in attn_out, divided by 16
    uint32_t hoff[NQ];                         // byte offset of the item's head inside a token row (column half 0)
    uint32_t col[NQ][SIDE], row[NQ][SIDE];     // byte offsets of the clamped tap columns / rows in k (and v)
    uint32_t wgt[NQ][2];
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        if (NCH == 1 && (i4 & 1)) continue;
        const int item = item0 + (g + 8 * (i4 >> 1)) * (4 * NCH) + t + 4 * (i4 & 1);
        const int qs = item / p.h;
        const int head = item - qs * p.h;
        int bq;
        if (p.sorted != nullptr) {
            valid[i4] = qs < total_q;
            bq = static_cast<int>(p.sorted[min(qs, total_q - 1)].x);
        } else {
            // unsorted: walk the map in 16 x 8 tiles
            const int tile = qs / (kMmaTileW * kMmaTileH);
            const int within = qs - tile * (kMmaTileW * kMmaTileH);
            const int tiles_y = (p.rows + kMmaTileH - 1) / kMmaTileH;
            const int bt = tile / p.tiles_x;
            const int tx = tile - bt * p.tiles_x;
            const int b = bt / tiles_y;
            const int ty = bt - b * tiles_y;
            int qx = tx * kMmaTileW + (within & (kMmaTileW - 1)), qy = ty * kMmaTileH + within / kMmaTileW;
            valid[i4] = b < p.B && qx < p.W && qy < p.rows;
            qx = min(qx, p.W - 1);
            qy = min(qy, p.rows - 1);
            bq = min(b, p.B - 1) * p.Nq + qy * p.W + qx;
        }
        qoff[i4] = static_cast<uint32_t>(bq) * RB + head * SLICE_BYTES;
        aoff[i4] = static_cast<uint32_t>(bq) * p.h + head;
        if (SAMEQ && (i4 & 1)) continue;        // same query, same window as the item to its left
        const int wq = SAMEQ ? (i4 >> 1) : i4;
        hoff[wq] = head * SLICE_BYTES;
        float x, y;
        DT<T>::load_xy(static_cast<const T *>(p.mo) + (static_cast<int64_t>(bq) * p.h + head) * 2, x, y);
        const float xf = floorf(x), yf = floorf(y);
        {
            float wf[4];
            bilinear_weights<T>(x, xf, y, yf, wf);
            wgt[wq][0] = DT<T>::pack(&wf[0]);
            wgt[wq][1] = DT<T>::pack(&wf[2]);
        }
        const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
        const uint32_t item_base = static_cast<uint32_t>(bq / p.Nq) * static_cast<uint32_t>(p.N);   // tokens before this batch item
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            col[wq][i] = static_cast<uint32_t>(min(max(x0 + i, 0), p.W - 1)) * RB + hoff[wq];
            row[wq][i] = (item_base + static_cast<uint32_t>(min(max(y0 + i, 0), p.H - 1)) * p.W) * RB;
        }
    }
#define MA_WQ(i4_) (SAMEQ ? ((i4_) >> 1) : (i4_))
#define MA_HEAD_SHIFT(i4_) ((SAMEQ && ((i4_) & 1)) ? 4 * SLICE_BYTES : 0)     // column half 1 is 4 heads further
    const char *kb = static_cast<const char *>(p.k);
    const char *vb = static_cast<const char *>(p.v);

    // ---- scores, one column half at a time; sc[m][ch] = tap m of the items in rows g and g+8
    uint32_t sc[NCH][M];
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
        const int ia = ch, ib = 2 + ch;
        uint32_t qa[NW], qb[NW];
        load_words<NW>(qa, static_cast<const char *>(p.q) + qoff[ia]);
        load_words<NW>(qb, static_cast<const char *>(p.q) + qoff[ib]);
#pragma unroll
        for (int j = 0; j < SIDE; ++j)
#pragma unroll
            for (int i = 0; i < SIDE; ++i) {
                uint32_t da[NW], db[NW];
                load_words<NW>(da, kb + (row[MA_WQ(ia)][j] + col[MA_WQ(ia)][i]) + MA_HEAD_SHIFT(ia));
                load_words<NW>(db, kb + (row[MA_WQ(ib)][j] + col[MA_WQ(ib)][i]) + MA_HEAD_SHIFT(ib));
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    da[w] = Mma<T>::absdiff2(qa[w], da[w]);
                    db[w] = Mma<T>::absdiff2(qb[w], db[w]);
                }
                float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int jj = 0; jj < NW / 2; ++jj)
                    Mma<T>::run(c, da[2 * jj], db[2 * jj], da[2 * jj + 1], db[2 * jj + 1], b_sum, b_sum);
                // c[0] = L1 sum of the row-g item, c[2] = of the row-(g+8) item; round, negate, scale
                const float l1[2] = {c[0], c[2]};
                uint32_t packed = DT<T>::pack(l1);
                if constexpr (POW2) {
                    packed = DT<T>::aw_mul(packed, DT<T>::aw_bcast(-p.scale));
                } else {
                    const float sf[2] = {DT<T>::rnd(-DT<T>::unpack(packed, 0) * p.scale),
                                         DT<T>::rnd(-DT<T>::unpack(packed, 1) * p.scale)};
                    packed = DT<T>::pack(sf);
                }
                sc[ch][j * SIDE + i] = packed;
            }
    }

    // ---- BilinearSoftmax per item
    uint32_t ap[4][M / 2];
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        if (NCH == 1 && (i4 & 1)) continue;
        bilinear_softmax_r1_packed<T>(sc[i4 & (NCH - 1)], i4 >> 1, wgt[MA_WQ(i4)], ap[i4]);
        if (p.attn != nullptr && valid[i4])
            store_words<M / 2>(static_cast<T *>(p.attn) + static_cast<int64_t>(aoff[i4]) * M, ap[i4]);
    }

    // ---- values: one column half after the other, two taps per matrix instruction
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
        const int ia = ch, ib = 2 + ch;
        float o[NW][4];
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[w][e] = 0.f;
#pragma unroll
        for (int m = 0; m < M; m += 2) {
            const int j0 = m / SIDE, i0 = m % SIDE, j1 = (m + 1) / SIDE, i1 = (m + 1) % SIDE;
            uint32_t va0[NW], va1[NW], vb0[NW], vb1[NW];
            load_words<NW>(va0, vb + (row[MA_WQ(ia)][j0] + col[MA_WQ(ia)][i0]) + MA_HEAD_SHIFT(ia));
            load_words<NW>(va1, vb + (row[MA_WQ(ia)][j1] + col[MA_WQ(ia)][i1]) + MA_HEAD_SHIFT(ia));
            load_words<NW>(vb0, vb + (row[MA_WQ(ib)][j0] + col[MA_WQ(ib)][i0]) + MA_HEAD_SHIFT(ib));
            load_words<NW>(vb1, vb + (row[MA_WQ(ib)][j1] + col[MA_WQ(ib)][i1]) + MA_HEAD_SHIFT(ib));
            const uint32_t a_lo = dup_lo(ap[ia][m / 2]), a_hi = dup_hi(ap[ia][m / 2]);
            const uint32_t b_lo = dup_lo(ap[ib][m / 2]), b_hi = dup_hi(ap[ib][m / 2]);
#pragma unroll
            for (int w = 0; w < NW; ++w)
                Mma<T>::run(o[w], Mma<T>::mul2(a_lo, va0[w]), Mma<T>::mul2(b_lo, vb0[w]), Mma<T>::mul2(a_hi, va1[w]),
                            Mma<T>::mul2(b_hi, vb1[w]), b_id, b_id);
        }
#pragma unroll
        for (int rh = 0; rh < 2; ++rh) {
            const int i4 = 2 * rh + ch;
            if (!valid[i4]) continue;
            uint32_t ow[NW];
#pragma unroll
            for (int w = 0; w < NW; ++w) ow[w] = DT<T>::pack(&o[w][2 * rh]);
            store_words<NW>(static_cast<char *>(p.out) + qoff[i4], ow);
        }
    }
#undef MA_WQ
#undef MA_HEAD_SHIFT
}

template <typename T>
cudaError_t launch_mma(const Params &p, int cpl, bool sameq, bool pow2, int nch, unsigned blocks, cudaStream_t stream);

}  // namespace matchattn
