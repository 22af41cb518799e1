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

// Items per block: 8 warps x 128.  Queries of a block form a tile_w x tile_h tile as in the scalar kernel.
template <typename T, int R, int CPL>
__global__ void __launch_bounds__(kThreads, 1) fused_forward_mma_kernel(const Params p)
{
    constexpr int SIDE = 2 * R + 2, M = SIDE * SIDE;
    constexpr int NW = CPL * 4;                 // 32-bit words per item and tap
    constexpr int SLICE = CPL * 8;              // = hd
    static_assert(M % 2 == 0, "taps are consumed in pairs");

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // constant selector fragments (see the header comment)
    const uint32_t ones = Mma<T>::kOneLo | Mma<T>::kOneHi;
    const uint32_t b_col0 = (g == 2 * t) ? ones : 0u;                     // k-slots of lane t -> column 2t
    const uint32_t b_col1 = (g == 2 * t + 1) ? ones : 0u;                 //                   -> column 2t+1
    const uint32_t b_id = (g == 2 * t) ? Mma<T>::kOneLo : ((g == 2 * t + 1) ? Mma<T>::kOneHi : 0u);

    // the lane's four items: i4 = 2*rowhalf + colhalf
    bool valid[4];
    int64_t bq[4];
    int lane_off[4], head_of[4];
    int col[4][SIDE], row[4][SIDE];
    uint32_t wgt[4][2];      // the four bilinear weights of an item, as two pairs of T
    const int b = blockIdx.y;
    const int tile_y = blockIdx.x / p.tiles_x;
    const int tile_x = blockIdx.x - tile_y * p.tiles_x;
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        const int item = warp * 128 + (g + 8 * (i4 >> 1)) * 8 + t + 4 * (i4 & 1);
        const int lq = item / p.h;
        const int head = item - lq * p.h;
        int qx = tile_x * p.tile_w + (lq & (p.tile_w - 1));
        int qy = tile_y * p.tile_h + (lq >> p.tile_w_shift);
        valid[i4] = (lq >> p.tile_w_shift) < p.tile_h && qx < p.W && qy < p.rows;
        qx = min(qx, p.W - 1);
        qy = min(qy, p.rows - 1);
        bq[i4] = static_cast<int64_t>(b) * p.Nq + qy * p.W + qx;
        lane_off[i4] = head * SLICE;
        head_of[i4] = head;
        float x, y;
        DT<T>::load_xy(static_cast<const T *>(p.mo) + (bq[i4] * p.h + head) * 2, x, y);
        const float xf = floorf(x), yf = floorf(y);
        {
            float wf[4];
            bilinear_weights<T>(x, xf, y, yf, wf);      // already rounded to T: the packing below is exact
            wgt[i4][0] = DT<T>::pack(&wf[0]);
            wgt[i4][1] = DT<T>::pack(&wf[2]);
        }
        const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            col[i4][i] = min(max(x0 + i, 0), p.W - 1) * p.C + lane_off[i4];
            row[i4][i] = min(max(y0 + i, 0), p.H - 1) * p.W * p.C;
        }
    }
    const int64_t kv_base = static_cast<int64_t>(b) * p.N * p.C;
    const T *kb = static_cast<const T *>(p.k) + kv_base;
    const T *vb = static_cast<const T *>(p.v) + kv_base;

    uint32_t qw[4][NW];
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) load_words<NW>(qw[i4], static_cast<const T *>(p.q) + bq[i4] * p.C + lane_off[i4]);

    // ---- scores, rounded and scaled like the reference's (so exactly representable in T), kept as
    //      pairs: sc[m][0] = items 0 and 1, sc[m][1] = items 2 and 3
    uint32_t sc[M][2];
#pragma unroll
    for (int j = 0; j < SIDE; ++j)
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            uint32_t d[4][NW];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) load_words<NW>(d[i4], kb + (row[i4][j] + col[i4][i]));
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4)
#pragma unroll
                for (int w = 0; w < NW; ++w) d[i4][w] = Mma<T>::absdiff2(qw[i4][w], d[i4][w]);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int jj = 0; jj < NW / 2; ++jj)
                Mma<T>::run(c, d[0][2 * jj], d[2][2 * jj], d[0][2 * jj + 1], d[2][2 * jj + 1], b_col0, b_col0);
#pragma unroll
            for (int jj = 0; jj < NW / 2; ++jj)
                Mma<T>::run(c, d[1][2 * jj], d[3][2 * jj], d[1][2 * jj + 1], d[3][2 * jj + 1], b_col1, b_col1);
            float fs[4];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) fs[i4] = finish_score<T>(c[i4], p.scale);
            sc[j * SIDE + i][0] = DT<T>::pack(&fs[0]);
            sc[j * SIDE + i][1] = DT<T>::pack(&fs[2]);
        }

    // ---- BilinearSoftmax per item; weights kept packed in pairs of taps
    uint32_t ap[4][M / 2];
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        {
            float s[M], wf[4];
#pragma unroll
            for (int m = 0; m < M; ++m) s[m] = DT<T>::unpack(sc[m][i4 >> 1], i4 & 1);
#pragma unroll
            for (int e = 0; e < 4; ++e) wf[e] = DT<T>::unpack(wgt[i4][e >> 1], e & 1);
            bilinear_softmax<T, R>(s, wf, ap[i4]);
        }
        if (p.attn != nullptr && valid[i4])
            store_words<M / 2>(static_cast<T *>(p.attn) + bq[i4] * p.attn_stride + head_of[i4] * M, ap[i4]);
    }

    // ---- values: two taps per matrix instruction, column halves one after the other
    float o[2][NW][4];
#pragma unroll
    for (int ch = 0; ch < 2; ++ch)
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[ch][w][e] = 0.f;
#pragma unroll
    for (int m = 0; m < M; m += 2) {
        const int j0 = m / SIDE, i0 = m % SIDE, j1 = (m + 1) / SIDE, i1 = (m + 1) % SIDE;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
            uint32_t v0[2][NW], v1[2][NW];
#pragma unroll
            for (int rh = 0; rh < 2; ++rh) {
                const int i4 = 2 * rh + ch;
                load_words<NW>(v0[rh], vb + (row[i4][j0] + col[i4][i0]));
                load_words<NW>(v1[rh], vb + (row[i4][j1] + col[i4][i1]));
            }
#pragma unroll
            for (int rh = 0; rh < 2; ++rh) {
                const int i4 = 2 * rh + ch;
                const uint32_t a_lo = dup_lo(ap[i4][m / 2]), a_hi = dup_hi(ap[i4][m / 2]);
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    v0[rh][w] = Mma<T>::mul2(a_lo, v0[rh][w]);
                    v1[rh][w] = Mma<T>::mul2(a_hi, v1[rh][w]);
                }
            }
#pragma unroll
            for (int w = 0; w < NW; ++w) Mma<T>::run(o[ch][w], v0[0][w], v0[1][w], v1[0][w], v1[1][w], b_id, b_id);
        }
    }

#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        if (!valid[i4]) continue;
        const int rh = i4 >> 1, ch = i4 & 1;
        uint32_t ow[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) ow[w] = DT<T>::pack(&o[ch][w][2 * rh]);
        store_words<NW>(static_cast<T *>(p.out) + bq[i4] * p.out_stride + lane_off[i4], ow);
    }
}

template <typename T>
cudaError_t launch_mma(const Params &p, int r, int cpl, dim3 grid, cudaStream_t stream);

}  // namespace matchattn
