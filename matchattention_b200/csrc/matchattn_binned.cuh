// Binned MatchAttention forward: queries are grouped by the tile of the token
// map their window falls into, each block stages that tile of K and V (plus a
// halo of one window) in shared memory once and serves all the queries of the
// bin from there.
//
// Why.  The direct kernels fetch the 2*(2r+2)^2 taps of every query from L2:
// 8 KB per query at C=128 in float16, six times the bytes the operator has to
// move.  When neighbouring queries look at unrelated places (offsets spread
// over tens of tokens) nothing of that is shared in L1 and the kernel is bound
// by L2->SM bandwidth.  Sorting the queries by where they look turns the
// scattered side of the gather around: K/V tiles are read once per bin
// (~1.6 tokens per query instead of 32 taps), and what becomes scattered is the
// query side, which is 3 whole-sector runs per query (q, out, attn_out).
//
// Passes (all on the caller's stream, scratch memory supplied by the caller):
//   1. bin_count   one thread per query: window origin -> tile -> bin, histogram;
//                  also checks that all heads of the query share one sampling
//                  centre (the cross-attention case).  If any query does not,
//                  a flag diverts the call to the direct kernel.
//   2. bin_scan    exclusive prefix sum of the histogram (one block).
//   3. bin_scatter counting-sort scatter of (query id, centre) records.
//   4. binned_forward_kernel  persistent blocks take bins from an atomic counter.
//
// The arithmetic of pass 4 is that of the matrix-instruction kernel
// (matchattn_mma.cuh): element-wise work on the 16-bit lanes, float32 sums on
// mma.sync with constant selector matrices; only the source of the taps
// differs (shared memory instead of global memory).
#pragma once

#include "matchattn_mma.cuh"

namespace matchattn {

// control words in the scratch area
enum { kCtrlBinCounter = 0, kCtrlNotShared = 1, kCtrlWords = 8 };

constexpr size_t kMaxBinnedSmem = 112 * 1024;  // dynamic shared memory of one block (two blocks per SM)
constexpr int kBinThreads = 256;              // threads of a block of pass 4 (two blocks per SM)
constexpr int kBinItemsPerPass = (kBinThreads / 32) * 128;

struct BinParams {
    Params p;
    uint32_t *counts;     // [nbins]
    uint32_t *starts;     // [nbins]
    uint32_t *cursors;    // [nbins]
    uint32_t *ctrl;       // [kCtrlWords]
    uint32_t *bin_of;     // [B * Nq]
    uint2 *sorted;        // [B * Nq]  x = query id (b*Nq + n), y = raw bits of the centre (16-bit x | y << 16)
    int bins_x, bins_y;   // bins per item in x and y
    int nbins;            // B * bins_x * bins_y
    int TX, TY;           // window origins per bin in x and y
    int RW, RH;           // staged region in tokens: TX + 2r + 1, TY + 2r + 1
    int region_bytes;     // RW * RH * C * sizeof(T): size of the K (or V) region in shared memory
};

// ---- helpers shared by the passes ----------------------------------------

template <typename T>
__device__ __forceinline__ void centre_from_bits(uint32_t bits, float &x, float &y);
template <>
__device__ __forceinline__ void centre_from_bits<__half>(uint32_t bits, float &x, float &y)
{
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&bits));
    x = f.x;
    y = f.y;
}
template <>
__device__ __forceinline__ void centre_from_bits<__nv_bfloat16>(uint32_t bits, float &x, float &y)
{
    x = __uint_as_float(bits << 16);
    y = __uint_as_float(bits & 0xffff0000u);
}

// ---- pass 1: histogram -----------------------------------------------------

template <typename T, int R>
__global__ void __launch_bounds__(256) bin_count_kernel(const BinParams bp)
{
    const Params &p = bp.p;
    const int64_t total = static_cast<int64_t>(p.B) * p.Nq;
    const int64_t bq = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (bq >= total) return;
    const uint32_t *mo = static_cast<const uint32_t *>(p.mo) + bq * p.h;   // one 32-bit word per head
    const uint32_t first = __ldg(mo);
    bool same = true;
    for (int hh = 1; hh < p.h; ++hh) same &= (__ldg(mo + hh) == first);
    if (!same) atomicOr(&bp.ctrl[kCtrlNotShared], 1u);
    float x, y;
    centre_from_bits<T>(first, x, y);
    const int x0 = min(max(window_origin(floorf(x), R, p.W) - R, 0), p.W - 1);
    const int y0 = min(max(window_origin(floorf(y), R, p.H) - R, 0), p.H - 1);
    const int b = static_cast<int>(bq / p.Nq);
    const uint32_t bin = (static_cast<uint32_t>(b) * bp.bins_y + y0 / bp.TY) * bp.bins_x + x0 / bp.TX;
    bp.bin_of[bq] = bin;
    atomicAdd(&bp.counts[bin], 1u);
}

// ---- pass 2: exclusive scan (one block of 1024 threads) ----------------------

static __global__ void __launch_bounds__(1024) bin_scan_kernel(const BinParams bp)
{
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        carry = 0;
        bp.ctrl[kCtrlBinCounter] = 0;
    }
    __syncthreads();
    for (int base = 0; base < bp.nbins; base += 1024) {
        const int i = base + tid;
        const uint32_t v = i < bp.nbins ? bp.counts[i] : 0u;
        uint32_t inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            uint32_t ws = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, ws, o);
                if (lane >= o) ws += n;
            }
            warp_sums[lane] = ws;
        }
        __syncthreads();
        const uint32_t before = carry + (warp ? warp_sums[warp - 1] : 0u) + inc - v;
        if (i < bp.nbins) {
            bp.starts[i] = before;
            bp.cursors[i] = before;
        }
        __syncthreads();
        if (tid == 1023) carry = before + v;
        __syncthreads();
    }
}

// ---- pass 3: scatter ---------------------------------------------------------

static __global__ void __launch_bounds__(256) bin_scatter_kernel(const BinParams bp)
{
    const Params &p = bp.p;
    const int64_t total = static_cast<int64_t>(p.B) * p.Nq;
    const int64_t bq = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (bq >= total) return;
    const uint32_t bin = bp.bin_of[bq];
    const uint32_t pos = atomicAdd(&bp.cursors[bin], 1u);
    const uint32_t bits = __ldg(static_cast<const uint32_t *>(p.mo) + bq * p.h);
    bp.sorted[pos] = make_uint2(static_cast<uint32_t>(bq), bits);
}

// ---- pass 4 --------------------------------------------------------------------

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void *gptr)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void lds_128(uint32_t *w, uint32_t smem_addr)
{
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(smem_addr));
}

// NW words of an item, 16 bytes at a time; `swz` (0 or 16) swaps the halves of every 32-byte pair
// so that the two queries of a quarter warp hit different banks.  The same permutation is applied
// to q, K, V and out, so the channel order inside a lane is consistent.
template <int NW>
__device__ __forceinline__ void lds_item(uint32_t (&w)[NW], uint32_t addr, uint32_t swz)
{
#pragma unroll
    for (int c = 0; c < NW / 4; ++c) lds_128(&w[4 * c], addr + ((16u * c) ^ swz));
}
template <int NW>
__device__ __forceinline__ void ldg_item(uint32_t (&w)[NW], const char *ptr, uint32_t swz)
{
#pragma unroll
    for (int c = 0; c < NW / 4; ++c) ld_nc_128(&w[4 * c], ptr + ((16u * c) ^ swz));
}
template <int NW>
__device__ __forceinline__ void stg_item(char *ptr, const uint32_t (&w)[NW], uint32_t swz)
{
#pragma unroll
    for (int c = 0; c < NW / 4; ++c) st_128(ptr + ((16u * c) ^ swz), &w[4 * c]);
}

// SAMEQ: the head count is a multiple of 8, so the two column halves of a row (columns t and t+4)
// are two heads of the SAME query and share its window; then a lane handles 2 queries x 2 heads
// and keeps one set of window coordinates per query instead of one per item.
template <typename T, int CPL, bool SAMEQ>
__global__ void __launch_bounds__(kBinThreads, 2) binned_forward_kernel(const BinParams bp)
{
    constexpr int R = 1, SIDE = 2 * R + 2, M = SIDE * SIDE;
    constexpr int NW = CPL * 4;
    constexpr int SLICE = CPL * 8;
    constexpr int NQ = SAMEQ ? 2 : 4;             // distinct windows per lane
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_bin;

    const Params &p = bp.p;
    if (bp.ctrl[kCtrlNotShared] != 0) return;      // the direct kernel launched after this one does the work

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t swz = (CPL % 2 == 0 && (g & 1)) ? 16u : 0u;
    const uint32_t ones = Mma<T>::kOneLo | Mma<T>::kOneHi;
    const uint32_t b_col0 = (g == 2 * t) ? ones : 0u;
    const uint32_t b_col1 = (g == 2 * t + 1) ? ones : 0u;
    const uint32_t b_id = (g == 2 * t) ? Mma<T>::kOneLo : ((g == 2 * t + 1) ? Mma<T>::kOneHi : 0u);
    const int RB = p.C * 2;                                   // bytes of a token row
    const uint32_t k_sm = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const uint32_t v_sm = k_sm + bp.region_bytes;

    for (;;) {
        __syncthreads();                                      // previous bin fully consumed, s_bin free
        if (tid == 0) s_bin = static_cast<int>(atomicAdd(&bp.ctrl[kCtrlBinCounter], 1u));
        __syncthreads();
        const int bin = s_bin;
        if (bin >= bp.nbins) break;
        const int cnt = static_cast<int>(bp.counts[bin]);
        if (cnt == 0) continue;
        const uint32_t start = bp.starts[bin];
        const int per_item = bp.bins_x * bp.bins_y;
        const int b = bin / per_item;
        const int rem = bin - b * per_item;
        const int by = rem / bp.bins_x, bx = rem - by * bp.bins_x;
        const int rx0 = bx * bp.TX, ry0 = by * bp.TY;
        const int ext_x = min(bp.RW, p.W - rx0), ext_y = min(bp.RH, p.H - ry0);

        // stage the K and V regions: rows of ext_x tokens, 16 bytes per copy
        {
            const int chunks = ext_x * (RB / 16);
            const char *kg = static_cast<const char *>(p.k) + (static_cast<int64_t>(b) * p.N + static_cast<int64_t>(ry0) * p.W + rx0) * RB;
            const char *vg = static_cast<const char *>(p.v) + (static_cast<int64_t>(b) * p.N + static_cast<int64_t>(ry0) * p.W + rx0) * RB;
            for (int rr = 0; rr < ext_y; ++rr) {
                const int64_t goff = static_cast<int64_t>(rr) * p.W * RB;
                const uint32_t soff = static_cast<uint32_t>(rr * bp.RW * RB);
                for (int c = tid; c < chunks; c += kBinThreads) {
                    cp_async_16(k_sm + soff + 16u * c, kg + goff + 16 * c);
                    cp_async_16(v_sm + soff + 16u * c, vg + goff + 16 * c);
                }
            }
            cp_async_wait_all();
        }
        __syncthreads();

        // each warp takes 128-item chunks of the bin on its own; the block meets again at the next bin
        const int items = cnt * p.h;
        for (int pass0 = warp * 128; pass0 < items; pass0 += kBinItemsPerPass) {
            // item i4 = 2*rowhalf + colhalf; window wq(i4) = its index into the per-query arrays
            bool valid[4];
            uint32_t qid[4];
            int head_of[4];
            int col[NQ][SIDE], row[NQ][SIDE];        // byte offsets inside a region, head 0
            uint32_t wgt[NQ][2];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                const int item = pass0 + (g + 8 * (i4 >> 1)) * 8 + t + 4 * (i4 & 1);
                int sq = item / p.h;
                head_of[i4] = item - sq * p.h;
                valid[i4] = sq < cnt;
                if (SAMEQ && (i4 & 1)) {               // same query as the item to its left
                    qid[i4] = qid[i4 - 1];
                    continue;
                }
                sq = min(sq, cnt - 1);
                const uint2 rec = bp.sorted[start + sq];
                qid[i4] = rec.x;
                const int wq = SAMEQ ? (i4 >> 1) : i4;
                float x, y;
                centre_from_bits<T>(rec.y, x, y);
                const float xf = floorf(x), yf = floorf(y);
                {
                    float wf[4];
                    bilinear_weights<T>(x, xf, y, yf, wf);
                    wgt[wq][0] = DT<T>::pack(&wf[0]);
                    wgt[wq][1] = DT<T>::pack(&wf[2]);
                }
                const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
#pragma unroll
                for (int i = 0; i < SIDE; ++i) {
                    col[wq][i] = (min(max(x0 + i, 0), p.W - 1) - rx0) * RB;
                    row[wq][i] = (min(max(y0 + i, 0), p.H - 1) - ry0) * bp.RW * RB;
                }
            }
            int hoff[4];                              // byte offset of the item's head inside a token row
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) hoff[i4] = head_of[i4] * (SLICE * 2);
#define MA_WQ(i4_) (SAMEQ ? ((i4_) >> 1) : (i4_))

            uint32_t qw[4][NW];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4)
                ldg_item<NW>(qw[i4], static_cast<const char *>(p.q) + static_cast<int64_t>(qid[i4]) * RB + hoff[i4], swz);

            // ---- scores
            uint32_t sc[M][2];
#pragma unroll
            for (int j = 0; j < SIDE; ++j)
#pragma unroll
                for (int i = 0; i < SIDE; ++i) {
                    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
                    {
                        uint32_t da[NW], db[NW];       // column half 0: items 0 (row g) and 2 (row g+8)
                        lds_item<NW>(da, k_sm + row[MA_WQ(0)][j] + col[MA_WQ(0)][i] + hoff[0], swz);
                        lds_item<NW>(db, k_sm + row[MA_WQ(2)][j] + col[MA_WQ(2)][i] + hoff[2], swz);
#pragma unroll
                        for (int w = 0; w < NW; ++w) {
                            da[w] = Mma<T>::absdiff2(qw[0][w], da[w]);
                            db[w] = Mma<T>::absdiff2(qw[2][w], db[w]);
                        }
#pragma unroll
                        for (int jj = 0; jj < NW / 2; ++jj)
                            Mma<T>::run(c0, da[2 * jj], db[2 * jj], da[2 * jj + 1], db[2 * jj + 1], b_col0, b_col0);
                    }
                    {
                        uint32_t da[NW], db[NW];       // column half 1: items 1 and 3
                        lds_item<NW>(da, k_sm + row[MA_WQ(1)][j] + col[MA_WQ(1)][i] + hoff[1], swz);
                        lds_item<NW>(db, k_sm + row[MA_WQ(3)][j] + col[MA_WQ(3)][i] + hoff[3], swz);
#pragma unroll
                        for (int w = 0; w < NW; ++w) {
                            da[w] = Mma<T>::absdiff2(qw[1][w], da[w]);
                            db[w] = Mma<T>::absdiff2(qw[3][w], db[w]);
                        }
#pragma unroll
                        for (int jj = 0; jj < NW / 2; ++jj)
                            Mma<T>::run(c1, da[2 * jj], db[2 * jj], da[2 * jj + 1], db[2 * jj + 1], b_col1, b_col1);
                    }
                    // the selectors leave c0's odd and c1's even entries at zero
                    const float fs[4] = {finish_score<T>(c0[0], p.scale), finish_score<T>(c1[1], p.scale),
                                         finish_score<T>(c0[2], p.scale), finish_score<T>(c1[3], p.scale)};
                    sc[j * SIDE + i][0] = DT<T>::pack(&fs[0]);
                    sc[j * SIDE + i][1] = DT<T>::pack(&fs[2]);
                }

            // ---- BilinearSoftmax per item
            uint32_t ap[4][M / 2];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                {
                    float s[M], wf[4];
#pragma unroll
                    for (int m = 0; m < M; ++m) s[m] = DT<T>::unpack(sc[m][i4 >> 1], i4 & 1);
#pragma unroll
                    for (int e = 0; e < 4; ++e) wf[e] = DT<T>::unpack(wgt[MA_WQ(i4)][e >> 1], e & 1);
                    bilinear_softmax<T, R>(s, wf, ap[i4]);
                }
                if (p.attn != nullptr && valid[i4])
                    store_words<M / 2>(static_cast<T *>(p.attn) + (static_cast<int64_t>(qid[i4]) * p.h + head_of[i4]) * M, ap[i4]);
            }

            // ---- values: one column half after the other, two taps per matrix instruction
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                float o[NW][4];
#pragma unroll
                for (int w = 0; w < NW; ++w)
#pragma unroll
                    for (int e = 0; e < 4; ++e) o[w][e] = 0.f;
                const int ia = ch, ib = 2 + ch;       // the items of rows g and g+8
#pragma unroll
                for (int m = 0; m < M; m += 2) {
                    const int j0 = m / SIDE, i0 = m % SIDE, j1 = (m + 1) / SIDE, i1 = (m + 1) % SIDE;
                    uint32_t va0[NW], va1[NW], vb0[NW], vb1[NW];
                    lds_item<NW>(va0, v_sm + row[MA_WQ(ia)][j0] + col[MA_WQ(ia)][i0] + hoff[ia], swz);
                    lds_item<NW>(va1, v_sm + row[MA_WQ(ia)][j1] + col[MA_WQ(ia)][i1] + hoff[ia], swz);
                    lds_item<NW>(vb0, v_sm + row[MA_WQ(ib)][j0] + col[MA_WQ(ib)][i0] + hoff[ib], swz);
                    lds_item<NW>(vb1, v_sm + row[MA_WQ(ib)][j1] + col[MA_WQ(ib)][i1] + hoff[ib], swz);
                    const uint32_t a_lo = dup_lo(ap[ia][m / 2]), a_hi = dup_hi(ap[ia][m / 2]);
                    const uint32_t b_lo = dup_lo(ap[ib][m / 2]), b_hi = dup_hi(ap[ib][m / 2]);
#pragma unroll
                    for (int w = 0; w < NW; ++w)
                        Mma<T>::run(o[w], Mma<T>::mul2(a_lo, va0[w]), Mma<T>::mul2(b_lo, vb0[w]),
                                    Mma<T>::mul2(a_hi, va1[w]), Mma<T>::mul2(b_hi, vb1[w]), b_id, b_id);
                }
#pragma unroll
                for (int rh = 0; rh < 2; ++rh) {
                    const int i4 = 2 * rh + ch;
                    if (!valid[i4]) continue;
                    uint32_t ow[NW];
#pragma unroll
                    for (int w = 0; w < NW; ++w) ow[w] = DT<T>::pack(&o[w][2 * rh]);
                    stg_item<NW>(static_cast<char *>(p.out) + static_cast<int64_t>(qid[i4]) * RB + hoff[i4], ow, swz);
                }
            }
#undef MA_WQ
        }
    }
}

// launchers (16-bit translation units)
template <typename T>
cudaError_t launch_binned(const BinParams &bp, int cpl, int grid_blocks, size_t smem_bytes, cudaStream_t stream);

}  // namespace matchattn
