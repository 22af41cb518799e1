// Staged MatchAttention forward for sm_100a: K/V tiles brought into shared memory by the tensor
// memory accelerator (cp.async.bulk.tensor, completion signalled on an mbarrier), taps read from there.
//
// When it pays.  The direct kernel issues one load instruction per tap and lane.  With one sampling
// centre per (query, head) -- the self-attention case -- every lane of such a load touches its own
// 128-byte line, and the L1 tag stage, not the data, limits the kernel (measured: with the arithmetic
// removed the direct kernel still needs 90 % of its time on such inputs).  When the centres of
// neighbouring queries stay close together (self attention, smooth disparity or flow fields) the taps of
// a tile of queries all fall into a small region of the token map, which is copied to shared memory
// once, as whole lines, by one instruction; tap reads then cost shared-memory bandwidth only.
//
// One block = one tile of QW x QH queries (all heads), IPT queries-with-heads per thread:
//   1. every thread reads the centres of its items and the block reduces the extent of all their
//      (clamped) windows;
//   2. if the extent fits the RW x RH region the tensor maps were encoded for, thread 0 requests the K
//      region; all threads wait on the mbarrier (bounded), compute scores and BilinearSoftmax for their
//      items from shared memory and write attn_out; the packed weights stay in thread-local memory;
//   3. after a block barrier the same buffer receives the V region and the weighted sums follow;
//   4. a tile whose windows spread further is served with the direct kernel's global loads by the same
//      block: no input is ever refused, the staging is an optimisation per tile.
// Two such blocks share an SM, so one computes while the other waits for its copy (strategy 6).  A second
// form keeps one persistent block per SM with a producer warp and 24 consumer warps (strategy 5, further
// down).  Measured on a B200 (384 x 384 tokens, 8 heads x 16, float16): L2->SM traffic falls 3.2x against the
// direct kernel (10 M instead of 34 M sectors per item), the run time does not (88-90 us against 86 us per item
// with one centre per head, 93-99 against 73 with shared centres): the operator is bound by instruction
// issue on every path.  Both forms are therefore selected on request, not automatically.  Taps outside the map
// are index-clamped exactly as in the direct kernel; the part of a region that sticks out of the map is
// zero-filled by the copy and never read.
//
// The tensor maps cover this GPU's own K and V only; the copy is the plain form, delivered to this block's
// shared memory alone.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "matchattn_binned.cuh"      // lds_128

namespace matchattn {

constexpr int kStagedThreads = 256;
constexpr int kStagedQW = 16;                       // tile width in queries
constexpr size_t kStagedRegionBytes = 110 * 1024;   // shared-memory region of one block (two blocks per SM)
constexpr int kStagedMaxIPT = 8;

struct StagedParams {
    Params p;
    int ipt;            // items (query, head) per thread = iterations over the tile
    int rows_per_it;    // query rows one iteration covers: (kStagedThreads / h) / kStagedQW
    int QH;             // tile height in queries = ipt * rows_per_it
    int RW, RH;         // staged region in tokens
    int tiles_x;
    uint32_t region_bytes;   // RW * RH * C * sizeof(T)
    unsigned long long *fallback_tiles;   // or null: counts the tiles served by global loads (diagnostics)
};

// ---- mbarrier / bulk-tensor copy primitives ---------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Waits for the phase with the given parity; gives up after `limit` polls (returns false) so that a copy
// that never completes cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (done) return true;
    }
    return false;
}

// One box of a rank-4 tensor (channels, x, y, item) into shared memory, completion on `bar`.
__device__ __forceinline__ void tma_load_box(void *dst, const CUtensorMap *map, int x, int y, int item, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(x), "r"(y), "r"(item),
                   "r"(smem_u32(bar))
                 : "memory");
}

// A lane's NW words of one tap.  STAGED: from the region in shared memory.  A lane's slice is 16 * NW / 4
// bytes at a 256-byte token pitch, so lanes 128 bytes apart would hit the same banks: they take their
// 16-byte pieces in rotated order (`rot`), and the caller keeps q and the output accumulators in the
// same rotated order.  Otherwise: from global memory, as the direct kernel does.
template <typename T, int NW, bool STAGED>
__device__ __forceinline__ void load_tap(uint32_t (&w)[NW], uint32_t smem_addr, int rot, const T *gptr)
{
    if constexpr (STAGED) {
        constexpr int PIECES = NW / 4;
#pragma unroll
        for (int c = 0; c < PIECES; ++c) lds_128(&w[4 * c], smem_addr + 16u * static_cast<uint32_t>((c + rot) & (PIECES - 1)));
    } else {
        load_words<NW>(w, gptr);
    }
}

// ---- the kernel --------------------------------------------------------------------------------

// geometry of one item of the tile
struct StagedItem {
    bool valid;
    int64_t bq;
    float x, y;
};

template <typename T, int CPL, bool POW2>
__global__ void __launch_bounds__(kStagedThreads, 2)
staged_forward_kernel(const StagedParams sp, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v)
{
    constexpr int R = 1, SIDE = 4, M = 16;
    constexpr int NW = CPL * DT<T>::kWordsPerChunk;       // 4 or 8 words per lane and tap
    constexpr int EPW = 2, NWA = M / EPW;
    constexpr int PIECES = NW / 4;
    static_assert(sizeof(T) == 2 && (CPL == 1 || CPL == 2), "16-bit types, 8 or 16 channels per head");
    const Params &p = sp.p;

    extern __shared__ unsigned char smem_raw[];
    unsigned char *region = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    __shared__ uint64_t bar;
    __shared__ int ext[4];              // min x, max x, min y, max y of the clamped windows of the tile

    const int tid = threadIdx.x;
    const int lq = tid / p.h, head = tid - lq * p.h;
    const int tile_y = blockIdx.x / sp.tiles_x, tile_x = blockIdx.x - tile_y * sp.tiles_x;
    const int b = blockIdx.y;
    const int qx = tile_x * kStagedQW + (lq & (kStagedQW - 1));
    const int qy_base = tile_y * sp.QH + (lq >> 4);
    const int lane_off = head * p.hd;                      // channels
    const uint32_t lane_byte = static_cast<uint32_t>(lane_off) * 2u;
    const int rot = (PIECES > 1) ? static_cast<int>((lane_byte >> 7) & (PIECES - 1)) : 0;

    if (tid == 0) {
        mbar_init(&bar, 1);
        ext[0] = 0x7fffffff; ext[1] = -0x7fffffff; ext[2] = 0x7fffffff; ext[3] = -0x7fffffff;
    }
    __syncthreads();

    auto item_of = [&](int it) {
        StagedItem s;
        const int qy = qy_base + it * sp.rows_per_it;
        s.valid = lq < (kStagedThreads / p.h) && qx < p.W && qy < p.rows;
        s.bq = static_cast<int64_t>(b) * p.Nq + static_cast<int64_t>(min(qy, p.rows - 1)) * p.W + min(qx, p.W - 1);
        DT<T>::load_xy(static_cast<const T *>(p.mo) + (s.bq * p.h + head) * 2, s.x, s.y);
        return s;
    };

    // 1. extent of the tile's windows
    {
        int lox = 0x7fffffff, hix = -0x7fffffff, loy = 0x7fffffff, hiy = -0x7fffffff;
#pragma unroll
        for (int it = 0; it < kStagedMaxIPT; ++it) {        // unrolled: the centre loads of all items are in flight together
            if (it >= sp.ipt) break;
            const StagedItem s = item_of(it);
            if (!s.valid) continue;
            const int x0 = window_origin(floorf(s.x), R, p.W) - R, y0 = window_origin(floorf(s.y), R, p.H) - R;
            lox = min(lox, min(max(x0, 0), p.W - 1));
            hix = max(hix, min(max(x0 + SIDE - 1, 0), p.W - 1));
            loy = min(loy, min(max(y0, 0), p.H - 1));
            hiy = max(hiy, min(max(y0 + SIDE - 1, 0), p.H - 1));
        }
        for (int o = 16; o > 0; o >>= 1) {
            lox = min(lox, __shfl_xor_sync(0xffffffffu, lox, o));
            hix = max(hix, __shfl_xor_sync(0xffffffffu, hix, o));
            loy = min(loy, __shfl_xor_sync(0xffffffffu, loy, o));
            hiy = max(hiy, __shfl_xor_sync(0xffffffffu, hiy, o));
        }
        if ((tid & 31) == 0) {
            atomicMin(&ext[0], lox); atomicMax(&ext[1], hix); atomicMin(&ext[2], loy); atomicMax(&ext[3], hiy);
        }
    }
    __syncthreads();
    const int lox = ext[0], hix = ext[1], loy = ext[2], hiy = ext[3];
    if (hix < lox) return;                                  // no valid item in this tile
    bool staged = (hix - lox + 1 <= sp.RW) && (hiy - loy + 1 <= sp.RH);

    constexpr uint32_t kWaitPolls = 1u << 24;              // far beyond any real copy; bounds the wait
    if (staged) {
        if (tid == 0) {
            mbar_expect_tx(&bar, sp.region_bytes);
            tma_load_box(region, &map_k, lox, loy, b, &bar);
        }
        const bool arrived = mbar_wait(&bar, 0, kWaitPolls);
        // a copy that did not arrive in time: wait once more (the buffer must not be abandoned while a
        // copy may still land in it), then serve the tile from global memory
        if (!__syncthreads_and(arrived)) {
            mbar_wait(&bar, 0, kWaitPolls);
            staged = false;
            __syncthreads();
        }
    }
    if (!staged && tid == 0 && sp.fallback_tiles != nullptr) atomicAdd(sp.fallback_tiles, 1ull);

    const uint32_t tok_bytes = static_cast<uint32_t>(p.C) * 2u;
    const uint32_t row_bytes = tok_bytes * static_cast<uint32_t>(sp.RW);
    const uint32_t region_lane = smem_u32(region) + lane_byte;
    const T *kg = static_cast<const T *>(p.k) + static_cast<int64_t>(b) * p.N * p.C + lane_off;
    const T *vg = static_cast<const T *>(p.v) + static_cast<int64_t>(b) * p.N * p.C + lane_off;

    uint32_t aw_all[kStagedMaxIPT][NWA];                    // packed attention weights of the thread's items

    // tap geometry of an item: byte offsets into the region (STAGED) or element offsets into K/V
    auto geometry = [&](const StagedItem &s, bool use_region, uint32_t (&col)[SIDE], uint32_t (&row)[SIDE], float (&wgt)[4]) {
        const float xf = floorf(s.x), yf = floorf(s.y);
        bilinear_weights<T>(s.x, xf, s.y, yf, wgt);
        const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            const int tx = min(max(x0 + i, 0), p.W - 1), ty = min(max(y0 + i, 0), p.H - 1);
            if (use_region) {
                col[i] = static_cast<uint32_t>(tx - lox) * tok_bytes;
                row[i] = static_cast<uint32_t>(ty - loy) * row_bytes;
            } else {
                col[i] = static_cast<uint32_t>(tx * p.C);
                row[i] = static_cast<uint32_t>(ty * p.W * p.C);
            }
        }
    };

    // 2. scores and BilinearSoftmax
    auto scores = [&](auto staged_tag) {
        constexpr bool ST = decltype(staged_tag)::value;
        // the centre and the query slice of the NEXT item are requested before the current item is worked
        // on, so that their latency hides behind it (the loop over the items is not unrolled)
        StagedItem s = item_of(0);
        uint32_t qw[NW];
        load_words<NW>(qw, static_cast<const T *>(p.q) + s.bq * p.C + lane_off);
        for (int it = 0; it < sp.ipt; ++it) {
            const StagedItem cur = s;
            uint32_t qr[NW];
#pragma unroll
            for (int w = 0; w < NW; ++w) qr[w] = (ST && rot) ? qw[(w + 4) & (NW - 1)] : qw[w];   // pieces in load order
            if (it + 1 < sp.ipt) {
                s = item_of(it + 1);
                load_words<NW>(qw, static_cast<const T *>(p.q) + s.bq * p.C + lane_off);
            }
            if (!cur.valid) continue;                       // (its window need not lie inside the region)
            uint32_t col[SIDE], row[SIDE];
            float wgt[4];
            geometry(cur, ST, col, row, wgt);
            float sc[M];
            uint32_t spk[POW2 ? M / 2 : 1];
            float part_even = 0.f;
#pragma unroll
            for (int j = 0; j < SIDE; ++j)
#pragma unroll
                for (int i = 0; i < SIDE; ++i) {
                    uint32_t kw[NW];
                    load_tap<T, NW, ST>(kw, region_lane + row[j] + col[i], rot, kg + row[j] + col[i]);
                    float a0 = 0.f, a1 = 0.f;
#pragma unroll
                    for (int w = 0; w < NW; ++w) DT<T>::absdiff(a0, a1, qr[w], kw[w]);
                    const float part = a0 + a1;
                    if constexpr (POW2) {
                        if (i & 1) spk[(j * SIDE + i) >> 1] = DT<T>::aw_mul(DT<T>::aw_from(-part_even, -part), DT<T>::aw_bcast(p.scale));
                        else part_even = part;
                    } else {
                        sc[j * SIDE + i] = finish_score<T>(part, p.scale);
                    }
                }
            if constexpr (POW2) {
#pragma unroll
                for (int m = 0; m < M; m += 2) {
                    sc[m] = DT<T>::unpack(spk[m >> 1], 0);
                    sc[m + 1] = DT<T>::unpack(spk[m >> 1], 1);
                }
            }
            uint32_t aw[NWA];
            bilinear_softmax<T, R>(sc, wgt, aw);
            if (p.attn != nullptr) store_words<NWA>(static_cast<T *>(p.attn) + (cur.bq * p.h + head) * M, aw);
#pragma unroll
            for (int w = 0; w < NWA; ++w) aw_all[it][w] = aw[w];
        }
    };

    // 3. weighted sums of the value taps
    auto values = [&](auto staged_tag) {
        constexpr bool ST = decltype(staged_tag)::value;
        StagedItem s = item_of(0);
        uint32_t awn[NWA];
#pragma unroll
        for (int w = 0; w < NWA; ++w) awn[w] = aw_all[0][w];
        for (int it = 0; it < sp.ipt; ++it) {
            const StagedItem cur = s;
            uint32_t aw[NWA];
#pragma unroll
            for (int w = 0; w < NWA; ++w) aw[w] = awn[w];
            if (it + 1 < sp.ipt) {                          // next item's centre and weights, ahead of their use
                s = item_of(it + 1);
#pragma unroll
                for (int w = 0; w < NWA; ++w) awn[w] = aw_all[it + 1][w];
            }
            if (!cur.valid) continue;
            uint32_t col[SIDE], row[SIDE];
            float wgt[4];
            geometry(cur, ST, col, row, wgt);
            float o[NW * EPW];
#pragma unroll
            for (int c = 0; c < NW * EPW; ++c) o[c] = 0.f;
#pragma unroll
            for (int j = 0; j < SIDE; ++j)
#pragma unroll
                for (int i = 0; i < SIDE; ++i) {
                    uint32_t vw[NW];
                    load_tap<T, NW, ST>(vw, region_lane + row[j] + col[i], rot, vg + row[j] + col[i]);
                    const typename DT<T>::Bcast am = DT<T>::aw_tap(aw, j * SIDE + i);
#pragma unroll
                    for (int w = 0; w < NW; ++w) DT<T>::wmul(am, vw[w], &o[w * EPW]);
                }
            uint32_t pk[NW], ow[NW];
#pragma unroll
            for (int w = 0; w < NW; ++w) pk[w] = DT<T>::pack(&o[w * EPW]);
#pragma unroll
            for (int w = 0; w < NW; ++w) ow[w] = (ST && rot) ? pk[(w + 4) & (NW - 1)] : pk[w];      // undo the rotation
            store_words<NW>(static_cast<T *>(p.out) + cur.bq * p.C + lane_off, ow);
        }
    };

    if (staged) {
        scores(std::true_type{});
        __syncthreads();                                   // every thread is done with the K region
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&bar, sp.region_bytes);
            tma_load_box(region, &map_v, lox, loy, b, &bar);
        }
        const bool arrived = mbar_wait(&bar, 1, kWaitPolls);
        if (!__syncthreads_and(arrived)) {
            mbar_wait(&bar, 1, kWaitPolls);
            __syncthreads();
            values(std::false_type{});
        } else {
            values(std::true_type{});
        }
    } else {
        scores(std::false_type{});
        values(std::false_type{});
    }
}

// ---- the persistent, warp-specialised form -----------------------------------------------------
//
// One block per SM, 25 warps: warp 0 is the producer, warps 1-24 (768 threads) are consumers, one
// (query, head) item per consumer thread and tile.  Shared memory holds ONE K region and ONE V region;
// the two are refilled alternately, so that every copy has a whole phase of the consumers to arrive in:
//
//   producer, tile t:   extent of the tile's windows (its 768 centres, 24 per lane)
//                       wait empty_K (consumers done with the scores of tile t-1)   -> copy K region of t
//                       wait empty_V (consumers done with the values of tile t-1)   -> copy V region of t
//   consumers, tile t:  wait full_K -> scores, BilinearSoftmax, attn_out           -> arrive empty_K
//                       wait full_V -> weighted value sums, out                    -> arrive empty_V
//
// While the consumers add up the values of tile t the K region of tile t+1 lands, and while they score
// tile t+1 its V region lands.  The attention weights of an item stay in its thread's registers between
// the two phases.  A tile whose windows do not fit the region is flagged in the tile's info slot and served
// with global loads.  Every wait is bounded: a wait that runs out raises the block's abort flag, which ends
// all roles (the remaining tiles of that block stay unwritten and the call's status word counts the event).

constexpr int kPersistConsumers = 768;
constexpr int kPersistThreads = kPersistConsumers + 32;
constexpr size_t kPersistRegionBytes = 96 * 1024;        // one K (or V) region; two of them per block

struct PersistParams {
    Params p;
    int QH;              // tile height in queries: (768 / h) / 16
    int RW, RH;          // staged region in tokens
    int tiles_x, tiles_y;
    long long total_tiles;   // tiles_x * tiles_y * B
    uint32_t region_bytes;   // RW * RH * C * sizeof(T) <= kPersistRegionBytes
    unsigned long long *status;   // or null: [0] += tiles served by global loads, bit 63 set when a wait ran out
};

struct TileInfo {
    int lox, loy;        // origin of the staged region in the token map
    int staged;          // 1: taps come from the regions, 0: from global memory
    int pad;
};

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// bounded wait that also gives up when another role has raised the abort flag
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < (1u << 26); ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (done) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

template <typename T, int CPL, bool POW2>
__global__ void __launch_bounds__(kPersistThreads, 1)
staged_persistent_kernel(const PersistParams sp, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v)
{
    constexpr int R = 1, SIDE = 4, M = 16;
    constexpr int NW = CPL * DT<T>::kWordsPerChunk;
    constexpr int EPW = 2, NWA = M / EPW;
    constexpr int PIECES = NW / 4;
    static_assert(sizeof(T) == 2 && (CPL == 1 || CPL == 2), "16-bit types, 8 or 16 channels per head");
    const Params &p = sp.p;

    extern __shared__ unsigned char smem_raw[];
    unsigned char *region_k = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    unsigned char *region_v = region_k + kPersistRegionBytes;
    __shared__ uint64_t full_k, full_v, empty_k, empty_v;
    __shared__ TileInfo info[2];
    __shared__ int abort_flag;

    const int tid = threadIdx.x;
    if (tid == 0) {
        mbar_init(&full_k, 1);
        mbar_init(&full_v, 1);
        mbar_init(&empty_k, kPersistConsumers / 32);
        mbar_init(&empty_v, kPersistConsumers / 32);
        abort_flag = 0;
    }
    __syncthreads();
    volatile int *abort_ptr = &abort_flag;

    const int per_item = sp.tiles_x * sp.tiles_y;
    const int qpt = kPersistConsumers / p.h;                 // queries per tile

    if (tid < 32) {
        // ---------------------------------------------------------------- producer warp
        unsigned long long fallbacks = 0;
        int it = 0;
        for (long long tile = blockIdx.x; tile < sp.total_tiles; tile += gridDim.x, ++it) {
            const int b = static_cast<int>(tile / per_item);
            const int rem = static_cast<int>(tile - static_cast<long long>(b) * per_item);
            const int tile_y = rem / sp.tiles_x, tile_x = rem - tile_y * sp.tiles_x;
            int lox = 0x7fffffff, hix = -0x7fffffff, loy = 0x7fffffff, hiy = -0x7fffffff;
            // the 768 centres of the tile, 24 per lane, eight loads in flight at a time
            for (int base = 0; base < kPersistConsumers; base += 256) {
                float cx[8], cy[8];
                bool ok8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int c = base + u * 32 + tid;
                    const int lq = c / p.h, head = c - lq * p.h;
                    const int qx = tile_x * kStagedQW + (lq & (kStagedQW - 1)), qy = tile_y * sp.QH + (lq >> 4);
                    ok8[u] = lq < qpt && qx < p.W && qy < p.rows;
                    const int64_t bq = static_cast<int64_t>(b) * p.Nq + static_cast<int64_t>(min(qy, p.rows - 1)) * p.W + min(qx, p.W - 1);
                    DT<T>::load_xy(static_cast<const T *>(p.mo) + (bq * p.h + min(head, p.h - 1)) * 2, cx[u], cy[u]);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (!ok8[u]) continue;
                    const int x0 = window_origin(floorf(cx[u]), R, p.W) - R, y0 = window_origin(floorf(cy[u]), R, p.H) - R;
                    lox = min(lox, min(max(x0, 0), p.W - 1));
                    hix = max(hix, min(max(x0 + SIDE - 1, 0), p.W - 1));
                    loy = min(loy, min(max(y0, 0), p.H - 1));
                    hiy = max(hiy, min(max(y0 + SIDE - 1, 0), p.H - 1));
                }
            }
            for (int o = 16; o > 0; o >>= 1) {
                lox = min(lox, __shfl_xor_sync(0xffffffffu, lox, o));
                hix = max(hix, __shfl_xor_sync(0xffffffffu, hix, o));
                loy = min(loy, __shfl_xor_sync(0xffffffffu, loy, o));
                hiy = max(hiy, __shfl_xor_sync(0xffffffffu, hiy, o));
            }
            const bool staged = hix >= lox && (hix - lox + 1 <= sp.RW) && (hiy - loy + 1 <= sp.RH);
            if (!staged) ++fallbacks;
            bool ok = true;
            if (tid == 0) {
                // K of this tile: the consumers must be done with the scores of the previous one
                if (it > 0) ok = mbar_wait_or_abort(&empty_k, static_cast<uint32_t>((it - 1) & 1), abort_ptr);
                if (ok) {
                    info[it & 1].lox = lox; info[it & 1].loy = loy; info[it & 1].staged = staged ? 1 : 0;
                    if (staged) {
                        mbar_expect_tx(&full_k, sp.region_bytes);
                        tma_load_box(region_k, &map_k, lox, loy, b, &full_k);
                    } else {
                        mbar_arrive(&full_k);
                    }
                    if (it > 0) ok = mbar_wait_or_abort(&empty_v, static_cast<uint32_t>((it - 1) & 1), abort_ptr);
                }
                if (ok) {
                    if (staged) {
                        mbar_expect_tx(&full_v, sp.region_bytes);
                        tma_load_box(region_v, &map_v, lox, loy, b, &full_v);
                    } else {
                        mbar_arrive(&full_v);
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
        }
        if (tid == 0 && sp.status != nullptr) {
            unsigned long long add = fallbacks;      // (every lane counted the same tiles)
            if (*abort_ptr) add |= 1ull << 63;
            if (add) atomicAdd(sp.status, add);
        }
        return;
    }

    // -------------------------------------------------------------------- consumer warps
    const int c = tid - 32;
    const int lq = c / p.h, head = c - lq * p.h;
    const int lane_off = head * p.hd;
    const uint32_t lane_byte = static_cast<uint32_t>(lane_off) * 2u;
    const int rot = (PIECES > 1) ? static_cast<int>((lane_byte >> 7) & (PIECES - 1)) : 0;
    const uint32_t tok_bytes = static_cast<uint32_t>(p.C) * 2u;
    const uint32_t row_bytes = tok_bytes * static_cast<uint32_t>(sp.RW);
    const uint32_t rk_lane = smem_u32(region_k) + lane_byte, rv_lane = smem_u32(region_v) + lane_byte;
    const bool lane0 = (tid & 31) == 0;

    int it = 0;
    for (long long tile = blockIdx.x; tile < sp.total_tiles; tile += gridDim.x, ++it) {
        const int b = static_cast<int>(tile / per_item);
        const int rem = static_cast<int>(tile - static_cast<long long>(b) * per_item);
        const int tile_y = rem / sp.tiles_x, tile_x = rem - tile_y * sp.tiles_x;
        const int qx = tile_x * kStagedQW + (lq & (kStagedQW - 1)), qy = tile_y * sp.QH + (lq >> 4);
        const bool valid = lq < qpt && qx < p.W && qy < p.rows;
        const int64_t bq = static_cast<int64_t>(b) * p.Nq + static_cast<int64_t>(min(qy, p.rows - 1)) * p.W + min(qx, p.W - 1);
        const T *kg = static_cast<const T *>(p.k) + static_cast<int64_t>(b) * p.N * p.C + lane_off;
        const T *vg = static_cast<const T *>(p.v) + static_cast<int64_t>(b) * p.N * p.C + lane_off;

        // requested before the wait: centre and query slice of this item
        float x, y;
        DT<T>::load_xy(static_cast<const T *>(p.mo) + (bq * p.h + head) * 2, x, y);
        uint32_t qw[NW];
        load_words<NW>(qw, static_cast<const T *>(p.q) + bq * p.C + lane_off);

        if (!mbar_wait_or_abort(&full_k, static_cast<uint32_t>(it & 1), abort_ptr)) return;
        const int lox = info[it & 1].lox, loy = info[it & 1].loy;
        const bool staged = info[it & 1].staged != 0;

        const float xf = floorf(x), yf = floorf(y);
        float wgt[4];
        bilinear_weights<T>(x, xf, y, yf, wgt);
        const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
        uint32_t col[SIDE], row[SIDE];
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            const int tx = min(max(x0 + i, 0), p.W - 1), ty = min(max(y0 + i, 0), p.H - 1);
            col[i] = staged ? static_cast<uint32_t>(tx - lox) * tok_bytes : static_cast<uint32_t>(tx * p.C);
            row[i] = staged ? static_cast<uint32_t>(ty - loy) * row_bytes : static_cast<uint32_t>(ty * p.W * p.C);
        }
        const bool swap = staged && rot != 0;
        uint32_t aw[NWA];
        if (valid) {
            uint32_t qr[NW];
#pragma unroll
            for (int w = 0; w < NW; ++w) qr[w] = swap ? qw[(w + 4) & (NW - 1)] : qw[w];
            float sc[M];
            uint32_t spk[POW2 ? M / 2 : 1];
            float part_even = 0.f;
            auto score_taps = [&](auto staged_tag) {
                constexpr bool ST = decltype(staged_tag)::value;
#pragma unroll
                for (int j = 0; j < SIDE; ++j)
#pragma unroll
                    for (int i = 0; i < SIDE; ++i) {
                        uint32_t kw[NW];
                        load_tap<T, NW, ST>(kw, rk_lane + row[j] + col[i], rot, kg + row[j] + col[i]);
                        float a0 = 0.f, a1 = 0.f;
#pragma unroll
                        for (int w = 0; w < NW; ++w) DT<T>::absdiff(a0, a1, qr[w], kw[w]);
                        const float part = a0 + a1;
                        if constexpr (POW2) {
                            if (i & 1) spk[(j * SIDE + i) >> 1] = DT<T>::aw_mul(DT<T>::aw_from(-part_even, -part), DT<T>::aw_bcast(p.scale));
                            else part_even = part;
                        } else {
                            sc[j * SIDE + i] = finish_score<T>(part, p.scale);
                        }
                    }
            };
            if (staged) score_taps(std::true_type{});
            else score_taps(std::false_type{});
            if constexpr (POW2) {
#pragma unroll
                for (int m = 0; m < M; m += 2) {
                    sc[m] = DT<T>::unpack(spk[m >> 1], 0);
                    sc[m + 1] = DT<T>::unpack(spk[m >> 1], 1);
                }
            }
            bilinear_softmax<T, R>(sc, wgt, aw);
            if (p.attn != nullptr) store_words<NWA>(static_cast<T *>(p.attn) + (bq * p.h + head) * M, aw);
        }
        __syncwarp();
        if (lane0) mbar_arrive(&empty_k);               // this warp no longer reads the K region

        if (!mbar_wait_or_abort(&full_v, static_cast<uint32_t>(it & 1), abort_ptr)) return;
        if (valid) {
            float o[NW * EPW];
#pragma unroll
            for (int cc = 0; cc < NW * EPW; ++cc) o[cc] = 0.f;
            auto value_taps = [&](auto staged_tag) {
                constexpr bool ST = decltype(staged_tag)::value;
#pragma unroll
                for (int j = 0; j < SIDE; ++j)
#pragma unroll
                    for (int i = 0; i < SIDE; ++i) {
                        uint32_t vw[NW];
                        load_tap<T, NW, ST>(vw, rv_lane + row[j] + col[i], rot, vg + row[j] + col[i]);
                        const typename DT<T>::Bcast am = DT<T>::aw_tap(aw, j * SIDE + i);
#pragma unroll
                        for (int w = 0; w < NW; ++w) DT<T>::wmul(am, vw[w], &o[w * EPW]);
                    }
            };
            if (staged) value_taps(std::true_type{});
            else value_taps(std::false_type{});
            uint32_t pk[NW], ow[NW];
#pragma unroll
            for (int w = 0; w < NW; ++w) pk[w] = DT<T>::pack(&o[w * EPW]);
#pragma unroll
            for (int w = 0; w < NW; ++w) ow[w] = swap ? pk[(w + 4) & (NW - 1)] : pk[w];
            store_words<NW>(static_cast<T *>(p.out) + bq * p.C + lane_off, ow);
        }
        __syncwarp();
        if (lane0) mbar_arrive(&empty_v);
    }
}

template <typename T>
cudaError_t launch_staged_persistent(const PersistParams &sp, int cpl, const CUtensorMap &map_k, const CUtensorMap &map_v,
                                     int grid_blocks, cudaStream_t stream);

template <typename T>
cudaError_t launch_staged(const StagedParams &sp, int cpl, const CUtensorMap &map_k, const CUtensorMap &map_v, dim3 grid,
                          size_t smem_bytes, cudaStream_t stream);

}  // namespace matchattn
