// C ABI of the MatchAttention operator (declared in include/matchattn.h):
// argument validation, choice of kernel variant and launch geometry.
#include "../../include/matchattn.h"

#include <stdint.h>
#include <stdio.h>

#include "matchattn_kernels.cuh"
#include "matchattn_mma.cuh"
#include "matchattn_binned.cuh"
#include "matchattn_staged.cuh"

namespace matchattn {
namespace {

struct Plan {
    bool fast;
    int cpl;   // chunks (8 channels) per lane
    int lph;   // lanes per head
    bool mma;  // 16-bit, one lane per head, r == 1: accumulate with matrix instructions
    int mma_nch = 2;   // items per lane of that kernel: 2 * mma_nch
};

constexpr int kVariantAuto = 0, kVariantScalar = 1, kVariantMma = 2, kVariantMma2 = 3;   // 3: two items per lane
constexpr int kStrategyAuto = 0, kStrategyDirect = 1, kStrategyBinned = 2, kStrategySorted = 3, kStrategySortedMma = 4,
              kStrategyStaged = 5, kStrategyStagedBlocks = 6;

// Geometry of the binned path; valid == false when the arguments are outside what it covers.
struct BinGeometry {
    bool valid;
    int TX, TY, RW, RH, bins_x, bins_y, nbins, region_bytes;
    size_t off_counts, off_ctrl, off_starts, off_cursors, off_bin_of, off_sorted, total_bytes;
};

BinGeometry bin_geometry(int B, int H, int W, int h, int hd, int r, int dtype, int rows)
{
    BinGeometry gmt{};
    if (dtype == MATCHATTN_F32 || r != 1 || hd % 8 != 0 || hd > 40 || h > 128) return gmt;
    const long long RB = 2LL * h * hd;
    int TX = 16, TY = 8;
    auto region = [&](int tx, int ty) { return (tx + 2 * r + 1LL) * (ty + 2 * r + 1LL) * RB; };
    while (2 * region(TX, TY) > static_cast<long long>(kMaxBinnedSmem) && (TX > 1 || TY > 1)) {
        if (TX >= TY * 2 || TY == 1) TX /= 2; else TY /= 2;
    }
    if (2 * region(TX, TY) > static_cast<long long>(kMaxBinnedSmem)) return gmt;
    gmt.TX = TX; gmt.TY = TY;
    gmt.RW = TX + 2 * r + 1; gmt.RH = TY + 2 * r + 1;
    gmt.bins_x = (W + TX - 1) / TX; gmt.bins_y = (H + TY - 1) / TY;
    const long long nbins = 1LL * B * gmt.bins_x * gmt.bins_y, nq = 1LL * B * rows * W;
    // the kernels index (query, head) items of one bin, and of the whole call, with 32-bit integers
    if (nbins >= (1LL << 30) || nq * h >= (1LL << 31)) return gmt;
    gmt.nbins = static_cast<int>(nbins);
    gmt.region_bytes = static_cast<int>(region(TX, TY));
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    size_t off = 0;
    gmt.off_counts = off;  off += 4 * static_cast<size_t>(nbins);      // counts and ctrl are cleared together
    gmt.off_ctrl = off;    off = up(off + 4 * kCtrlWords);
    gmt.off_starts = off;  off = up(off + 4 * static_cast<size_t>(nbins));
    gmt.off_cursors = off; off = up(off + 4 * static_cast<size_t>(nbins));
    gmt.off_bin_of = off;  off = up(off + 4 * static_cast<size_t>(nq));
    gmt.off_sorted = off;  off = up(off + 8 * static_cast<size_t>(nq));
    gmt.total_bytes = off;
    gmt.valid = true;
    return gmt;
}
// ---- staged path: geometry and tensor maps ------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (the library does not link libcuda).
EncodeTiledFn encode_tiled()
{
    static const EncodeTiledFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return static_cast<EncodeTiledFn>(nullptr);
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

struct StagedGeometry {
    bool valid;
    int ipt, rows_per_it, QH, RW, RH;
};

// Tile and region of the staged path; valid == false when the arguments are outside what it covers.
StagedGeometry staged_geometry(int h, int hd, int r, int dtype)
{
    StagedGeometry g{};
    if (dtype == MATCHATTN_F32 || r != 1 || (hd != 8 && hd != 16)) return g;
    if (h != 1 && h != 2 && h != 4 && h != 8 && h != 16) return g;
    const int C = h * hd;
    if (C > 256) return g;                               // a box dimension holds at most 256 elements
    const int qpi = kStagedThreads / h;                  // queries per iteration
    g.rows_per_it = qpi / kStagedQW;
    g.ipt = 8 / g.rows_per_it;
    if (g.ipt < 1) g.ipt = 1;
    if (g.ipt > kStagedMaxIPT) g.ipt = kStagedMaxIPT;
    g.QH = g.ipt * g.rows_per_it;
    const long long tokens = static_cast<long long>(kStagedRegionBytes) / (2LL * C);
    int S = -1;
    while ((kStagedQW + 3 + 2 * (S + 1)) * 1LL * (g.QH + 3 + 2 * (S + 1)) <= tokens && kStagedQW + 3 + 2 * (S + 1) <= 256 &&
           g.QH + 3 + 2 * (S + 1) <= 256)
        ++S;
    if (S < 0) return g;
    g.RW = kStagedQW + 3 + 2 * S;
    g.RH = g.QH + 3 + 2 * S;
    g.valid = true;
    return g;
}

// Tile and region of the persistent staged kernel: 768 (query, head) items per tile, 16 queries wide.
StagedGeometry persist_geometry(int h, int hd, int r, int dtype)
{
    StagedGeometry g{};
    if (dtype == MATCHATTN_F32 || r != 1 || (hd != 8 && hd != 16)) return g;
    if (h != 1 && h != 2 && h != 4 && h != 8 && h != 16) return g;
    const int C = h * hd;
    if (C > 256) return g;
    g.ipt = 1;
    g.rows_per_it = (kPersistConsumers / h) / kStagedQW;
    g.QH = g.rows_per_it;
    const long long tokens = static_cast<long long>(kPersistRegionBytes) / (2LL * C);
    int S = -1;
    while ((kStagedQW + 3 + 2 * (S + 1)) * 1LL * (g.QH + 3 + 2 * (S + 1)) <= tokens && kStagedQW + 3 + 2 * (S + 1) <= 256 &&
           g.QH + 3 + 2 * (S + 1) <= 256)
        ++S;
    if (S < 0) return g;
    g.RW = kStagedQW + 3 + 2 * S;
    g.RH = g.QH + 3 + 2 * S;
    g.valid = true;
    return g;
}

bool make_kv_map(CUtensorMap *map, const void *base, int dtype, int B, int H, int W, int C, int RW, int RH)
{
    const EncodeTiledFn enc = encode_tiled();
    if (enc == nullptr) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                                static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[3] = {2ull * C, 2ull * C * W, 2ull * C * W * H};          // bytes, dimensions 1..3
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(C), static_cast<cuuint32_t>(RW), static_cast<cuuint32_t>(RH), 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUtensorMapDataType dt = dtype == MATCHATTN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    return enc(map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool is_pow2_float(float v)
{
    int e = 0;
    return v > 0.f && frexpf(v, &e) == 0.5f;
}

inline bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }
inline int ilog2(int v)
{
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

// How a head of hd channels is spread over lanes.  hd/8 = odd * 2^k; a lane
// takes `odd` chunks times a power of two, at most four chunks (five when
// odd == 5), and the remaining power of two becomes lanes per head.
Plan make_plan(int h, int hd, int r, int cpl_request)
{
    Plan pl{false, 0, 0, false, 2};
    if (hd % 8 != 0 || (r != 1 && r != 2)) return pl;
    const int hd8 = hd / 8;
    int odd = hd8;
    while ((odd & 1) == 0) odd >>= 1;
    if (odd > 5) return pl;
    int cpl = odd;
    if (cpl_request > 0) {
        if (cpl_request > 5 || hd8 % cpl_request != 0 || !is_pow2(hd8 / cpl_request)) return pl;
        cpl = cpl_request;
    } else {
        // r = 2 keeps a 36-tap window per lane: narrower slices (more lanes per head) leave room for it
        const int cap = r == 2 ? 2 : 4;
        while (cpl * 2 <= cap && hd8 % (cpl * 2) == 0) cpl *= 2;
    }
    const int lph = hd8 / cpl;
    if (lph > 32 || h * lph > kThreads) return pl;
    pl.fast = true;
    pl.cpl = cpl;
    pl.lph = lph;
    return pl;
}

// SMs of the current device (148 when the query fails)
inline int sm_count()
{
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return 148;
    return sms > 0 ? sms : 148;
}

inline bool aligned(const void *p, uintptr_t a) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// The matrix-instruction kernel: unsorted (walks the map in tiles) or in sorted order.  In sorted
// order with h a multiple of 8 the shared-window build runs when the sorting pass found all heads
// of every query looking at one place (guard word == 0) and the general build otherwise; both are
// enqueued, one of them returns at once.
template <typename T>
cudaError_t run_mma(Params p, int cpl, const uint32_t *not_shared_flag, int nch, cudaStream_t stream)
{
    if constexpr (sizeof(T) != 2) {
        return cudaErrorInvalidValue;
    } else {
        const bool pow2 = is_pow2_float(p.scale);
        long long items;
        p.tiles_x = (p.W + kMmaTileW - 1) / kMmaTileW;
        if (p.sorted != nullptr) {
            items = 1LL * p.B * p.Nq * p.h;
        } else {
            const long long tiles_y = (p.rows + kMmaTileH - 1) / kMmaTileH;
            items = 1LL * p.B * tiles_y * p.tiles_x * kMmaTileW * kMmaTileH * p.h;
        }
        const long long per_block = (kThreads / 32) * 64LL * nch;
        if (items >= (1LL << 31) - per_block) return cudaErrorInvalidValue;
        const unsigned blocks = static_cast<unsigned>((items + per_block - 1) / per_block);
        if (nch == 2 && p.sorted != nullptr && not_shared_flag != nullptr && p.h % 8 == 0) {
            p.guard = not_shared_flag;
            p.guard_run_if = 0;
            cudaError_t e = launch_mma<T>(p, cpl, true, pow2, 2, blocks, stream);
            if (e != cudaSuccess) return e;
            p.guard_run_if = 1;
            return launch_mma<T>(p, cpl, false, pow2, 2, blocks, stream);
        }
        p.guard = nullptr;
        return launch_mma<T>(p, cpl, false, pow2, nch, blocks, stream);
    }
}

template <typename T>
int run(Params &p, const Plan &pl, int r, int tile_w_request, cudaStream_t stream)
{
    cudaError_t err;
    if (pl.fast) {
        p.lph = pl.lph;
        p.lph_shift = ilog2(pl.lph);
        p.G = p.h * pl.lph;
        if (pl.mma) {
            err = run_mma<T>(p, pl.cpl, p.sorted != nullptr ? p.guard : nullptr, pl.mma_nch, stream);
            return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
        }
        int threads = kThreads;
        long long blocks = 0;
        const long long fill = 2LL * sm_count();
        for (;;) {
            const int qpb = threads / p.G;               // queries per block (>= 1)
            const int qpw = p.G >= 32 ? 1 : 32 / p.G;    // queries a warp covers, kept in one row
            int tw;
            if (tile_w_request > 0) {
                tw = 1;
                while (tw * 2 <= tile_w_request && tw * 2 <= qpb) tw *= 2;
            } else {
                tw = 1;
                while (tw * tw < qpb) tw *= 2;           // about square
                while (tw * 2 <= qpw) tw *= 2;       // at least a warp's queries wide, as a power of two
            }
            while (tw > qpb) tw >>= 1;
            if (tw < 1) tw = 1;
            p.tile_w = tw;
            p.tile_w_shift = ilog2(tw);
            p.tile_h = qpb / tw;
            p.tiles_x = (p.W + p.tile_w - 1) / p.tile_w;
            const int tiles_y = (p.rows + p.tile_h - 1) / p.tile_h;
            blocks = 1LL * p.tiles_x * tiles_y;
            // A launch too small to give every SM two blocks is bound by the latency of one warp's
            // chain of taps: narrower blocks (the kernels only bound their size from above) spread
            // the same queries over more SMs.
            if (threads <= 64 || threads / 2 < p.G || blocks * p.B >= fill) break;
            threads /= 2;
        }
        unsigned grid_y = p.B;
        if (p.sorted != nullptr) {       // one flat list of queries over all batch items
            const long long per_block = 1LL * p.tile_w * p.tile_h;
            blocks = (1LL * p.B * p.Nq + per_block - 1) / per_block;
            grid_y = 1;
        }
        if (blocks > 2147483647LL) return MATCHATTN_ERR_TOO_LARGE;
        const dim3 grid(static_cast<unsigned>(blocks), grid_y);
        err = launch_fast<T>(p, r, pl.cpl, pl.lph > 1, grid, threads, stream);
    } else {
        const long long per_item = 1LL * p.Nq * p.h;
        const long long blocks = (per_item + kThreads - 1) / kThreads;
        if (blocks > 2147483647LL) return MATCHATTN_ERR_TOO_LARGE;
        err = launch_generic<T>(p, dim3(static_cast<unsigned>(blocks), p.B), stream);
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}

// Up to sixteen block copies in one launch (matchattn_copy_blocks): grid.y picks the block, the grid.x
// CTAs of a block stride over its 16-byte words, four loads in flight per thread before the stores.
constexpr int kCopyBatch = 16;
constexpr int kCopyBlocksPerCopy = 64;
struct CopyBatch {
    uint4 *dst[kCopyBatch];
    const uint4 *src[kCopyBatch];
    unsigned long long words[kCopyBatch];
};

__global__ void __launch_bounds__(kThreads) copy_blocks_kernel(const CopyBatch cb)
{
    const uint4 *__restrict__ src = cb.src[blockIdx.y];
    uint4 *__restrict__ dst = cb.dst[blockIdx.y];
    const unsigned long long n = cb.words[blockIdx.y];
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
    unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * kThreads + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
        const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
        dst[i] = a;
        dst[i + stride] = b;
        dst[i + 2 * stride] = c;
        dst[i + 3 * stride] = d;
    }
    for (; i < n; i += stride) dst[i] = src[i];
}

// caller-side glue folded into the call (matchattn_fused_forward_glue); all off by default
struct Glue {
    const void *gate = nullptr;
    int clamp = 0;
    long long out_stride = 0, attn_stride = 0;      // 0 = natural
    unsigned long long *debug = nullptr;            // checked entry point: status words
    int kv_shift = 0;                               // keys / values of item b come from item (b + kv_shift) mod B
};

int forward_impl(const void *max_offset, const void *q, const void *k, const void *v, void *out, void *attn_out,
                 int B, int H, int W, int h, int hd, int rx, int ry, int dtype, int attn_type, float scale,
                 int q_row_begin, int q_row_end, void *cuda_stream, int tile_w, int force_generic, int cpl_request,
                 int variant, void *workspace = nullptr, size_t workspace_bytes = 0, int strategy = kStrategyDirect,
                 const Glue &glue = Glue())
{
    if (!max_offset || !q || !k || !v || !out) return MATCHATTN_ERR_NULL;
    if (dtype != MATCHATTN_F32 && dtype != MATCHATTN_F16 && dtype != MATCHATTN_BF16) return MATCHATTN_ERR_DTYPE;
    if (attn_type != MATCHATTN_L1_NORM && attn_type != MATCHATTN_DOT_PRODUCT) return MATCHATTN_ERR_ATTN_TYPE;
    if (attn_type == MATCHATTN_DOT_PRODUCT) {
        // the dot product runs on the general kernel only
        if ((strategy != kStrategyAuto && strategy != kStrategyDirect) || variant != 0) return MATCHATTN_ERR_VARIANT;
        force_generic = 1;
    }
    if (B <= 0 || H <= 0 || W <= 0 || h <= 0 || hd <= 0) return MATCHATTN_ERR_SHAPE;
    if (q_row_begin < 0 || q_row_end > H || q_row_begin >= q_row_end) return MATCHATTN_ERR_SHAPE;
    if (rx != ry || rx < 0 || rx > MATCHATTN_MAX_R) return MATCHATTN_ERR_WINDOW;
    if (2 * rx + 2 > W || 2 * ry + 2 > H) return MATCHATTN_ERR_WINDOW_FIT;
    const int r = rx;
    const int M = (2 * r + 2) * (2 * r + 2);
    const long long C = 1LL * h * hd, N = 1LL * H * W, Nq = 1LL * (q_row_end - q_row_begin) * W;
    // index ranges the kernels rely on: per-item offsets in 32 bits, batch on grid.y
    if (C > 65536 || N * C >= 2147483647LL || Nq * h * M >= 2147483647LL || B > 65535) return MATCHATTN_ERR_TOO_LARGE;
    const uintptr_t esize = dtype == MATCHATTN_F32 ? 4 : 2;
    // a tap's column is an unsigned 32-bit byte offset within its row
    if (1LL * W * C * static_cast<long long>(esize) >= (1LL << 32)) return MATCHATTN_ERR_TOO_LARGE;
    const long long out_stride = glue.out_stride > 0 ? glue.out_stride : C;
    const long long attn_stride = glue.attn_stride > 0 ? glue.attn_stride : 1LL * h * M;
    if (out_stride < C || attn_stride < 1LL * h * M || out_stride >= (1LL << 30) || attn_stride >= (1LL << 30))
        return MATCHATTN_ERR_SHAPE;
    const bool has_glue = glue.gate != nullptr || glue.clamp != 0 || out_stride != C || attn_stride != 1LL * h * M ||
                          glue.debug != nullptr || glue.kv_shift != 0;
    if (has_glue && (strategy == kStrategyBinned || variant == kVariantMma || variant == kVariantMma2)) return MATCHATTN_ERR_VARIANT;
    if (!aligned(glue.gate, esize)) return MATCHATTN_ERR_ALIGN;
    if (!aligned(max_offset, 2 * esize) || !aligned(q, esize) || !aligned(k, esize) || !aligned(v, esize) ||
        !aligned(out, esize) || !aligned(attn_out, esize))
        return MATCHATTN_ERR_ALIGN;

    Plan pl = force_generic ? Plan{false, 0, 0, false, 2} : make_plan(h, hd, r, cpl_request);
    if (pl.fast) {
        // vector width of a lane's slice decides the alignment the specialised kernel needs
        const int slice_bytes = pl.cpl * 8 * static_cast<int>(esize);
        const uintptr_t need = (slice_bytes % 32 == 0) ? 32 : 16;
        const uintptr_t need_attn = (M * esize) % 32 == 0 ? 32 : ((M * esize) % 16 == 0 ? 16 : 8);
        if (!aligned(q, need) || !aligned(k, need) || !aligned(v, need) || !aligned(out, need) ||
            !aligned(attn_out, need_attn) || !aligned(glue.gate, need) || (out_stride * esize) % need != 0 ||
            (attn_stride * esize) % need_attn != 0)
            pl.fast = false;
    }
    if (pl.fast) {
        // the matrix-instruction kernel addresses q/out, k/v and attn_out with 32-bit byte offsets
        const bool mma_ok = esize == 2 && r == 1 && pl.lph == 1 && !has_glue && aligned(attn_out, 32) &&
                            1LL * B * N * C * 2 < (1LL << 32) && 1LL * B * Nq * C * 2 < (1LL << 32) &&
                            1LL * B * Nq * h * M * 2 < (1LL << 32);
        const bool want_mma = variant == kVariantMma || variant == kVariantMma2 || strategy == kStrategySortedMma;
        pl.mma = mma_ok && want_mma;
        pl.mma_nch = variant == kVariantMma2 ? 1 : 2;
        if (want_mma && !mma_ok) return MATCHATTN_ERR_VARIANT;
    } else if (variant == kVariantMma || variant == kVariantMma2 || strategy == kStrategySortedMma) {
        return MATCHATTN_ERR_VARIANT;
    }

    Params p{};
    p.mo = max_offset; p.q = q; p.k = k; p.v = v; p.out = out; p.attn = attn_out;
    p.B = B; p.H = H; p.W = W; p.h = h; p.hd = hd; p.C = static_cast<int>(C);
    p.rows = q_row_end - q_row_begin;
    p.Nq = static_cast<int>(Nq);
    p.N = static_cast<int>(N);
    p.r = r;
    p.scale = scale;
    {   // a power of two that both 16-bit types hold exactly as a normal number
        int e = 0;
        p.scale_pow2 = dtype != MATCHATTN_F32 && scale > 0.f && frexpf(scale, &e) == 0.5f && e >= -12 && e <= 15;
    }
    p.guard = nullptr;
    p.guard_run_if = 1;
    p.sorted = nullptr;
    p.gate = glue.gate;
    p.out_stride = static_cast<int>(out_stride);
    p.attn_stride = static_cast<int>(attn_stride);
    p.clamp = glue.clamp;
    p.debug = glue.debug;
    p.kv_shift = glue.kv_shift;
    p.dot = attn_type == MATCHATTN_DOT_PRODUCT;
    if (glue.clamp) {
        // the caller's bounds (models/attention_blocks.py:49-52), rounded to the tensor type as there
        const float hx = static_cast<float>(W - 1 - r - 1e-3), hy = static_cast<float>(H - 1 - r - 1e-3);
        p.clamp_lo = static_cast<float>(r);
        p.clamp_hi_x = dtype == MATCHATTN_F16   ? __half2float(__float2half_rn(hx))
                       : dtype == MATCHATTN_BF16 ? __bfloat162float(__float2bfloat16_rn(hx)) : hx;
        p.clamp_hi_y = dtype == MATCHATTN_F16   ? __half2float(__float2half_rn(hy))
                       : dtype == MATCHATTN_BF16 ? __bfloat162float(__float2bfloat16_rn(hy)) : hy;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    // staged path, persistent form: one block per SM, a producer warp keeps the K and V regions of the next
    // tile arriving (cp.async.bulk.tensor on mbarriers) while 24 consumer warps work on the current one
    if (strategy == kStrategyStaged) {
        const StagedGeometry sg = persist_geometry(h, hd, r, dtype);
        if (!sg.valid || !pl.fast || pl.lph != 1 || has_glue || !aligned(k, 16) || !aligned(v, 16))
            return MATCHATTN_ERR_VARIANT;
        CUtensorMap map_k, map_v;
        if (!make_kv_map(&map_k, k, dtype, B, H, W, static_cast<int>(C), sg.RW, sg.RH) ||
            !make_kv_map(&map_v, v, dtype, B, H, W, static_cast<int>(C), sg.RW, sg.RH))
            return MATCHATTN_ERR_VARIANT;
        PersistParams sp{};
        sp.p = p;
        sp.QH = sg.QH; sp.RW = sg.RW; sp.RH = sg.RH;
        sp.tiles_x = (W + kStagedQW - 1) / kStagedQW;
        sp.tiles_y = (p.rows + sg.QH - 1) / sg.QH;
        sp.total_tiles = 1LL * sp.tiles_x * sp.tiles_y * B;
        sp.region_bytes = static_cast<uint32_t>(2LL * C * sg.RW * sg.RH);
        sp.status = nullptr;
        if (1LL * sp.tiles_x * sp.tiles_y > 2147483647LL) return MATCHATTN_ERR_TOO_LARGE;
        if (workspace != nullptr && workspace_bytes >= 8 && aligned(workspace, 8)) {
            sp.status = static_cast<unsigned long long *>(workspace);
            cudaError_t e = cudaMemsetAsync(workspace, 0, 8, stream);
            if (e != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(e);
        }
        const long long sms = sm_count();
        const int grid_blocks = static_cast<int>(sp.total_tiles < sms ? sp.total_tiles : sms);
        cudaError_t err = dtype == MATCHATTN_F16 ? launch_staged_persistent<__half>(sp, pl.cpl, map_k, map_v, grid_blocks, stream)
                                                 : launch_staged_persistent<__nv_bfloat16>(sp, pl.cpl, map_k, map_v, grid_blocks, stream);
        return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
    }

    // staged path, one block per tile (two blocks per SM; kept for comparison, strategy 6)
    if (strategy == kStrategyStagedBlocks) {
        const StagedGeometry sg = staged_geometry(h, hd, r, dtype);
        if (!sg.valid || !pl.fast || pl.lph != 1 || has_glue || !aligned(k, 16) || !aligned(v, 16) || H > 65535 * 8)
            return MATCHATTN_ERR_VARIANT;
        CUtensorMap map_k, map_v;
        if (!make_kv_map(&map_k, k, dtype, B, H, W, static_cast<int>(C), sg.RW, sg.RH) ||
            !make_kv_map(&map_v, v, dtype, B, H, W, static_cast<int>(C), sg.RW, sg.RH))
            return MATCHATTN_ERR_VARIANT;
        StagedParams sp{};
        sp.p = p;
        sp.ipt = sg.ipt; sp.rows_per_it = sg.rows_per_it; sp.QH = sg.QH; sp.RW = sg.RW; sp.RH = sg.RH;
        sp.tiles_x = (W + kStagedQW - 1) / kStagedQW;
        sp.region_bytes = static_cast<uint32_t>(2LL * C * sg.RW * sg.RH);
        sp.fallback_tiles = nullptr;
        if (workspace != nullptr && workspace_bytes >= 8 && aligned(workspace, 8)) {
            sp.fallback_tiles = static_cast<unsigned long long *>(workspace);
            cudaError_t e = cudaMemsetAsync(workspace, 0, 8, stream);
            if (e != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(e);
        }
        const long long tiles = 1LL * sp.tiles_x * ((p.rows + sg.QH - 1) / sg.QH);
        if (tiles > 2147483647LL) return MATCHATTN_ERR_TOO_LARGE;
        const dim3 grid(static_cast<unsigned>(tiles), B);
        const size_t smem = sp.region_bytes + 128;
        cudaError_t err = dtype == MATCHATTN_F16 ? launch_staged<__half>(sp, pl.cpl, map_k, map_v, grid, smem, stream)
                                                 : launch_staged<__nv_bfloat16>(sp, pl.cpl, map_k, map_v, grid, smem, stream);
        return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
    }

    // binned path: sort the queries by target tile, serve each tile from shared memory
    if (strategy != kStrategyDirect) {
        const BinGeometry gmt = bin_geometry(B, H, W, h, hd, r, dtype, p.rows);
        const bool usable = gmt.valid && pl.fast && pl.lph == 1 && workspace != nullptr &&
                            workspace_bytes >= gmt.total_bytes && aligned(workspace, 256) &&
                            aligned(q, 16) && aligned(k, 16) && aligned(v, 16) && aligned(out, 16) &&
                            aligned(attn_out, 32) && aligned(max_offset, 4);
        if (strategy >= kStrategyBinned && !usable) return MATCHATTN_ERR_VARIANT;
        // The sorting passes and the staging do not beat the direct kernel on any shape measured, so the
        // automatic choice (strategy 0) is the direct kernel and the binned path runs on request only.
        if (usable && strategy >= kStrategyBinned) {
            char *ws = static_cast<char *>(workspace);
            BinParams bp{};
            bp.p = p;
            bp.counts = reinterpret_cast<uint32_t *>(ws + gmt.off_counts);
            bp.ctrl = reinterpret_cast<uint32_t *>(ws + gmt.off_ctrl);
            bp.starts = reinterpret_cast<uint32_t *>(ws + gmt.off_starts);
            bp.cursors = reinterpret_cast<uint32_t *>(ws + gmt.off_cursors);
            bp.bin_of = reinterpret_cast<uint32_t *>(ws + gmt.off_bin_of);
            bp.sorted = reinterpret_cast<uint2 *>(ws + gmt.off_sorted);
            bp.bins_x = gmt.bins_x; bp.bins_y = gmt.bins_y; bp.nbins = gmt.nbins;
            bp.TX = gmt.TX; bp.TY = gmt.TY; bp.RW = gmt.RW; bp.RH = gmt.RH; bp.region_bytes = gmt.region_bytes;
            cudaError_t err = cudaMemsetAsync(bp.counts, 0, 4 * static_cast<size_t>(gmt.nbins) + 4 * kCtrlWords, stream);
            if (err != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(err);
            int dev = 0, sms = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            const int grid_blocks = 2 * (sms > 0 ? sms : 148);
            const size_t smem_bytes = 2 * static_cast<size_t>(gmt.region_bytes);
            const int main_cpl = strategy == kStrategyBinned ? pl.cpl : 0;     // 0: sorting passes only
            err = dtype == MATCHATTN_F16 ? launch_binned<__half>(bp, main_cpl, grid_blocks, smem_bytes, stream)
                                         : launch_binned<__nv_bfloat16>(bp, main_cpl, grid_blocks, smem_bytes, stream);
            if (err != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(err);
            if (strategy == kStrategySorted) {
                // the direct kernel below walks the queries in sorted order; correct whatever the heads do
                p.sorted = bp.sorted;
            } else if (strategy == kStrategySortedMma) {
                p.sorted = bp.sorted;
                p.guard = bp.ctrl + kCtrlNotShared;      // picks the shared-window or the general build
            } else {
                // queries whose heads look at different places: the direct kernel below runs instead
                p.guard = bp.ctrl + kCtrlNotShared;
                pl.mma = false;
            }
        }
    }
    switch (dtype) {
    case MATCHATTN_F32: return run<float>(p, pl, r, tile_w, stream);
    case MATCHATTN_F16: return run<__half>(p, pl, r, tile_w, stream);
    default: return run<__nv_bfloat16>(p, pl, r, tile_w, stream);
    }
}

}  // namespace
}  // namespace matchattn

extern "C" {

int matchattn_fused_forward(const void *max_offset, const void *q, const void *k, const void *v, void *out,
                            void *attn_out, int B, int H, int W, int h, int hd, int rx, int ry, int dtype,
                            int attn_type, float scale, int q_row_begin, int q_row_end, void *cuda_stream)
{
    return matchattn::forward_impl(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, rx, ry, dtype, attn_type,
                                   scale, q_row_begin, q_row_end, cuda_stream, 0, 0, 0, 0);
}

int matchattn_fused_forward_ex(const void *max_offset, const void *q, const void *k, const void *v, void *out,
                               void *attn_out, int B, int H, int W, int h, int hd, int rx, int ry, int dtype,
                               int attn_type, float scale, int q_row_begin, int q_row_end, void *cuda_stream,
                               int tile_w, int force_generic, int chunks_per_lane, int variant)
{
    return matchattn::forward_impl(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, rx, ry, dtype, attn_type,
                                   scale, q_row_begin, q_row_end, cuda_stream, tile_w, force_generic,
                                   chunks_per_lane, variant);
}

int matchattn_fused_forward_glue(const void *max_offset, const void *q, const void *k, const void *v,
                                 const void *gate, void *out, void *attn_out, int B, int H, int W, int h, int hd,
                                 int rx, int ry, int dtype, int attn_type, float scale, int q_row_begin,
                                 int q_row_end, int clamp_offsets, long long out_row_stride,
                                 long long attn_row_stride, int kv_item_shift, void *cuda_stream)
{
    if (kv_item_shift < 0 || kv_item_shift >= (B > 0 ? B : 1)) return MATCHATTN_ERR_SHAPE;
    matchattn::Glue glue;
    glue.kv_shift = kv_item_shift;
    glue.gate = gate;
    glue.clamp = clamp_offsets;
    glue.out_stride = out_row_stride;
    glue.attn_stride = attn_row_stride;
    return matchattn::forward_impl(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, rx, ry, dtype, attn_type,
                                   scale, q_row_begin, q_row_end, cuda_stream, 0, 0, 0, 0, nullptr, 0,
                                   matchattn::kStrategyDirect, glue);
}

int matchattn_fused_forward_checked(const void *max_offset, const void *q, const void *k, const void *v, void *out,
                                    void *attn_out, int B, int H, int W, int h, int hd, int rx, int ry, int dtype,
                                    int attn_type, float scale, int q_row_begin, int q_row_end, void *status,
                                    void *cuda_stream)
{
    if (status == nullptr || (reinterpret_cast<uintptr_t>(status) & 7)) return MATCHATTN_ERR_NULL;
    cudaError_t e = cudaMemsetAsync(status, 0, 16, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(e);
    matchattn::Glue glue;
    glue.debug = static_cast<unsigned long long *>(status);
    return matchattn::forward_impl(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, rx, ry, dtype, attn_type,
                                   scale, q_row_begin, q_row_end, cuda_stream, 0, 0, 0, 0, nullptr, 0,
                                   matchattn::kStrategyDirect, glue);
}

size_t matchattn_workspace_bytes(int B, int H, int W, int h, int hd, int r, int dtype, int q_row_begin, int q_row_end)
{
    if (B <= 0 || H <= 0 || W <= 0 || h <= 0 || hd <= 0 || q_row_begin < 0 || q_row_end > H || q_row_begin >= q_row_end)
        return 0;
    const matchattn::BinGeometry gmt = matchattn::bin_geometry(B, H, W, h, hd, r, dtype, q_row_end - q_row_begin);
    return gmt.valid ? gmt.total_bytes : 0;
}

int matchattn_fused_forward_ws(const void *max_offset, const void *q, const void *k, const void *v, void *out,
                               void *attn_out, int B, int H, int W, int h, int hd, int rx, int ry, int dtype,
                               int attn_type, float scale, int q_row_begin, int q_row_end, void *cuda_stream,
                               void *workspace, size_t workspace_bytes, int strategy)
{
    return matchattn::forward_impl(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, rx, ry, dtype, attn_type,
                                   scale, q_row_begin, q_row_end, cuda_stream, 0, 0, 0, 0, workspace,
                                   workspace_bytes, strategy);
}

const char *matchattn_describe_dispatch(int h, int hd, int r, int dtype, int pointers_32B_aligned)
{
    static thread_local char text[64];
    if (dtype != MATCHATTN_F32 && dtype != MATCHATTN_F16 && dtype != MATCHATTN_BF16) return nullptr;
    if (h <= 0 || hd <= 0 || r < 0 || r > MATCHATTN_MAX_R) return nullptr;
    matchattn::Plan pl = matchattn::make_plan(h, hd, r, 0);
    if (pl.fast && !pointers_32B_aligned) {
        const int esize = dtype == MATCHATTN_F32 ? 4 : 2;
        if ((pl.cpl * 8 * esize) % 32 == 0) pl.fast = false;
    }
    if (!pl.fast) return "generic";
    snprintf(text, sizeof(text), "fast cpl=%d lph=%d", pl.cpl, pl.lph);
    return text;
}

int matchattn_copy_blocks(void *const *dst, const void *const *src, const size_t *bytes, int count, int use_kernel,
                          void *cuda_stream)
{
    using namespace matchattn;
    if (count < 0 || (count > 0 && (!dst || !src || !bytes))) return MATCHATTN_ERR_NULL;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    CopyBatch batch{};
    int filled = 0;
    const auto flush = [&]() -> cudaError_t {
        if (filled == 0) return cudaSuccess;
        copy_blocks_kernel<<<dim3(kCopyBlocksPerCopy, filled), kThreads, 0, stream>>>(batch);
        filled = 0;
        return cudaGetLastError();
    };
    for (int i = 0; i < count; ++i) {
        if (bytes[i] == 0) continue;
        if (!dst[i] || !src[i]) return MATCHATTN_ERR_NULL;
        const bool vec = use_kernel && aligned(dst[i], 16) && aligned(src[i], 16) && bytes[i] % 16 == 0;
        cudaError_t err = cudaSuccess;
        if (vec) {
            batch.dst[filled] = static_cast<uint4 *>(dst[i]);
            batch.src[filled] = static_cast<const uint4 *>(src[i]);
            batch.words[filled] = bytes[i] / 16;
            if (++filled == kCopyBatch) err = flush();
        } else {
            err = cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyDefault, stream);
        }
        if (err != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(err);
    }
    const cudaError_t err = flush();
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}

int matchattn_version(void) { return 102; }

const char *matchattn_strerror(int status)
{
    switch (status) {
    case MATCHATTN_OK: return "ok";
    case MATCHATTN_ERR_NULL: return "a required pointer is NULL";
    case MATCHATTN_ERR_SHAPE: return "bad shape: a size is not positive or the query row band is empty or outside the map";
    case MATCHATTN_ERR_WINDOW_FIT: return "the (2r+2) window does not fit the token map";
    case MATCHATTN_ERR_DTYPE: return "unsupported element type";
    case MATCHATTN_ERR_ATTN_TYPE: return "attn_type: unknown, or not covered by this entry point (forward: l1_norm 0, dot_product 1; backward: l1_norm)";
    case MATCHATTN_ERR_WINDOW: return "unsupported window: rx must equal ry and 0 <= r <= 4";
    case MATCHATTN_ERR_ALIGN: return "a pointer is not aligned to its element size";
    case MATCHATTN_ERR_TOO_LARGE: return "sizes exceed the supported index range";
    case MATCHATTN_ERR_VARIANT: return "the requested kernel variant does not cover these arguments";
    case MATCHATTN_ERR_SCRATCH_LIMIT:
        return "the problem needs more scratch than the built-in area holds (MATCHATTN_STATIC_SCRATCH_BYTES); "
               "use matchattn_fused_forward_ws with your own scratch or split the call";
    default: break;
    }
    if (status >= MATCHATTN_ERR_CUDA) return cudaGetErrorString(static_cast<cudaError_t>(status - MATCHATTN_ERR_CUDA));
    return "unknown status";
}

}  // extern "C"
