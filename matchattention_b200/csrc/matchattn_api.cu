// C ABI of the MatchAttention operator (declared in include/matchattn.h):
// argument validation, choice of kernel variant and launch geometry.
#include "../../include/matchattn.h"

#include <stdint.h>
#include <stdio.h>

#include "matchattn_kernels.cuh"
#include "matchattn_mma.cuh"

namespace matchattn {
namespace {

struct Plan {
    bool fast;
    int cpl;   // chunks (8 channels) per lane
    int lph;   // lanes per head
    bool mma;  // 16-bit, one lane per head, r == 1: accumulate with matrix instructions
};

constexpr int kVariantAuto = 0, kVariantScalar = 1, kVariantMma = 2;
constexpr int kMmaItemsPerBlock = 1024;   // 8 warps x 128 items

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
    Plan pl{false, 0, 0, false};
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
        while (cpl * 2 <= 4 && hd8 % (cpl * 2) == 0) cpl *= 2;
    }
    const int lph = hd8 / cpl;
    if (lph > 32 || h * lph > kThreads) return pl;
    pl.fast = true;
    pl.cpl = cpl;
    pl.lph = lph;
    return pl;
}

inline bool aligned(const void *p, uintptr_t a) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <typename T>
cudaError_t launch_mma_if_16bit(const Params &p, int r, int cpl, dim3 grid, cudaStream_t stream)
{
    if constexpr (sizeof(T) == 2) return launch_mma<T>(p, r, cpl, grid, stream);
    else return cudaErrorInvalidValue;
}

template <typename T>
int run(Params &p, const Plan &pl, int r, int tile_w_request, cudaStream_t stream)
{
    cudaError_t err;
    if (pl.fast) {
        p.lph = pl.lph;
        p.lph_shift = ilog2(pl.lph);
        p.G = p.h * pl.lph;
        const int lanes_per_block = pl.mma ? kMmaItemsPerBlock : kThreads;
        const int qpb = lanes_per_block / p.G;       // queries per block (>= 1)
        const int qpw = p.G >= 32 ? 1 : 32 / p.G;    // queries a warp covers, kept in one row
        int tw;
        if (tile_w_request > 0) {
            tw = 1;
            while (tw * 2 <= tile_w_request && tw * 2 <= qpb) tw *= 2;
        } else {
            tw = 1;
            while (tw * tw < qpb) tw *= 2;           // about square
            if (tw < qpw) tw = qpw;
        }
        while (tw > qpb) tw >>= 1;
        if (tw < 1) tw = 1;
        p.tile_w = tw;
        p.tile_w_shift = ilog2(tw);
        p.tile_h = qpb / tw;
        p.tiles_x = (p.W + p.tile_w - 1) / p.tile_w;
        const int tiles_y = (p.rows + p.tile_h - 1) / p.tile_h;
        const long long blocks = 1LL * p.tiles_x * tiles_y;
        if (blocks > 2147483647LL) return MATCHATTN_ERR_TOO_LARGE;
        const dim3 grid(static_cast<unsigned>(blocks), p.B);
        err = pl.mma ? launch_mma_if_16bit<T>(p, r, pl.cpl, grid, stream)
                     : launch_fast<T>(p, r, pl.cpl, pl.lph > 1, grid, stream);
    } else {
        const long long per_item = 1LL * p.Nq * p.h;
        const long long blocks = (per_item + kThreads - 1) / kThreads;
        if (blocks > 2147483647LL) return MATCHATTN_ERR_TOO_LARGE;
        err = launch_generic<T>(p, dim3(static_cast<unsigned>(blocks), p.B), stream);
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}

int forward_impl(const void *max_offset, const void *q, const void *k, const void *v, void *out, void *attn_out,
                 int B, int H, int W, int h, int hd, int rx, int ry, int dtype, int attn_type, float scale,
                 int q_row_begin, int q_row_end, void *cuda_stream, int tile_w, int force_generic, int cpl_request,
                 int variant)
{
    if (!max_offset || !q || !k || !v || !out) return MATCHATTN_ERR_NULL;
    if (dtype != MATCHATTN_F32 && dtype != MATCHATTN_F16 && dtype != MATCHATTN_BF16) return MATCHATTN_ERR_DTYPE;
    if (attn_type != MATCHATTN_L1_NORM) return MATCHATTN_ERR_ATTN_TYPE;
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
    if (!aligned(max_offset, 2 * esize) || !aligned(q, esize) || !aligned(k, esize) || !aligned(v, esize) ||
        !aligned(out, esize) || !aligned(attn_out, esize))
        return MATCHATTN_ERR_ALIGN;

    Plan pl = force_generic ? Plan{false, 0, 0, false} : make_plan(h, hd, r, cpl_request);
    if (pl.fast) {
        // vector width of a lane's slice decides the alignment the specialised kernel needs
        const int slice_bytes = pl.cpl * 8 * static_cast<int>(esize);
        const uintptr_t need = (slice_bytes % 32 == 0) ? 32 : 16;
        const uintptr_t need_attn = (M * esize) % 32 == 0 ? 32 : ((M * esize) % 16 == 0 ? 16 : 8);
        if (!aligned(q, need) || !aligned(k, need) || !aligned(v, need) || !aligned(out, need) ||
            !aligned(attn_out, need_attn))
            pl.fast = false;
    }
    if (pl.fast) {
        const bool mma_ok = esize == 2 && r == 1 && pl.lph == 1 && h <= kMmaItemsPerBlock;
        // the direct-gather form of the matrix-instruction kernel runs at one block per SM and is
        // latency-bound; it is selected only on request
        pl.mma = mma_ok && variant == kVariantMma;
        if (variant == kVariantMma && !mma_ok) return MATCHATTN_ERR_VARIANT;
    } else if (variant == kVariantMma) {
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
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
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

int matchattn_version(void) { return 100; }

const char *matchattn_strerror(int status)
{
    switch (status) {
    case MATCHATTN_OK: return "ok";
    case MATCHATTN_ERR_NULL: return "a required pointer is NULL";
    case MATCHATTN_ERR_SHAPE: return "bad shape: a size is not positive or the query row band is empty or outside the map";
    case MATCHATTN_ERR_WINDOW_FIT: return "the (2r+2) window does not fit the token map";
    case MATCHATTN_ERR_DTYPE: return "unsupported element type";
    case MATCHATTN_ERR_ATTN_TYPE: return "unsupported attn_type: only l1_norm is implemented";
    case MATCHATTN_ERR_WINDOW: return "unsupported window: rx must equal ry and 0 <= r <= 4";
    case MATCHATTN_ERR_ALIGN: return "a pointer is not aligned to its element size";
    case MATCHATTN_ERR_TOO_LARGE: return "sizes exceed the supported index range";
    case MATCHATTN_ERR_VARIANT: return "the requested kernel variant does not cover these arguments";
    default: break;
    }
    if (status >= MATCHATTN_ERR_CUDA) return cudaGetErrorString(static_cast<cudaError_t>(status - MATCHATTN_ERR_CUDA));
    return "unknown status";
}

}  // extern "C"
