// Convex upsampling of a field: MatchStereo.upsample_field of the reference
// (models/match_stereo.py:73-84) as one kernel.
//
//   field [B, H, W, D], mask [B, 9*f*f, H, W]  ->  out [B, f*H, f*W, D]
//   out[b, h*f+i, w*f+j, d] = sum_k softmax_k(mask[b, (k*f+i)*f+j, h, w]) * (f * field[b, h+ky-1, w+kx-1, d])
//
// The reference does this with a view, a softmax, an unfold, a broadcast multiply that materialises
// a [B, D, 9, f, f, H, W] tensor, a sum and a permute: about six passes over 4-5x the data.  Here one
// thread owns one coarse cell (b, h, w): it reads its 9*f*f mask logits (each a coalesced read across
// the threads of a warp, the mask is the bulk of the traffic and is read exactly once), the 3x3
// neighbourhood of the field, and writes the f x f block of fine cells.  HBM-bound: 9*f*f + ~D reads and
// f*f*D writes per thread.  Rounding in the 16-bit types follows eager PyTorch: softmax result, field*f
// and every product rounded to the tensor type, nine-term sum in float32.
#include "../../include/matchattn.h"

#include <stdint.h>

#include "matchattn_kernels.cuh"

namespace matchattn {
namespace {

constexpr int kMaxD = 8;

template <typename T, int F>
__global__ void __launch_bounds__(128) upsample_field_kernel(const T *__restrict__ field, const T *__restrict__ mask,
                                                             T *__restrict__ out, int B, int H, int W, int D)
{
    const int w = blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    if (w >= W) return;
    const int64_t plane = static_cast<int64_t>(H) * W;

    // 3x3 neighbourhood of the field, times f, rounded to T; zero outside the map
    float nb[9][kMaxD];
#pragma unroll
    for (int k = 0; k < 9; ++k) {
        const int hh = h + k / 3 - 1, ww = w + k % 3 - 1;
        const bool inside = hh >= 0 && hh < H && ww >= 0 && ww < W;
        const T *src = field + ((static_cast<int64_t>(b) * H + (inside ? hh : h)) * W + (inside ? ww : w)) * D;
#pragma unroll
        for (int d = 0; d < kMaxD; ++d)
            nb[k][d] = (inside && d < D) ? DT<T>::rnd(load_one<T>(src + d) * static_cast<float>(F)) : 0.f;
    }

    const T *mrow = mask + static_cast<int64_t>(b) * 9 * F * F * plane + static_cast<int64_t>(h) * W + w;
    for (int i = 0; i < F; ++i) {
        T *orow = out + ((static_cast<int64_t>(b) * H * F + static_cast<int64_t>(h) * F + i) * W * F + static_cast<int64_t>(w) * F) * D;
#pragma unroll
        for (int j = 0; j < F; ++j) {
            float p[9];
            float mx = -INFINITY;
#pragma unroll
            for (int k = 0; k < 9; ++k) {
                p[k] = load_one<T>(mrow + static_cast<int64_t>((k * F + i) * F + j) * plane);
                mx = fmaxf(mx, p[k]);
            }
            float den = 0.f;
#pragma unroll
            for (int k = 0; k < 9; ++k) {
                p[k] = expf(p[k] - mx);
                den += p[k];
            }
            const float inv = __frcp_rn(den);
#pragma unroll
            for (int k = 0; k < 9; ++k) p[k] = DT<T>::rnd(p[k] * inv);
#pragma unroll
            for (int d = 0; d < kMaxD; ++d) {
                if (d >= D) break;
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < 9; ++k) acc += DT<T>::rnd(p[k] * nb[k][d]);
                store_one<T>(orow + j * D + d, acc);
            }
        }
    }
}

// 2^x by the special-function unit (the weights are rounded to the tensor type right after)
__device__ __forceinline__ float exp2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// a packed 32-bit word of two 16-bit values as the pair type of the element-wise helpers
template <typename T>
__device__ __forceinline__ typename DT<T>::Bcast word_as_pair(uint32_t w);
template <>
__device__ __forceinline__ float word_as_pair<float>(uint32_t w) { return __uint_as_float(w); }
template <>
__device__ __forceinline__ __half2 word_as_pair<__half>(uint32_t w) { return *reinterpret_cast<const __half2 *>(&w); }
template <>
__device__ __forceinline__ __nv_bfloat162 word_as_pair<__nv_bfloat16>(uint32_t w) { return *reinterpret_cast<const __nv_bfloat162 *>(&w); }


// Vector path for the shapes the model uses (F*D <= 8, W a multiple of VW = 4): one thread owns four
// consecutive coarse cells of one row h and ONE fine row i.  Its mask reads are 8- or 16-byte loads (four
// cells of one channel), and the 4*f fine cells it produces are one contiguous run of 4*F*D elements of the
// output row, stored 16 bytes at a time.  Four cells keep the thread light (about 110 registers, ~1000
// threads resident per SM); the softmax exponentials use the fast intrinsic (the weights are rounded to the
// tensor type right after, which hides its error in all but ~0.1 % of the 16-bit cases).
template <typename T, int F, int D>
__global__ void __launch_bounds__(128) upsample_field_vec_kernel(const T *__restrict__ field, const T *__restrict__ mask,
                                                                 T *__restrict__ out, int B, int H, int W)
{
    constexpr int VW = 4;                           // cells per thread
    constexpr int EPW = DT<T>::kElemsPerWord;
    const int wq = blockIdx.x * blockDim.x + threadIdx.x;        // group of VW cells
    const int w0 = wq * VW;
    if (w0 >= W) return;
    const int hi = blockIdx.y, b = blockIdx.z;
    const int h = hi / F, i = hi - h * F;
    const int64_t plane = static_cast<int64_t>(H) * W;

    // field * f for rows h-1..h+1, columns w0-1..w0+VW, rounded to T; zero outside the map
    float nb[3][VW + 2][D];
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
        const int hh = h + ky - 1;
#pragma unroll
        for (int c = 0; c < VW + 2; ++c) {
            const int ww = w0 + c - 1;
            const bool inside = hh >= 0 && hh < H && ww >= 0 && ww < W;
            const T *src = field + ((static_cast<int64_t>(b) * H + (inside ? hh : h)) * W + (inside ? ww : w0)) * D;
#pragma unroll
            for (int d = 0; d < D; ++d) nb[ky][c][d] = inside ? DT<T>::rnd(load_one<T>(src + d) * static_cast<float>(F)) : 0.f;
        }
    }

    [[maybe_unused]] uint32_t nbw[3][VW + 2];
    if constexpr (EPW == 2 && D == 2) {
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
            for (int c = 0; c < VW + 2; ++c) nbw[ky][c] = DT<T>::aw_from(nb[ky][c][0], nb[ky][c][1]);
    }

    float res[VW][F][D];
    const T *mbase = mask + static_cast<int64_t>(b) * 9 * F * F * plane + static_cast<int64_t>(h) * W + w0;
#pragma unroll
    for (int j = 0; j < F; ++j) {
        float lg[9][VW];
#pragma unroll
        for (int k = 0; k < 9; ++k) {
            uint32_t wds[VW / EPW];
            const T *src = mbase + static_cast<int64_t>((k * F + i) * F + j) * plane;
            if constexpr (EPW == 2) {
                const uint2 t2 = __ldg(reinterpret_cast<const uint2 *>(src));
                wds[0] = t2.x;
                wds[1] = t2.y;
            } else {
                ld_nc_128(wds, src);
            }
#pragma unroll
            for (int c = 0; c < VW; ++c) {
                if constexpr (EPW == 2) lg[k][c] = DT<T>::unpack(wds[c >> 1], c & 1);
                else lg[k][c] = __uint_as_float(wds[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < VW; ++c) {
            float mx = lg[0][c];
#pragma unroll
            for (int k = 1; k < 9; ++k) mx = fmaxf(mx, lg[k][c]);
            // exp(l - mx) as 2^(l * log2e - mx * log2e), one fused multiply-add and one special-function op
            constexpr float kLog2e = 1.4426950408889634f;
            const float shift = -mx * kLog2e;
            float p[9], den = 0.f;
#pragma unroll
            for (int k = 0; k < 9; ++k) {
                p[k] = exp2_approx(fmaf(lg[k][c], kLog2e, shift));
                den += p[k];
            }
            const float inv = __frcp_rn(den);
#pragma unroll
            for (int d = 0; d < D; ++d) res[c][j][d] = 0.f;
            if constexpr (EPW == 2 && D == 2) {
                // both components of a neighbour are one packed word: weight (rounded to T, broadcast)
                // times word in one packed multiply, each rounded product added to its float32 sum
#pragma unroll
                for (int k = 0; k < 9; ++k) {
                    const float pf = p[k] * inv;
                    DT<T>::wmul(word_as_pair<T>(DT<T>::aw_from(pf, pf)), nbw[k / 3][c + k % 3], &res[c][j][0]);
                }
            } else {
#pragma unroll
                for (int k = 0; k < 9; ++k) {
                    const float pk = DT<T>::rnd(p[k] * inv);
#pragma unroll
                    for (int d = 0; d < D; ++d) res[c][j][d] += DT<T>::rnd(pk * nb[k / 3][c + k % 3][d]);
                }
            }
        }
    }

    // VW*F*D consecutive elements of the fine row h*F+i
    T *orow = out + ((static_cast<int64_t>(b) * H * F + hi) * W * F + static_cast<int64_t>(w0) * F) * D;
    constexpr int NEL = VW * F * D;
    const float *flat = &res[0][0][0];
    if constexpr ((NEL * sizeof(T)) % 16 == 0) {
        constexpr int NWORDS = NEL / EPW;
        uint32_t ow[NWORDS];
#pragma unroll
        for (int x = 0; x < NWORDS; ++x) ow[x] = DT<T>::pack(&flat[x * EPW]);
#pragma unroll
        for (int x = 0; x < NWORDS / 4; ++x) st_128(reinterpret_cast<char *>(orow) + 16 * x, &ow[4 * x]);
    } else {
#pragma unroll
        for (int x = 0; x < NEL; ++x) store_one<T>(orow + x, flat[x]);
    }
}

template <typename T, int F, int D>
bool try_vec(const T *f, const T *m, T *o, int B, int H, int W, cudaStream_t stream)
{
    constexpr int VW = 4;
    if (W % VW != 0 || (reinterpret_cast<uintptr_t>(m) % 16) != 0 || (reinterpret_cast<uintptr_t>(o) % 16) != 0 ||
        1LL * H * F > 65535)
        return false;
    const dim3 grid((W / VW + 127) / 128, H * F, B), block(128);
    upsample_field_vec_kernel<T, F, D><<<grid, block, 0, stream>>>(f, m, o, B, H, W);
    return true;
}

template <typename T>
cudaError_t launch(const void *field, const void *mask, void *out, int B, int H, int W, int D, int factor,
                   cudaStream_t stream)
{
    const dim3 grid((W + 127) / 128, H, B), block(128);
    const T *f = static_cast<const T *>(field), *m = static_cast<const T *>(mask);
    T *o = static_cast<T *>(out);
    // the model's shapes: a 2-component field, factor 2 between stages and 4 at the end
    if (D == 2 && factor == 2 && try_vec<T, 2, 2>(f, m, o, B, H, W, stream)) return cudaGetLastError();
    if (D == 2 && factor == 4 && try_vec<T, 4, 2>(f, m, o, B, H, W, stream)) return cudaGetLastError();
    switch (factor) {
    case 1: upsample_field_kernel<T, 1><<<grid, block, 0, stream>>>(f, m, o, B, H, W, D); break;
    case 2: upsample_field_kernel<T, 2><<<grid, block, 0, stream>>>(f, m, o, B, H, W, D); break;
    case 4: upsample_field_kernel<T, 4><<<grid, block, 0, stream>>>(f, m, o, B, H, W, D); break;
    case 8: upsample_field_kernel<T, 8><<<grid, block, 0, stream>>>(f, m, o, B, H, W, D); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace
}  // namespace matchattn

extern "C" int matchattn_upsample_field(const void *field, const void *mask, void *out, int B, int H, int W, int D,
                                        int factor, int dtype, void *cuda_stream)
{
    if (!field || !mask || !out) return MATCHATTN_ERR_NULL;
    if (B <= 0 || H <= 0 || W <= 0 || D <= 0 || D > matchattn::kMaxD) return MATCHATTN_ERR_SHAPE;
    if (factor != 1 && factor != 2 && factor != 4 && factor != 8) return MATCHATTN_ERR_SHAPE;
    if (H > 65535 || B > 65535 || 1LL * B * 9 * factor * factor * H * W >= (1LL << 40)) return MATCHATTN_ERR_TOO_LARGE;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t err;
    switch (dtype) {
    case MATCHATTN_F32: err = matchattn::launch<float>(field, mask, out, B, H, W, D, factor, stream); break;
    case MATCHATTN_F16: err = matchattn::launch<__half>(field, mask, out, B, H, W, D, factor, stream); break;
    case MATCHATTN_BF16: err = matchattn::launch<__nv_bfloat16>(field, mask, out, B, H, W, D, factor, stream); break;
    default: return MATCHATTN_ERR_DTYPE;
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}
