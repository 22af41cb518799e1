// Two small steps of the model that sit either side of the MatchAttention blocks, each as one kernel:
//
//   consistency_mask   MatchAttentionLayer.consistency_mask (models/attention_blocks.py:130-138 with
//                      utils/utils.py:31-48): once per layer, 26 times per forward.  The reference runs
//                      about fifteen small kernels (grid, normalise, permutes, grid_sample, abs, sum, compare).
//   local_disparity    local_disparity_estimator + disp_to_flow (models/cost_volume.py:123-178): the step
//                      between the cost volume and the first block (about twenty kernels in the reference).
//
// Rounding of the 16-bit types follows eager PyTorch on the GPU: every elementwise tensor op rounds to
// the tensor type, reductions and the bilinear sampler accumulate in float32 and round once.
#include "../../include/matchattn.h"

#include <stdint.h>

#include "matchattn_kernels.cuh"

namespace matchattn {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) consistency_mask_kernel(const T *__restrict__ field, T *__restrict__ mask,
                                                                T *__restrict__ diff_out, int B, int H, int W, float A)
{
    const int64_t px = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t plane = static_cast<int64_t>(H) * W;
    if (px >= B * plane) return;
    const int b = static_cast<int>(px / plane);
    const int rem = static_cast<int>(px - b * plane);
    const int y = rem / W, x = rem - y * W;
    const int tb = b + (b < B / 2 ? B / 2 : -(B / 2));          // the other view

    const float f0 = load_one<T>(field + px * 2), f1 = load_one<T>(field + px * 2 + 1);
    // offset = field + grid, then the reference's normalisation 2 * o / (size - 1) - 1, op by op
    const float ox = DT<T>::rnd(f0 + static_cast<float>(x)), oy = DT<T>::rnd(f1 + static_cast<float>(y));
    const float gx = DT<T>::rnd(DT<T>::rnd(__fdiv_rn(DT<T>::rnd(2.f * ox), static_cast<float>(W - 1))) - 1.f);
    const float gy = DT<T>::rnd(DT<T>::rnd(__fdiv_rn(DT<T>::rnd(2.f * oy), static_cast<float>(H - 1))) - 1.f);
    // bilinear sampler, align_corners, zero padding, float32 inside
    const float ix = __fmul_rn(__fdiv_rn(gx + 1.f, 2.f), static_cast<float>(W - 1));
    const float iy = __fmul_rn(__fdiv_rn(gy + 1.f, 2.f), static_cast<float>(H - 1));
    const float fx0 = floorf(ix), fy0 = floorf(iy);
    const float wx1 = ix - fx0, wx0 = (fx0 + 1.f) - ix, wy1 = iy - fy0, wy0 = (fy0 + 1.f) - iy;
    const float wgt[4] = {__fmul_rn(wx0, wy0), __fmul_rn(wx1, wy0), __fmul_rn(wx0, wy1), __fmul_rn(wx1, wy1)};
    const T *other = field + static_cast<int64_t>(tb) * plane * 2;
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const float cx = fx0 + static_cast<float>(t & 1), cy = fy0 + static_cast<float>(t >> 1);
        if (cx >= 0.f && cx <= static_cast<float>(W - 1) && cy >= 0.f && cy <= static_cast<float>(H - 1)) {
            const T *src = other + (static_cast<int64_t>(static_cast<int>(cy)) * W + static_cast<int>(cx)) * 2;
            acc0 = fmaf(load_one<T>(src), wgt[t], acc0);
            acc1 = fmaf(load_one<T>(src + 1), wgt[t], acc1);
        }
    }
    const float d = DT<T>::rnd(fabsf(DT<T>::rnd(f0 + DT<T>::rnd(acc0))) + fabsf(DT<T>::rnd(f1 + DT<T>::rnd(acc1))));
    if (diff_out != nullptr) store_one<T>(diff_out + px, d);
    store_one<T>(mask + px, d < A ? 1.f : 0.f);
}

template <typename T>
__global__ void __launch_bounds__(128) local_disparity_kernel(const T *__restrict__ cv, T *__restrict__ flow,
                                                               T *__restrict__ blur_out, int *__restrict__ centre_out,
                                                               int B, int D, int H, int W, float tiny)
{
    const int64_t plane = static_cast<int64_t>(H) * W;
    const int64_t px = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (px >= plane) return;
    const int b = blockIdx.y;
    const T *col = cv + static_cast<int64_t>(b) * D * plane + px;      // this pixel's D values, `plane` apart

    // 5-tap box average over D (zero padded, divided by 5), first arg max
    float w0 = 0.f, w1 = 0.f, w2 = load_one<T>(col), w3 = load_one<T>(col + plane), w4;
    float best = -INFINITY;
    int arg = 0;
    for (int d = 0; d < D; ++d) {
        w4 = d + 2 < D ? load_one<T>(col + static_cast<int64_t>(d + 2) * plane) : 0.f;
        // the sum runs over the taps inside [0, D) in ascending order, as the pooling kernel adds them
        float acc = 0.f;
        if (d >= 2) acc += w0;
        if (d >= 1) acc += w1;
        acc += w2;
        if (d + 1 < D) acc += w3;
        if (d + 2 < D) acc += w4;
        const float bl = DT<T>::rnd(__fdiv_rn(acc, 5.f));
        if (bl > best) {
            best = bl;
            arg = d;
        }
        w0 = w1; w1 = w2; w2 = w3; w3 = w4;
    }
    const int centre = min(max(arg, 2), D - 3);
    // PyTorch converts the scalar 1/D to the tensor type before it compares
    const float mean = DT<T>::rnd(static_cast<float>(1.0 / static_cast<double>(D)));
    float p[5], sum = 0.f;
#pragma unroll
    for (int t = 0; t < 5; ++t) {
        p[t] = load_one<T>(col + static_cast<int64_t>(centre - 2 + t) * plane);
        if (p[t] < mean) p[t] = 0.f;
        sum += p[t];
    }
    sum = fmaxf(DT<T>::rnd(sum), tiny);
    float disp = 0.f;
#pragma unroll
    for (int t = 0; t < 5; ++t)
        disp += DT<T>::rnd(DT<T>::rnd(__fdiv_rn(p[t], sum)) * DT<T>::rnd(static_cast<float>(centre - 2 + t)));
    disp = DT<T>::rnd(disp);
    if (b < B / 2) disp = -disp;
    const int64_t o = static_cast<int64_t>(b) * plane + px;
    store_one<T>(flow + o * 2, disp);
    store_one<T>(flow + o * 2 + 1, 0.f);
    if (blur_out != nullptr) store_one<T>(blur_out + o, best);
    if (centre_out != nullptr) centre_out[o] = centre;
}

template <typename T>
cudaError_t run_mask(const void *field, void *mask, void *diff, int B, int H, int W, float A, cudaStream_t stream)
{
    const int64_t total = static_cast<int64_t>(B) * H * W;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    consistency_mask_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T *>(field), static_cast<T *>(mask),
                                                          static_cast<T *>(diff), B, H, W, A);
    return cudaGetLastError();
}

template <typename T>
cudaError_t run_disparity(const void *cv, void *flow, void *blur, int *centre, int B, int D, int H, int W, float tiny,
                          cudaStream_t stream)
{
    const int64_t plane = static_cast<int64_t>(H) * W;
    const dim3 grid(static_cast<unsigned>((plane + 127) / 128), B);
    local_disparity_kernel<T><<<grid, 128, 0, stream>>>(static_cast<const T *>(cv), static_cast<T *>(flow),
                                                       static_cast<T *>(blur), centre, B, D, H, W, tiny);
    return cudaGetLastError();
}

}  // namespace
}  // namespace matchattn

extern "C" int matchattn_consistency_mask(const void *field, void *noc_mask, void *field_diff, int B, int H, int W,
                                          float threshold, int dtype, void *cuda_stream)
{
    if (!field || !noc_mask) return MATCHATTN_ERR_NULL;
    if (B <= 0 || (B & 1) || H <= 1 || W <= 1) return MATCHATTN_ERR_SHAPE;
    if (1LL * B * H * W >= (1LL << 31) * 256) return MATCHATTN_ERR_TOO_LARGE;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t err;
    switch (dtype) {
    case MATCHATTN_F32: err = matchattn::run_mask<float>(field, noc_mask, field_diff, B, H, W, threshold, stream); break;
    case MATCHATTN_F16: err = matchattn::run_mask<__half>(field, noc_mask, field_diff, B, H, W, threshold, stream); break;
    case MATCHATTN_BF16: err = matchattn::run_mask<__nv_bfloat16>(field, noc_mask, field_diff, B, H, W, threshold, stream); break;
    default: return MATCHATTN_ERR_DTYPE;
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}

extern "C" int matchattn_local_disparity(const void *volume, void *flow, void *blur_max, int *centre, int B, int D,
                                         int H, int W, int dtype, void *cuda_stream)
{
    if (!volume || !flow) return MATCHATTN_ERR_NULL;
    if (B <= 0 || (B & 1) || D < 5 || H <= 0 || W <= 0) return MATCHATTN_ERR_SHAPE;
    if (B > 65535 || 1LL * D * H * W >= (1LL << 40)) return MATCHATTN_ERR_TOO_LARGE;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t err;
    switch (dtype) {
    case MATCHATTN_F32: err = matchattn::run_disparity<float>(volume, flow, blur_max, centre, B, D, H, W, 1.17549435e-38f, stream); break;
    case MATCHATTN_F16: err = matchattn::run_disparity<__half>(volume, flow, blur_max, centre, B, D, H, W, 6.103515625e-05f, stream); break;
    case MATCHATTN_BF16: err = matchattn::run_disparity<__nv_bfloat16>(volume, flow, blur_max, centre, B, D, H, W, 1.17549435e-38f, stream); break;
    default: return MATCHATTN_ERR_DTYPE;
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}
