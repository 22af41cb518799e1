// Cost volume of the stereo branch of GlobalCorrelation (models/cost_volume.py:26-51) as one kernel.
//
//   corr [B, H, W, W]  (reference column, then target column, of one image row)
//   vol  [2B, D = W, H, W]
//     left  view: vol[b, d, h, w]   = corr[b, h, w, w-d]  (w >= d, else 0)
//     right view: vol[B+b, d, h, w] = corr[b, h, w+d, w]  (w+d < W, else 0)
//   softmax over d, then the out-of-view fill (left: columns w < d take column d; right: columns
//   w > W-1-d take column W-1-d).
//
// The reference builds this with two Python loops over the W disparities (2 x W slice assignments,
// W more for the fill: about 300 tiny launches at W = 48) around a softmax.  Here one block owns one
// (view, batch item, row): it stages the row's W x W correlation slice in shared memory (coalesced),
// every thread takes columns w and does the softmax over d for them out of shared memory, the
// probabilities go back to shared memory as [d][w], and the block writes the W rows of W outputs
// with the fill applied, coalesced along w.  HBM traffic: corr once, vol once.
#include "../../include/matchattn.h"

#include <stdint.h>

#include "matchattn_kernels.cuh"

namespace matchattn {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) stereo_volume_kernel(const T *__restrict__ corr, T *__restrict__ vol, int B, int H, int W)
{
    extern __shared__ float sm[];                 // [W][W + 1]: first corr[w][j], then prob[d][w]
    const int h = blockIdx.x, b2 = blockIdx.y;
    const bool right = b2 >= B;
    const int b = right ? b2 - B : b2;
    const int P = W + 1;                          // padded pitch: column walks hit different banks
    const T *src = corr + (static_cast<int64_t>(b) * H + h) * W * W;
    for (int e = threadIdx.x; e < W * W; e += blockDim.x) sm[(e / W) * P + (e % W)] = load_one<T>(src + e);
    __syncthreads();

    // per column w: gather the shifted diagonal into registers-by-recompute, softmax over d.
    // Two passes over shared memory (max, then exp/sum), a third to normalise; results are written to a
    // second array so that other columns still see the correlation.
    float *prob = sm + W * P;                     // [D][W + 1]
    for (int w = threadIdx.x; w < W; w += blockDim.x) {
        float mx = -INFINITY;
        for (int d = 0; d < W; ++d) {
            float val = 0.f;
            if (!right && w >= d) val = sm[w * P + (w - d)];
            if (right && w + d < W) val = sm[(w + d) * P + w];
            mx = fmaxf(mx, val);
        }
        float den = 0.f;
        for (int d = 0; d < W; ++d) {
            float val = 0.f;
            if (!right && w >= d) val = sm[w * P + (w - d)];
            if (right && w + d < W) val = sm[(w + d) * P + w];
            const float e = expf(val - mx);
            prob[d * P + w] = e;
            den += e;
        }
        const float inv = __frcp_rn(den);
        for (int d = 0; d < W; ++d) prob[d * P + w] = DT<T>::rnd(prob[d * P + w] * inv);
    }
    __syncthreads();

    for (int e = threadIdx.x; e < W * W; e += blockDim.x) {
        const int d = e / W, w = e - d * W;
        int from = w;
        if (!right && w < d) from = d;
        if (right && w > W - 1 - d) from = W - 1 - d;
        store_one<T>(vol + ((static_cast<int64_t>(b2) * W + d) * H + h) * W + w, prob[d * P + from]);
    }
}

template <typename T>
cudaError_t launch(const void *corr, void *vol, int B, int H, int W, size_t smem, cudaStream_t stream)
{
    // per-device attribute of the kernel: set on every launch (cheap, idempotent, thread-safe)
    cudaError_t e = cudaFuncSetAttribute(stereo_volume_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return e;
    stereo_volume_kernel<T><<<dim3(H, 2 * B), 256, smem, stream>>>(static_cast<const T *>(corr), static_cast<T *>(vol), B, H, W);
    return cudaGetLastError();
}

}  // namespace
}  // namespace matchattn

extern "C" int matchattn_stereo_volume(const void *correlation, void *volume, int B, int H, int W, int dtype,
                                       void *cuda_stream)
{
    if (!correlation || !volume) return MATCHATTN_ERR_NULL;
    if (B <= 0 || H <= 0 || W <= 0) return MATCHATTN_ERR_SHAPE;
    const size_t smem = 2 * sizeof(float) * static_cast<size_t>(W) * (W + 1);
    if (smem > 200 * 1024 || 2LL * B > 65535) return MATCHATTN_ERR_TOO_LARGE;      // W <= 159
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t err;
    switch (dtype) {
    case MATCHATTN_F32: err = matchattn::launch<float>(correlation, volume, B, H, W, smem, stream); break;
    case MATCHATTN_F16: err = matchattn::launch<__half>(correlation, volume, B, H, W, smem, stream); break;
    case MATCHATTN_BF16: err = matchattn::launch<__nv_bfloat16>(correlation, volume, B, H, W, smem, stream); break;
    default: return MATCHATTN_ERR_DTYPE;
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}
