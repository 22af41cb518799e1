// Flow branch of GlobalCorrelation after its matmul, with local_flow_estimator
// (models/cost_volume.py:61-69 and :71-121), as five kernels and no temporaries beyond a small scratch:
//
//   corr [B, N, N] (N = H*W; scaled q.k^T, reference token then target token)
//   prob [2B, N, N]   written: softmax over the last axis of corr[b] and of corr[b]^T
//   flow [2B, H, W, 2] written
//
// The reference materialises the concatenation [corr; corr^T] (2 x N^2), its softmax, the 5x5-pooled copy
// (avg_pool2d over the N x N "image"), arg max, a [2B, N, 25, 2] gather of coordinates and a dozen
// elementwise temporaries.  Here: row softmax of corr; column statistics of corr and a tiled transposed
// normalise for the second half; one pass that pools and takes the arg max without storing the pooled
// volume; one thread per token for the 5x5 window estimate.
// Rounding of the 16-bit types as eager PyTorch on the GPU: softmax, pooling and sums accumulate in float32
// and round once, every elementwise op rounds.
#include "../../include/matchattn.h"

#include <stdint.h>

#include "matchattn_kernels.cuh"

namespace matchattn {
namespace {

constexpr int kFlowThreads = 256;

__device__ __forceinline__ float block_reduce_max(float v, float *sm)
{
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sm[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) r = fmaxf(r, sm[w]);
    __syncthreads();
    return r;
}

__device__ __forceinline__ float block_reduce_sum(float v, float *sm)
{
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) r += sm[w];
    __syncthreads();
    return r;
}

// prob[b, i, :] = softmax(corr[b, i, :]); one block per row
template <typename T>
__global__ void __launch_bounds__(kFlowThreads) flow_row_softmax_kernel(const T *__restrict__ corr, T *__restrict__ prob, int64_t N)
{
    __shared__ float sm[kFlowThreads / 32];
    const T *src = corr + (static_cast<int64_t>(blockIdx.y) * N + blockIdx.x) * N;
    T *dst = prob + (static_cast<int64_t>(blockIdx.y) * N + blockIdx.x) * N;
    float mx = -INFINITY;
    for (int64_t j = threadIdx.x; j < N; j += blockDim.x) mx = fmaxf(mx, load_one<T>(src + j));
    mx = block_reduce_max(mx, sm);
    float den = 0.f;
    for (int64_t j = threadIdx.x; j < N; j += blockDim.x) den += expf(load_one<T>(src + j) - mx);
    den = block_reduce_sum(den, sm);
    for (int64_t j = threadIdx.x; j < N; j += blockDim.x) store_one<T>(dst + j, __fdiv_rn(expf(load_one<T>(src + j) - mx), den));
}

// column maximum and sum of exponentials of corr[b]: 64 columns per block, four row groups
template <typename T>
__global__ void __launch_bounds__(kFlowThreads) flow_col_stats_kernel(const T *__restrict__ corr, float *__restrict__ cmax,
                                                                       float *__restrict__ csum, int64_t N)
{
    __shared__ float sm[4][64];
    const int c = threadIdx.x & 63, g = threadIdx.x >> 6;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * 64 + c;
    const T *src = corr + static_cast<int64_t>(blockIdx.y) * N * N;
    float mx = -INFINITY;
    if (col < N)
        for (int64_t j = g; j < N; j += 4) mx = fmaxf(mx, load_one<T>(src + j * N + col));
    sm[g][c] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(sm[0][c], sm[1][c]), fmaxf(sm[2][c], sm[3][c]));
    __syncthreads();
    float den = 0.f;
    if (col < N)
        for (int64_t j = g; j < N; j += 4) den += expf(load_one<T>(src + j * N + col) - mx);
    sm[g][c] = den;
    __syncthreads();
    if (g == 0 && col < N) {
        cmax[blockIdx.y * N + col] = mx;
        csum[blockIdx.y * N + col] = (sm[0][c] + sm[1][c]) + (sm[2][c] + sm[3][c]);
    }
}

// prob[B + b, i, j] = exp(corr[b, j, i] - cmax[i]) / csum[i], through a 32 x 32 shared-memory tile
template <typename T>
__global__ void __launch_bounds__(kFlowThreads) flow_transposed_softmax_kernel(const T *__restrict__ corr, const float *__restrict__ cmax,
                                                                                const float *__restrict__ csum, T *__restrict__ prob_t,
                                                                                int64_t N)
{
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;       // 32 x 8
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * 32, j0 = static_cast<int64_t>(blockIdx.y) * 32;
    const T *src = corr + static_cast<int64_t>(blockIdx.z) * N * N;
    T *dst = prob_t + static_cast<int64_t>(blockIdx.z) * N * N;
    for (int k = ty; k < 32; k += 8) {
        const int64_t j = j0 + k, i = i0 + tx;
        tile[k][tx] = (j < N && i < N) ? load_one<T>(src + j * N + i) : 0.f;
    }
    __syncthreads();
    for (int k = ty; k < 32; k += 8) {
        const int64_t i = i0 + k, j = j0 + tx;
        if (i < N && j < N)
            store_one<T>(dst + i * N + j, __fdiv_rn(expf(tile[tx][k] - cmax[blockIdx.z * N + i]), csum[blockIdx.z * N + i]));
    }
}

// per (b2, i): maximum over j of the 5 x 5 box average of prob[b2] around (i, j), and its first arg max.
// A block takes kPoolRows consecutive rows i: the kPoolRows + 4 rows of probabilities they need are staged
// once per column chunk in shared memory (1.5 reads per element instead of 5), every thread keeps the
// 12 x 5 neighbourhood of its column in registers and forms the 25-term sums of its eight outputs from
// them, in the reference's order (row-major over the window, out-of-range taps skipped).
constexpr int kPoolRows = 8;

template <typename T>
__global__ void __launch_bounds__(kFlowThreads) flow_pool_argmax_kernel(const T *__restrict__ prob, T *__restrict__ blur_max,
                                                                         int *__restrict__ arg_out, int64_t N)
{
    __shared__ float rows[kPoolRows + 4][kFlowThreads + 4];
    __shared__ float best_v[kPoolRows][kFlowThreads / 32];
    __shared__ int best_j[kPoolRows][kFlowThreads / 32];
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kPoolRows;
    const T *base = prob + static_cast<int64_t>(blockIdx.y) * N * N;
    float best[kPoolRows];
    int arg[kPoolRows];
#pragma unroll
    for (int r = 0; r < kPoolRows; ++r) {
        best[r] = -INFINITY;
        arg[r] = 0x7fffffff;
    }
    for (int64_t c0 = 0; c0 < N; c0 += kFlowThreads) {
        for (int e = threadIdx.x; e < (kPoolRows + 4) * (kFlowThreads + 4); e += kFlowThreads) {
            const int di = e / (kFlowThreads + 4), cc = e - di * (kFlowThreads + 4);
            const int64_t ii = i0 + di - 2, jj = c0 + cc - 2;
            rows[di][cc] = (ii >= 0 && ii < N && jj >= 0 && jj < N) ? load_one<T>(base + ii * N + jj) : 0.f;
        }
        __syncthreads();
        const int64_t j = c0 + threadIdx.x;
        if (j < N) {
            float w[kPoolRows + 4][5];
#pragma unroll
            for (int di = 0; di < kPoolRows + 4; ++di)
#pragma unroll
                for (int dj = 0; dj < 5; ++dj) w[di][dj] = rows[di][threadIdx.x + dj];
#pragma unroll
            for (int r = 0; r < kPoolRows; ++r) {
                const int64_t i = i0 + r;
                if (i >= N) break;
                float acc = 0.f;
#pragma unroll
                for (int di = 0; di < 5; ++di)
#pragma unroll
                    for (int dj = 0; dj < 5; ++dj) {
                        const int64_t ii = i + di - 2, jj = j + dj - 2;
                        if (ii >= 0 && ii < N && jj >= 0 && jj < N) acc += w[r + di][dj];
                    }
                const float bl = DT<T>::rnd(__fdiv_rn(acc, 25.f));
                if (bl > best[r]) {
                    best[r] = bl;
                    arg[r] = static_cast<int>(j);
                }
            }
        }
        __syncthreads();
    }
    // block arg max per row: larger value wins, equal values keep the smaller index
#pragma unroll
    for (int r = 0; r < kPoolRows; ++r) {
        float bv = best[r];
        int bj = arg[r];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oj = __shfl_xor_sync(0xffffffffu, bj, o);
            if (ov > bv || (ov == bv && oj < bj)) {
                bv = ov;
                bj = oj;
            }
        }
        if ((threadIdx.x & 31) == 0) {
            best_v[r][threadIdx.x >> 5] = bv;
            best_j[r][threadIdx.x >> 5] = bj;
        }
    }
    __syncthreads();
    if (threadIdx.x < kPoolRows && i0 + threadIdx.x < N) {
        const int r = threadIdx.x;
        float bv = best_v[r][0];
        int bj = best_j[r][0];
        for (int w = 1; w < kFlowThreads / 32; ++w)
            if (best_v[r][w] > bv || (best_v[r][w] == bv && best_j[r][w] < bj)) {
                bv = best_v[r][w];
                bj = best_j[r][w];
            }
        arg_out[blockIdx.y * N + i0 + r] = bj;
        if (blur_max != nullptr) store_one<T>(blur_max + blockIdx.y * N + i0 + r, bv);
    }
}

// per (b2, i): 5 x 5 window of probabilities around the clamped arg max -> expected target position - own position
template <typename T>
__global__ void __launch_bounds__(kFlowThreads) flow_window_kernel(const T *__restrict__ prob, const int *__restrict__ arg_in,
                                                                    T *__restrict__ flow, int *__restrict__ centre_out, int H, int W,
                                                                    int64_t total, float tiny)
{
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= total) return;
    const int64_t N = static_cast<int64_t>(H) * W;
    const int64_t b2 = t / N, i = t - b2 * N;
    const int arg = arg_in[t];
    const int cy = min(max(arg / W, 2), H - 3), cx = min(max(arg % W, 2), W - 3);
    const T *row = prob + (b2 * N + i) * N;
    const float mean = DT<T>::rnd(static_cast<float>(1.0 / static_cast<double>(N)));   // the scalar is converted to T first
    float p[25], sum = 0.f;
#pragma unroll
    for (int k = 0; k < 25; ++k) {
        p[k] = load_one<T>(row + static_cast<int64_t>(cy + k / 5 - 2) * W + (cx + k % 5 - 2));
        if (p[k] < mean) p[k] = 0.f;
        sum += p[k];
    }
    sum = fmaxf(DT<T>::rnd(sum), tiny);
    float ax = 0.f, ay = 0.f;
#pragma unroll
    for (int k = 0; k < 25; ++k) {
        const float np = DT<T>::rnd(__fdiv_rn(p[k], sum));
        ax += DT<T>::rnd(np * DT<T>::rnd(static_cast<float>(cx + k % 5 - 2)));
        ay += DT<T>::rnd(np * DT<T>::rnd(static_cast<float>(cy + k / 5 - 2)));
    }
    const int qy = static_cast<int>(i / W), qx = static_cast<int>(i - static_cast<int64_t>(qy) * W);
    store_one<T>(flow + t * 2, DT<T>::rnd(DT<T>::rnd(ax) - DT<T>::rnd(static_cast<float>(qx))));
    store_one<T>(flow + t * 2 + 1, DT<T>::rnd(DT<T>::rnd(ay) - DT<T>::rnd(static_cast<float>(qy))));
    if (centre_out != nullptr) centre_out[t] = cy * W + cx;
}

template <typename T>
cudaError_t run_flow_init(const void *corr_, void *prob_, void *flow_, void *blur_, int *centre, void *scratch, int B, int H,
                          int W, float tiny, cudaStream_t stream)
{
    const int64_t N = static_cast<int64_t>(H) * W;
    const T *corr = static_cast<const T *>(corr_);
    T *prob = static_cast<T *>(prob_);
    float *cmax = static_cast<float *>(scratch), *csum = cmax + B * N;
    int *arg = reinterpret_cast<int *>(csum + B * N);
    flow_row_softmax_kernel<T><<<dim3(static_cast<unsigned>(N), B), kFlowThreads, 0, stream>>>(corr, prob, N);
    flow_col_stats_kernel<T><<<dim3(static_cast<unsigned>((N + 63) / 64), B), kFlowThreads, 0, stream>>>(corr, cmax, csum, N);
    const unsigned tiles = static_cast<unsigned>((N + 31) / 32);
    flow_transposed_softmax_kernel<T><<<dim3(tiles, tiles, B), kFlowThreads, 0, stream>>>(corr, cmax, csum, prob + B * N * N, N);
    flow_pool_argmax_kernel<T><<<dim3(static_cast<unsigned>((N + kPoolRows - 1) / kPoolRows), 2 * B), kFlowThreads, 0, stream>>>(
        prob, static_cast<T *>(blur_), arg, N);
    const int64_t total = 2 * B * N;
    flow_window_kernel<T><<<static_cast<unsigned>((total + kFlowThreads - 1) / kFlowThreads), kFlowThreads, 0, stream>>>(
        prob, arg, static_cast<T *>(flow_), centre, H, W, total, tiny);
    return cudaGetLastError();
}

}  // namespace
}  // namespace matchattn

extern "C" size_t matchattn_flow_init_scratch_bytes(int B, int H, int W)
{
    if (B <= 0 || H <= 0 || W <= 0) return 0;
    return static_cast<size_t>(B) * H * W * (2 * sizeof(float) + 2 * sizeof(int));
}

extern "C" int matchattn_flow_init(const void *correlation, void *prob, void *flow, void *blur_max, int *centre,
                                   void *scratch, size_t scratch_bytes, int B, int H, int W, int dtype, void *cuda_stream)
{
    if (!correlation || !prob || !flow || !scratch) return MATCHATTN_ERR_NULL;
    if (B <= 0 || H < 5 || W < 5) return MATCHATTN_ERR_SHAPE;
    const long long N = 1LL * H * W;
    if (N > 65535LL * 32 || 2LL * B > 65535 || N >= (1LL << 31)) return MATCHATTN_ERR_TOO_LARGE;
    if (scratch_bytes < matchattn_flow_init_scratch_bytes(B, H, W) || (reinterpret_cast<uintptr_t>(scratch) & 15))
        return MATCHATTN_ERR_ALIGN;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t err;
    switch (dtype) {
    case MATCHATTN_F32: err = matchattn::run_flow_init<float>(correlation, prob, flow, blur_max, centre, scratch, B, H, W, 1.17549435e-38f, stream); break;
    case MATCHATTN_F16: err = matchattn::run_flow_init<__half>(correlation, prob, flow, blur_max, centre, scratch, B, H, W, 6.103515625e-05f, stream); break;
    case MATCHATTN_BF16: err = matchattn::run_flow_init<__nv_bfloat16>(correlation, prob, flow, blur_max, centre, scratch, B, H, W, 1.17549435e-38f, stream); break;
    default: return MATCHATTN_ERR_DTYPE;
    }
    return err == cudaSuccess ? MATCHATTN_OK : MATCHATTN_ERR_CUDA + static_cast<int>(err);
}
