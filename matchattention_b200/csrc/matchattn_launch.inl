// Included once per element type with MATCHATTN_T defined: instantiates the
// specialised kernels for that type and the switch that picks one.
#include "matchattn_kernels.cuh"
#ifdef MATCHATTN_T_IS_16BIT
#include "matchattn_mma.cuh"
#include "matchattn_binned.cuh"
#include "matchattn_staged.cuh"
#endif

namespace matchattn {

template <typename T, int R>
static cudaError_t launch_fast_r(const Params &p, int cpl, bool multi, dim3 grid, int threads, cudaStream_t stream)
{
    const bool extras = p.guard != nullptr || p.sorted != nullptr || p.gate != nullptr || p.clamp != 0 || p.debug != nullptr || p.kv_shift != 0 ||
                        p.out_stride != p.C || p.attn_stride != p.h * (2 * R + 2) * (2 * R + 2);
    // power-of-two scale: a build of the plain kernel that finishes two scores per packed instruction
    constexpr bool kCanPack = sizeof(T) == 2;
    const bool pow2 = kCanPack && p.scale_pow2 != 0 && !extras;
#define MA_CASE(CPL_, MULTI_)                                                              \
    if (cpl == CPL_ && multi == MULTI_) {                                                  \
        if (extras) fused_forward_kernel<T, R, CPL_, MULTI_, true><<<grid, threads, 0, stream>>>(p);   \
        else if (pow2) fused_forward_kernel<T, R, CPL_, MULTI_, false, kCanPack><<<grid, threads, 0, stream>>>(p);  \
        else fused_forward_kernel<T, R, CPL_, MULTI_, false><<<grid, threads, 0, stream>>>(p);         \
        return cudaGetLastError();                                                         \
    }
    MA_CASE(1, false) MA_CASE(1, true)
    MA_CASE(2, false) MA_CASE(2, true)
    MA_CASE(3, false) MA_CASE(3, true)
    MA_CASE(4, false) MA_CASE(4, true)
    MA_CASE(5, false) MA_CASE(5, true)
#undef MA_CASE
    return cudaErrorInvalidValue;
}

template <>
cudaError_t launch_fast<MATCHATTN_T>(const Params &p, int r, int cpl, bool multi, dim3 grid, int threads, cudaStream_t stream)
{
    if (r == 1) return launch_fast_r<MATCHATTN_T, 1>(p, cpl, multi, grid, threads, stream);
    if (r == 2) return launch_fast_r<MATCHATTN_T, 2>(p, cpl, multi, grid, threads, stream);
    return cudaErrorInvalidValue;
}

#ifdef MATCHATTN_T_IS_16BIT
template <typename T, int CPL>
static cudaError_t launch_mma_cpl(const Params &p, bool sameq, bool pow2, int nch, unsigned blocks, cudaStream_t stream)
{
    if (nch == 1) {
        if (pow2) fused_forward_mma_kernel<T, CPL, false, true, 1><<<blocks, kThreads, 0, stream>>>(p);
        else fused_forward_mma_kernel<T, CPL, false, false, 1><<<blocks, kThreads, 0, stream>>>(p);
    } else if (sameq && pow2) fused_forward_mma_kernel<T, CPL, true, true, 2><<<blocks, kThreads, 0, stream>>>(p);
    else if (sameq) fused_forward_mma_kernel<T, CPL, true, false, 2><<<blocks, kThreads, 0, stream>>>(p);
    else if (pow2) fused_forward_mma_kernel<T, CPL, false, true, 2><<<blocks, kThreads, 0, stream>>>(p);
    else fused_forward_mma_kernel<T, CPL, false, false, 2><<<blocks, kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

template <>
cudaError_t launch_mma<MATCHATTN_T>(const Params &p, int cpl, bool sameq, bool pow2, int nch, unsigned blocks,
                                    cudaStream_t stream)
{
    switch (cpl) {
    case 1: return launch_mma_cpl<MATCHATTN_T, 1>(p, sameq, pow2, nch, blocks, stream);
    case 2: return launch_mma_cpl<MATCHATTN_T, 2>(p, sameq, pow2, nch, blocks, stream);
    case 3: return launch_mma_cpl<MATCHATTN_T, 3>(p, sameq, pow2, nch, blocks, stream);
    case 4: return launch_mma_cpl<MATCHATTN_T, 4>(p, sameq, pow2, nch, blocks, stream);
    case 5: return launch_mma_cpl<MATCHATTN_T, 5>(p, sameq, pow2, nch, blocks, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <typename T, int CPL, bool SAMEQ>
static cudaError_t launch_binned_one(const BinParams &bp, int grid_blocks, size_t smem_bytes, cudaStream_t stream)
{
    // The opt-in to large dynamic shared memory is a per-device attribute of the kernel: it is set on
    // every launch (cheap, idempotent, safe from any host thread) rather than remembered per process.
    cudaError_t e = cudaFuncSetAttribute(binned_forward_kernel<T, CPL, SAMEQ>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMaxBinnedSmem));
    if (e != cudaSuccess) return e;
    binned_forward_kernel<T, CPL, SAMEQ><<<grid_blocks, kBinThreads, smem_bytes, stream>>>(bp);
    return cudaGetLastError();
}

template <typename T, int CPL>
static cudaError_t launch_binned_cpl(const BinParams &bp, int grid_blocks, size_t smem_bytes, cudaStream_t stream)
{
    return bp.p.h % 8 == 0 ? launch_binned_one<T, CPL, true>(bp, grid_blocks, smem_bytes, stream)
                           : launch_binned_one<T, CPL, false>(bp, grid_blocks, smem_bytes, stream);
}

template <>
cudaError_t launch_binned<MATCHATTN_T>(const BinParams &bp, int cpl, int grid_blocks, size_t smem_bytes,
                                       cudaStream_t stream)
{
    const Params &p = bp.p;
    const long long total = 1LL * p.B * p.Nq;
    const unsigned qblocks = static_cast<unsigned>((total + 255) / 256);
    bin_count_kernel<MATCHATTN_T, 1><<<qblocks, 256, 0, stream>>>(bp);
    bin_scan_kernel<<<1, 1024, 0, stream>>>(bp);
    bin_scatter_kernel<<<qblocks, 256, 0, stream>>>(bp);
    switch (cpl) {
    case 0: return cudaGetLastError();       // sorting passes only
    case 1: return launch_binned_cpl<MATCHATTN_T, 1>(bp, grid_blocks, smem_bytes, stream);
    case 2: return launch_binned_cpl<MATCHATTN_T, 2>(bp, grid_blocks, smem_bytes, stream);
    case 3: return launch_binned_cpl<MATCHATTN_T, 3>(bp, grid_blocks, smem_bytes, stream);
    case 4: return launch_binned_cpl<MATCHATTN_T, 4>(bp, grid_blocks, smem_bytes, stream);
    case 5: return launch_binned_cpl<MATCHATTN_T, 5>(bp, grid_blocks, smem_bytes, stream);
    default: return cudaErrorInvalidValue;
    }
}
#endif

#ifdef MATCHATTN_T_IS_16BIT
template <typename T, int CPL, bool POW2>
static cudaError_t launch_staged_one(const StagedParams &sp, const CUtensorMap &map_k, const CUtensorMap &map_v, dim3 grid,
                                     size_t smem_bytes, cudaStream_t stream)
{
    // per-device attribute of the kernel: set on every launch (cheap, idempotent, thread-safe)
    cudaError_t e = cudaFuncSetAttribute(staged_forward_kernel<T, CPL, POW2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kStagedRegionBytes + 128));
    if (e != cudaSuccess) return e;
    staged_forward_kernel<T, CPL, POW2><<<grid, kStagedThreads, smem_bytes, stream>>>(sp, map_k, map_v);
    return cudaGetLastError();
}

template <typename T, int CPL, bool POW2>
static cudaError_t launch_persist_one(const PersistParams &sp, const CUtensorMap &map_k, const CUtensorMap &map_v,
                                      int grid_blocks, cudaStream_t stream)
{
    const size_t smem_bytes = 2 * kPersistRegionBytes + 128;
    cudaError_t e = cudaFuncSetAttribute(staged_persistent_kernel<T, CPL, POW2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem_bytes));
    if (e != cudaSuccess) return e;
    staged_persistent_kernel<T, CPL, POW2><<<grid_blocks, kPersistThreads, smem_bytes, stream>>>(sp, map_k, map_v);
    return cudaGetLastError();
}

template <>
cudaError_t launch_staged_persistent<MATCHATTN_T>(const PersistParams &sp, int cpl, const CUtensorMap &map_k,
                                                  const CUtensorMap &map_v, int grid_blocks, cudaStream_t stream)
{
    const bool pow2 = sp.p.scale_pow2 != 0;
    if (cpl == 1) return pow2 ? launch_persist_one<MATCHATTN_T, 1, true>(sp, map_k, map_v, grid_blocks, stream)
                              : launch_persist_one<MATCHATTN_T, 1, false>(sp, map_k, map_v, grid_blocks, stream);
    if (cpl == 2) return pow2 ? launch_persist_one<MATCHATTN_T, 2, true>(sp, map_k, map_v, grid_blocks, stream)
                              : launch_persist_one<MATCHATTN_T, 2, false>(sp, map_k, map_v, grid_blocks, stream);
    return cudaErrorInvalidValue;
}

template <>
cudaError_t launch_staged<MATCHATTN_T>(const StagedParams &sp, int cpl, const CUtensorMap &map_k, const CUtensorMap &map_v,
                                       dim3 grid, size_t smem_bytes, cudaStream_t stream)
{
    const bool pow2 = sp.p.scale_pow2 != 0;
    if (cpl == 1) return pow2 ? launch_staged_one<MATCHATTN_T, 1, true>(sp, map_k, map_v, grid, smem_bytes, stream)
                              : launch_staged_one<MATCHATTN_T, 1, false>(sp, map_k, map_v, grid, smem_bytes, stream);
    if (cpl == 2) return pow2 ? launch_staged_one<MATCHATTN_T, 2, true>(sp, map_k, map_v, grid, smem_bytes, stream)
                              : launch_staged_one<MATCHATTN_T, 2, false>(sp, map_k, map_v, grid, smem_bytes, stream);
    return cudaErrorInvalidValue;
}
#endif

template <>
cudaError_t launch_generic<MATCHATTN_T>(const Params &p, dim3 grid, cudaStream_t stream)
{
    generic_forward_kernel<MATCHATTN_T><<<grid, kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace matchattn
