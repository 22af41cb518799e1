// Included once per element type with MATCHATTN_T defined: instantiates the
// specialised kernels for that type and the switch that picks one.
#include "matchattn_kernels.cuh"
#ifdef MATCHATTN_T_IS_16BIT
#include "matchattn_mma.cuh"
#endif

namespace matchattn {

template <typename T, int R>
static cudaError_t launch_fast_r(const Params &p, int cpl, bool multi, dim3 grid, cudaStream_t stream)
{
#define MA_CASE(CPL_, MULTI_)                                                              \
    if (cpl == CPL_ && multi == MULTI_) {                                                  \
        fused_forward_kernel<T, R, CPL_, MULTI_><<<grid, kThreads, 0, stream>>>(p);        \
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
cudaError_t launch_fast<MATCHATTN_T>(const Params &p, int r, int cpl, bool multi, dim3 grid, cudaStream_t stream)
{
    if (r == 1) return launch_fast_r<MATCHATTN_T, 1>(p, cpl, multi, grid, stream);
    if (r == 2) return launch_fast_r<MATCHATTN_T, 2>(p, cpl, multi, grid, stream);
    return cudaErrorInvalidValue;
}

#ifdef MATCHATTN_T_IS_16BIT
template <>
cudaError_t launch_mma<MATCHATTN_T>(const Params &p, int r, int cpl, dim3 grid, cudaStream_t stream)
{
    if (r != 1) return cudaErrorInvalidValue;
#define MA_CASE(CPL_)                                                                      \
    if (cpl == CPL_) {                                                                     \
        fused_forward_mma_kernel<MATCHATTN_T, 1, CPL_><<<grid, kThreads, 0, stream>>>(p);  \
        return cudaGetLastError();                                                         \
    }
    MA_CASE(1) MA_CASE(2) MA_CASE(3) MA_CASE(4) MA_CASE(5)
#undef MA_CASE
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
