// The operator for callers that cannot allocate device memory.
//
// Some hosts hand a plugin its tensors and a stream but no allocator: an
// inference server whose memory plan is frozen after start-up, a per-frame
// camera loop running under a fixed device-memory budget, an embedding
// application that forbids cudaMalloc outside its own pool because the call
// synchronises the device.  Such a caller can use the direct kernels (they need
// no scratch at all), but not the binned path, whose counting sort needs a few
// megabytes of scratch.  This file gives that path a scratch area that is part
// of the library image itself: a file-scope __device__ array.  Nothing here
// calls cudaMalloc, cudaFree or any other allocating routine.
//
// The price: every GPU on which the library is used holds
// MATCHATTN_STATIC_SCRATCH_BYTES of device memory from the moment the module is
// loaded until the process exits, and the problem size is limited by it.
#include "../../include/matchattn.h"

#include <cuda_runtime.h>
#include <mutex>

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime
// (a host-side stand-in): it is never passed to a kernel.  The device address is
// asked for with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[MATCHATTN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_address[kMaxDevices] = {};   // device address of g_static_scratch, per device
bool g_scratch_ready[kMaxDevices] = {};

// Device address of the scratch array on the current device; looked up once per device.
int scratch_on_current_device(void **address)
{
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(err);
    if (dev < 0 || dev >= kMaxDevices) return MATCHATTN_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ready[dev]) {
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_static_scratch);      // with device `dev` current
        if (err != cudaSuccess) return MATCHATTN_ERR_CUDA + static_cast<int>(err);
        if (ptr == nullptr) return MATCHATTN_ERR_NULL;
        g_scratch_address[dev] = ptr;
        g_scratch_ready[dev] = true;
    }
    *address = g_scratch_address[dev];
    return MATCHATTN_OK;
}

}  // namespace

extern "C" int matchattn_fused_forward_static(const void *max_offset, const void *q, const void *k, const void *v,
                                              void *out, void *attn_out, int B, int H, int W, int h, int hd, int rx,
                                              int ry, int dtype, int attn_type, float scale, int q_row_begin,
                                              int q_row_end, void *cuda_stream)
{
    if (rx != ry) return MATCHATTN_ERR_WINDOW;
    if (B <= 0 || H <= 0 || W <= 0 || h <= 0 || hd <= 0 || q_row_begin < 0 || q_row_end > H || q_row_begin >= q_row_end)
        return MATCHATTN_ERR_SHAPE;
    // sizes first: nothing is launched and no address is looked up for a problem that does not fit
    const size_t need = matchattn_workspace_bytes(B, H, W, h, hd, rx, dtype, q_row_begin, q_row_end);
    if (need == 0) return MATCHATTN_ERR_VARIANT;             // the binned path does not cover these arguments
    if (need > static_cast<size_t>(MATCHATTN_STATIC_SCRATCH_BYTES)) return MATCHATTN_ERR_SCRATCH_LIMIT;
    void *scratch = nullptr;
    const int rc = scratch_on_current_device(&scratch);
    if (rc != MATCHATTN_OK) return rc;
    // The sorting passes clear the histogram and the control words of the scratch themselves at the
    // start of every call; everything else in it is overwritten before it is read.
    return matchattn_fused_forward_ws(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, rx, ry, dtype, attn_type,
                                      scale, q_row_begin, q_row_end, cuda_stream, scratch, need,
                                      /*strategy: binned*/ 2);
}
