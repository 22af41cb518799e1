/*
 * matchattn.h -- C ABI of the B200 (sm_100a) MatchAttention operator.
 *
 * The library replaces the native side of the reference's 'cuda' path:
 *   - pybind entry  match_attention.fused_forward      models/src/match_former_cuda.cpp:24-44
 *   - host driver   match_former_fused_forward          models/src/match_former_fused_forward.cu:461-628
 * and computes what the reference's 'pytorch' path computes
 * (models/mat_pytorch_impl.py:3-178 as driven by models/attention_blocks.py:82-91).
 *
 * Conventions
 *   - plain pointers and sizes only; every buffer is owned by the caller;
 *   - all pointers are DEVICE pointers on the current CUDA device;
 *   - nothing is allocated, nothing is synchronised: each call enqueues its
 *     kernels on `cuda_stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) and returns;
 *   - outputs are fully overwritten, they need not be zeroed beforehand;
 *   - the return value is 0 on success, otherwise a status that
 *     matchattn_strerror() turns into text.  A bad argument never reaches the
 *     device.
 */
#ifndef MATCHATTN_H_
#define MATCHATTN_H_

#include <stddef.h>

#if defined(__GNUC__)
#define MATCHATTN_API __attribute__((visibility("default")))
#else
#define MATCHATTN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types (argument `dtype`) */
#define MATCHATTN_F32  0
#define MATCHATTN_F16  1
#define MATCHATTN_BF16 2

/* scoring functions (argument `attn_type`).  The negative L1 distance is the
 * only one the reference models select (models/attention_blocks.py:93) and the
 * one the tuned kernels compute.  The dot product exists in the reference only
 * as an unused native kernel (models/src/match_former_fused_forward.cu:222-251)
 * with no PyTorch form to compare with; here it runs on the general kernel
 * (any head width, one thread per query and head; no tuned variant, no
 * strategy other than 0 or 1), checked against a restatement of that kernel. */
#define MATCHATTN_L1_NORM     0
#define MATCHATTN_DOT_PRODUCT 1

/* status codes */
#define MATCHATTN_OK                 0
#define MATCHATTN_ERR_NULL           1  /* a required pointer is NULL                         */
#define MATCHATTN_ERR_SHAPE          2  /* a size is <= 0, or the row band is empty / outside */
#define MATCHATTN_ERR_WINDOW_FIT     3  /* 2r+2 exceeds H or W (models/attention_blocks.py:64) */
#define MATCHATTN_ERR_DTYPE          4  /* unknown element type                               */
#define MATCHATTN_ERR_ATTN_TYPE      5  /* unknown scoring function                            */
#define MATCHATTN_ERR_WINDOW         6  /* rx != ry, r < 0 or r above the supported maximum    */
#define MATCHATTN_ERR_ALIGN          7  /* a pointer is not aligned to its element size       */
#define MATCHATTN_ERR_TOO_LARGE      8  /* sizes overflow the 32-bit index ranges in use      */
#define MATCHATTN_ERR_VARIANT        9  /* the kernel variant asked for does not cover the arguments */
#define MATCHATTN_ERR_SCRATCH_LIMIT 10  /* the problem needs more than the built-in scratch area     */
#define MATCHATTN_ERR_CUDA         100  /* 100 + cudaError_t of a failed launch               */

/* largest window radius accepted */
#define MATCHATTN_MAX_R 4

/*
 * The fused MatchAttention forward.
 * Replaces mf_fused_forward (models/src/match_former_cuda.cpp:24-39) and the
 * seven-launch driver behind it (models/src/match_former_fused_forward.cu:461-628).
 *
 *   max_offset [B, Nq, h, 2]  absolute sampling centre (x, y) of every (query, head), token units
 *   q          [B, Nq, h*hd]
 *   k, v       [B, H*W, h*hd]
 *   out        [B, Nq, h*hd]                      written
 *   attn_out   [B, Nq, h, (2r+2)^2]               written; may be NULL to skip it
 *
 * Nq = (q_row_end - q_row_begin) * W.  With q_row_begin = 0 and q_row_end = H
 * this is the whole op.  Otherwise the query-side arrays (max_offset, q, out,
 * attn_out) hold only the rows [q_row_begin, q_row_end) of the token map while
 * k and v still hold all of it: the row-band form used to split one large
 * pair across GPUs.
 *
 * Window taps outside the map are clamped to the nearest border token
 * (models/mat_pytorch_impl.py:58-59); max_offset itself may lie anywhere.
 * rx must equal ry.  `scale` multiplies the negative L1 score
 * (models/attention_blocks.py:86).
 */
MATCHATTN_API int matchattn_fused_forward(const void *max_offset, const void *q, const void *k, const void *v,
                            void *out, void *attn_out,
                            int B, int H, int W, int h, int hd, int rx, int ry,
                            int dtype, int attn_type, float scale,
                            int q_row_begin, int q_row_end, void *cuda_stream);

/*
 * Tuning knobs for the call above; same contract and results.
 *   tile_w        width in queries of the 2-D query tile that one thread block covers
 *                 (0 = choose automatically);
 *   force_generic non-zero selects the slow any-shape kernel even where a
 *                 specialised one exists (used by the tests to cover it);
 *   chunks_per_lane  how many 8-channel chunks of a head one lane owns (0 =
 *                 choose automatically; a value that does not divide hd/8 into a
 *                 power-of-two number of lanes falls back to the any-shape kernel);
 *   variant       0 = choose automatically; 1 = the scalar kernel (float32 sums on the
 *                 CUDA cores); 2 = the kernel that sums with warp matrix instructions
 *                 (16-bit types, r = 1, head width <= 40; MATCHATTN_ERR_VARIANT otherwise).
 * No counterpart in the reference.
 */
MATCHATTN_API int matchattn_fused_forward_ex(const void *max_offset, const void *q, const void *k, const void *v,
                               void *out, void *attn_out,
                               int B, int H, int W, int h, int hd, int rx, int ry,
                               int dtype, int attn_type, float scale,
                               int q_row_begin, int q_row_end, void *cuda_stream,
                               int tile_w, int force_generic, int chunks_per_lane, int variant);

/*
 * The operator with the caller's glue folded in.  In the reference, MatchAttention.forward
 * clamps the centres before the op (models/attention_blocks.py:45-59,79) and, in the cross
 * branch, multiplies the result by a gate and concatenates the attention weights to it before
 * the output projection (models/attention_blocks.py:95-98); these are five small kernels and
 * two extra passes over the outputs per call.  Here:
 *   clamp_offsets    non-zero: every centre is first clamped to [r, W-1-r-1e-3] x [r, H-1-r-1e-3]
 *                    in the tensor type (the upper bound rounded to that type), NaN kept;
 *   gate             [B, Nq, h*hd] or NULL: out is rounded to the tensor type and then
 *                    multiplied by it element-wise;
 *   out_row_stride   elements from one query's out to the next (0 = h*hd);
 *   attn_row_stride  elements from one query's attn_out to the next (0 = h*(2r+2)^2).
 *   kv_item_shift    keys and values of batch item b are read from item (b + kv_item_shift) mod B
 *                    (0 <= kv_item_shift < B).  The cross branch pairs every view with the other one
 *                    (models/attention_blocks.py:67-71: tgt = cat((tgt_, ref_))); with B/2 here the caller
 *                    projects K and V of the un-swapped batch and skips that copy.
 * With out = buf, attn_out = buf + h*hd and both strides = h*hd + h*(2r+2)^2 the kernel writes
 * the concatenated [B, Nq, h*hd + h*(2r+2)^2] tensor the projection consumes.  Direct kernel only.
 */
MATCHATTN_API int matchattn_fused_forward_glue(const void *max_offset, const void *q, const void *k, const void *v,
                                               const void *gate, void *out, void *attn_out,
                                               int B, int H, int W, int h, int hd, int rx, int ry,
                                               int dtype, int attn_type, float scale,
                                               int q_row_begin, int q_row_end,
                                               int clamp_offsets, long long out_row_stride,
                                               long long attn_row_stride, int kv_item_shift, void *cuda_stream);

/*
 * The operator with every index checked on the device: the debugging aid for hosts that cannot run a
 * memory checker.  Same arguments and results as matchattn_fused_forward (direct kernels), plus
 *   status  16 bytes of device memory, 8-byte aligned; cleared by the call, then
 *           [0] = number of indices (key/value taps, query-side rows) that left their array,
 *           [1] = the first offender as block << 32 | thread << 8 | kind (1 tap, 2 query row), 0 if none.
 * An index that fails the check is only recorded; the access itself is the clamped one of the normal
 * kernel, so the call never faults.  Read `status` after synchronising the stream.  Runs the build of the
 * kernel that also honours the rarely used options, which is a few per cent slower than the plain one.
 * No counterpart in the reference (its driver checks nothing, models/src/match_former_fused_forward.cu:461-628).
 */
MATCHATTN_API int matchattn_fused_forward_checked(const void *max_offset, const void *q, const void *k, const void *v,
                                                  void *out, void *attn_out,
                                                  int B, int H, int W, int h, int hd, int rx, int ry,
                                                  int dtype, int attn_type, float scale,
                                                  int q_row_begin, int q_row_end, void *status, void *cuda_stream);

/*
 * Backward of the operator: gradients with respect to q, k, v and max_offset, given the gradients of both
 * outputs.  The reference's native path has none (models/match_former_ops.py registers no autograd; the
 * attn_sum buffer "for backward" of models/src/match_former_fused_forward.cu:409,495 is never read); what is
 * computed is what autograd computes over the reference's 'pytorch' path (models/mat_pytorch_impl.py:3-178
 * driven by models/attention_blocks.py:82-91).
 *   d_out        [B, Nq, h*hd]            gradient of out
 *   d_attn       [B, Nq, h, (2r+2)^2]     gradient of attn_out, or NULL (the self branch discards attn_out)
 *   d_q          [B, Nq, h*hd]            written (tensor type)
 *   d_k, d_v     [B, H*W, h*hd] float32   ACCUMULATED with atomic adds: the caller zeroes them (or passes running sums)
 *   d_max_offset [B, Nq, h, 2]            written, or NULL: through the bilinear weights (floor has no gradient)
 * Nothing is saved by the forward; the kernel recomputes what it needs, in float32 whatever the tensor type.
 * Allocates nothing, launches on `cuda_stream`.
 */
MATCHATTN_API int matchattn_fused_backward(const void *max_offset, const void *q, const void *k, const void *v,
                                           const void *d_out, const void *d_attn,
                                           void *d_q, float *d_k, float *d_v, void *d_max_offset,
                                           int B, int H, int W, int h, int hd, int rx, int ry,
                                           int dtype, int attn_type, float scale,
                                           int q_row_begin, int q_row_end, void *cuda_stream);

/*
 * The same operator with scratch memory from the caller, which opens the binned
 * path: the queries are counting-sorted by the tile of the token map their window
 * falls into and each tile of K/V is staged in shared memory once for all the
 * queries that look at it.  It pays when sampling centres are spread widely
 * (neighbouring queries then share no taps and the direct kernel is bound by
 * L2 bandwidth).  Covered: float16 / bfloat16, r = 1, head width <= 40, one
 * sampling centre per query shared by all heads; a call whose heads differ is
 * detected on the device and served by the direct kernel in the same call.
 *
 *   workspace        device scratch of at least matchattn_workspace_bytes(...) bytes,
 *                    256-byte aligned; contents need not be preserved between calls,
 *                    but two calls that overlap on the device must not share it;
 *   strategy         0 = let the library choose (currently always the direct kernel);
 *                    1 = direct kernel (workspace may be NULL);
 *                    2 = binned path, or MATCHATTN_ERR_VARIANT when it does not apply;
 *                    3 = the sorting passes only, then the direct kernel walking the queries
 *                        in sorted order (the tiles are then shared through L1 instead of
 *                        shared memory; heads may look at different places).
 *                    5, 6 = staged tiles: per tile of 16 x QH queries the extent of the windows is found
 *                        and, when it fits the shared-memory region, the tensor memory accelerator copies
 *                        that K region and V region in with one cp.async.bulk.tensor each (completion on an
 *                        mbarrier); taps are then read from shared memory.  5: one persistent block per SM,
 *                        a producer warp keeps the next regions arriving while 24 consumer warps compute;
 *                        6: one block per tile.  A tile whose
 *                        windows spread further is served with global loads by the same block, so every
 *                        input is accepted; it pays when neighbouring queries look at neighbouring places
 *                        (self attention, smooth disparity / flow).  16-bit types, r = 1, head width 8 or
 *                        16, 1/2/4/8/16 heads, at most 256 channels; MATCHATTN_ERR_VARIANT otherwise.  Needs
 *                        no scratch; if `workspace` holds at least 8 bytes its first 8 receive the number
 *                        of tiles that fell back to global loads (a 64-bit counter, cleared by the call).
 * Still allocates nothing and does not synchronise.  No counterpart in the reference
 * (its driver allocates its own temporaries, models/src/match_former_fused_forward.cu:492-508).
 */
MATCHATTN_API int matchattn_fused_forward_ws(const void *max_offset, const void *q, const void *k, const void *v,
                                             void *out, void *attn_out,
                                             int B, int H, int W, int h, int hd, int rx, int ry,
                                             int dtype, int attn_type, float scale,
                                             int q_row_begin, int q_row_end, void *cuda_stream,
                                             void *workspace, size_t workspace_bytes, int strategy);

/* Scratch bytes the binned path needs for these sizes; 0 when it does not apply. */
MATCHATTN_API size_t matchattn_workspace_bytes(int B, int H, int W, int h, int hd, int r, int dtype,
                                               int q_row_begin, int q_row_end);

/*
 * The binned path for callers that cannot allocate device memory (a server whose
 * memory plan is frozen after start-up, a frame loop with a fixed device budget, a
 * host application that owns every allocation and hands a plugin only tensors and a
 * stream).  Same arguments and results as matchattn_fused_forward_ws with strategy 2,
 * but the scratch is a fixed area inside the library image, so the caller passes
 * none and the library allocates none: no cudaMalloc, cudaFree or other allocating
 * call is made.
 *
 *   - The area is MATCHATTN_STATIC_SCRATCH_BYTES large.  Every GPU on which the
 *     library's module is loaded holds that much device memory until the process
 *     exits.  A problem that needs more (see matchattn_workspace_bytes) is refused
 *     with MATCHATTN_ERR_SCRATCH_LIMIT; one the binned path does not cover
 *     (float32, r != 1, head width > 40) with MATCHATTN_ERR_VARIANT.  With the
 *     present size, 8 heads x 16 channels in float16 fit up to about 690 000
 *     queries per call (the 4 x 384 x 384 headline shape needs 7.1 MB).
 *   - The first call on a device looks up the device address of the area (once per
 *     device, with that device current).  Make that first call outside any stream
 *     capture.
 *   - All calls on a device share the one area and it keeps whatever the last call
 *     left in it.  Each call clears the parts that must start at zero itself, on
 *     its own stream.  Two calls that can overlap on the device (different streams,
 *     different host threads) race on it: serialise them, or give the others
 *     their own scratch through matchattn_fused_forward_ws.
 * No counterpart in the reference.
 */
#define MATCHATTN_STATIC_SCRATCH_BYTES (8u << 20)
MATCHATTN_API int matchattn_fused_forward_static(const void *max_offset, const void *q, const void *k, const void *v,
                                                 void *out, void *attn_out,
                                                 int B, int H, int W, int h, int hd, int rx, int ry,
                                                 int dtype, int attn_type, float scale,
                                                 int q_row_begin, int q_row_end, void *cuda_stream);

/*
 * Convex upsampling of a field, the step either side of the operator in the model:
 * MatchStereo.upsample_field (models/match_stereo.py:73-84) as one kernel instead of a
 * softmax, an unfold, a broadcast product, a sum and a permute.
 *   field [B, H, W, D]           D <= 8
 *   mask  [B, 9*f*f, H, W]       channel (k*f + i)*f + j, k = 3x3 neighbour (row-major, zero padding)
 *   out   [B, f*H, f*W, D]       written; f = factor in {1, 2, 4, 8}
 *   out[b, h*f+i, w*f+j, d] = sum_k softmax_k(mask[b, (k,i,j), h, w]) * (f * field[b, h+ky-1, w+kx-1, d])
 * Allocates nothing, launches on `cuda_stream`.
 */
MATCHATTN_API int matchattn_upsample_field(const void *field, const void *mask, void *out,
                                           int B, int H, int W, int D, int factor, int dtype, void *cuda_stream);

/*
 * Cost volume of the stereo branch of GlobalCorrelation, the step before the first MatchAttention
 * block (models/cost_volume.py:26-51: masks, the two Python loops over the disparities, the softmax
 * over disparity and the out-of-view fill), as one kernel.
 *   correlation [B, H, W, W]     scaled q.k^T of a row: reference column, then target column
 *   volume      [2B, W, H, W]    written: left view in the first B items, right view in the last B
 * W <= 159 (the row's W x W slice is staged in shared memory).  Allocates nothing.
 */
MATCHATTN_API int matchattn_stereo_volume(const void *correlation, void *volume, int B, int H, int W, int dtype,
                                          void *cuda_stream);

/*
 * Consistency (non-occlusion) mask of a bidirectional field, once per layer in the model:
 * MatchAttentionLayer.consistency_mask (models/attention_blocks.py:130-138; the sampler is
 * bilinear_sample_by_offset, utils/utils.py:39-48) as one kernel.
 *   field      [B, H, W, 2]   (x, y) per pixel; items [0, B/2) are one view, [B/2, B) the other; B even
 *   noc_mask   [B, H, W, 1]   written: 1 where sum_c |field_c + other_view_field_c(sampled at pixel + field)| < threshold
 *   field_diff [B, H, W, 1]   or NULL: the sum itself (the reference does not return it; tests use it)
 * The other view's field is sampled bilinearly with zero padding at the normalised coordinate
 * 2*x/(W-1) - 1 rounded as the reference's tensor ops round it.  Allocates nothing.
 */
MATCHATTN_API int matchattn_consistency_mask(const void *field, void *noc_mask, void *field_diff,
                                             int B, int H, int W, float threshold, int dtype, void *cuda_stream);

/*
 * From the cost volume to the initial field: local_disparity_estimator + disp_to_flow
 * (models/cost_volume.py:123-178) as one kernel.
 *   volume   [B, D, H, W]     softmaxed cost volume (matchattn_stereo_volume's output); B even, D >= 5
 *   flow     [B, H, W, 2]     written: (-disp, 0) for the first B/2 items, (disp, 0) for the rest
 *   blur_max [B, H, W]        or NULL: maximum over D of the 5-tap box average (tests)
 *   centre   [B, H, W] int32  or NULL: first arg max, clamped to [2, D-3] (tests)
 * disp = sum of the five probabilities around the centre, those below 1/D dropped, normalised, times
 * their disparities.  Allocates nothing.
 */
MATCHATTN_API int matchattn_local_disparity(const void *volume, void *flow, void *blur_max, int *centre,
                                            int B, int D, int H, int W, int dtype, void *cuda_stream);

/*
 * Flow branch of GlobalCorrelation after its matmul, with local_flow_estimator
 * (models/cost_volume.py:61-69 and :71-121): the step before the first MatchAttention block of MatchFlow.
 *   correlation [B, N, N]      N = H*W; scaled q.k^T, reference token then target token
 *   prob        [2B, N, N]     written: softmax over the last axis of correlation[b] (items [0, B)) and of its
 *                              transpose (items [B, 2B)); the reference returns it viewed as [2B, H, W, N]
 *   flow        [2B, H, W, 2]  written: expected target position within the 5x5 window around the arg max of the
 *                              5x5-pooled probabilities, minus the token's own position
 *   blur_max    [2B, N]        or NULL: the pooled maximum (tests)
 *   centre      [2B, N] int32  or NULL: the clamped window centre as y*W + x (tests)
 *   scratch     at least matchattn_flow_init_scratch_bytes(B, H, W) bytes of device memory, 16-byte aligned
 * H, W >= 5.  Allocates nothing; five kernels on `cuda_stream`.
 */
MATCHATTN_API size_t matchattn_flow_init_scratch_bytes(int B, int H, int W);
MATCHATTN_API int matchattn_flow_init(const void *correlation, void *prob, void *flow, void *blur_max, int *centre,
                                      void *scratch, size_t scratch_bytes, int B, int H, int W, int dtype,
                                      void *cuda_stream);

/* Name of the kernel variant the arguments would dispatch to ("fast cpl=2 lph=1",
 * "generic", ...) or NULL if they are rejected.  Launches nothing. */
MATCHATTN_API const char *matchattn_describe_dispatch(int h, int hd, int r, int dtype, int pointers_32B_aligned);

/*
 * Row-band helper (no counterpart in the reference, which has no multi-GPU code): enqueue `count`
 * device-to-device copies dst[i] <- src[i] of bytes[i] bytes on `cuda_stream`.  Source and destination
 * may live on different GPUs of the box when the caller has mapped the peer's memory into this process
 * (the halo rows of K / V that a band pulls out of its neighbours' buffers, matchattention_b200/band.py).
 * use_kernel == 0: one cudaMemcpyAsync per block (copy engines).  use_kernel != 0: one kernel launch per
 * sixteen blocks reads the sources with plain 16-byte loads (over NVLink when they are a peer's) and
 * stores locally; blocks whose addresses or sizes are not multiples of 16 bytes still go through
 * cudaMemcpyAsync.  Nothing is allocated; the arrays are host memory read before return.
 */
MATCHATTN_API int matchattn_copy_blocks(void *const *dst, const void *const *src, const size_t *bytes, int count,
                                        int use_kernel, void *cuda_stream);

/* version of this ABI: major * 100 + minor */
MATCHATTN_API int matchattn_version(void);

/* text for a status code; never NULL */
MATCHATTN_API const char *matchattn_strerror(int status);

#ifdef __cplusplus
}
#endif
#endif /* MATCHATTN_H_ */
