/*
 * CPU oracle for the MatchAttention operator.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the algorithm of the reference's
 * 'pytorch' MatchAttention path.  It exists so that the CUDA kernels can be
 * checked against it and so that the benchmark can time a CPU baseline; it is
 * never linked into, imported by or called from the shipped library.
 *
 * Parity status: pinned.  The restatement is compared, in the CPU test suite,
 * with golden vectors produced by executing the reference's own Python
 * functions (models/mat_pytorch_impl.py) on seeded inputs; the script that
 * made the vectors is tests/golden/make_golden.py.
 * One exception, PARITY UNPINNED: the dot-product scoring (attn_type 1 of
 * matchattn_oracle_forward_scored).  The reference has it only as an unused
 * native kernel (models/src/match_former_fused_forward.cu:222-251), which cannot
 * run without a GPU, and has no PyTorch form of it; its vectors come from the
 * reference's functions with the one scoring line swapped for the product form.
 *
 * What is restated (reference file:line):
 *   - window origin  floor(max_offset)            models/attention_blocks.py:82
 *   - bilinear weights [nw, ne, sw, se]           models/mat_pytorch_impl.py:3-27
 *   - tap grid, replicate-border index clamp,
 *     negative L1 score                            models/mat_pytorch_impl.py:29-76
 *   - score * scale                                models/attention_blocks.py:86
 *   - BilinearSoftmax: four shifted (2r+1)^2
 *     sub-windows, one softmax each, weighted,
 *     summed back in the order nw, ne, sw, se      models/mat_pytorch_impl.py:78-165
 *   - weighted sum of the gathered values          models/mat_pytorch_impl.py:167-178
 *
 * Rounding model for the 16-bit types.  Eager PyTorch evaluates each
 * elementwise op in fp32 and rounds the result to the tensor dtype, and it
 * accumulates reductions (sum, softmax) in fp32 and rounds once.  RND() below
 * marks every place where such a rounding happens; for fp32 it is the
 * identity.
 *
 * A second, smaller function restates the convex upsampling of a field that sits
 * on either side of the operator in the model (models/match_stereo.py:73-84).
 *
 * Layout (all arrays contiguous, row-major):
 *   max_offset [B, Nq, h, 2]   absolute (x, y) sampling centre in token units
 *   q          [B, Nq, h*hd]
 *   k, v       [B, H*W, h*hd]
 *   out        [B, Nq, h*hd]
 *   attn_out   [B, Nq, h, (2r+2)^2]      (may be NULL)
 * with Nq = (q_row_end - q_row_begin) * W: the query arrays hold only the rows
 * of the band, keys and values always hold the whole map.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define MA_MAX_R 4
#define MA_MAX_TAPS ((2 * MA_MAX_R + 2) * (2 * MA_MAX_R + 2))

enum { MA_F32 = 0, MA_F16 = 1, MA_BF16 = 2 };

/* ---- 16-bit float conversions, written out so that the result does not
 * depend on compiler flags or on F16C being present ---------------------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static float g_half_table[65536];
static int g_half_table_ready = 0;

static float half_bits_to_float_slow(uint16_t hbits)
{
    uint32_t sign = (uint32_t)(hbits & 0x8000u) << 16;
    uint32_t expo = (hbits >> 10) & 0x1fu;
    uint32_t mant = hbits & 0x3ffu;
    if (expo == 0x1fu) return u2f(sign | 0x7f800000u | (mant << 13));
    if (expo == 0) {
        /* zero or subnormal: value = mant * 2^-24, exact in fp32 */
        float mag = (float)mant * (1.0f / 16777216.0f);
        return sign ? -mag : mag;
    }
    return u2f(sign | ((expo + 112u) << 23) | (mant << 13));
}

static void ensure_half_table(void)
{
    if (g_half_table_ready) return;
    for (uint32_t i = 0; i < 65536u; ++i) g_half_table[i] = half_bits_to_float_slow((uint16_t)i);
    g_half_table_ready = 1;
}

/* fp32 -> fp16 bits, round to nearest even, with subnormals, inf and nan */
static inline uint16_t float_to_half_bits(float f)
{
    uint32_t u = f2u(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t au = u & 0x7fffffffu;
    if (au >= 0x7f800000u) /* inf or nan */
        return (uint16_t)(sign | 0x7c00u | ((au > 0x7f800000u) ? 0x200u : 0u));
    if (au >= 0x477ff000u) /* rounds to or beyond 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    if (au < 0x38800000u) { /* below 2^-14: subnormal half (or zero) */
        /* adding 0.5 (fp32) aligns the value so that the low mantissa bits
         * are the subnormal half, already rounded to nearest even */
        float shifted = u2f(au) + 0.5f;
        return (uint16_t)(sign | (f2u(shifted) - 0x3f000000u));
    }
    uint32_t lsb = (au >> 13) & 1u;
    au += 0xfffu + lsb;              /* round to nearest even on bit 13 */
    return (uint16_t)(sign | ((au - 0x38000000u) >> 13));
}

static inline float bf16_bits_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }

static inline uint16_t float_to_bf16_bits(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float load_elem(const void *p, int64_t i, const int dt)
{
    if (dt == MA_F32) return ((const float *)p)[i];
    if (dt == MA_F16) return g_half_table[((const uint16_t *)p)[i]];
    return bf16_bits_to_float(((const uint16_t *)p)[i]);
}

static inline void store_elem(void *p, int64_t i, float val, const int dt)
{
    if (dt == MA_F32) ((float *)p)[i] = val;
    else if (dt == MA_F16) ((uint16_t *)p)[i] = float_to_half_bits(val);
    else ((uint16_t *)p)[i] = float_to_bf16_bits(val);
}

/* round an fp32 value to the tensor dtype and return it as fp32 */
static inline float rnd(float val, const int dt)
{
    if (dt == MA_F32) return val;
    if (dt == MA_F16) return g_half_table[float_to_half_bits(val)];
    return bf16_bits_to_float(float_to_bf16_bits(val));
}
#define RND(v) rnd((v), dt)

/* floor of a coordinate, limited to the range in which the replicate clamp
 * of the taps still gives the same answer; keeps the int conversion defined */
static inline int origin_of(float coord, int r, int extent)
{
    float fl = floorf(coord);
    float lo = (float)(-(r + 2)), hi = (float)(extent + r + 1);
    if (!(fl >= lo)) fl = lo;
    if (fl > hi) fl = hi;
    return (int)fl;
}

static inline int clampi(int a, int lo, int hi) { return a < lo ? lo : (a > hi ? hi : a); }

/* One (query, head): everything from the window origin to the output slice.
 * always_inline + a literal dt at the call sites gives one specialised copy
 * per dtype. */
static inline __attribute__((always_inline)) void
one_query_head(const void *mo, const void *q, const void *k, const void *v, void *out, void *attn_out,
               int64_t bq /* b*Nq + nq */, int64_t kbase /* b*H*W */, int head,
               int H, int W, int h, int hd, int r, float scale, const int dt, const int dot)
{
    const int side = 2 * r + 2, sub = 2 * r + 1, M = side * side;
    const int C = h * hd;
    const int64_t lh = bq * h + head;

    /* models/mat_pytorch_impl.py:11-25 */
    const float x = load_elem(mo, lh * 2, dt), y = load_elem(mo, lh * 2 + 1, dt);
    const float dx = RND(x - floorf(x)), dy = RND(y - floorf(y));
    const float ex = RND(1.0f - dx), ey = RND(1.0f - dy);
    const float wgt[4] = { RND(ex * ey), RND(dx * ey), RND(ex * dy), RND(dx * dy) };

    /* models/attention_blocks.py:82 and models/mat_pytorch_impl.py:45-61 */
    const int x0 = origin_of(x, r, W), y0 = origin_of(y, r, H);
    int64_t tap_tok[MA_MAX_TAPS];
    for (int j = 0; j < side; ++j) {
        const int ty = clampi(y0 - r + j, 0, H - 1);
        for (int i = 0; i < side; ++i) {
            const int tx = clampi(x0 - r + i, 0, W - 1);
            tap_tok[j * side + i] = kbase + (int64_t)ty * W + tx;
        }
    }

    /* models/mat_pytorch_impl.py:74 then models/attention_blocks.py:86.  dot != 0: the dot-product
     * scoring of models/src/match_former_fused_forward.cu:222-251, which has no PyTorch counterpart in the
     * reference (PARITY UNPINNED for it): line 74 restated as (q.unsqueeze(3) * k_sampled).sum(-1), each
     * product rounded to the tensor type, the sum accumulated in float32. */
    float score[MA_MAX_TAPS];
    const int64_t qoff = bq * C + (int64_t)head * hd;
    for (int m = 0; m < M; ++m) {
        const int64_t koff = tap_tok[m] * C + (int64_t)head * hd;
        float acc = 0.0f;
        if (dot) {
            for (int c = 0; c < hd; ++c)     /* built with -ffp-contract=off: product and sum stay separate */
                acc += RND(load_elem(q, qoff + c, dt) * load_elem(k, koff + c, dt));
            score[m] = RND(RND(acc) * scale);
        } else {
            for (int c = 0; c < hd; ++c)
                acc += fabsf(RND(load_elem(q, qoff + c, dt) - load_elem(k, koff + c, dt)));
            score[m] = RND(RND(-RND(acc)) * scale);
        }
    }

    /* models/mat_pytorch_impl.py:148-165: sub-window t is shifted by
     * (row t/2, column t%2); softmax, weight, then accumulate in place */
    float a[MA_MAX_TAPS];
    for (int m = 0; m < M; ++m) a[m] = 0.0f;
    for (int t = 0; t < 4; ++t) {
        const int oy = t >> 1, ox = t & 1;
        float mx = -INFINITY;
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) {
                const float s = score[(j + oy) * side + i + ox];
                mx = s > mx ? s : mx;
            }
        float e[(2 * MA_MAX_R + 1) * (2 * MA_MAX_R + 1)];
        float den = 0.0f;
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) {
                const float ev = expf(score[(j + oy) * side + i + ox] - mx);
                e[j * sub + i] = ev;
                den += ev;
            }
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) {
                const int m = (j + oy) * side + i + ox;
                const float p = RND(e[j * sub + i] / den);
                a[m] = RND(a[m] + RND(wgt[t] * p));
            }
    }
    if (attn_out)
        for (int m = 0; m < M; ++m) store_elem(attn_out, lh * M + m, a[m], dt);

    /* models/mat_pytorch_impl.py:176 */
    for (int c = 0; c < hd; ++c) {
        float acc = 0.0f;
        for (int m = 0; m < M; ++m)
            acc += RND(a[m] * load_elem(v, tap_tok[m] * C + (int64_t)head * hd + c, dt));
        store_elem(out, qoff + c, acc, dt);
    }
}

const char *matchattn_oracle_strerror(int code)
{
    switch (code) {
    case 0: return "ok";
    case 1: return "null pointer";
    case 2: return "bad shape";
    case 3: return "window does not fit the token map";
    case 4: return "unsupported dtype";
    case 5: return "window radius too large for the oracle";
    case 6: return "unknown scoring function";
    default: return "unknown";
    }
}

/* Work of one thread: a contiguous range of (batch, query) indices. */
typedef struct {
    const void *mo, *q, *k, *v;
    void *out, *attn_out;
    int64_t first, last, Nq, N;
    int H, W, h, hd, r, dtype, dot;
    float scale;
} ma_job;

static void *run_job(void *arg)
{
    const ma_job *jb = (const ma_job *)arg;
    for (int64_t bq = jb->first; bq < jb->last; ++bq) {
        const int64_t kbase = (bq / jb->Nq) * jb->N;
        for (int head = 0; head < jb->h; ++head) {
            switch (jb->dtype) {
            case MA_F32:
                one_query_head(jb->mo, jb->q, jb->k, jb->v, jb->out, jb->attn_out, bq, kbase, head,
                               jb->H, jb->W, jb->h, jb->hd, jb->r, jb->scale, MA_F32, jb->dot);
                break;
            case MA_F16:
                one_query_head(jb->mo, jb->q, jb->k, jb->v, jb->out, jb->attn_out, bq, kbase, head,
                               jb->H, jb->W, jb->h, jb->hd, jb->r, jb->scale, MA_F16, jb->dot);
                break;
            default:
                one_query_head(jb->mo, jb->q, jb->k, jb->v, jb->out, jb->attn_out, bq, kbase, head,
                               jb->H, jb->W, jb->h, jb->hd, jb->r, jb->scale, MA_BF16, jb->dot);
                break;
            }
        }
    }
    return NULL;
}

int matchattn_oracle_max_threads(void)
{
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* Returns 0 on success.  nthreads <= 0 means "all online cores".  attn_type: 0 = negative L1 distance
 * (the reference's models), 1 = dot product (restated, see one_query_head). */
int matchattn_oracle_forward_scored(const void *max_offset, const void *q, const void *k, const void *v,
                                    void *out, void *attn_out,
                                    int B, int H, int W, int h, int hd, int r, int dtype, int attn_type, float scale,
                                    int q_row_begin, int q_row_end, int nthreads)
{
    if (!max_offset || !q || !k || !v || !out) return 1;
    if (attn_type != 0 && attn_type != 1) return 6;
    if (B <= 0 || H <= 0 || W <= 0 || h <= 0 || hd <= 0 || r < 0) return 2;
    if (q_row_begin < 0 || q_row_end > H || q_row_begin >= q_row_end) return 2;
    if (2 * r + 2 > H || 2 * r + 2 > W) return 3; /* models/attention_blocks.py:64 */
    if (dtype != MA_F32 && dtype != MA_F16 && dtype != MA_BF16) return 4;
    if (r > MA_MAX_R) return 5;
    ensure_half_table();

    const int64_t Nq = (int64_t)(q_row_end - q_row_begin) * W;
    const int64_t total = (int64_t)B * Nq;
    if (nthreads <= 0) nthreads = matchattn_oracle_max_threads();
    if (nthreads > 256) nthreads = 256;
    if ((int64_t)nthreads > total) nthreads = (int)total;

    ma_job jobs[256];
    pthread_t tids[256];
    for (int t = 0; t < nthreads; ++t) {
        ma_job *jb = &jobs[t];
        jb->mo = max_offset; jb->q = q; jb->k = k; jb->v = v; jb->out = out; jb->attn_out = attn_out;
        jb->first = total * t / nthreads;
        jb->last = total * (t + 1) / nthreads;
        jb->Nq = Nq; jb->N = (int64_t)H * W;
        jb->H = H; jb->W = W; jb->h = h; jb->hd = hd; jb->r = r; jb->dtype = dtype; jb->scale = scale;
        jb->dot = attn_type;
    }
    int started = 0;
    for (int t = 1; t < nthreads; ++t) {
        if (pthread_create(&tids[t], NULL, run_job, &jobs[t]) != 0) break;
        started = t;
    }
    run_job(&jobs[0]);
    /* a thread that could not be started has its range done here */
    for (int t = started + 1; t < nthreads; ++t) run_job(&jobs[t]);
    for (int t = 1; t <= started; ++t) pthread_join(tids[t], NULL);
    return 0;
}

int matchattn_oracle_forward(const void *max_offset, const void *q, const void *k, const void *v,
                             void *out, void *attn_out,
                             int B, int H, int W, int h, int hd, int r, int dtype, float scale,
                             int q_row_begin, int q_row_end, int nthreads)
{
    return matchattn_oracle_forward_scored(max_offset, q, k, v, out, attn_out, B, H, W, h, hd, r, dtype, 0, scale,
                                           q_row_begin, q_row_end, nthreads);
}

/*
 * Convex upsampling of a field, MatchStereo.upsample_field (models/match_stereo.py:73-84):
 *   field [B, H, W, D], mask [B, 9*f*f, H, W] (channel = (k*f + i)*f + j, k = 3x3 neighbour, row-major,
 *   zero padding), out [B, f*H, f*W, D]:
 *   out[b, h*f+i, w*f+j, d] = sum_k softmax_k(mask[b, (k,i,j), h, w]) * (f * field[b, h+ky-1, w+kx-1, d]).
 * Rounding in the 16-bit types as eager PyTorch: the softmax result, field*f and each product are
 * rounded to the tensor type, the sum over the nine neighbours accumulates in float32.
 */
int matchattn_oracle_upsample_field(const void *field, const void *mask, void *out, int B, int H, int W, int D,
                                    int factor, int dtype)
{
    if (!field || !mask || !out) return 1;
    if (B <= 0 || H <= 0 || W <= 0 || D <= 0 || factor <= 0) return 2;
    if (dtype != MA_F32 && dtype != MA_F16 && dtype != MA_BF16) return 4;
    ensure_half_table();
    const int dt = dtype, f = factor;
    const int64_t plane = (int64_t)H * W;
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h)
            for (int w = 0; w < W; ++w)
                for (int i = 0; i < f; ++i)
                    for (int j = 0; j < f; ++j) {
                        float logit[9], mx = -INFINITY, den = 0.0f, p[9];
                        for (int k = 0; k < 9; ++k) {
                            const int64_t ch = ((int64_t)k * f + i) * f + j;
                            logit[k] = load_elem(mask, ((int64_t)b * 9 * f * f + ch) * plane + (int64_t)h * W + w, dt);
                            mx = logit[k] > mx ? logit[k] : mx;
                        }
                        for (int k = 0; k < 9; ++k) { p[k] = expf(logit[k] - mx); den += p[k]; }
                        for (int k = 0; k < 9; ++k) p[k] = RND(p[k] / den);
                        for (int d = 0; d < D; ++d) {
                            float acc = 0.0f;
                            for (int k = 0; k < 9; ++k) {
                                const int hh = h + k / 3 - 1, ww = w + k % 3 - 1;
                                float val = 0.0f;
                                if (hh >= 0 && hh < H && ww >= 0 && ww < W)
                                    val = RND(load_elem(field, (((int64_t)b * H + hh) * W + ww) * D + d, dt) * (float)f);
                                acc += RND(p[k] * val);
                            }
                            store_elem(out, ((((int64_t)b * H * f + (int64_t)h * f + i) * W * f) + (int64_t)w * f + j) * D + d,
                                       acc, dt);
                        }
                    }
    return 0;
}

/*
 * Cost volume of the stereo branch of GlobalCorrelation (models/cost_volume.py:26-51), from the
 * correlation [B, H, W, W] (reference index, then target index along a row) to the volume
 * [2B, D = W, H, W] the module returns:
 *   first half  (left view):   vol[b, d, h, w]   = corr[b, h, w, w - d]   for w >= d, else 0
 *   second half (right view):  vol[B+b, d, h, w] = corr[b, h, w + d, w]   for w + d < W, else 0
 * (the positions the reference masks with -1e9 / -1e4 are exactly the ones these shifts never read),
 * then a softmax over d, rounded to the tensor type, and the out-of-view fill: the left view copies
 * column d into columns w < d, the right view copies column W-1-d into columns w > W-1-d.
 */
int matchattn_oracle_stereo_volume(const void *corr, void *volume, int B, int H, int W, int dtype)
{
    if (!corr || !volume) return 1;
    if (B <= 0 || H <= 0 || W <= 0) return 2;
    if (dtype != MA_F32 && dtype != MA_F16 && dtype != MA_BF16) return 4;
    ensure_half_table();
    const int dt = dtype, D = W;
    float *sm = (float *)malloc(sizeof(float) * (size_t)D * W);
    if (!sm) return 2;
    for (int b2 = 0; b2 < 2 * B; ++b2)
        for (int h = 0; h < H; ++h) {
            const int right = b2 >= B, b = right ? b2 - B : b2;
            const int64_t row = ((int64_t)b * H + h) * W * W;          /* corr[b, h, :, :] */
            for (int w = 0; w < W; ++w) {
                float mx = -INFINITY, den = 0.0f;
                for (int d = 0; d < D; ++d) {
                    float val = 0.0f;
                    if (!right && w >= d) val = load_elem(corr, row + (int64_t)w * W + (w - d), dt);
                    if (right && w + d < W) val = load_elem(corr, row + (int64_t)(w + d) * W + w, dt);
                    sm[(size_t)d * W + w] = val;
                    mx = val > mx ? val : mx;
                }
                for (int d = 0; d < D; ++d) {
                    const float e = expf(sm[(size_t)d * W + w] - mx);
                    sm[(size_t)d * W + w] = e;
                    den += e;
                }
                for (int d = 0; d < D; ++d) sm[(size_t)d * W + w] = RND(sm[(size_t)d * W + w] / den);
            }
            for (int d = 0; d < D; ++d)
                for (int w = 0; w < W; ++w) {
                    int src = w;
                    if (!right && w < d) src = d;
                    if (right && w > W - 1 - d) src = W - 1 - d;
                    store_elem(volume, (((int64_t)b2 * D + d) * H + h) * W + w, sm[(size_t)d * W + src], dt);
                }
        }
    free(sm);
    return 0;
}

/*
 * Consistency (non-occlusion) mask, MatchAttentionLayer.consistency_mask
 * (models/attention_blocks.py:130-138 with utils/utils.py:31-48):
 *   field [B, H, W, 2] (x, y), the first B/2 items one view, the last B/2 the other;
 *   offset   = field + pixel grid
 *   sampled  = bilinear sample (align_corners, zero padding) of the OTHER view's field at offset,
 *              through normalised coordinates 2*x/(W-1) - 1 as the reference computes them
 *   diff     = sum_c |field_c + sampled_c|
 *   mask     = diff < A
 * Rounding model of the 16-bit types: every elementwise tensor op rounds to the tensor type; the
 * sampler itself works in float32 from the rounded normalised coordinate (as PyTorch's CUDA
 * grid sampler does) and rounds its result once.  diff_out (may be NULL) receives diff.
 */
int matchattn_oracle_consistency_mask(const void *field, void *mask_out, void *diff_out, int B, int H, int W,
                                      float A, int dtype)
{
    if (!field || !mask_out) return 1;
    if (B <= 0 || (B & 1) || H <= 1 || W <= 1) return 2;
    if (dtype != MA_F32 && dtype != MA_F16 && dtype != MA_BF16) return 4;
    ensure_half_table();
    const int dt = dtype;
    for (int b = 0; b < B; ++b) {
        const int tb = (b + B / 2) % B;
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x) {
                const int64_t px = ((int64_t)b * H + y) * W + x;
                const float f0 = load_elem(field, px * 2, dt), f1 = load_elem(field, px * 2 + 1, dt);
                const float ox = RND(f0 + (float)x), oy = RND(f1 + (float)y);
                const float gx = RND(RND(RND(2.0f * ox) / (float)(W - 1)) - 1.0f);
                const float gy = RND(RND(RND(2.0f * oy) / (float)(H - 1)) - 1.0f);
                const float ix = ((gx + 1.0f) / 2.0f) * (float)(W - 1), iy = ((gy + 1.0f) / 2.0f) * (float)(H - 1);
                const float fx0 = floorf(ix), fy0 = floorf(iy);
                const float wx1 = ix - fx0, wx0 = (fx0 + 1.0f) - ix, wy1 = iy - fy0, wy0 = (fy0 + 1.0f) - iy;
                const float wgt[4] = { wx0 * wy0, wx1 * wy0, wx0 * wy1, wx1 * wy1 };
                float diff = 0.0f;
                for (int c = 0; c < 2; ++c) {
                    float acc = 0.0f;
                    for (int t = 0; t < 4; ++t) {
                        const float cx = fx0 + (float)(t & 1), cy = fy0 + (float)(t >> 1);
                        if (cx >= 0.0f && cx <= (float)(W - 1) && cy >= 0.0f && cy <= (float)(H - 1))
                            acc = fmaf(load_elem(field, ((((int64_t)tb * H + (int)cy) * W) + (int)cx) * 2 + c, dt), wgt[t], acc);
                    }
                    const float sampled = RND(acc);
                    diff += fabsf(RND((c == 0 ? f0 : f1) + sampled));
                }
                diff = RND(diff);
                if (diff_out) store_elem(diff_out, px, diff, dt);
                store_elem(mask_out, px, diff < A ? 1.0f : 0.0f, dt);
            }
    }
    return 0;
}

/*
 * Local disparity estimator, local_disparity_estimator + disp_to_flow (models/cost_volume.py:123-178):
 *   cv [B, D, H, W] (softmaxed cost volume) -> flow [B, H, W, 2].
 *   blur   = 5-tap box average over D (zero padded, always divided by 5)
 *   centre = first arg max of blur over D, clamped to [2, D-3]
 *   p_k    = cv at centre-2 .. centre+2, zeroed where below 1/D, normalised by their sum
 *            (sum floored at the smallest normal number of the tensor type)
 *   disp   = sum_k p_k * (centre - 2 + k); negated for the first B/2 items; flow = (disp, 0).
 * blur_out / centre_out (may be NULL) receive the blurred maximum and the clamped centre: the tests
 * gate the discrete choice on them.
 */
int matchattn_oracle_local_disparity(const void *cv, void *flow, void *blur_out, int *centre_out, int B, int D, int H,
                                     int W, int dtype)
{
    if (!cv || !flow) return 1;
    if (B <= 0 || (B & 1) || D < 5 || H <= 0 || W <= 0) return 2;
    if (dtype != MA_F32 && dtype != MA_F16 && dtype != MA_BF16) return 4;
    ensure_half_table();
    const int dt = dtype;
    const int64_t plane = (int64_t)H * W;
    const float tiny = dt == MA_F32 ? 1.17549435e-38f : (dt == MA_F16 ? 6.103515625e-05f : 1.17549435e-38f);
    const float mean = RND((float)(1.0 / D));      /* PyTorch converts the scalar to the tensor type before comparing */
    for (int b = 0; b < B; ++b)
        for (int64_t px = 0; px < plane; ++px) {
            const int64_t base = (int64_t)b * D * plane + px;
            float best = -INFINITY;
            int arg = 0;
            for (int d = 0; d < D; ++d) {
                float acc = 0.0f;
                for (int t = d - 2; t <= d + 2; ++t)
                    if (t >= 0 && t < D) acc += load_elem(cv, base + (int64_t)t * plane, dt);
                const float bl = RND(acc / 5.0f);
                if (bl > best) { best = bl; arg = d; }
            }
            int centre = arg < 2 ? 2 : (arg > D - 3 ? D - 3 : arg);
            float p[5], sum = 0.0f;
            for (int t = 0; t < 5; ++t) {
                p[t] = load_elem(cv, base + (int64_t)(centre - 2 + t) * plane, dt);
                if (p[t] < mean) p[t] = 0.0f;
                sum += p[t];
            }
            sum = RND(sum);
            if (sum < tiny) sum = tiny;
            float disp = 0.0f;
            for (int t = 0; t < 5; ++t) disp += RND(RND(p[t] / sum) * RND((float)(centre - 2 + t)));
            disp = RND(disp);
            if (b < B / 2) disp = -disp;
            store_elem(flow, ((int64_t)b * plane + px) * 2, disp, dt);
            store_elem(flow, ((int64_t)b * plane + px) * 2 + 1, 0.0f, dt);
            if (blur_out) store_elem(blur_out, (int64_t)b * plane + px, best, dt);
            if (centre_out) centre_out[(int64_t)b * plane + px] = centre;
        }
    return 0;
}

/*
 * Flow branch of GlobalCorrelation with its estimator (models/cost_volume.py:56-69 and
 * local_flow_estimator :71-121), from the scaled all-pairs correlation to the initial flow:
 *   corr [B, N, N], N = H*W (reference token, then target token)
 *   prob [2B, N, N]   prob[b] = softmax over the last axis of corr[b], prob[B+b] = the same of corr[b]^T
 *   blur  = 5x5 box average of prob[b2] taken as an N x N IMAGE (zero padded, divided by 25): the reference
 *           applies avg_pool2d to the 3-D tensor, so the window runs over neighbouring reference AND target
 *           token indices (models/cost_volume.py:86)
 *   centre = first arg max of blur over the target axis, as (y, x) = (idx / W, idx % W), clamped to
 *            [2, H-3] x [2, W-3]
 *   p_k   = prob at the 5x5 tokens around the centre, zeroed where below 1/N, normalised by their sum
 *           (floored at the smallest normal number of the type)
 *   flow  = sum_k p_k * (x_k, y_k) - (x, y) of the reference token
 * blur_max_out [2B, N] and centre_out [2B, N] (flat target index after the clamp) may be NULL.
 */
int matchattn_oracle_flow_init(const void *corr, void *prob, void *flow, void *blur_max_out, int *centre_out,
                               int B, int H, int W, int dtype)
{
    if (!corr || !prob || !flow) return 1;
    if (B <= 0 || H < 5 || W < 5) return 2;
    if (dtype != MA_F32 && dtype != MA_F16 && dtype != MA_BF16) return 4;
    ensure_half_table();
    const int dt = dtype;
    const int64_t N = (int64_t)H * W;
    const float tiny = dt == MA_F16 ? 6.103515625e-05f : 1.17549435e-38f;
    const float mean = RND((float)(1.0 / (double)N));
    float *row = (float *)malloc(sizeof(float) * (size_t)N);
    if (!row) return 2;
    /* softmax of every row of corr[b] and of corr[b]^T */
    for (int b2 = 0; b2 < 2 * B; ++b2) {
        const int tr = b2 >= B, b = tr ? b2 - B : b2;
        for (int64_t i = 0; i < N; ++i) {
            float mx = -INFINITY, den = 0.0f;
            for (int64_t j = 0; j < N; ++j) {
                row[j] = load_elem(corr, (int64_t)b * N * N + (tr ? j * N + i : i * N + j), dt);
                mx = row[j] > mx ? row[j] : mx;
            }
            for (int64_t j = 0; j < N; ++j) { row[j] = expf(row[j] - mx); den += row[j]; }
            for (int64_t j = 0; j < N; ++j) store_elem(prob, ((int64_t)b2 * N + i) * N + j, row[j] / den, dt);
        }
    }
    for (int b2 = 0; b2 < 2 * B; ++b2)
        for (int64_t i = 0; i < N; ++i) {
            const int64_t pb = (int64_t)b2 * N * N;
            float best = -INFINITY;
            int64_t arg = 0;
            for (int64_t j = 0; j < N; ++j) {
                float acc = 0.0f;
                for (int64_t ii = i - 2; ii <= i + 2; ++ii)
                    for (int64_t jj = j - 2; jj <= j + 2; ++jj)
                        if (ii >= 0 && ii < N && jj >= 0 && jj < N) acc += load_elem(prob, pb + ii * N + jj, dt);
                const float bl = RND(acc / 25.0f);
                if (bl > best) { best = bl; arg = j; }
            }
            int cy = (int)(arg / W), cx = (int)(arg % W);
            cy = cy < 2 ? 2 : (cy > H - 3 ? H - 3 : cy);
            cx = cx < 2 ? 2 : (cx > W - 3 ? W - 3 : cx);
            float p[25], sum = 0.0f;
            for (int t = 0; t < 25; ++t) {
                const int sy = cy + t / 5 - 2, sx = cx + t % 5 - 2;
                p[t] = load_elem(prob, pb + i * N + (int64_t)sy * W + sx, dt);
                if (p[t] < mean) p[t] = 0.0f;
                sum += p[t];
            }
            sum = RND(sum);
            if (sum < tiny) sum = tiny;
            float ax = 0.0f, ay = 0.0f;
            for (int t = 0; t < 25; ++t) {
                const int sy = cy + t / 5 - 2, sx = cx + t % 5 - 2;
                const float np_ = RND(p[t] / sum);
                ax += RND(np_ * RND((float)sx));
                ay += RND(np_ * RND((float)sy));
            }
            const int qy = (int)(i / W), qx = (int)(i % W);
            store_elem(flow, ((int64_t)b2 * N + i) * 2, RND(RND(ax) - RND((float)qx)), dt);
            store_elem(flow, ((int64_t)b2 * N + i) * 2 + 1, RND(RND(ay) - RND((float)qy)), dt);
            if (blur_max_out) store_elem(blur_max_out, (int64_t)b2 * N + i, best, dt);
            if (centre_out) centre_out[(int64_t)b2 * N + i] = cy * W + cx;
        }
    free(row);
    return 0;
}
