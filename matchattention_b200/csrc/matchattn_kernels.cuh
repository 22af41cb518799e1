// MatchAttention forward kernels for sm_100a.
//
// One launch does the whole operator: window origin and bilinear weights from
// the sampling centre, replicate-clamped gather of the (2r+2)^2 key taps,
// negative L1 scores, BilinearSoftmax (four shifted (2r+1)^2 softmaxes blended
// by the bilinear weights) and the weighted sum of the value taps.  Nothing is
// written to global memory except the two outputs.
//
// Work split.  A head's hd channels are cut into "chunks" of 8 channels.  One
// lane owns CPL consecutive chunks of one head of one query; LPH lanes (a power
// of two, inside one warp) together own a head and add their partial L1 sums
// with xor shuffles.  The h*LPH lanes of a query sit next to each other, so a
// warp reads and writes q / out / attn_out / max_offset as contiguous runs, and
// a block covers a 2-D tile of queries so that neighbouring windows overlap in
// L1.  Key/value taps are fetched straight from global memory with 128- or
// 256-bit loads through L1/L2 (each tap of a lane is a whole number of 32-byte
// sectors or a 16-byte half sector).
//
// Arithmetic.  For float16 / bfloat16 every rounding the eager PyTorch
// evaluation of the algorithm performs is reproduced (q-k, the L1 sum, the
// scale, the softmax result, weight*p, the four accumulating adds, a*v, the
// final sum); all reductions accumulate in float32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace matchattn {

constexpr int kThreads = 256;

struct Params {
    const void *mo, *q, *k, *v;
    void *out, *attn;
    int B, H, W, h, hd, C;
    int rows;       // query rows of the band
    int Nq;         // rows * W
    int N;          // H * W
    int r;          // window radius (generic kernel only)
    int lph;        // lanes per head
    int lph_shift;  // log2(lph)
    int G;          // lanes per query = h * lph
    int tile_w;     // query tile of a block: tile_w (power of two) x tile_h
    int tile_w_shift;
    int tile_h;
    int tiles_x;
    float scale;
    const uint32_t *guard;   // when not null the kernel runs only if (*guard != 0) == (guard_run_if != 0)
    int guard_run_if;
    const uint2 *sorted;     // when not null: queries are taken in this order (x = b*Nq + n), see matchattn_binned.cuh
    // caller-side glue folded into the kernel (all off by default)
    const void *gate;        // [B, Nq, C] or null: out is multiplied by it element-wise (after rounding to T)
    int out_stride;          // elements between consecutive queries of out (C unless out is part of a wider row)
    int attn_stride;         // elements between consecutive queries of attn_out (h*M by default)
    int clamp;               // non-zero: clamp the centre to [lo, hi_x] x [lo, hi_y] first, as the caller would
    float clamp_lo, clamp_hi_x, clamp_hi_y;   // bounds, already rounded to T
    int scale_pow2;          // non-zero: 16-bit type and `scale` is a power of two that the type represents exactly
    unsigned long long *debug;   // when not null (checked entry point): [0] counts out-of-range indices, [1] keeps the first
    int kv_shift;            // keys / values of batch item b are read from item (b + kv_shift) mod B (0: the same item)
    int dot;                 // non-zero: scores are sum(q*k) instead of -sum|q-k| (general kernel only)
};

// Records an index that left its array (checked entry point only): a count and the first offender as
// (block << 32 | thread << 8 | what), what = 1 key/value tap, 2 query-side row.
__device__ __forceinline__ void debug_record(unsigned long long *dbg, unsigned what)
{
    atomicAdd(&dbg[0], 1ull);
    atomicCAS(&dbg[1], 0ull, (static_cast<unsigned long long>(blockIdx.x) << 32) | (threadIdx.x << 8) | what);
}

// torch.clamp semantics: NaN stays NaN
__device__ __forceinline__ float clamp_keep_nan(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ------------------------------------------------------------------ loads / stores

__device__ __forceinline__ void ld_nc_256(uint32_t *w, const void *p)
{
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
}
__device__ __forceinline__ void ld_nc_128(uint32_t *w, const void *p)
{
    asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                 : "l"(p));
}
__device__ __forceinline__ void st_256(void *p, const uint32_t *w)
{
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}
__device__ __forceinline__ void st_128(void *p, const uint32_t *w)
{
    asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                 : "memory");
}
__device__ __forceinline__ void st_64(void *p, const uint32_t *w)
{
    asm volatile("st.global.v2.b32 [%0], {%1,%2};" ::"l"(p), "r"(w[0]), "r"(w[1]) : "memory");
}

// NW 32-bit words from an address aligned to 32 bytes when NW % 8 == 0, else to 16 bytes.
template <int NW>
__device__ __forceinline__ void load_words(uint32_t (&w)[NW], const void *p)
{
    static_assert(NW % 4 == 0, "a lane's slice is a multiple of 16 bytes");
    if constexpr (NW % 8 == 0) {
#pragma unroll
        for (int i = 0; i < NW / 8; ++i) ld_nc_256(&w[8 * i], static_cast<const char *>(p) + 32 * i);
    } else {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i) ld_nc_128(&w[4 * i], static_cast<const char *>(p) + 16 * i);
    }
}

// NW words to an address whose alignment is the largest of 32/16/8 bytes dividing 4*NW.
template <int NW>
__device__ __forceinline__ void store_words(void *p, const uint32_t (&w)[NW])
{
    static_assert(NW % 2 == 0, "stores are at least 8 bytes wide");
    if constexpr (NW % 8 == 0) {
#pragma unroll
        for (int i = 0; i < NW / 8; ++i) st_256(static_cast<char *>(p) + 32 * i, &w[8 * i]);
    } else if constexpr (NW % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i) st_128(static_cast<char *>(p) + 16 * i, &w[4 * i]);
    } else {
#pragma unroll
        for (int i = 0; i < NW / 2; ++i) st_64(static_cast<char *>(p) + 8 * i, &w[2 * i]);
    }
}

// row pointer + unsigned byte offset (one widening multiply-add instead of a 64-bit add with carry)
template <typename T>
__device__ __forceinline__ const T *tap_ptr(const T *row, uint32_t byte_off)
{
    return reinterpret_cast<const T *>(reinterpret_cast<const char *>(row) + byte_off);
}

// float32 accumulator += float16 addend in one instruction (PTX ISA 8.6, sm_100+)
__device__ __forceinline__ float add_f32_f16(float acc, unsigned short h)
{
    asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(acc) : "h"(h));
    return acc;
}

__device__ __forceinline__ float add_f32_bf16(float acc, unsigned short h)
{
    asm("add.rn.f32.bf16 %0, %1, %0;" : "+f"(acc) : "h"(h));
    return acc;
}

// packed float32 arithmetic of sm_100: two lanes of a 64-bit register per instruction
__device__ __forceinline__ void fma_f32x2(float &d0, float &d1, float a, float b0, float b1)
{
    asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
        "mov.b64 ra, {%2, %2};\n\t"
        "mov.b64 rb, {%3, %4};\n\t"
        "mov.b64 rc, {%0, %1};\n\t"
        "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "+f"(d0), "+f"(d1)
        : "f"(a), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void sub_f32x2(float &d0, float &d1, float a0, float a1, float b0, float b1)
{
    asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "sub.rn.f32x2 rc, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// ------------------------------------------------------------------ per-dtype arithmetic

template <typename T>
struct DT;

template <>
struct DT<float> {
    static constexpr int kWordsPerChunk = 8;   // 8 channels * 4 bytes
    static constexpr int kElemsPerWord = 1;
    static constexpr bool kHalfPipe = false;
    static __device__ __forceinline__ float rnd(float x) { return x; }
    static __device__ __forceinline__ void load_xy(const void *p, float &x, float &y)
    {
        const float2 t = __ldg(static_cast<const float2 *>(p));
        x = t.x;
        y = t.y;
    }
    // acc += |q - k| over the elements of one word
    static __device__ __forceinline__ void absdiff(float &a0, float &, uint32_t qw, uint32_t kw)
    {
        a0 += fabsf(__uint_as_float(qw) - __uint_as_float(kw));
    }
    using Bcast = float;
    static __device__ __forceinline__ Bcast bcast(float a) { return a; }
    // o += a * v over the elements of one word (o points at this word's accumulators)
    static __device__ __forceinline__ void wmul(Bcast a, uint32_t vw, float *o) { o[0] = fmaf(a, __uint_as_float(vw), o[0]); }
    static __device__ __forceinline__ uint32_t pack(const float *o) { return __float_as_uint(o[0]); }
    static __device__ __forceinline__ float unpack(uint32_t w, int) { return __uint_as_float(w); }
    // word of packed outputs times word of the gate, rounded to T
    static __device__ __forceinline__ uint32_t gate_mul(uint32_t o, uint32_t gw) { return __float_as_uint(__fmul_rn(__uint_as_float(o), __uint_as_float(gw))); }
    // attention weights live in 32-bit words holding kElemsPerWord of them ("lo" element first)
    static __device__ __forceinline__ uint32_t aw_from(float lo, float) { return __float_as_uint(lo); }
    static __device__ __forceinline__ uint32_t aw_bcast(float w) { return __float_as_uint(w); }
    static __device__ __forceinline__ uint32_t aw_mul(uint32_t x, uint32_t y) { return __float_as_uint(__fmul_rn(__uint_as_float(x), __uint_as_float(y))); }
    static __device__ __forceinline__ uint32_t aw_add(uint32_t x, uint32_t y) { return __float_as_uint(__fadd_rn(__uint_as_float(x), __uint_as_float(y))); }
    static __device__ __forceinline__ Bcast aw_tap(const uint32_t *aw, int m) { return __uint_as_float(aw[m]); }
};

template <>
struct DT<__half> {
    static constexpr int kWordsPerChunk = 4;   // 8 channels * 2 bytes
    static constexpr int kElemsPerWord = 2;
    static constexpr bool kHalfPipe = true;    // 16-bit arithmetic needs few enough registers for 3 blocks per SM
    static __device__ __forceinline__ float rnd(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ void load_xy(const void *p, float &x, float &y)
    {
        const uint32_t u = __ldg(static_cast<const uint32_t *>(p));
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u));
        x = f.x;
        y = f.y;
    }
    static __device__ __forceinline__ void absdiff(float &a0, float &a1, uint32_t qw, uint32_t kw)
    {
        // the difference is rounded to float16 (as the reference does); its magnitude is added to the
        // float32 sums with the mixed-precision add (two chains, even and odd channels)
        const __half2 d = __habs2(__hsub2(*reinterpret_cast<const __half2 *>(&qw), *reinterpret_cast<const __half2 *>(&kw)));
        a0 = add_f32_f16(a0, __half_as_ushort(__low2half(d)));
        a1 = add_f32_f16(a1, __half_as_ushort(__high2half(d)));
    }
    using Bcast = __half2;
    static __device__ __forceinline__ Bcast bcast(__half a) { return __half2half2(a); }
    static __device__ __forceinline__ void wmul(Bcast a, uint32_t vw, float *o)
    {
        // product rounded to float16, then added to the float32 sum by the mixed-precision add of sm_100
        const __half2 pr = __hmul2_rn(a, *reinterpret_cast<const __half2 *>(&vw));
        const uint32_t u = *reinterpret_cast<const uint32_t *>(&pr);
        o[0] = add_f32_f16(o[0], static_cast<unsigned short>(u & 0xffffu));
        o[1] = add_f32_f16(o[1], static_cast<unsigned short>(u >> 16));
    }
    static __device__ __forceinline__ uint32_t pack(const float *o)
    {
        const __half2 t = __floats2half2_rn(o[0], o[1]);
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ float unpack(uint32_t w, int hi)
    {
        const __half2 t = *reinterpret_cast<const __half2 *>(&w);
        return hi ? __high2float(t) : __low2float(t);
    }
    static __device__ __forceinline__ uint32_t gate_mul(uint32_t o, uint32_t gw)
    {
        const __half2 t = __hmul2_rn(*reinterpret_cast<const __half2 *>(&o), *reinterpret_cast<const __half2 *>(&gw));
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ uint32_t aw_from(float lo, float hi)
    {
        const __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ uint32_t aw_bcast(float w) { return aw_from(w, w); }
    // the _rn forms are never contracted into a fused multiply-add: the product must round on its own
    static __device__ __forceinline__ uint32_t aw_mul(uint32_t x, uint32_t y)
    {
        const __half2 t = __hmul2_rn(*reinterpret_cast<const __half2 *>(&x), *reinterpret_cast<const __half2 *>(&y));
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ uint32_t aw_add(uint32_t x, uint32_t y)
    {
        const __half2 t = __hadd2_rn(*reinterpret_cast<const __half2 *>(&x), *reinterpret_cast<const __half2 *>(&y));
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ Bcast aw_tap(const uint32_t *aw, int m)
    {
        const uint32_t u = (m & 1) ? __byte_perm(aw[m >> 1], 0, 0x3232) : __byte_perm(aw[m >> 1], 0, 0x1010);
        return *reinterpret_cast<const __half2 *>(&u);
    }
};

template <>
struct DT<__nv_bfloat16> {
    static constexpr int kWordsPerChunk = 4;
    static constexpr int kElemsPerWord = 2;
    static constexpr bool kHalfPipe = true;
    static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ void load_xy(const void *p, float &x, float &y)
    {
        const uint32_t u = __ldg(static_cast<const uint32_t *>(p));
        x = __uint_as_float(u << 16);
        y = __uint_as_float(u & 0xffff0000u);
    }
    static __device__ __forceinline__ void absdiff(float &a0, float &a1, uint32_t qw, uint32_t kw)
    {
        const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&qw),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&kw));
        const uint32_t u = *reinterpret_cast<const uint32_t *>(&d) & 0x7fff7fffu;
        a0 = add_f32_bf16(a0, static_cast<unsigned short>(u & 0xffffu));
        a1 = add_f32_bf16(a1, static_cast<unsigned short>(u >> 16));
    }
    using Bcast = __nv_bfloat162;
    static __device__ __forceinline__ Bcast bcast(__nv_bfloat16 a) { return __bfloat162bfloat162(a); }
    static __device__ __forceinline__ void wmul(Bcast a, uint32_t vw, float *o)
    {
        const __nv_bfloat162 t = __hmul2_rn(a, *reinterpret_cast<const __nv_bfloat162 *>(&vw));
        const uint32_t u = *reinterpret_cast<const uint32_t *>(&t);
        o[0] = add_f32_bf16(o[0], static_cast<unsigned short>(u & 0xffffu));
        o[1] = add_f32_bf16(o[1], static_cast<unsigned short>(u >> 16));
    }
    static __device__ __forceinline__ uint32_t pack(const float *o)
    {
        const __nv_bfloat162 t = __floats2bfloat162_rn(o[0], o[1]);
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ float unpack(uint32_t w, int hi)
    {
        return __uint_as_float(hi ? (w & 0xffff0000u) : (w << 16));
    }
    static __device__ __forceinline__ uint32_t gate_mul(uint32_t o, uint32_t gw)
    {
        const __nv_bfloat162 t = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162 *>(&o),
                                            *reinterpret_cast<const __nv_bfloat162 *>(&gw));
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ uint32_t aw_from(float lo, float hi)
    {
        const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ uint32_t aw_bcast(float w) { return aw_from(w, w); }
    static __device__ __forceinline__ uint32_t aw_mul(uint32_t x, uint32_t y)
    {
        const __nv_bfloat162 t = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162 *>(&x),
                                            *reinterpret_cast<const __nv_bfloat162 *>(&y));
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ uint32_t aw_add(uint32_t x, uint32_t y)
    {
        const __nv_bfloat162 t = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162 *>(&x),
                                            *reinterpret_cast<const __nv_bfloat162 *>(&y));
        return *reinterpret_cast<const uint32_t *>(&t);
    }
    static __device__ __forceinline__ Bcast aw_tap(const uint32_t *aw, int m)
    {
        const uint32_t u = (m & 1) ? __byte_perm(aw[m >> 1], 0, 0x3232) : __byte_perm(aw[m >> 1], 0, 0x1010);
        return *reinterpret_cast<const __nv_bfloat162 *>(&u);
    }
};

// ------------------------------------------------------------------ shared pieces

// exp for the softmax.  expf() (2 ulp) is what eager PyTorch uses on the GPU; the
// fast intrinsic is 2 + |1.2 x| ulp, which after rounding to 16 bits flips the
// last bit of several per cent of the attention weights.
#ifndef MATCHATTN_FAST_EXP
#define MATCHATTN_FAST_EXP 0
#endif
__device__ __forceinline__ float softmax_exp(float x)
{
#if MATCHATTN_FAST_EXP
    return __expf(x);
#else
    return expf(x);
#endif
}
// Correctly rounded 1/x: the quotient e/den then matches the reference's division to the last
// float32 bit or one off.  (The one-ulp approximate reciprocal was measured to flip enough 16-bit
// roundings of dominant weights to push single outputs past the tolerance.)
__device__ __forceinline__ float softmax_rcp(float x) { return __frcp_rn(x); }

// Window origin: floor of the centre, limited to the range in which the
// replicate clamp of the taps cannot tell the difference (keeps the int
// conversion defined for huge or NaN centres; NaN still poisons the weights).
__device__ __forceinline__ int window_origin(float fl, int r, int extent)
{
    return static_cast<int>(fminf(fmaxf(fl, static_cast<float>(-(r + 2))), static_cast<float>(extent + r + 1)));
}

// Bilinear weights nw, ne, sw, se, each rounded to T where the reference rounds.
template <typename T>
__device__ __forceinline__ void bilinear_weights(float x, float xf, float y, float yf, float (&w)[4])
{
    const float dx = DT<T>::rnd(x - xf), dy = DT<T>::rnd(y - yf);
    const float ex = DT<T>::rnd(1.f - dx), ey = DT<T>::rnd(1.f - dy);
    w[0] = DT<T>::rnd(ex * ey);
    w[1] = DT<T>::rnd(dx * ey);
    w[2] = DT<T>::rnd(ex * dy);
    w[3] = DT<T>::rnd(dx * dy);
}

// Raw L1 sums -> scaled scores, with the reference's roundings.
template <typename T>
__device__ __forceinline__ float finish_score(float l1, float scale)
{
    return DT<T>::rnd(DT<T>::rnd(-l1) * scale);
}

// BilinearSoftmax over a (2R+2)^2 score window held in registers: four shifted
// (2R+1)^2 sub-windows, a softmax in each, blended by the bilinear weights in
// the order nw, ne, sw, se with a rounding to T after every step.
//
// softmax(x)_m = exp(x_m - c) / sum exp(x - c) for any c, so the exponentials
// are taken once per tap around the maximum of the whole window and shared by
// the four sub-windows (their sums are built from shared row and column
// partial sums).  If a sub-window's own maximum lies so far below the global
// one that its exponentials could underflow, every sub-window is evaluated
// around its own maximum instead.  Everything is unrolled with constant
// indices so that the arrays stay in registers.
//
// The result is written as 32-bit words `aw` holding kElemsPerWord consecutive
// taps each, which is the layout of attn_out; in the 16-bit types the rounding
// chain p -> w*p -> a + w*p runs on such pairs (a column that a sub-window does
// not cover contributes w * 0 = +0, which leaves the sum unchanged).
template <typename T, int R, typename ExpMinus>
__device__ __forceinline__ void blend_subwindow(uint32_t (&aw)[(2 * R + 2) * (2 * R + 2) / DT<T>::kElemsPerWord],
                                                const int t, const float wt, const float inv, ExpMinus e_of)
{
    constexpr int SIDE = 2 * R + 2, SUB = 2 * R + 1, EPW = DT<T>::kElemsPerWord;
    const int oy = t >> 1, ox = t & 1;
    const uint32_t wt_w = DT<T>::aw_bcast(wt);
#pragma unroll
    for (int j = 0; j < SUB; ++j)
#pragma unroll
        for (int iw = 0; iw < SIDE / EPW; ++iw) {
            const int i0 = iw * EPW, i1 = i0 + EPW - 1;          // columns of this word
            const bool in0 = i0 >= ox && i0 < ox + SUB, in1 = i1 >= ox && i1 < ox + SUB;
            if (!in0 && !in1) continue;
            const int m0 = (j + oy) * SIDE + i0;
            const float p0 = in0 ? e_of(m0) * inv : 0.f;
            const float p1 = (EPW == 2 && in1) ? e_of(m0 + 1) * inv : 0.f;
            uint32_t &dst = aw[m0 / EPW];
            dst = DT<T>::aw_add(dst, DT<T>::aw_mul(wt_w, DT<T>::aw_from(p0, p1)));
        }
}

template <typename T, int R>
__device__ __forceinline__ void bilinear_softmax(const float (&s)[(2 * R + 2) * (2 * R + 2)], const float (&w)[4],
                                                 uint32_t (&aw)[(2 * R + 2) * (2 * R + 2) / DT<T>::kElemsPerWord])
{
    constexpr int SIDE = 2 * R + 2, SUB = 2 * R + 1, M = SIDE * SIDE, EPW = DT<T>::kElemsPerWord;
    static_assert(SIDE % EPW == 0, "a word never straddles two window rows");
#pragma unroll
    for (int m = 0; m < M / EPW; ++m) aw[m] = 0u;

    // sub-window maxima from shared column / row partial maxima
    float sub_max[4];
    {
        float top[SIDE], bot[SIDE];
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            float mid = s[SIDE + i];
#pragma unroll
            for (int j = 2; j < SUB; ++j) mid = fmaxf(mid, s[j * SIDE + i]);
            top[i] = fmaxf(s[i], mid);
            bot[i] = fmaxf(mid, s[(SIDE - 1) * SIDE + i]);
        }
        float mt = top[1], mb = bot[1];
#pragma unroll
        for (int i = 2; i < SUB; ++i) {
            mt = fmaxf(mt, top[i]);
            mb = fmaxf(mb, bot[i]);
        }
        sub_max[0] = fmaxf(top[0], mt);
        sub_max[1] = fmaxf(mt, top[SIDE - 1]);
        sub_max[2] = fmaxf(bot[0], mb);
        sub_max[3] = fmaxf(mb, bot[SIDE - 1]);
    }
    const float gmax = fmaxf(fmaxf(sub_max[0], sub_max[1]), fmaxf(sub_max[2], sub_max[3]));
    const float gmin = fminf(fminf(sub_max[0], sub_max[1]), fminf(sub_max[2], sub_max[3]));

    if (gmax - gmin < 60.f) {
        float e[M];
#pragma unroll
        for (int m = 0; m < M; ++m) e[m] = softmax_exp(s[m] - gmax);
        float top[SIDE], bot[SIDE];
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            float mid = e[SIDE + i];
#pragma unroll
            for (int j = 2; j < SUB; ++j) mid += e[j * SIDE + i];
            top[i] = e[i] + mid;
            bot[i] = mid + e[(SIDE - 1) * SIDE + i];
        }
        float mt = top[1], mb = bot[1];
#pragma unroll
        for (int i = 2; i < SUB; ++i) {
            mt += top[i];
            mb += bot[i];
        }
        const float den[4] = {top[0] + mt, mt + top[SIDE - 1], bot[0] + mb, mb + bot[SIDE - 1]};
#pragma unroll
        for (int t = 0; t < 4; ++t)
            blend_subwindow<T, R>(aw, t, w[t], softmax_rcp(den[t]), [&](int m) { return e[m]; });
    } else {   // rare: widely spread scores, or a NaN score
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int oy = t >> 1, ox = t & 1;
            const float mx = sub_max[t];
            float den = 0.f;
#pragma unroll
            for (int j = 0; j < SUB; ++j)
#pragma unroll
                for (int i = 0; i < SUB; ++i) den += softmax_exp(s[(j + oy) * SIDE + i + ox] - mx);
            blend_subwindow<T, R>(aw, t, w[t], softmax_rcp(den), [&](int m) { return softmax_exp(s[m] - mx); });
        }
    }
}

// ------------------------------------------------------------------ the specialised kernel

// resident blocks per SM the register allocation is held to (more warps hide the gather latency)
template <typename T, int R, int CPL>
constexpr int min_blocks()
{
    // r = 2 holds a 36-tap window per lane: one block per SM without a register limit, two (128
    // registers, a few spilled words) for the 16-bit types up to four chunks per lane
    if (R != 1) return (DT<T>::kHalfPipe && CPL <= 4) ? 2 : 1;
    return (DT<T>::kHalfPipe && CPL <= 2) ? 3 : 2;
}

// EXTRAS selects the build of the kernel that also honours the rarely used Params fields (sorted
// query order, guard, clamp, gate, strided outputs); the plain build ignores them and keeps the
// hot path free of their branches and registers.
// POW2: the host found `scale` to be a power of two that the 16-bit type T represents exactly.
template <typename T, int R, int CPL, bool MULTI, bool EXTRAS, bool POW2 = false>
__global__ void __launch_bounds__(kThreads, min_blocks<T, R, CPL>()) fused_forward_kernel(const Params p)
{
    constexpr int SIDE = 2 * R + 2, M = SIDE * SIDE;
    constexpr int NW = CPL * DT<T>::kWordsPerChunk;        // 32-bit words of K (or V, q, out) per lane and tap
    constexpr int EPW = DT<T>::kElemsPerWord;
    constexpr int SLICE = CPL * 8;                          // channels per lane

    if constexpr (EXTRAS) {
        if (p.guard != nullptr && ((*p.guard != 0u) != (p.guard_run_if != 0))) return;
    }

    // lane -> (query of the tile, head, slice of the head)
    const int tid = threadIdx.x;
    const int lq = tid / p.G;
    const int g = tid - lq * p.G;
    int head, sl;
    if constexpr (MULTI) {
        head = g >> p.lph_shift;
        sl = g & (p.lph - 1);
    } else {
        head = g;
        sl = 0;
    }
    bool valid;
    int b;
    int64_t bq;
    if (EXTRAS && p.sorted != nullptr) {
        // queries in the order of the sorted list: neighbours in the list look at the same tile of
        // the map, so their taps hit in L1
        const int qpb = p.tile_w * p.tile_h;
        const int64_t total = static_cast<int64_t>(p.B) * p.Nq;
        const int64_t qs = static_cast<int64_t>(blockIdx.x) * qpb + lq;
        valid = lq < qpb && qs < total;
        if constexpr (!MULTI) {
            if (!valid) return;
        }
        bq = p.sorted[min(qs, total - 1)].x;
        b = static_cast<int>(bq / p.Nq);
    } else {
        const int tile_y = blockIdx.x / p.tiles_x;
        const int tile_x = blockIdx.x - tile_y * p.tiles_x;
        int qx = tile_x * p.tile_w + (lq & (p.tile_w - 1));
        int qy = tile_y * p.tile_h + (lq >> p.tile_w_shift);
        valid = (lq >> p.tile_w_shift) < p.tile_h && qx < p.W && qy < p.rows;
        if constexpr (!MULTI) {
            if (!valid) return;
        } else {
            // lanes without a query stay for the shuffles and redo a neighbour's work
            qx = min(qx, p.W - 1);
            qy = min(qy, p.rows - 1);
        }
        b = blockIdx.y;
        bq = static_cast<int64_t>(b) * p.Nq + qy * p.W + qx;
    }

    // sampling centre -> origin, weights, clamped tap rows / columns (in elements)
    float x, y;
    DT<T>::load_xy(static_cast<const T *>(p.mo) + (bq * p.h + head) * 2, x, y);
    if (EXTRAS && p.clamp) {
        x = clamp_keep_nan(x, p.clamp_lo, p.clamp_hi_x);
        y = clamp_keep_nan(y, p.clamp_lo, p.clamp_hi_y);
    }
    const float xf = floorf(x), yf = floorf(y);
    float wgt[4];
    bilinear_weights<T>(x, xf, y, yf, wgt);
    const int x0 = window_origin(xf, R, p.W) - R, y0 = window_origin(yf, R, p.H) - R;
    // a tap's address is its row's pointer plus an unsigned 32-bit byte offset of its column
    uint32_t col[SIDE];
    int row[SIDE];
#pragma unroll
    for (int i = 0; i < SIDE; ++i) {
        col[i] = static_cast<uint32_t>(min(max(x0 + i, 0), p.W - 1) * p.C) * static_cast<uint32_t>(sizeof(T));
        row[i] = min(max(y0 + i, 0), p.H - 1) * p.W * p.C;
    }

    const int lane_off = head * p.hd + sl * SLICE;
    // the cross branch reads the other view's keys / values: the caller's batch roll folded into the index
    const int b_kv = (EXTRAS && p.kv_shift != 0) ? (b + p.kv_shift >= p.B ? b + p.kv_shift - p.B : b + p.kv_shift) : b;
    const int64_t kv_base = static_cast<int64_t>(b_kv) * p.N * p.C + lane_off;
    const T *kb = static_cast<const T *>(p.k) + kv_base;
    const T *vb = static_cast<const T *>(p.v) + kv_base;

    if (EXTRAS && p.debug != nullptr) {
        // checked entry point: every index this lane is about to use, against the extent of its array
        const int64_t item_elems = static_cast<int64_t>(p.N) * p.C;
#pragma unroll
        for (int j = 0; j < SIDE; ++j)
#pragma unroll
            for (int i = 0; i < SIDE; ++i) {
                const int64_t first = static_cast<int64_t>(row[j]) + col[i] / static_cast<uint32_t>(sizeof(T)) + lane_off;
                if (row[j] < 0 || first < 0 || first + SLICE > item_elems) debug_record(p.debug, 1u);
            }
        if (bq < 0 || bq >= static_cast<int64_t>(p.B) * p.Nq || lane_off + SLICE > p.C || b < 0 || b >= p.B)
            debug_record(p.debug, 2u);
    }

    uint32_t qw[NW];
    load_words<NW>(qw, static_cast<const T *>(p.q) + bq * p.C + lane_off);

    // scores.  With a power-of-two scale that T holds exactly (POW2), round16(h * scale) is an exact
    // 16-bit product: two neighbouring taps share one packed negate-and-round and one packed multiply,
    // and the finished scores stay packed (eight registers instead of sixteen) until the softmax, which
    // leaves room for one more tap load in flight.  The roundings are the reference's either way.
    float s[M];
    uint32_t sp[POW2 ? M / 2 : 1];
    float part_even = 0.f;
#pragma unroll
    for (int j = 0; j < SIDE; ++j)
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            uint32_t kw[NW];
            load_words<NW>(kw, tap_ptr(kb + row[j], col[i]));
            float a0 = 0.f, a1 = 0.f;
            if constexpr (EPW == 1) {
                // float32: two channels per packed subtract (same roundings as the scalar form)
#pragma unroll
                for (int w = 0; w < NW; w += 2) {
                    float d0, d1;
                    sub_f32x2(d0, d1, __uint_as_float(qw[w]), __uint_as_float(qw[w + 1]), __uint_as_float(kw[w]),
                              __uint_as_float(kw[w + 1]));
                    a0 += fabsf(d0);
                    a1 += fabsf(d1);
                }
            } else {
#pragma unroll
                for (int w = 0; w < NW; ++w) DT<T>::absdiff(a0, a1, qw[w], kw[w]);
            }
            float part = a0 + a1;
            if constexpr (MULTI) {
                for (int o = p.lph >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            }
            if constexpr (POW2) {
                if (i & 1) sp[(j * SIDE + i) >> 1] = DT<T>::aw_mul(DT<T>::aw_from(-part_even, -part), DT<T>::aw_bcast(p.scale));
                else part_even = part;
            } else {
                s[j * SIDE + i] = finish_score<T>(part, p.scale);
            }
        }
    if constexpr (POW2) {
#pragma unroll
        for (int m = 0; m < M; m += 2) {
            s[m] = DT<T>::unpack(sp[m >> 1], 0);
            s[m + 1] = DT<T>::unpack(sp[m >> 1], 1);
        }
    }

    // the first value taps are requested before the softmax so that their latency overlaps it
    // (two taps: measured best, more of them spill)
    constexpr int VPF = (R == 1 && CPL <= 2) ? 2 : 0;
    uint32_t vpre[VPF > 0 ? VPF : 1][NW];
#pragma unroll
    for (int t = 0; t < VPF; ++t) load_words<NW>(vpre[t], tap_ptr(vb + row[t / SIDE], col[t % SIDE]));

    constexpr int NWA = M / EPW;
    uint32_t aw[NWA];
    bilinear_softmax<T, R>(s, wgt, aw);

    if (p.attn != nullptr && sl == 0 && valid)
        store_words<NWA>(static_cast<T *>(p.attn) + (EXTRAS ? bq * p.attn_stride + head * M : (bq * p.h + head) * M), aw);

    // weighted sum of the value taps
    float o[NW * EPW];
#pragma unroll
    for (int c = 0; c < NW * EPW; ++c) o[c] = 0.f;
#pragma unroll
    for (int j = 0; j < SIDE; ++j)
#pragma unroll
        for (int i = 0; i < SIDE; ++i) {
            uint32_t vw[NW];
            if (j * SIDE + i < VPF) {
#pragma unroll
                for (int w = 0; w < NW; ++w) vw[w] = vpre[j * SIDE + i][w];
            } else {
                load_words<NW>(vw, tap_ptr(vb + row[j], col[i]));
            }
            const typename DT<T>::Bcast am = DT<T>::aw_tap(aw, j * SIDE + i);
            if constexpr (EPW == 1) {
                // float32: two channels per packed fused multiply-add
#pragma unroll
                for (int w = 0; w < NW; w += 2)
                    fma_f32x2(o[w], o[w + 1], __uint_as_float(aw[j * SIDE + i]), __uint_as_float(vw[w]), __uint_as_float(vw[w + 1]));
                (void)am;
            } else {
#pragma unroll
                for (int w = 0; w < NW; ++w) DT<T>::wmul(am, vw[w], &o[w * EPW]);
            }
        }

    if (valid) {
        uint32_t ow[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) ow[w] = DT<T>::pack(&o[w * EPW]);
        if (EXTRAS && p.gate != nullptr) {
            uint32_t gw[NW];
            load_words<NW>(gw, static_cast<const T *>(p.gate) + bq * p.C + lane_off);
#pragma unroll
            for (int w = 0; w < NW; ++w) ow[w] = DT<T>::gate_mul(ow[w], gw[w]);
        }
        store_words<NW>(static_cast<T *>(p.out) + bq * (EXTRAS ? p.out_stride : p.C) + lane_off, ow);
    }
}

// ------------------------------------------------------------------ the any-shape kernel
//
// One thread per (query, head); scalar loads; any head width, any radius up to
// kMaxR, pointers aligned to the element size only.  Slow: the fallback for
// shapes the specialised kernel does not cover.

constexpr int kMaxR = 4;
constexpr int kMaxTaps = (2 * kMaxR + 2) * (2 * kMaxR + 2);

template <typename T>
__device__ __forceinline__ float load_one(const T *p);
template <>
__device__ __forceinline__ float load_one<float>(const float *p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_one<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <>
__device__ __forceinline__ float load_one<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(__ldg(p)); }

template <typename T>
__device__ __forceinline__ void store_one(T *p, float x);
template <>
__device__ __forceinline__ void store_one<float>(float *p, float x) { *p = x; }
template <>
__device__ __forceinline__ void store_one<__half>(__half *p, float x) { *p = __float2half_rn(x); }
template <>
__device__ __forceinline__ void store_one<__nv_bfloat16>(__nv_bfloat16 *p, float x) { *p = __float2bfloat16_rn(x); }

template <typename T>
__global__ void __launch_bounds__(kThreads) generic_forward_kernel(const Params p)
{
    if (p.guard != nullptr && ((*p.guard != 0u) != (p.guard_run_if != 0))) return;
    const int64_t per_item = static_cast<int64_t>(p.Nq) * p.h;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (t >= per_item) return;
    const int b = blockIdx.y;
    const int head = static_cast<int>(t % p.h);
    const int64_t bq = static_cast<int64_t>(b) * p.Nq + t / p.h;
    const int r = p.r, side = 2 * r + 2, sub = 2 * r + 1, M = side * side;

    const T *mo = static_cast<const T *>(p.mo) + (bq * p.h + head) * 2;
    float x = load_one<T>(mo), y = load_one<T>(mo + 1);
    if (p.clamp) {
        x = clamp_keep_nan(x, p.clamp_lo, p.clamp_hi_x);
        y = clamp_keep_nan(y, p.clamp_lo, p.clamp_hi_y);
    }
    const float xf = floorf(x), yf = floorf(y);
    float wgt[4];
    bilinear_weights<T>(x, xf, y, yf, wgt);
    const int x0 = window_origin(xf, r, p.W) - r, y0 = window_origin(yf, r, p.H) - r;

    const T *qp = static_cast<const T *>(p.q) + bq * p.C + head * p.hd;
    const int b_kv = b + p.kv_shift >= p.B ? b + p.kv_shift - p.B : b + p.kv_shift;
    const int64_t kv_base = static_cast<int64_t>(b_kv) * p.N * p.C + head * p.hd;
    const T *kb = static_cast<const T *>(p.k) + kv_base;
    const T *vb = static_cast<const T *>(p.v) + kv_base;

    float s[kMaxTaps], a[kMaxTaps];
    for (int j = 0; j < side; ++j) {
        const int ty = min(max(y0 + j, 0), p.H - 1);
        for (int i = 0; i < side; ++i) {
            const int tx = min(max(x0 + i, 0), p.W - 1);
            if (p.debug != nullptr && (ty < 0 || ty >= p.H || tx < 0 || tx >= p.W)) debug_record(p.debug, 1u);
            const T *kp = kb + static_cast<int64_t>(ty * p.W + tx) * p.C;
            float acc = 0.f;
            if (p.dot) {     // products rounded to T, summed in float32; finish_score negates its argument
                for (int c = 0; c < p.hd; ++c) acc -= DT<T>::rnd(__fmul_rn(load_one<T>(qp + c), load_one<T>(kp + c)));
            } else {
                for (int c = 0; c < p.hd; ++c) acc += fabsf(DT<T>::rnd(load_one<T>(qp + c) - load_one<T>(kp + c)));
            }
            s[j * side + i] = finish_score<T>(acc, p.scale);
            a[j * side + i] = 0.f;
        }
    }
    for (int tq = 0; tq < 4; ++tq) {
        const int oy = tq >> 1, ox = tq & 1;
        float mx = s[oy * side + ox];
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) mx = fmaxf(mx, s[(j + oy) * side + i + ox]);
        float den = 0.f;
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) den += __expf(s[(j + oy) * side + i + ox] - mx);
        const float inv = __frcp_rn(den);
        for (int j = 0; j < sub; ++j)
            for (int i = 0; i < sub; ++i) {
                const int m = (j + oy) * side + i + ox;
                const float pr = DT<T>::rnd(__expf(s[m] - mx) * inv);
                a[m] = DT<T>::rnd(a[m] + DT<T>::rnd(wgt[tq] * pr));
            }
    }
    if (p.attn != nullptr) {
        T *ap = static_cast<T *>(p.attn) + bq * p.attn_stride + head * M;
        for (int m = 0; m < M; ++m) store_one<T>(ap + m, a[m]);
    }
    T *op = static_cast<T *>(p.out) + bq * p.out_stride + head * p.hd;
    const T *gp = p.gate != nullptr ? static_cast<const T *>(p.gate) + bq * p.C + head * p.hd : nullptr;
    for (int c = 0; c < p.hd; ++c) {
        float acc = 0.f;
        for (int j = 0; j < side; ++j) {
            const int ty = min(max(y0 + j, 0), p.H - 1);
            for (int i = 0; i < side; ++i) {
                const int tx = min(max(x0 + i, 0), p.W - 1);
                const float vv = load_one<T>(vb + static_cast<int64_t>(ty * p.W + tx) * p.C + c);
                if (sizeof(T) == 4) acc = fmaf(a[j * side + i], vv, acc);
                else acc += DT<T>::rnd(a[j * side + i] * vv);
            }
        }
        if (gp != nullptr) acc = DT<T>::rnd(acc) * load_one<T>(gp + c);
        store_one<T>(op + c, acc);
    }
}

// Launchers, one translation unit per element type.
template <typename T>
cudaError_t launch_fast(const Params &p, int r, int cpl, bool multi, dim3 grid, int threads, cudaStream_t stream);
template <typename T>
cudaError_t launch_generic(const Params &p, dim3 grid, cudaStream_t stream);

}  // namespace matchattn
