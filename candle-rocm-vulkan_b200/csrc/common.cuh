// Shared device helpers of libb200attn: bit-exact element codecs, PTX wrappers (mbarrier, bulk
// copies, mma.sync, packed conversions) and the host-side error plumbing. sm_100a only.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200attn.h"

namespace b200 {

// ---------------------------------------------------------------------------------------------
// host: error reporting
// ---------------------------------------------------------------------------------------------
int set_error(int code, const char *fmt, ...);
int check_launch(const char *what);

// Diagnostic switches select between code paths that give the same results, so that each can be tested and timed
// alone. They exist only in builds with -DB200_DIAG (read from the environment, once per process); the library
// proper reads no environment variable.
#ifdef B200_DIAG
#include <cstdlib>
inline const char *diag_env(const char *name) { return getenv(name); }
#else
inline const char *diag_env(const char *) { return nullptr; }
#endif

// ---------------------------------------------------------------------------------------------
// bit casts
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ float u2f(uint32_t u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}
__host__ __device__ __forceinline__ uint32_t f2u(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

// ---------------------------------------------------------------------------------------------
// Element codecs, bit-exact with candle-core/kernels/accel_common.h:131-236 (same integer
// algorithm; divisions and roundings are IEEE, the library is built without fast-math).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float e4m3_to_f(uint32_t c) {
    const uint32_t mag = c & 0x7fu;
    const float nrm = u2f((mag << 20) + (120u << 23));
    const float sub = (float)mag * 0.001953125f;
    float v = mag >= 8u ? nrm : sub;
    v = (c & 0x80u) ? -v : v;
    return mag == 0x7fu ? u2f(0x7fc00000u) : v;
}

__device__ __forceinline__ uint32_t f_to_e4m3(float f) {
    const uint32_t x = f2u(f);
    const uint32_t s = (x >> 24) & 0x80u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return s | 0x7fu;
    const float a = u2f(ax);
    if (a >= 448.0f) return s | 0x7eu;
    if (a < 0.015625f) return s | (uint32_t)rintf(a * 512.0f);
    const uint32_t r = ax + 0x7ffffu + ((ax >> 20) & 1u);
    uint32_t code = (((r >> 23) - 120u) << 3) | ((r >> 20) & 7u);
    if (code > 0x7eu) code = 0x7eu;
    return s | code;
}

__device__ __forceinline__ float fp4_to_f(uint32_t c) {
    const uint32_t e = (c >> 1) & 3u, m = c & 1u;
    const float v = e == 0 ? 0.5f * (float)m : u2f(((e + 126u) << 23) | (m << 22));
    return (c & 8u) ? -v : v;
}

__device__ __forceinline__ uint32_t f_to_fp4(float f) {
    const uint32_t s = (f2u(f) >> 28) & 8u;
    const float a = fabsf(f);
    uint32_t c;
    if (!(a > 0.25f)) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return s | c;
}

__device__ __forceinline__ float e8m0_to_f(uint32_t c) { return c == 0 ? u2f(0x00400000u) : u2f(c << 23); }
// 1 / e8m0_to_f(c) = 2^(127 - c), itself a float (2^-127 is a subnormal, 1 / inf is 0): the product x * e8m0_recip(c) and
// the IEEE quotient x / e8m0_to_f(c) round the same real number, so they agree bit for bit, overflow and subnormal
// results included
__device__ __forceinline__ float e8m0_recip(uint32_t c) {
    return c >= 254u ? (c == 254u ? u2f(0x00400000u) : 0.0f) : u2f((254u - c) << 23);
}

__device__ __forceinline__ uint32_t mx_scale_code(float amax, int emax_elem) {
    int e = -127;
    const uint32_t bits = f2u(amax);
    const int be = (int)((bits >> 23) & 0xffu);
    if (amax > 0.0f && be != 0xff && be != 0) e = be - 127 - emax_elem;
    e = max(e, -127);
    e = min(e, 127);
    return (uint32_t)(e + 127);
}

// bf16 / f16 storage <-> f32 (exact widening; RNE narrowing like ax_f2h / ax_f2bf)
__device__ __forceinline__ float bf16_bits_to_f(uint16_t b) { return u2f(((uint32_t)b) << 16); }
__device__ __forceinline__ uint16_t f_to_bf16_bits(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float f16_bits_to_f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }

template <int DT>
__device__ __forceinline__ float load_elem(const void *p, uint64_t i) {
    if (DT == B200_F32) return reinterpret_cast<const float *>(p)[i];
    if (DT == B200_F16) return f16_bits_to_f(reinterpret_cast<const uint16_t *>(p)[i]);
    if (DT == B200_BF16) return bf16_bits_to_f(reinterpret_cast<const uint16_t *>(p)[i]);
    return e4m3_to_f(reinterpret_cast<const uint8_t *>(p)[i]);
}

__device__ __forceinline__ float load_elem_rt(const void *p, uint64_t i, int dt) {
    if (dt == B200_F32) return load_elem<B200_F32>(p, i);
    if (dt == B200_F16) return load_elem<B200_F16>(p, i);
    if (dt == B200_BF16) return load_elem<B200_BF16>(p, i);
    return load_elem<B200_FP8>(p, i);
}

__device__ __forceinline__ void store_elem_rt(void *p, uint64_t i, float v, int dt) {
    if (dt == B200_F32) reinterpret_cast<float *>(p)[i] = v;
    else if (dt == B200_F16) reinterpret_cast<uint16_t *>(p)[i] = f_to_f16_bits(v);
    else reinterpret_cast<uint16_t *>(p)[i] = f_to_bf16_bits(v);
}

__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == B200_F32 ? 4 : (dt == B200_FP8 ? 1 : 2); }

// ---------------------------------------------------------------------------------------------
// packed conversions to f16x2 (sm_100a: cvt.rn.f16x2.{e4m3x2,e2m1x2})
// ---------------------------------------------------------------------------------------------
// two e4m3 bytes (low 16 bits of x) -> f16x2, low byte in the low half
__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint32_t x) {
    uint32_t d;
    asm("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %1;\n cvt.rn.f16x2.e4m3x2 %0, lo;\n}" : "=r"(d) : "r"(x));
    return d;
}
__device__ __forceinline__ uint32_t cvt_e4m3x2_hi_f16x2(uint32_t x) {
    uint32_t d;
    asm("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %1;\n cvt.rn.f16x2.e4m3x2 %0, hi;\n}" : "=r"(d) : "r"(x));
    return d;
}
// the four bytes of x, each two e2m1 nibbles -> four f16x2 (low nibble in the low half)
__device__ __forceinline__ void cvt_e2m1x8_f16x2(uint32_t x, uint32_t &d0, uint32_t &d1, uint32_t &d2, uint32_t &d3) {
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
        : "r"(x));
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B (accumulator starts at zero, no register is cleared for it)
__device__ __forceinline__ void mma_f16_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk copy (TMA, no multicast)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll already blocks for a hardware defined
// time slice) and returns false, so a copy that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = 1u << 22) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

} // namespace b200
