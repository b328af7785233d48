// Row quantizer / dequantizer and the fused quantize-on-append of the compressed KV cache.
//
// One warp owns one row (lane l holds elements l, l + 32, l + 64, ...): the row maximum and the
// per-block maxima are warp shuffles instead of the seven-barrier shared-memory trees of the
// reference's one-workgroup-per-row kernel (candle-core/kernels/turbo_quant_impl.h:71-159), and
// the packed row goes straight to its slot of the capacity buffer. Codes, block scales and rsc0
// are bit-exact with that kernel: maxima do not depend on the reduction order, the sum of
// squares of the codebook formats reproduces the order of its 128-lane tree
// (candle-core/kernels/accel_common.h:255-267), all divisions are IEEE (by a power of two: the
// exact product with its reciprocal).
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace b200 {

constexpr int QW = 4;  // warps (rows in flight) per block

struct QuantSideParams {
    const void *src;
    uint32_t *dst;
    const float *tab;
    const float *signs;
    const int32_t *pos;
    uint64_t s_b, s_h, s_t;  // source strides (elements)
    uint64_t c_b, c_h, c_t;  // destination strides (words)
    int32_t pos0;
    int32_t mode, cb, code_words, aux_words, row_words;
    int32_t rot;
    uint32_t cap;      // rows per (batch entry, head) slab of the destination; 0 = not given, positions are not checked
    int32_t *status;   // set to 3 when a row's position lies outside [0, cap): that row is not written
};

struct QuantParams {
    QuantSideParams side[2];
    uint32_t nb, nh, nt, d;
    int32_t src_dtype;
    uint32_t nt_mul, nt_shr, nh_mul, nh_shr;  // fastdiv invariants of nt and nh (rows128 kernel)
    uint32_t after_prev;  // launched as a programmatic dependent of the stream's previous kernel (B200_KV_AFTER_PREV)
};

// A grid launched while the stream's previous kernel still runs (that kernel neither reads the rows written here nor
// writes this call's inputs) lets its own dependents be scheduled at once, and before it ends waits for that kernel:
// so this grid's completion still implies the completion of everything before it in the stream.
__device__ __forceinline__ void after_prev_begin(const QuantParams &p) {
    if (p.after_prev) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void after_prev_end(const QuantParams &p) {
    if (p.after_prev) asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// EPL: elements per lane (D <= 32 * EPL); DT: source dtype
template <int EPL, int DT>
__global__ void __launch_bounds__(QW * 32) quant_rows_kernel(const QuantParams p) {
    __shared__ __align__(16) uint8_t s_codes[QW][32 * EPL];
    __shared__ uint32_t s_scales[QW][2 * EPL];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const QuantSideParams &sp = p.side[blockIdx.y];
    const uint32_t D = p.d;
    const int nk = (int)((D + 31) / 32);
    const uint64_t rows = (uint64_t)p.nb * p.nh * p.nt;
    uint8_t *codes = s_codes[warp];
    uint32_t *sc = s_scales[warp];
    after_prev_begin(p);

    const bool small = rows < 0x80000000ull;  // 32-bit row arithmetic (the 64-bit divisions cost more than the codecs)
    for (uint64_t row = (uint64_t)blockIdx.x * QW + warp; row < rows; row += (uint64_t)gridDim.x * QW) {
        uint32_t t, h, b;
        if (small) {
            const uint32_t r32 = (uint32_t)row, bh = r32 / p.nt;
            t = r32 - bh * p.nt;
            b = bh / p.nh;
            h = bh - b * p.nh;
        } else {
            t = (uint32_t)(row % p.nt);
            h = (uint32_t)((row / p.nt) % p.nh);
            b = (uint32_t)(row / ((uint64_t)p.nt * p.nh));
        }
        const char *src = reinterpret_cast<const char *>(sp.src) + (b * sp.s_b + h * sp.s_h + t * sp.s_t) * (uint64_t)dtype_size(DT);
        const int64_t pos = (sp.pos ? (int64_t)sp.pos[b] + sp.pos0 : (int64_t)sp.pos0) + (int64_t)t;
        if (pos < 0 || (sp.cap && pos >= (int64_t)sp.cap)) {
            // a stale or corrupt device position: nothing is written outside the slab (the whole warp takes this branch)
            if (lane == 0 && sp.status) atomicExch(sp.status, 3);
            continue;
        }
        uint32_t *orow = sp.dst + b * sp.c_b + h * sp.c_h + (uint64_t)pos * sp.c_t;

        float x[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) {
            const uint32_t j = lane + 32 * k;
            x[k] = (k < nk && j < D) ? load_elem<DT>(src, j) : 0.0f;
        }

        if (sp.rot == B200_ROT_HADAMARD) {
            // y = H diag(sign) x / sqrt(D): signs, Walsh-Hadamard butterflies (element index bits
            // 0-4 across lanes, higher bits across registers), then the scale
#pragma unroll
            for (int k = 0; k < EPL; ++k) {
                const uint32_t j = lane + 32 * k;
                if (k < nk && j < D) x[k] *= sp.signs[j];
            }
            for (uint32_t o = 1; o < 32 && o < D; o <<= 1) {
#pragma unroll
                for (int k = 0; k < EPL; ++k) {
                    const float y = __shfl_xor_sync(0xffffffffu, x[k], o);
                    x[k] = (lane & o) ? y - x[k] : x[k] + y;
                }
            }
#pragma unroll
            for (int o = 1; o < EPL; o <<= 1) {
                if (o < nk) {
#pragma unroll
                    for (int k = 0; k < EPL; ++k) {
                        if (!(k & o)) {
                            const float a = x[k], c = x[k | o];
                            x[k] = a + c;
                            x[k | o] = a - c;
                        }
                    }
                }
            }
            const float s = 1.0f / sqrtf((float)D);
#pragma unroll
            for (int k = 0; k < EPL; ++k) x[k] *= s;
        }

        const uint32_t mode = sp.mode, cb = sp.cb;
        float rsc0 = 1.0f;
        uint32_t c[EPL];
        if (mode <= B200_TURBO_PROD) {
            // sum of squares in the order of the reference's 128 lanes: lane t adds j = t,
            // t + 128, ..., then red[t] += red[t + s] for s = 64 ... 1
            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int k = 0; k < EPL; ++k) part[k & 3] = __fadd_rn(part[k & 3], __fmul_rn(x[k], x[k]));
            float ss = __fadd_rn(__fadd_rn(part[0], part[2]), __fadd_rn(part[1], part[3]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, o));
            ss = __shfl_sync(0xffffffffu, ss, 0);
            const float norm = __fsqrt_rn(ss);
            const float inv = norm > 0.0f ? __fdiv_rn(1.0f, norm) : 0.0f;
            const uint32_t nbnd = (1u << cb) - 1u;
            rsc0 = norm;
#pragma unroll
            for (int k = 0; k < EPL; ++k) {
                const float u = __fmul_rn(x[k], inv);
                uint32_t idx = 0;
                for (uint32_t bi = 0; bi < nbnd; ++bi) idx += u >= __ldg(sp.tab + 16 + bi) ? 1u : 0u;
                c[k] = idx;
            }
        } else if (mode == B200_MXFP4 || mode == B200_MXFP8) {
            const int emax = mode == B200_MXFP4 ? 2 : 8;
#pragma unroll
            for (int k = 0; k < EPL; ++k) {
                const float bm = warp_max(fabsf(x[k]));  // block k = elements [32 k, 32 k + 32)
                const uint32_t code = mx_scale_code(bm, emax);
                const float qv = __fmul_rn(x[k], e8m0_recip(code));  // = x / e8m0_to_f(code), bit for bit
                c[k] = code == 0 ? 0u : (mode == B200_MXFP4 ? f_to_fp4(qv) : f_to_e4m3(qv));
                if (lane == 0 && k < nk) sc[k] = code;
            }
        } else {
            float am = 0.0f;
#pragma unroll
            for (int k = 0; k < EPL; ++k) am = fmaxf(am, fabsf(x[k]));
            am = warp_max(am);
            if (mode == B200_NVFP4) {
                const float g = am > 0.0f ? __fdiv_rn(am, 2688.0f) : 1.0f;
                rsc0 = g;
#pragma unroll
                for (int k = 0; k < EPL; ++k) {
                    float bm = fabsf(x[k]);  // blocks 2 k (lanes 0-15) and 2 k + 1 (lanes 16-31)
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
                    const uint32_t scode = f_to_e4m3(__fdiv_rn(__fdiv_rn(bm, 6.0f), g));
                    const float eff = __fmul_rn(e4m3_to_f(scode), g);
                    c[k] = eff > 0.0f ? f_to_fp4(__fdiv_rn(x[k], eff)) : 0u;
                    if ((lane & 15) == 0 && k < nk) sc[2 * k + (lane >> 4)] = scode;
                }
            } else {
                const float s = am > 0.0f ? __fdiv_rn(am, 448.0f) : 1.0f;
                rsc0 = s;
#pragma unroll
                for (int k = 0; k < EPL; ++k) c[k] = f_to_e4m3(__fdiv_rn(x[k], s));
            }
        }

#pragma unroll
        for (int k = 0; k < EPL; ++k)
            if (k < nk) codes[lane + 32 * k] = (uint8_t)c[k];
        __syncwarp();

        // pack: element e at bit e * cb of the little-endian word stream
        const uint32_t mask = (1u << cb) - 1u;
        if (cb == 8 && (D & 3u) == 0) {
            // a word = four code bytes
            for (uint32_t w = lane; w < (uint32_t)sp.code_words; w += 32) orow[w] = reinterpret_cast<const uint32_t *>(codes)[w];
        } else if (cb == 4 && (D & 7u) == 0) {
            // a word = the low nibbles of eight code bytes
            for (uint32_t w = lane; w < (uint32_t)sp.code_words; w += 32) {
                const uint2 v = reinterpret_cast<const uint2 *>(codes)[w];
                const uint32_t a = v.x & 0x0f0f0f0fu, c4 = v.y & 0x0f0f0f0fu;
                const uint32_t lo = (a | (a >> 4)) & 0x00ff00ffu, hi = (c4 | (c4 >> 4)) & 0x00ff00ffu;
                orow[w] = ((lo | (lo >> 8)) & 0xffffu) | (((hi | (hi >> 8)) & 0xffffu) << 16);
            }
        } else
        for (uint32_t w = lane; w < (uint32_t)sp.code_words; w += 32) {
            const uint32_t bit0 = w * 32u;
            const uint32_t e0 = bit0 / cb;
            uint32_t e1 = (bit0 + 31u) / cb + 1u;
            e1 = min(e1, D);
            uint32_t word = 0;
            for (uint32_t e = e0; e < e1; ++e) {
                const int sh = (int)(e * cb) - (int)bit0;
                const uint32_t cc = codes[e] & mask;
                word |= sh >= 0 ? (cc << sh) : (cc >> (-sh));
            }
            orow[w] = word;
        }
        const bool scales = mode == B200_MXFP4 || mode == B200_MXFP8 || mode == B200_NVFP4;
        const uint32_t nblk = mode == B200_NVFP4 ? (D >> 4) : (D >> 5);
        for (uint32_t w = lane; w < (uint32_t)sp.aux_words; w += 32) {
            uint32_t word = 0;
            if (scales)
                for (uint32_t e = 0; e < 4u; ++e)
                    if (w * 4u + e < nblk) word |= (sc[w * 4u + e] & 0xffu) << (8u * e);
            orow[sp.code_words + w] = word;
        }
        if (lane == 0) {
            orow[sp.code_words + sp.aux_words] = f2u(rsc0);
            orow[sp.code_words + sp.aux_words + 1] = 0u;
        }
        __syncwarp();
    }
    after_prev_end(p);
}

// ---------------------------------------------------------------------------------------------
// Rows of 128 elements in the block-scaled formats. Eight lanes share a row (four rows per warp): lane l of the eight owns
// elements 16 l .. 16 l + 15 (two or four 16-byte loads), which is exactly one NVFP4 scale block and half an MX block, so the
// block arithmetic runs once per 16 elements, the row maximum is three shuffles, and a lane's codes are already the 8 or
// 16 bytes of the row that it stores. The codes come from the hardware conversions (cvt.rn.satfinite.e2m1x2 /
// e4m3x2: round to nearest even, saturating), which agree with the integer codecs of common.cuh on every input that is
// not a NaN; a lane that holds a NaN or an infinity (the only sources of a NaN quotient) gives NaNs those codecs' codes
// explicitly. Maxima do not depend on the order of the reduction, every division is IEEE, so rows are bit-identical to
// quant_rows_kernel's. Row -> (batch entry, head, token) uses multiply-high division by the launch's invariants.
// ---------------------------------------------------------------------------------------------
constexpr int Q128_WARPS = 8, Q128_RPW = 4;  // warps per block, rows per warp

// one value -> its e4m3 code
__device__ __forceinline__ uint32_t e4m3_hw(float f) {
    uint32_t d;
    asm("{\n .reg .b16 t;\n cvt.rn.satfinite.e4m3x2.f32 t, %1, %1;\n cvt.u32.u16 %0, t;\n}" : "=r"(d) : "f"(f));
    d &= 0xffu;
    return f != f ? (((f2u(f) >> 24) & 0x80u) | 0x7fu) : d;
}
// two values -> two e4m3 codes (lo in the low byte); FIX: NaNs get the sign of the input and 0x7f
template <bool FIX>
__device__ __forceinline__ uint32_t e4m3x2_hw(float lo, float hi) {
    uint32_t d;
    asm("{\n .reg .b16 t;\n cvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\n cvt.u32.u16 %0, t;\n}" : "=r"(d) : "f"(hi), "f"(lo));
    if (FIX) {
        if (lo != lo) d = (d & 0xff00u) | ((f2u(lo) >> 24) & 0x80u) | 0x7fu;
        if (hi != hi) d = (d & 0x00ffu) | ((((f2u(hi) >> 24) & 0x80u) | 0x7fu) << 8);
    }
    return d;
}
// two values -> one byte of e2m1 codes (lo in the low nibble); FIX: a NaN keeps its sign and gets magnitude 0
template <bool FIX>
__device__ __forceinline__ uint32_t fp4x2_hw(float lo, float hi) {
    if (FIX) {
        lo = lo != lo ? u2f(f2u(lo) & 0x80000000u) : lo;
        hi = hi != hi ? u2f(f2u(hi) & 0x80000000u) : hi;
    }
    uint32_t d;
    asm("{\n .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n cvt.u32.u8 %0, t;\n}" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
// x / s as the reference computes it. MUL: s is a power of two and `s` holds its reciprocal (e8m0_recip): the product is
// the same float as the IEEE quotient and costs one instruction instead of a division sequence.
template <bool MUL>
__device__ __forceinline__ float scaled(float x, float s) { return MUL ? __fmul_rn(x, s) : __fdiv_rn(x, s); }
// the lane's 16 elements divided by s -> 16 e2m1 codes (two words)
template <bool FIX, bool MUL = false>
__device__ __forceinline__ void fp4x16_div(const float (&x)[16], float s, uint32_t (&w)[2]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) v |= fp4x2_hw<FIX>(scaled<MUL>(x[8 * h + 2 * i], s), scaled<MUL>(x[8 * h + 2 * i + 1], s)) << (8 * i);
        w[h] = v;
    }
}
// ... -> 16 e4m3 codes (four words)
template <bool FIX, bool MUL = false>
__device__ __forceinline__ void e4m3x16_div(const float (&x)[16], float s, uint32_t (&w)[4]) {
#pragma unroll
    for (int h = 0; h < 4; ++h)
        w[h] = e4m3x2_hw<FIX>(scaled<MUL>(x[4 * h], s), scaled<MUL>(x[4 * h + 1], s)) |
               (e4m3x2_hw<FIX>(scaled<MUL>(x[4 * h + 2], s), scaled<MUL>(x[4 * h + 3], s)) << 16);
}

template <int DT>
__device__ __forceinline__ void load16(const char *src, int l8, float (&x)[16]) {
    if (DT == B200_F32) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(src) + 4 * l8 + q);
            x[4 * q] = v.x, x[4 * q + 1] = v.y, x[4 * q + 2] = v.z, x[4 * q + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src) + 2 * l8 + q);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (DT == B200_BF16) {
                    x[8 * q + 2 * i] = u2f(w[i] << 16);
                    x[8 * q + 2 * i + 1] = u2f(w[i] & 0xffff0000u);
                } else {
                    x[8 * q + 2 * i] = f16_bits_to_f((uint16_t)w[i]);
                    x[8 * q + 2 * i + 1] = f16_bits_to_f((uint16_t)(w[i] >> 16));
                }
            }
        }
    }
}

// n / d for n < 2^31 with the invariants of fastdiv_init
__device__ __forceinline__ uint32_t fastdiv(uint32_t n, uint32_t mul, uint32_t shr) { return (__umulhi(n, mul) + n) >> shr; }

template <int DT>
__global__ void __launch_bounds__(Q128_WARPS * 32) quant_rows128_kernel(const QuantParams p) {
    const QuantSideParams &sp = p.side[blockIdx.y];
    const int lane = threadIdx.x & 31, l8 = lane & 7;
    const uint32_t rows = p.nb * p.nh * p.nt;
    const uint32_t mode = sp.mode;
    after_prev_begin(p);
    for (uint32_t base = (blockIdx.x * Q128_WARPS + (threadIdx.x >> 5)) * Q128_RPW; base < rows; base += gridDim.x * Q128_WARPS * Q128_RPW) {
        bool live = base + (lane >> 3) < rows;  // a row past the end repeats the last one and stores nothing
        const uint32_t row = live ? base + (lane >> 3) : rows - 1;
        const uint32_t bh = fastdiv(row, p.nt_mul, p.nt_shr), t = row - bh * p.nt, b = fastdiv(bh, p.nh_mul, p.nh_shr), h = bh - b * p.nh;
        const char *src = reinterpret_cast<const char *>(sp.src) + (b * sp.s_b + h * sp.s_h + t * sp.s_t) * (uint64_t)dtype_size(DT);
        int64_t pos = (sp.pos ? (int64_t)sp.pos[b] + sp.pos0 : (int64_t)sp.pos0) + (int64_t)t;
        if (pos < 0 || (sp.cap && pos >= (int64_t)sp.cap)) {
            // a stale or corrupt device position: the row is computed like the others (the lanes of a row shuffle among
            // themselves) but nothing is written outside the slab
            if (live && l8 == 0 && sp.status) atomicExch(sp.status, 3);
            live = false;
            pos = 0;
        }
        uint32_t *orow = sp.dst + b * sp.c_b + h * sp.c_h + (uint64_t)pos * sp.c_t;
        float x[16];
        load16<DT>(src, l8, x);

        if (sp.rot == B200_ROT_HADAMARD) {
            // element index bits 0-3 across the registers, bits 4-6 across the lanes: the butterflies run in the same
            // order (bit 0 first) as in quant_rows_kernel
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 sg = __ldg(reinterpret_cast<const float4 *>(sp.signs) + 4 * l8 + q);
                x[4 * q] *= sg.x, x[4 * q + 1] *= sg.y, x[4 * q + 2] *= sg.z, x[4 * q + 3] *= sg.w;
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) {
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    if (!(k & o)) {
                        const float a = x[k], c = x[k | o];
                        x[k] = a + c;
                        x[k | o] = a - c;
                    }
                }
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const float y = __shfl_xor_sync(0xffffffffu, x[k], o);
                    x[k] = (lane & o) ? y - x[k] : x[k] + y;
                }
            }
            const float s = 1.0f / sqrtf(128.0f);
#pragma unroll
            for (int k = 0; k < 16; ++k) x[k] *= s;
        }

        // the lane's maximum; a NaN survives only if all sixteen are NaNs (fmaxf drops a NaN operand). z is a NaN when
        // the lane holds a NaN or an infinity.
        float bm = fabsf(x[0]), z = x[0] * 0.0f;
#pragma unroll
        for (int k = 1; k < 16; ++k) {
            bm = fmaxf(bm, fabsf(x[k]));
            z = fmaf(x[k], 0.0f, z);
        }
        const bool special = z != z;
        float rsc0 = 1.0f;
        uint32_t cw;  // words of codes before the scales
        if (mode == B200_NVFP4) {
            cw = 16;
            float am = fmaxf(0.0f, bm);
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
            const float g = am > 0.0f ? __fdiv_rn(am, 2688.0f) : 1.0f;
            rsc0 = g;
            const uint32_t scode = e4m3_hw(__fdiv_rn(__fdiv_rn(bm, 6.0f), g));  // the lane's 16 elements are one scale block
            const float eff = __fmul_rn(e4m3_to_f(scode), g);
            uint32_t w[2] = {0u, 0u};
            if (eff > 0.0f) {
                if (special) fp4x16_div<true>(x, eff, w);
                else fp4x16_div<false>(x, eff, w);
            }
            if (live) {
                *reinterpret_cast<uint2 *>(orow + 2 * l8) = make_uint2(w[0], w[1]);
                reinterpret_cast<uint8_t *>(orow + 16)[l8] = (uint8_t)scode;
            }
        } else if (mode == B200_FP8) {
            cw = 32;
            float am = fmaxf(0.0f, bm);
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
            const float s = am > 0.0f ? __fdiv_rn(am, 448.0f) : 1.0f;
            rsc0 = s;
            uint32_t w[4];
            if (special) e4m3x16_div<true>(x, s, w);
            else e4m3x16_div<false>(x, s, w);
            if (live) {
#pragma unroll
                for (int i = 0; i < 4; ++i) orow[4 * l8 + i] = w[i];
            }
        } else {
            // MXFP4 / MXFP8: a block of 32 = two neighbouring lanes
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            const uint32_t code = mx_scale_code(bm, mode == B200_MXFP4 ? 2 : 8);
            const float s = e8m0_recip(code);  // the divisor is a power of two: multiply by its reciprocal, same bits
            if (mode == B200_MXFP4) {
                cw = 16;
                uint32_t w[2] = {0u, 0u};
                if (code != 0) {
                    if (special) fp4x16_div<true, true>(x, s, w);
                    else fp4x16_div<false, true>(x, s, w);
                }
                if (live) orow[2 * l8] = w[0], orow[2 * l8 + 1] = w[1];  // rows of 19 words: 4-byte alignment only
            } else {
                cw = 32;
                uint32_t w[4] = {0u, 0u, 0u, 0u};
                if (code != 0) {
                    if (special) e4m3x16_div<true, true>(x, s, w);
                    else e4m3x16_div<false, true>(x, s, w);
                }
                if (live) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) orow[4 * l8 + i] = w[i];
                }
            }
            if (live && (l8 & 1) == 0) reinterpret_cast<uint8_t *>(orow + cw)[l8 >> 1] = (uint8_t)code;
        }
        if (live && l8 < 2) orow[cw + (uint32_t)sp.aux_words + l8] = l8 ? 0u : f2u(rsc0);
    }
    after_prev_end(p);
}

// rsc0 * element for every element (candle-core/kernels/turbo_quant_impl.h:44-53,208-218)
__global__ void __launch_bounds__(256) dequant_rows_kernel(const uint32_t *__restrict__ data, const float *__restrict__ tab,
                                                          float *__restrict__ out, uint64_t rows, uint32_t D,
                                                          uint64_t stride, uint32_t mode, uint32_t cb,
                                                          uint32_t code_words, uint32_t rsc_off, float *__restrict__ zs) {
    const uint64_t n = rows * D;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = idx / D;
        const uint32_t j = (uint32_t)(idx % D);
        const uint32_t *r = data + row * stride;
        const uint32_t pos = j * cb, wi = pos >> 5, sh = pos & 31u;
        uint32_t c = r[wi] >> sh;
        if (sh + cb > 32u) c |= r[wi + 1] << (32u - sh);
        c &= (1u << cb) - 1u;
        const uint32_t *aux = r + code_words;
        float e;
        if (mode <= B200_TURBO_PROD) e = tab[c];
        else if (mode == B200_MXFP4) e = __fmul_rn(fp4_to_f(c), e8m0_to_f((aux[j >> 7] >> (((j >> 5) & 3u) * 8u)) & 0xffu));
        else if (mode == B200_NVFP4) e = __fmul_rn(fp4_to_f(c), e4m3_to_f((aux[j >> 6] >> (((j >> 4) & 3u) * 8u)) & 0xffu));
        else if (mode == B200_MXFP8) e = __fmul_rn(e4m3_to_f(c), e8m0_to_f((aux[j >> 7] >> (((j >> 5) & 3u) * 8u)) & 0xffu));
        else e = e4m3_to_f(c);
        out[idx] = __fmul_rn(u2f(r[rsc_off]), e);
        if (zs) {
            // prod rows: the QJL coefficient of element j (candle-core/kernels/turbo_quant_impl.h:219-222)
            const float c = __fdiv_rn(__fmul_rn(__fmul_rn(u2f(r[rsc_off]), u2f(r[rsc_off + 1])), 1.2533141f), (float)D);
            zs[idx] = ((r[code_words + (j >> 5)] >> (j & 31u)) & 1u) ? c : -c;
        }
    }
}

// Residual of the unit vectors to their codebook values (candle-core/kernels/turbo_quant_impl.h:161-177), with that
// kernel's roundings: inv = 1 / rsc0 (0 for a zero row), u = x * inv, resid = u - centroid, none of them fused.
template <int DT>
__global__ void __launch_bounds__(256) resid_rows_kernel(const void *__restrict__ src, const uint32_t *__restrict__ data, const float *__restrict__ tab,
                                                        float *__restrict__ resid, uint64_t rows, uint32_t D, uint64_t src_stride,
                                                        uint64_t data_stride, uint32_t cb, uint32_t rsc_off) {
    const uint64_t n = rows * D;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = idx / D;
        const uint32_t j = (uint32_t)(idx % D);
        const uint32_t *r = data + row * data_stride;
        const float norm = u2f(r[rsc_off]);
        const float inv = norm > 0.0f ? __fdiv_rn(1.0f, norm) : 0.0f;
        const float u = __fmul_rn(load_elem<DT>(reinterpret_cast<const char *>(src) + row * src_stride * dtype_size(DT), j), inv);
        const uint32_t pos = j * cb, wi = pos >> 5, sh = pos & 31u;
        uint32_t c = r[wi] >> sh;
        if (sh + cb > 32u) c |= r[wi + 1] << (32u - sh);
        c &= (1u << cb) - 1u;
        resid[idx] = __fsub_rn(u, tab[c]);
    }
}

// Sign bits of the projected residual and the residual's norm into prod rows (candle-core/kernels/
// turbo_quant_impl.h:179-206). One warp per row; the sum of squares runs in the order of the reference's 128 lanes
// (lane t adds j = t, t + 128, ..., then the halving tree), so rsc1 is bit-identical.
__global__ void __launch_bounds__(128) signs_rows_kernel(const uint32_t *__restrict__ in, const float *__restrict__ proj, const float *__restrict__ resid,
                                                        uint32_t *__restrict__ out, uint64_t rows, uint32_t D, uint32_t code_words,
                                                        uint32_t row_words) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sign_words = (D + 31u) / 32u;
    for (uint64_t row = (uint64_t)blockIdx.x * 4 + warp; row < rows; row += (uint64_t)gridDim.x * 4) {
        // reference lane t = (lane + 32 k) mod 128 holds part[k & 3] of this lane
        float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t k = 0; lane + 32u * k < D; ++k) {
            const float v = resid[row * D + lane + 32u * k];
            part[k & 3] = __fadd_rn(part[k & 3], __fmul_rn(v, v));
        }
        float ss = __fadd_rn(__fadd_rn(part[0], part[2]), __fadd_rn(part[1], part[3]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, o));
        ss = __shfl_sync(0xffffffffu, ss, 0);
        const uint32_t *ir = in + row * row_words;
        uint32_t *orow = out + row * row_words;
        for (uint32_t w = lane; w < row_words; w += 32) {
            uint32_t word = ir[w];
            if (w >= code_words && w < code_words + sign_words) {
                word = 0;
                const uint32_t base = (w - code_words) * 32u;
                for (uint32_t e = 0; e < 32u && base + e < D; ++e)
                    if (proj[row * D + base + e] >= 0.0f) word |= 1u << e;
            } else if (w == code_words + sign_words + 1u) {
                word = f2u(__fsqrt_rn(ss));
            }
            orow[w] = word;
        }
    }
}

// y = H diag(s) x / sqrt(D) (forward) or x = diag(s) H y / sqrt(D) (back), one warp per row, f32
__global__ void __launch_bounds__(128) hadamard_rows_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                           const float *__restrict__ signs, uint64_t rows, uint32_t D,
                                                           int inverse) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = (int)((D + 31) / 32);
    for (uint64_t row = (uint64_t)blockIdx.x * 4 + warp; row < rows; row += (uint64_t)gridDim.x * 4) {
        float x[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const uint32_t j = lane + 32 * k;
            x[k] = (k < nk && j < D) ? in[row * D + j] * (inverse ? 1.0f : signs[j]) : 0.0f;
        }
        for (uint32_t o = 1; o < 32 && o < D; o <<= 1) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                const float y = __shfl_xor_sync(0xffffffffu, x[k], o);
                x[k] = (lane & o) ? y - x[k] : x[k] + y;
            }
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            if (o < nk) {
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    if (!(k & o)) {
                        const float a = x[k], c = x[k | o];
                        x[k] = a + c;
                        x[k | o] = a - c;
                    }
                }
            }
        }
        const float s = 1.0f / sqrtf((float)D);
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const uint32_t j = lane + 32 * k;
            if (k < nk && j < D) out[row * D + j] = x[k] * s * (inverse ? signs[j] : 1.0f);
        }
    }
}

static int fill_side(QuantSideParams &sp, const B200QuantSide &q, uint32_t d) {
    B200RowLayout l;
    const int rc = b200_row_layout(q.mode, q.bits, (int)d, &l);
    if (rc) return rc;
    if (q.mode <= B200_TURBO_PROD && !q.tab) return set_error(B200_ERR_BAD_ARG, "turbo formats need the codebook table");
    if (q.rotation == B200_ROT_HADAMARD) {
        if (!q.signs) return set_error(B200_ERR_BAD_ARG, "hadamard rotation needs the sign vector");
        if (d & (d - 1)) return set_error(B200_ERR_BAD_ARG, "hadamard rotation needs a power of two length, got %u", d);
    } else if (q.rotation != B200_ROT_NONE) {
        return set_error(B200_ERR_UNSUPPORTED_SHAPE, "only none / hadamard rotations are fused");
    }
    sp.tab = q.tab;
    sp.signs = q.signs;
    sp.rot = q.rotation;
    sp.mode = q.mode;
    sp.cb = l.code_bits;
    sp.code_words = l.code_words;
    sp.aux_words = l.aux_words;
    sp.row_words = l.row_words;
    return B200_OK;
}

// n / d == (umulhi(n, mul) + n) >> shr for every n < 2^31: mul = ceil(2^(32 + shr) / d) - 2^32, shr = ceil(log2 d)
static void fastdiv_init(uint32_t d, uint32_t &mul, uint32_t &shr) {
    shr = 0;
    while ((1ull << shr) < d) ++shr;
    const unsigned __int128 one = 1;
    mul = (uint32_t)((((one << (32 + shr)) + d - 1) / d) - (one << 32));
}

// rows of 128 block-scaled elements whose source rows can be read as 16-byte vectors
static bool rows128_takes(const QuantParams &p, int sides) {
    static const bool off = diag_env("B200_QUANT_GENERIC") != nullptr;
    if (off || p.d != 128 || (uint64_t)p.nb * p.nh * p.nt >= 0x7fffff00ull) return false;
    const uint64_t vec = p.src_dtype == B200_F32 ? 3 : 7;  // elements per 16 bytes - 1
    for (int s = 0; s < sides; ++s) {
        const QuantSideParams &sp = p.side[s];
        if (sp.mode != B200_MXFP4 && sp.mode != B200_NVFP4 && sp.mode != B200_MXFP8 && sp.mode != B200_FP8) return false;
        if (((uintptr_t)sp.src & 15) || (sp.s_b & vec) || (sp.s_h & vec) || (sp.s_t & vec)) return false;
        if (sp.rot == B200_ROT_HADAMARD && ((uintptr_t)sp.signs & 15)) return false;
        // NVFP4 code words are stored in pairs
        if (sp.mode == B200_NVFP4 && (((uintptr_t)sp.dst & 7) || (sp.c_b & 1) || (sp.c_h & 1) || (sp.c_t & 1))) return false;
    }
    return true;
}

// a plain launch, or (after_prev) one that may be scheduled while the stream's previous kernel still runs
static int launch_maybe_after_prev(void (*kern)(const QuantParams), dim3 grid, dim3 block, cudaStream_t stream, const QuantParams &p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.after_prev ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "tq_quantize: %s", cudaGetErrorString(e));
    return check_launch("tq_quantize");
}

static int launch_quant(const QuantParams &p, int sides, cudaStream_t stream) {
    const uint64_t rows = (uint64_t)p.nb * p.nh * p.nt;
    if (rows == 0) return B200_OK;
    if (rows128_takes(p, sides)) {
        QuantParams q = p;
        fastdiv_init(p.nt, q.nt_mul, q.nt_shr);
        fastdiv_init(p.nh, q.nh_mul, q.nh_shr);
        const uint64_t per_block = Q128_WARPS * Q128_RPW;
        // as many blocks as are resident at once, shared by the sides
        static const int resident = [] {
            int per_sm = 4, sms = 148, dev = 0;
            cudaGetDevice(&dev);
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_rows128_kernel<B200_BF16>, Q128_WARPS * 32, 0);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            return std::max(per_sm, 1) * std::max(sms, 1);
        }();
        const dim3 grid((unsigned)std::min<uint64_t>((rows + per_block - 1) / per_block, (uint64_t)std::max(resident / sides, 1)), sides), block(Q128_WARPS * 32);
        if (p.src_dtype == B200_F32) return launch_maybe_after_prev(quant_rows128_kernel<B200_F32>, grid, block, stream, q);
        if (p.src_dtype == B200_F16) return launch_maybe_after_prev(quant_rows128_kernel<B200_F16>, grid, block, stream, q);
        return launch_maybe_after_prev(quant_rows128_kernel<B200_BF16>, grid, block, stream, q);
    }
    const unsigned gx = (unsigned)std::min<uint64_t>((rows + QW - 1) / QW, 148ull * 64);
    const dim3 grid(gx, sides), block(QW * 32);
#define B200_QUANT_LAUNCH(EPL)                                                                      \
    do {                                                                                            \
        if (p.src_dtype == B200_F32) return launch_maybe_after_prev(quant_rows_kernel<EPL, B200_F32>, grid, block, stream, p);      \
        if (p.src_dtype == B200_F16) return launch_maybe_after_prev(quant_rows_kernel<EPL, B200_F16>, grid, block, stream, p);      \
        return launch_maybe_after_prev(quant_rows_kernel<EPL, B200_BF16>, grid, block, stream, p);                                  \
    } while (0)
    if (p.d <= 128) B200_QUANT_LAUNCH(4);
    else if (p.d <= 256) B200_QUANT_LAUNCH(8);
    else B200_QUANT_LAUNCH(32);
#undef B200_QUANT_LAUNCH
}

} // namespace b200

using namespace b200;

extern "C" int b200_tq_quantize(const B200TqQuantArgs *a, b200_stream_t stream) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "tq_quantize: null args");
    if (a->rows == 0) return B200_OK;
    if (!a->src || !a->out) return set_error(B200_ERR_BAD_ARG, "tq_quantize: null pointer");
    if (a->src_dtype != B200_F32 && a->src_dtype != B200_F16 && a->src_dtype != B200_BF16)
        return set_error(B200_ERR_BAD_ARG, "tq_quantize: source dtype must be f32, f16 or bf16");
    QuantParams p;
    memset(&p, 0, sizeof(p));
    B200QuantSide q = {a->mode, a->bits, a->tab, B200_ROT_NONE, nullptr};
    const int rc = fill_side(p.side[0], q, a->dim);
    if (rc) return rc;
    QuantSideParams &sp = p.side[0];
    sp.src = a->src;
    sp.dst = a->out;
    sp.s_t = a->src_stride;
    sp.c_t = a->out_stride ? a->out_stride : (uint64_t)sp.row_words;
    if (sp.c_t < (uint64_t)sp.row_words) return set_error(B200_ERR_BAD_ARG, "tq_quantize: output stride below the row size");
    if (a->rows > 0xffffffffull) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_quantize: too many rows");
    p.nb = 1;
    p.nh = 1;
    p.nt = (uint32_t)a->rows;
    p.d = a->dim;
    p.src_dtype = a->src_dtype;
    return launch_quant(p, 1, (cudaStream_t)stream);
}

extern "C" int b200_kv_append(const B200KvAppendArgs *a, b200_stream_t stream) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "kv_append: null args");
    if ((uint64_t)a->b * a->hkv * a->t == 0) return B200_OK;
    if (!a->k || !a->v || !a->k_cache || !a->v_cache) return set_error(B200_ERR_BAD_ARG, "kv_append: null pointer");
    if (a->src_dtype != B200_F32 && a->src_dtype != B200_F16 && a->src_dtype != B200_BF16)
        return set_error(B200_ERR_BAD_ARG, "kv_append: source dtype must be f32, f16 or bf16");
    if (!a->pos && a->pos0 < 0) return set_error(B200_ERR_BAD_ARG, "kv_append: negative position");
    if (!a->pos && a->cap && (uint64_t)a->pos0 + a->t > (uint64_t)a->cap)
        return set_error(B200_ERR_BAD_ARG, "kv_append: rows [%d, %llu) do not fit a cache of %u rows", a->pos0,
                         (unsigned long long)a->pos0 + a->t, a->cap);
    QuantParams p;
    memset(&p, 0, sizeof(p));
    int rc = fill_side(p.side[0], a->kq, a->d);
    if (rc) return rc;
    rc = fill_side(p.side[1], a->vq, a->d);
    if (rc) return rc;
    const void *srcs[2] = {a->k, a->v};
    uint32_t *dsts[2] = {a->k_cache, a->v_cache};
    const uint64_t *ss[2] = {a->k_strides, a->v_strides};
    const uint64_t *cs[2] = {a->k_cache_strides, a->v_cache_strides};
    for (int s = 0; s < 2; ++s) {
        QuantSideParams &sp = p.side[s];
        sp.src = srcs[s];
        sp.dst = dsts[s];
        sp.s_b = ss[s][0];
        sp.s_h = ss[s][1];
        sp.s_t = ss[s][2];
        sp.c_b = cs[s][0];
        sp.c_h = cs[s][1];
        sp.c_t = cs[s][2];
        sp.pos = a->pos;
        sp.pos0 = a->pos0;
        sp.cap = a->cap;
        sp.status = a->status;
        if (sp.c_t < (uint64_t)sp.row_words) return set_error(B200_ERR_BAD_ARG, "kv_append: cache row stride below the row size");
    }
    p.nb = a->b;
    p.nh = a->hkv;
    p.nt = a->t;
    p.d = a->d;
    p.src_dtype = a->src_dtype;
    p.after_prev = (a->flags & B200_KV_AFTER_PREV) ? 1u : 0u;
    return launch_quant(p, 2, (cudaStream_t)stream);
}

extern "C" int b200_tq_dequantize(const B200TqDequantArgs *a, b200_stream_t stream) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "tq_dequantize: null args");
    if (a->rows == 0) return B200_OK;
    if (!a->data || !a->out) return set_error(B200_ERR_BAD_ARG, "tq_dequantize: null pointer");
    B200RowLayout l;
    const int rc = b200_row_layout(a->mode, a->bits, (int)a->dim, &l);
    if (rc) return rc;
    if (a->mode <= B200_TURBO_PROD && !a->tab) return set_error(B200_ERR_BAD_ARG, "turbo formats need the codebook table");
    const uint64_t stride = a->data_stride ? a->data_stride : (uint64_t)l.row_words;
    const uint64_t n = a->rows * a->dim;
    const unsigned grid = (unsigned)std::min<uint64_t>((n + 255) / 256, 148ull * 32);
    if (a->zs && a->mode != B200_TURBO_PROD) return set_error(B200_ERR_BAD_ARG, "tq_dequantize: QJL coefficients exist for prod rows only");
    dequant_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a->data, a->tab, a->out, a->rows, a->dim, stride, a->mode,
                                                               l.code_bits, l.code_words, l.rsc_offset, a->zs);
    return check_launch("tq_dequantize");
}

extern "C" int b200_tq_residual(const B200TqResidArgs *a, b200_stream_t stream) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "tq_residual: null args");
    if (a->rows == 0) return B200_OK;
    if (!a->src || !a->data || !a->tab || !a->resid) return set_error(B200_ERR_BAD_ARG, "tq_residual: null pointer");
    B200RowLayout l;
    const int rc = b200_row_layout(B200_TURBO_PROD, a->bits, (int)a->dim, &l);
    if (rc) return rc;
    const uint64_t ds = a->data_stride ? a->data_stride : (uint64_t)l.row_words;
    if (ds < (uint64_t)l.row_words) return set_error(B200_ERR_BAD_ARG, "tq_residual: row stride below the row size");
    const uint64_t n = a->rows * a->dim;
    const unsigned grid = (unsigned)std::min<uint64_t>((n + 255) / 256, 148ull * 32);
    cudaStream_t st = (cudaStream_t)stream;
    if (a->src_dtype == B200_F32)
        resid_rows_kernel<B200_F32><<<grid, 256, 0, st>>>(a->src, a->data, a->tab, a->resid, a->rows, a->dim, a->src_stride, ds, l.code_bits, l.rsc_offset);
    else if (a->src_dtype == B200_F16)
        resid_rows_kernel<B200_F16><<<grid, 256, 0, st>>>(a->src, a->data, a->tab, a->resid, a->rows, a->dim, a->src_stride, ds, l.code_bits, l.rsc_offset);
    else if (a->src_dtype == B200_BF16)
        resid_rows_kernel<B200_BF16><<<grid, 256, 0, st>>>(a->src, a->data, a->tab, a->resid, a->rows, a->dim, a->src_stride, ds, l.code_bits, l.rsc_offset);
    else
        return set_error(B200_ERR_BAD_ARG, "tq_residual: source dtype must be f32, f16 or bf16");
    return check_launch("tq_residual");
}

extern "C" int b200_tq_signs(const B200TqSignsArgs *a, b200_stream_t stream) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "tq_signs: null args");
    if (a->rows == 0) return B200_OK;
    if (!a->in || !a->proj || !a->resid || !a->out) return set_error(B200_ERR_BAD_ARG, "tq_signs: null pointer");
    B200RowLayout l;
    const int rc = b200_row_layout(B200_TURBO_PROD, a->bits, (int)a->dim, &l);
    if (rc) return rc;
    const unsigned grid = (unsigned)std::min<uint64_t>((a->rows + 3) / 4, 148ull * 16);
    signs_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(a->in, a->proj, a->resid, a->out, a->rows, a->dim, l.code_words, l.row_words);
    return check_launch("tq_signs");
}

extern "C" int b200_tq_rotate(const float *in, float *out, const float *signs, uint64_t rows, uint32_t dim, int inverse,
                              b200_stream_t stream) {
    if (rows == 0) return B200_OK;
    if (!in || !out || !signs) return set_error(B200_ERR_BAD_ARG, "tq_rotate: null pointer");
    if (dim == 0 || dim > 1024 || (dim & (dim - 1)))
        return set_error(B200_ERR_BAD_ARG, "hadamard rotation needs a power of two length up to 1024, got %u", dim);
    const unsigned grid = (unsigned)std::min<uint64_t>((rows + 3) / 4, 148ull * 32);
    hadamard_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(in, out, signs, rows, dim, inverse);
    return check_launch("tq_rotate");
}

// y = x Pi^T (inverse: x = y Pi) for a caller-supplied row-major dim x dim matrix: the rotation of head dims that are
// not powers of two (candle-nn/src/turbo_quant.rs:182-196, a library matmul there). One warp per row, the row in
// shared memory, lane l computes outputs l, l + 32, ...; products and sums in index order, unfused, so the result has
// the bits of the plain f32 loop.
__global__ void __launch_bounds__(128) dense_rotate_rows_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                               const float *__restrict__ pi, uint64_t rows, uint32_t D, int inverse) {
    extern __shared__ float xrow[];  // [4][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *x = xrow + (size_t)warp * D;
    for (uint64_t row = (uint64_t)blockIdx.x * 4 + warp; row < rows; row += (uint64_t)gridDim.x * 4) {
        __syncwarp();
        for (uint32_t j = lane; j < D; j += 32) x[j] = in[row * D + j];
        __syncwarp();
        for (uint32_t i = lane; i < D; i += 32) {
            float acc = 0.0f;
            if (!inverse)
                for (uint32_t j = 0; j < D; ++j) acc = __fadd_rn(acc, __fmul_rn(__ldg(pi + (size_t)i * D + j), x[j]));
            else
                for (uint32_t j = 0; j < D; ++j) acc = __fadd_rn(acc, __fmul_rn(__ldg(pi + (size_t)j * D + i), x[j]));
            out[row * D + i] = acc;
        }
    }
}

extern "C" int b200_tq_rotate_dense(const float *in, float *out, const float *pi, uint64_t rows, uint32_t dim, int inverse,
                                    b200_stream_t stream) {
    if (rows == 0) return B200_OK;
    if (!in || !out || !pi) return set_error(B200_ERR_BAD_ARG, "tq_rotate_dense: null pointer");
    if (in == out) return set_error(B200_ERR_BAD_ARG, "tq_rotate_dense: in and out must differ");
    if (dim == 0 || dim > 1024) return set_error(B200_ERR_BAD_ARG, "tq_rotate_dense: dim %u outside 1..1024", dim);
    const unsigned grid = (unsigned)std::min<uint64_t>((rows + 3) / 4, 148ull * 16);
    dense_rotate_rows_kernel<<<grid, 128, 4 * dim * sizeof(float), (cudaStream_t)stream>>>(in, out, pi, rows, dim, inverse);
    return check_launch("tq_rotate_dense");
}
