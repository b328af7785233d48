// Decode attention over packed K/V rows (FP8, MXFP8, MXFP4, NVFP4, TurboQuant 4-bit): kernel body.
//
// Work split: block = (key chunk, pack of up to 8 query rows that share a kv head, batch entry).
// Each of the 4 warps streams its own 32-key tiles of the chunk through a private ring of shared
// memory stages filled by bulk copies (cp.async.bulk + mbarrier, no multicast), so no block-wide
// barrier sits in the key loop. Per 16 keys a warp
//   1. dequantizes K in registers to f16 (packed cvt from e2m1 / e4m3, or a 256-entry pair table
//      for the codebook format; block scales relative to the row's largest block exponent, the rest
//      of the scale stays in f32) and multiplies with the f16 query fragments on mma.sync m16n8k16
//      (A = query rows, B = keys): lane (g, c) owns key g of an 8-key group and the quarter
//      [c D/4, (c + 1) D/4) of its row, a permutation of the contraction index shared with the
//      query fragments, so every byte of a row is read once, as 32-bit words;
//   2. runs the online softmax in f32 on the accumulator fragments (log2 domain). The per-key value
//      scale sigma_j = rsc0_v * 2^(largest block exponent) is folded into the exponent:
//      w_j = exp2(s_j + log2 sigma_j - M) <= 1 is the f16 operand of the second product, while the
//      normalizer sums exp2(s_j - M) in f32, so value scales of any magnitude stay exact;
//   3. dequantizes V (lane (g, c) owns keys {2c, 2c+1, 2c+8, 2c+9} x dims [g D/8, (g+1) D/8), bytes
//      or nibbles of two keys interleaved before the packed cvt so that the f16 pairs run along
//      the contraction index) and accumulates O^T = V^T P^T (A = V^T, B = P^T straight from the
//      score fragments).
// The warps' states are merged through shared memory; the block writes either the final rows
// (one chunk) or a normalized partial and its log-sum-exp for the combine kernel.
//
// Semantics: candle-core/kernels/turbo_quant_impl.h:232-401 (tq_attn): score = scale * rsc0_k *
// sum_d elem_k q_d, softcap, ALiBi, bottom-right aligned windows, value weight p * rsc0_v, zeros
// for rows without keys.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int DW = 4;         // warps per block
constexpr int WK = 32;        // keys per warp tile
constexpr int NS_MAX = 3;     // stages per warp (fewer when the rows are large)
constexpr int PACK = 8;       // query rows per block
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct DecodeSide {
    int32_t mode, code_words, rsc_off;
    int32_t rot;
    const float *tab;
    const float *signs;
};

struct DecodeParams {
    const void *q;
    void *out;
    int32_t q_dtype, out_dtype;
    uint64_t q_sb, q_sh, q_ss, o_sb, o_sh, o_ss;
    const uint32_t *k_rows, *v_rows;
    uint64_t k_sb, k_sh, k_ss, v_sb, v_sh, v_ss;  // words
    const int32_t *kv_len;
    uint32_t b, lq, lk, hq, hkv, d, group;
    uint32_t rows_per_kv, packs;
    DecodeSide k, v;
    float scale, softcap;
    int32_t wl, wr;
    const float *alibi;
    uint32_t alibi_bs;
    uint32_t chunk, max_splits;
    float *part_o;     // [b][ny][max_splits][PACK][d]
    float *part_lse;   // [b][ny][max_splits][PACK]
    int32_t *meta;     // [b][ny] live splits
    int32_t *status;
    uint32_t k_stage_bytes, v_stage_bytes;
    uint32_t ns;       // stages per warp
};

__host__ __device__ constexpr bool fmt_is4(int m) { return m == B200_MXFP4 || m == B200_NVFP4 || m == B200_TURBO_MSE; }

// largest byte of a word
__device__ __forceinline__ uint32_t max_byte(uint32_t w) {
    const uint32_t m = __vmaxu4(w, w >> 16);
    return max(m & 0xffu, (m >> 8) & 0xffu);
}
// f16x2 {2^da, 2^db} for da, db <= 0 (flushes to zero below 2^-14)
__device__ __forceinline__ uint32_t pow2_f16x2(int da, int db) {
    return ((uint32_t)max(da + 15, 0) << 10) | ((uint32_t)max(db + 15, 0) << 26);
}
__device__ __forceinline__ float pow2_e8m0(uint32_t e) { return u2f(max(e, 1u) << 23); }  // 2^(e-127), e >= 1

// Largest E8M0 exponent byte over the blocks of a row (MX formats), aux words at row[cw...].
template <int HD>
__device__ __forceinline__ uint32_t mx_row_emax(const uint32_t *row, int cw) {
    uint32_t w = row[cw];
    if (HD > 128) w = __vmaxu4(w, row[cw + 1]);
    return max_byte(w);
}

// ---------------------------------------------------------------------------------------------
// K side: lane (g, c) holds elements [c HD/4, (c+1) HD/4) of key g: per k-step s the B fragment
// (b0, b1) = elements 4s .. 4s+3 of that range. Returns kappa, the f32 factor of the row.
// ---------------------------------------------------------------------------------------------
template <int KM, int HD, bool QSPLIT>
__device__ __forceinline__ float qk_group(const uint32_t *krow, int c, const DecodeSide &ks, const uint32_t *lut,
                                          const uint32_t (&qh0)[HD / 16], const uint32_t (&qh2)[HD / 16],
                                          const uint32_t (&ql0)[HD / 16], const uint32_t (&ql2)[HD / 16],
                                          float (&acc)[4]) {
    constexpr int STEPS = HD / 16;
    float kappa = u2f(krow[ks.rsc_off]);
    if (fmt_is4(KM)) {
        constexpr int WORDS = HD / 32;  // words of this lane
        uint32_t sc[WORDS];             // f16x2 scale per word (8 elements)
        if (KM == B200_MXFP4) {
            const uint32_t emax = mx_row_emax<HD>(krow, ks.code_words);
            kappa *= pow2_e8m0(emax);
            constexpr int NB = HD >= 128 ? HD / 128 : 1;  // 32-blocks in this lane's range
            uint32_t sb[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int blk = HD >= 128 ? c * NB + i : c >> 1;
                const int e = (int)((krow[ks.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu);
                sb[i] = pow2_f16x2(e - (int)emax, e - (int)emax);
            }
#pragma unroll
            for (int w = 0; w < WORDS; ++w) sc[w] = sb[(8 * w) / 32];
        } else if (KM == B200_NVFP4) {
            constexpr int NB = HD / 64;  // 16-blocks in this lane's range
            uint32_t sb[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int blk = c * NB + i;
                const uint32_t byte = (krow[ks.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu;
                sb[i] = cvt_e4m3x2_f16x2(byte | (byte << 8));
            }
#pragma unroll
            for (int w = 0; w < WORDS; ++w) sc[w] = sb[(8 * w) / 16];
        }
#pragma unroll
        for (int w = 0; w < WORDS; ++w) {
            const uint32_t x = krow[c * WORDS + w];
            uint32_t h0, h1, h2, h3;
            if (KM == B200_TURBO_MSE) {
                h0 = lut[x & 0xffu];
                h1 = lut[(x >> 8) & 0xffu];
                h2 = lut[(x >> 16) & 0xffu];
                h3 = lut[x >> 24];
            } else {
                cvt_e2m1x8_f16x2(x, h0, h1, h2, h3);
                h0 = hmul2_u32(h0, sc[w]);
                h1 = hmul2_u32(h1, sc[w]);
                h2 = hmul2_u32(h2, sc[w]);
                h3 = hmul2_u32(h3, sc[w]);
            }
            mma_f16_16816(acc, qh0[2 * w], 0u, qh2[2 * w], 0u, h0, h1);
            mma_f16_16816(acc, qh0[2 * w + 1], 0u, qh2[2 * w + 1], 0u, h2, h3);
            if (QSPLIT) {
                mma_f16_16816(acc, ql0[2 * w], 0u, ql2[2 * w], 0u, h0, h1);
                mma_f16_16816(acc, ql0[2 * w + 1], 0u, ql2[2 * w + 1], 0u, h2, h3);
            }
        }
    } else {
        constexpr int NB = HD >= 128 ? HD / 128 : 1;  // 32-blocks in this lane's range
        uint32_t sb[NB];
        if (KM == B200_MXFP8) {
            const uint32_t emax = mx_row_emax<HD>(krow, ks.code_words);
            kappa *= pow2_e8m0(emax);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int blk = HD >= 128 ? c * NB + i : c >> 1;
                const int e = (int)((krow[ks.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu);
                sb[i] = pow2_f16x2(e - (int)emax, e - (int)emax);
            }
        }
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const uint32_t x = krow[c * STEPS + s];
            uint32_t h0 = cvt_e4m3x2_f16x2(x), h1 = cvt_e4m3x2_hi_f16x2(x);
            if (KM == B200_MXFP8) {
                h0 = hmul2_u32(h0, sb[(4 * s) / 32]);
                h1 = hmul2_u32(h1, sb[(4 * s) / 32]);
            }
            mma_f16_16816(acc, qh0[s], 0u, qh2[s], 0u, h0, h1);
            if (QSPLIT) mma_f16_16816(acc, ql0[s], 0u, ql2[s], 0u, h0, h1);
        }
    }
    return kappa;
}

// ---------------------------------------------------------------------------------------------
// V side metadata of one key: log2 of the f32 factor sigma = rsc0 [* 2^emax] (clamped; -inf -> the
// key adds nothing to the output) and the row's largest block exponent.
// ---------------------------------------------------------------------------------------------
template <int VM, int HD>
__device__ __forceinline__ void v_meta(const uint32_t *vrow, const DecodeSide &vs, float &lsig, bool &live, uint32_t &emax) {
    const float r0 = u2f(vrow[vs.rsc_off]);
    emax = 0;
    float l = fast_log2(r0);
    if (VM == B200_MXFP4 || VM == B200_MXFP8) {
        emax = mx_row_emax<HD>(vrow, vs.code_words);
        l += (float)((int)max(emax, 1u) - 127);
    }
    live = r0 > 0.0f && r0 < INFINITY;
    lsig = live ? fminf(fmaxf(l, -100.0f), 100.0f) : -100.0f;
}

// V fragments of one pair of keys (rows va, vb) for this lane's dims [g HD/8, (g+1) HD/8):
// lo[mt] = {va[2 mt], vb[2 mt]}, hi[mt] = {va[2 mt + 1], vb[2 mt + 1]} as f16x2.
template <int VM, int HD>
__device__ __forceinline__ void v_pair(const uint32_t *va, const uint32_t *vb, int g, const DecodeSide &vs,
                                       const uint32_t *lut, uint32_t ea, uint32_t eb, uint32_t (&lo)[HD / 16],
                                       uint32_t (&hi)[HD / 16]) {
    if (fmt_is4(VM)) {
        constexpr int WORDS = HD / 64 > 0 ? HD / 64 : 1;  // words per key of this lane (8 dims = 1 word at HD 64)
        constexpr int EPW = 8;
#pragma unroll
        for (int w = 0; w < WORDS; ++w) {
            const uint32_t xa = va[g * WORDS + w], xb = vb[g * WORDS + w];
            const uint32_t tl = (xa & 0x0f0f0f0fu) | ((xb & 0x0f0f0f0fu) << 4);
            const uint32_t th = ((xa >> 4) & 0x0f0f0f0fu) | (xb & 0xf0f0f0f0u);
            uint32_t l0, l1, l2, l3, h0, h1, h2, h3;
            if (VM == B200_TURBO_MSE) {
                l0 = lut[tl & 0xffu]; l1 = lut[(tl >> 8) & 0xffu]; l2 = lut[(tl >> 16) & 0xffu]; l3 = lut[tl >> 24];
                h0 = lut[th & 0xffu]; h1 = lut[(th >> 8) & 0xffu]; h2 = lut[(th >> 16) & 0xffu]; h3 = lut[th >> 24];
            } else {
                cvt_e2m1x8_f16x2(tl, l0, l1, l2, l3);
                cvt_e2m1x8_f16x2(th, h0, h1, h2, h3);
                uint32_t scl;
                const int d0 = g * (HD / 8) + EPW * w;
                if (VM == B200_MXFP4) {
                    const int blk = d0 / 32;
                    const int e0 = (int)((va[vs.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu);
                    const int e1 = (int)((vb[vs.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu);
                    scl = pow2_f16x2(e0 - (int)ea, e1 - (int)eb);
                } else {
                    const int blk = d0 / 16;
                    const uint32_t b0 = (va[vs.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu;
                    const uint32_t b1 = (vb[vs.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu;
                    scl = cvt_e4m3x2_f16x2(b0 | (b1 << 8));
                }
                l0 = hmul2_u32(l0, scl); l1 = hmul2_u32(l1, scl); l2 = hmul2_u32(l2, scl); l3 = hmul2_u32(l3, scl);
                h0 = hmul2_u32(h0, scl); h1 = hmul2_u32(h1, scl); h2 = hmul2_u32(h2, scl); h3 = hmul2_u32(h3, scl);
            }
            lo[4 * w] = l0; lo[4 * w + 1] = l1; lo[4 * w + 2] = l2; lo[4 * w + 3] = l3;
            hi[4 * w] = h0; hi[4 * w + 1] = h1; hi[4 * w + 2] = h2; hi[4 * w + 3] = h3;
        }
    } else {
        constexpr int WORDS = HD / 32;  // words per key of this lane
#pragma unroll
        for (int w = 0; w < WORDS; ++w) {
            const uint32_t xa = va[g * WORDS + w], xb = vb[g * WORDS + w];
            const uint32_t t0 = __byte_perm(xa, xb, 0x5140);  // a0 b0 a1 b1
            const uint32_t t1 = __byte_perm(xa, xb, 0x7362);  // a2 b2 a3 b3
            uint32_t l0 = cvt_e4m3x2_f16x2(t0), h0 = cvt_e4m3x2_hi_f16x2(t0);
            uint32_t l1 = cvt_e4m3x2_f16x2(t1), h1 = cvt_e4m3x2_hi_f16x2(t1);
            if (VM == B200_MXFP8) {
                const int blk = (g * (HD / 8) + 4 * w) / 32;
                const int e0 = (int)((va[vs.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu);
                const int e1 = (int)((vb[vs.code_words + (blk >> 2)] >> ((blk & 3) * 8)) & 0xffu);
                const uint32_t scl = pow2_f16x2(e0 - (int)ea, e1 - (int)eb);
                l0 = hmul2_u32(l0, scl); h0 = hmul2_u32(h0, scl); l1 = hmul2_u32(l1, scl); h1 = hmul2_u32(h1, scl);
            }
            lo[2 * w] = l0; hi[2 * w] = h0; lo[2 * w + 1] = l1; hi[2 * w + 1] = h1;
        }
    }
}

// In-place Walsh-Hadamard transform of `n` floats (power of two, n <= 32 * EPL... n <= 256 here) by
// one warp, with the sign vector applied before (rotate: y = H diag(s) x / sqrt(n)) or after
// (rotate back: x = diag(s) H y / sqrt(n)).
__device__ __forceinline__ void warp_hadamard(float *row, int n, const float *signs, bool signs_first, int lane) {
    float x[8];
    const int nk = (n + 31) / 32;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int j = lane + 32 * k;
        x[k] = (k < nk && j < n) ? row[j] * (signs_first ? signs[j] : 1.0f) : 0.0f;
    }
    for (int o = 1; o < 32 && o < n; o <<= 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float y = __shfl_xor_sync(0xffffffffu, x[k], o);
            x[k] = (lane & o) ? y - x[k] : x[k] + y;
        }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        if (o < nk) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (!(k & o)) {
                    const float a = x[k], c = x[k | o];
                    x[k] = a + c;
                    x[k | o] = a - c;
                }
            }
        }
    }
    const float s = 1.0f / sqrtf((float)n);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int j = lane + 32 * k;
        if (k < nk && j < n) row[j] = x[k] * s * (signs_first ? 1.0f : signs[j]);
    }
}

template <int KM, int VM, int HD, bool QSPLIT>
__global__ void __launch_bounds__(DW * 32) tq_decode_kernel(const DecodeParams p) {
    constexpr int STEPS = HD / 16;  // k-steps of q k^T == m-tiles of the output
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);                       // [DW][NS_MAX]
    const int NS = (int)p.ns;
    uint32_t *lut_k = reinterpret_cast<uint32_t *>(smem + 128);                // 256
    uint32_t *lut_v = lut_k + 256;                                             // 256
    float *mbuf = reinterpret_cast<float *>(smem + 128 + 2048);                // [DW][PACK][HD]
    float *m_M = mbuf + DW * PACK * HD;                                        // [DW][PACK]
    float *m_L = m_M + DW * PACK;                                              // [DW][PACK]
    uint8_t *stages = reinterpret_cast<uint8_t *>(m_L + DW * PACK);
    const uint32_t stage_bytes = p.k_stage_bytes + p.v_stage_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const uint32_t split = blockIdx.x, y = blockIdx.y, b = blockIdx.z;
    const uint32_t hk = y / p.packs, pack = y % p.packs;
    const uint32_t G = p.group, R = p.rows_per_kv;
    const long long lk_b = p.kv_len ? (long long)p.kv_len[b] : (long long)p.lk;

    // visible key range of query row r of this kv head (r = token * G + head in group)
    auto row_range = [&](uint32_t r, long long &lo, long long &hi, long long &pos) {
        const long long i = r / G;
        pos = i + lk_b - (long long)p.lq;
        lo = p.wl >= 0 ? max(pos - p.wl, 0ll) : 0ll;
        hi = p.wr >= 0 ? min(pos + p.wr + 1, lk_b) : lk_b;
        lo = min(lo, lk_b);
        hi = max(hi, lo);
    };
    long long LO = lk_b, HI = 0;
    for (uint32_t rr = 0; rr < PACK; ++rr) {
        const uint32_t r = pack * PACK + rr;
        if (r < R) {
            long long lo, hi, pos;
            row_range(r, lo, hi, pos);
            if (lo < hi) {
                LO = min(LO, lo);
                HI = max(HI, hi);
            }
        }
    }
    if (HI < LO) HI = LO;
    const uint32_t nsplit = (uint32_t)((HI - LO + p.chunk - 1) / p.chunk);
    if (split == 0 && tid == 0) p.meta[(size_t)b * gridDim.y + y] = (int32_t)nsplit;
    if (split >= max(nsplit, 1u)) return;
    const long long c_lo = LO + (long long)split * p.chunk;
    const long long c_hi = min(c_lo + (long long)p.chunk, HI);

    // this lane's query row (row g of the pack)
    const uint32_t my_r = pack * PACK + g;
    const bool my_valid = my_r < R;
    long long my_lo = 0, my_hi = 0, my_pos = 0;
    if (my_valid) row_range(my_r, my_lo, my_hi, my_pos);
    const uint32_t my_head = hk * G + (my_valid ? my_r % G : 0);
    const float my_slope = (p.alibi && my_valid) ? p.alibi[(size_t)b * p.alibi_bs + my_head] : 0.0f;

    // ------------------------------------------------------------------ prologue
    if (tid == 0) {
        for (int i = 0; i < DW * NS_MAX; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    if (KM == B200_TURBO_MSE)
        for (int i = tid; i < 256; i += DW * 32) lut_k[i] = pack_f16x2(p.k.tab[i & 15], p.k.tab[i >> 4]);
    if (VM == B200_TURBO_MSE)
        for (int i = tid; i < 256; i += DW * 32) lut_v[i] = pack_f16x2(p.v.tab[i & 15], p.v.tab[i >> 4]);
    // queries -> f32 rows in shared memory (rows of the pack; missing rows are zero)
    float *qbuf = mbuf;  // [PACK][HD]
    for (int idx = tid; idx < PACK * HD; idx += DW * 32) {
        const uint32_t rr = idx / HD, dd = idx % HD;
        const uint32_t r = pack * PACK + rr;
        float v = 0.0f;
        if (r < R) {
            const uint32_t i = r / G, h = hk * G + r % G;
            v = load_elem_rt(p.q, b * p.q_sb + h * p.q_sh + i * p.q_ss + dd, p.q_dtype);
        }
        qbuf[idx] = v;
    }
    __syncthreads();
    if (p.k.rot == B200_ROT_HADAMARD) {
        for (int rr = warp; rr < PACK; rr += DW) warp_hadamard(qbuf + rr * HD, HD, p.k.signs, true, lane);
        __syncthreads();
    }
    // power of two normalization of row g, then f16 fragments (hi / lo halves when QSPLIT)
    uint32_t qh0[STEPS], qh2[STEPS], ql0[STEPS], ql2[STEPS];
    float qscale;
    {
        const float *qr = qbuf + g * HD;
        float am = 0.0f;
        for (int dd = c; dd < HD; dd += 4) am = fmaxf(am, fabsf(qr[dd]));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        int e = 0;
        if (am > 0.0f && am < INFINITY) e = (int)((f2u(am) >> 23) & 0xffu) - 127 - 7;
        e = max(min(e, 100), -100);
        const float down = u2f((uint32_t)(127 - e) << 23), up = u2f((uint32_t)(127 + e) << 23);
        qscale = p.scale * up;
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const float *q4 = qr + c * (HD / 4) + 4 * s;
            const float x0 = q4[0] * down, x1 = q4[1] * down, x2 = q4[2] * down, x3 = q4[3] * down;
            qh0[s] = pack_f16x2(x0, x1);
            qh2[s] = pack_f16x2(x2, x3);
            if (QSPLIT) {
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&qh0[s]));
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&qh2[s]));
                ql0[s] = pack_f16x2(x0 - f0.x, x1 - f0.y);
                ql2[s] = pack_f16x2(x2 - f2.x, x3 - f2.y);
            } else {
                ql0[s] = 0u;
                ql2[s] = 0u;
            }
        }
    }
    __syncthreads();  // qbuf is reused by the merge; barriers are initialized

    // ------------------------------------------------------------------ per-warp key loop
    const uint32_t *kbase = p.k_rows + (size_t)b * p.k_sb + (size_t)hk * p.k_sh;
    const uint32_t *vbase = p.v_rows + (size_t)b * p.v_sb + (size_t)hk * p.v_sh;
    const uint32_t krb = (uint32_t)p.k_ss * 4u, vrb = (uint32_t)p.v_ss * 4u;  // row bytes
    const int ntiles = (int)((c_hi - c_lo + WK - 1) / WK);
    const int my_tiles = ntiles > warp ? (ntiles - warp + DW - 1) / DW : 0;
    uint8_t *wstage = stages + (size_t)warp * NS * stage_bytes;
    uint64_t *wbar = bars + warp * NS_MAX;
    bool wait_failed = false;

    // copies tile n of this warp into its stage n % NS
    auto issue = [&](int n) {
        const long long key0 = c_lo + (long long)(warp + n * DW) * WK;
        const int nkeys = (int)min((long long)WK, c_hi - key0);
        uint8_t *st = wstage + (size_t)(n % NS) * stage_bytes;
        const uintptr_t ka = reinterpret_cast<uintptr_t>(kbase) + (uintptr_t)key0 * krb;
        const uintptr_t va = reinterpret_cast<uintptr_t>(vbase) + (uintptr_t)key0 * vrb;
        const uintptr_t ka0 = ka & ~(uintptr_t)15, va0 = va & ~(uintptr_t)15;
        const uintptr_t ke = ka + (uintptr_t)nkeys * krb, ve = va + (uintptr_t)nkeys * vrb;
        // Rows below lk_b are readable; the 16-byte round up may only run past a tile that is not
        // the last one of its sequence. The last tile copies the round down and fetches the few
        // remaining words with plain loads.
        const bool last = key0 + nkeys >= lk_b;
        const uintptr_t ke1 = last ? (ke & ~(uintptr_t)15) : ((ke + 15) & ~(uintptr_t)15);
        const uintptr_t ve1 = last ? (ve & ~(uintptr_t)15) : ((ve + 15) & ~(uintptr_t)15);
        const uint32_t kb = ke1 > ka0 ? (uint32_t)(ke1 - ka0) : 0u, vb = ve1 > va0 ? (uint32_t)(ve1 - va0) : 0u;
        if (last) {
            if (lane < 4) {
                const uintptr_t a = ke1 + 4u * lane;
                if (a >= ka && a < ke) *reinterpret_cast<uint32_t *>(st + (a - ka0)) = *reinterpret_cast<const uint32_t *>(a);
            } else if (lane < 8) {
                const uintptr_t a = ve1 + 4u * (lane - 4);
                if (a >= va && a < ve)
                    *reinterpret_cast<uint32_t *>(st + p.k_stage_bytes + (a - va0)) = *reinterpret_cast<const uint32_t *>(a);
            }
            __syncwarp();
        }
        if (lane == 0) {
            mbar_expect_tx(&wbar[n % NS], kb + vb);
            if (kb) bulk_g2s(st, reinterpret_cast<const void *>(ka0), kb, &wbar[n % NS]);
            if (vb) bulk_g2s(st + p.k_stage_bytes, reinterpret_cast<const void *>(va0), vb, &wbar[n % NS]);
        }
    };

    float M = -INFINITY, lsum = 0.0f;  // row g: running max (log2 domain, value scale folded in), partial normalizer
    float oacc[STEPS][4];
#pragma unroll
    for (int mt = 0; mt < STEPS; ++mt) oacc[mt][0] = oacc[mt][1] = oacc[mt][2] = oacc[mt][3] = 0.0f;

    for (int n = 0; n < min(NS, my_tiles); ++n) issue(n);

    for (int n = 0; n < my_tiles; ++n) {
        if (!mbar_wait_bounded(&wbar[n % NS], (uint32_t)((n / NS) & 1))) {
            wait_failed = true;
            break;
        }
        const long long key0 = c_lo + (long long)(warp + n * DW) * WK;
        const int nkeys = (int)min((long long)WK, c_hi - key0);
        uint8_t *st = wstage + (size_t)(n % NS) * stage_bytes;
        const uint32_t koff = (uint32_t)((reinterpret_cast<uintptr_t>(kbase) + (uintptr_t)key0 * krb) & 15u);
        const uint32_t voff = (uint32_t)((reinterpret_cast<uintptr_t>(vbase) + (uintptr_t)key0 * vrb) & 15u);
        uint32_t *ktile = reinterpret_cast<uint32_t *>(st + koff);
        uint32_t *vtile = reinterpret_cast<uint32_t *>(st + p.k_stage_bytes + voff);
        if (nkeys < WK) {
            // rows past the chunk hold stale bytes: clear them so that masked keys decode to finite values
            const int nround = ((nkeys + 15) & ~15);
            for (uint32_t w = nkeys * p.k_ss + lane; w < nround * p.k_ss; w += 32) ktile[w] = 0u;
            for (uint32_t w = nkeys * p.v_ss + lane; w < nround * p.v_ss; w += 32) vtile[w] = 0u;
            __syncwarp();
        }
#pragma unroll 1
        for (int u = 0; u < WK / 16; ++u) {
            if (u * 16 >= nkeys) break;
            // ---- scores of 16 keys: two groups of 8 (lane's key: g)
            float sacc[2][4];
            float kap[2];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.0f;
                const uint32_t *krow = ktile + (size_t)(16 * u + 8 * nt + g) * p.k_ss;
                kap[nt] = qk_group<KM, HD, QSPLIT>(krow, c, p.k, lut_k, qh0, qh2, ql0, ql2, sacc[nt]);
            }
            // ---- value rows of this lane: keys 2c, 2c+1, 2c+8, 2c+9 of the 16
            const uint32_t *vr[4];
            float lsig[4];
            bool live[4];
            uint32_t vemax[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kk = 16 * u + 2 * c + (i & 1) + 8 * (i >> 1);
                vr[i] = vtile + (size_t)kk * p.v_ss;
                v_meta<VM, HD>(vr[i], p.v, lsig[i], live[i], vemax[i]);
            }
            // ---- online softmax for row g over the columns 2c, 2c+1 (group 0) and 8+2c, 9+2c (group 1)
            float s2[4], t2[4];
            float cmax = -INFINITY;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int nt = i >> 1, e = i & 1;
                const float kappa = __shfl_sync(0xffffffffu, kap[nt], (2 * c + e) * 4);
                const long long j = key0 + 16 * u + 8 * nt + 2 * c + e;
                float s = sacc[nt][e] * kappa * qscale;
                if (p.softcap > 0.0f) s = p.softcap * tanhf(s / p.softcap);
                if (my_slope != 0.0f) s -= my_slope * fabsf((float)(my_pos - j));
                const bool vis = my_valid && j >= my_lo && j < my_hi && j < c_hi;
                s2[i] = vis ? s * LOG2E : -INFINITY;
                t2[i] = vis ? s2[i] + lsig[i] : -INFINITY;
                cmax = fmaxf(cmax, t2[i]);
            }
            cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 1));
            cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 2));
            const float m_new = fmaxf(M, cmax);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const bool grew = m_new > M;
            if (__any_sync(0xffffffffu, grew)) {
                const float alpha = fast_exp2(M - m_use);  // 0 when M was -inf
                lsum *= alpha;
                const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * c) * 4);
                const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * c + 1) * 4);
#pragma unroll
                for (int mt = 0; mt < STEPS; ++mt) {
                    oacc[mt][0] *= a0;
                    oacc[mt][1] *= a1;
                    oacc[mt][2] *= a0;
                    oacc[mt][3] *= a1;
                }
            }
            M = m_new;
            float wgt[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lsum += fast_exp2(s2[i] - m_use);
                wgt[i] = live[i] ? fast_exp2(t2[i] - m_use) : 0.0f;
            }
            const uint32_t pb0 = pack_f16x2(wgt[0], wgt[1]), pb1 = pack_f16x2(wgt[2], wgt[3]);
            // ---- O^T += V^T P^T
            uint32_t lo0[STEPS], hi0[STEPS], lo1[STEPS], hi1[STEPS];
            v_pair<VM, HD>(vr[0], vr[1], g, p.v, lut_v, vemax[0], vemax[1], lo0, hi0);
            v_pair<VM, HD>(vr[2], vr[3], g, p.v, lut_v, vemax[2], vemax[3], lo1, hi1);
#pragma unroll
            for (int mt = 0; mt < STEPS; ++mt) mma_f16_16816(oacc[mt], lo0[mt], hi0[mt], lo1[mt], hi1[mt], pb0, pb1);
        }
        // the stage was read (and possibly patched) through the generic proxy: order that before the
        // bulk copy of the next tile into it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (n + NS < my_tiles) issue(n + NS);
    }
    if (wait_failed && p.status) atomicExch(p.status, 1);

    // ------------------------------------------------------------------ merge the warps
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
    __syncthreads();
    if (c == 0) {
        m_M[warp * PACK + g] = M;
        m_L[warp * PACK + g] = lsum;
    }
#pragma unroll
    for (int mt = 0; mt < STEPS; ++mt) {
        const int d0 = g * (HD / 8) + 2 * mt;
        float *o0 = mbuf + ((size_t)warp * PACK + 2 * c) * HD + d0;
        float *o1 = o0 + HD;
        *reinterpret_cast<float2 *>(o0) = make_float2(oacc[mt][0], oacc[mt][2]);
        *reinterpret_cast<float2 *>(o1) = make_float2(oacc[mt][1], oacc[mt][3]);
    }
    __syncthreads();
    // thread -> (row, slice of dims); the result of row rr goes to mbuf[rr] of warp slot 0
    constexpr int TPR = DW * 32 / PACK;  // threads per row
    constexpr int DPT = HD / TPR;        // dims per thread
    const int rr = tid / TPR, dsl = (tid % TPR) * DPT;
    float mstar = -INFINITY;
#pragma unroll
    for (int w = 0; w < DW; ++w) mstar = fmaxf(mstar, m_M[w * PACK + rr]);
    float L = 0.0f, f[DW];
#pragma unroll
    for (int w = 0; w < DW; ++w) {
        const float mw = m_M[w * PACK + rr];
        f[w] = mw == -INFINITY ? 0.0f : fast_exp2(mw - mstar);
        L += f[w] * m_L[w * PACK + rr];
    }
    const float invL = L > 0.0f ? 1.0f / L : 0.0f;
    float res[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        float a = 0.0f;
#pragma unroll
        for (int w = 0; w < DW; ++w) a += f[w] * mbuf[((size_t)w * PACK + rr) * HD + dsl + i];
        res[i] = a * invL;
    }
    const uint32_t r = pack * PACK + rr;
    if (nsplit > 1) {
        if (r < R) {
            const size_t slot = (((size_t)b * gridDim.y + y) * p.max_splits + split) * PACK + rr;
            float *po = p.part_o + slot * HD + dsl;
#pragma unroll
            for (int i = 0; i < DPT; ++i) po[i] = res[i];
            if (tid % TPR == 0) p.part_lse[slot] = L > 0.0f ? mstar * LN2 + logf(L) : -INFINITY;
        }
        return;
    }
    // single chunk: final rows (rotated back with the value signs when the cache is rotated)
    __syncthreads();
#pragma unroll
    for (int i = 0; i < DPT; ++i) mbuf[(size_t)rr * HD + dsl + i] = res[i];
    __syncthreads();
    if (p.v.rot == B200_ROT_HADAMARD) {
        for (int q = warp; q < PACK; q += DW) warp_hadamard(mbuf + q * HD, HD, p.v.signs, false, lane);
        __syncthreads();
    }
    if (r < R) {
        const uint32_t i0 = r / G, h = hk * G + r % G;
        const size_t obase = b * p.o_sb + h * p.o_sh + i0 * p.o_ss;
#pragma unroll
        for (int i = 0; i < DPT; ++i) store_elem_rt(p.out, obase + dsl + i, mbuf[(size_t)rr * HD + dsl + i], p.out_dtype);
    }
}

// Merges the chunks of one output row (candle-core/kernels/turbo_quant_impl.h:659-685), rotates it
// back and casts it. Rows whose block wrote the final result itself (one chunk) are skipped.
template <int HD>
__global__ void __launch_bounds__(128) tq_combine_kernel(const DecodeParams p) {
    __shared__ float rowbuf[4][HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rows = (size_t)p.b * p.hq * p.lq;
    const uint32_t ny = p.hkv * p.packs;
    for (size_t row = (size_t)blockIdx.x * 4 + warp; row < rows; row += (size_t)gridDim.x * 4) {
        const uint32_t i = (uint32_t)(row % p.lq);
        const uint32_t h = (uint32_t)((row / p.lq) % p.hq);
        const uint32_t b = (uint32_t)(row / ((size_t)p.lq * p.hq));
        const uint32_t hk = h / p.group, r = i * p.group + h % p.group;
        const uint32_t y = hk * p.packs + r / PACK, rr = r % PACK;
        const int ns = p.meta[(size_t)b * ny + y];
        if (ns <= 1) continue;
        const size_t slot0 = (((size_t)b * ny + y) * p.max_splits) * PACK + rr;
        float mx = -INFINITY;
        for (int s = 0; s < ns; ++s) mx = fmaxf(mx, p.part_lse[slot0 + (size_t)s * PACK]);
        float acc[HD / 32];
#pragma unroll
        for (int k = 0; k < HD / 32; ++k) acc[k] = 0.0f;
        float wsum = 0.0f;
        for (int s = 0; s < ns; ++s) {
            const float e = p.part_lse[slot0 + (size_t)s * PACK];
            const float w = e == -INFINITY ? 0.0f : expf(e - mx);
            wsum += w;
            if (w != 0.0f) {
                const float *po = p.part_o + (slot0 + (size_t)s * PACK) * HD;
#pragma unroll
                for (int k = 0; k < HD / 32; ++k) acc[k] += w * po[lane + 32 * k];
            }
        }
        float *rb = rowbuf[warp];
#pragma unroll
        for (int k = 0; k < HD / 32; ++k) rb[lane + 32 * k] = wsum > 0.0f ? acc[k] / wsum : 0.0f;
        __syncwarp();
        if (p.v.rot == B200_ROT_HADAMARD) {
            warp_hadamard(rb, HD, p.v.signs, false, lane);
            __syncwarp();
        }
        const size_t obase = b * p.o_sb + h * p.o_sh + i * p.o_ss;
#pragma unroll
        for (int k = 0; k < HD / 32; ++k) store_elem_rt(p.out, obase + lane + 32 * k, rb[lane + 32 * k], p.out_dtype);
        __syncwarp();
    }
}

}  // namespace b200
