// Decode attention over packed K/V rows (FP8, MXFP8, MXFP4, NVFP4, TurboQuant 4-bit): kernel body.
//
// Work split: block = (key chunk, pack of up to 8 query rows that share a kv head, batch entry).
// Each of the 4 warps streams its own 32-key tiles of the chunk through a private ring of shared
// memory stages filled by bulk copies (cp.async.bulk + mbarrier, no multicast), so no block-wide
// barrier sits in the key loop. Per tile the warp first derives the per-key scalars once (lane =
// key): f32 key scales, the value scale sigma = rsc0_v * 2^(largest block exponent) with its log2,
// and the f16 block scales of V relative to that exponent. Then per 16 keys it
//   1. dequantizes K in registers to f16 (packed cvt from e2m1 / e4m3, or a 256-entry pair table
//      for the codebook format) as the A operand of mma.sync m16n8k16 (rows = keys g and g + 8 of
//      lane (g, c)), with the f16 query fragments as B (columns = query rows). The contraction
//      index is permuted, identically for K and Q, so that a lane reads whole 32-bit words of its
//      rows. MX formats accumulate each 32-element block separately and apply the E8M0 block
//      scale times rsc0 in f32; the other formats apply rsc0 in f32 after the product;
//   2. runs the online softmax in f32 on the accumulator fragments (log2 domain). The value scale
//      is folded into the running maximum (M tracks s_j + log2 sigma_j), so the f16 weights
//      w_j = exp2(s_j - M) * sigma_j stay in range for value scales of any magnitude while the
//      normalizer sums exp2(s_j - M) in f32. M only moves when a score exceeds it by 2^8 (warp
//      vote), which keeps the cross-lane maximum out of the common path;
//   3. transposes the weights with movmatrix into the B operand of the second product and
//      dequantizes V as A = V^T (lane (g, c) owns keys {2c, 2c+1, 2c+8, 2c+9} x dims
//      [g D/8, (g+1) D/8); bytes or nibbles of two keys are interleaved before the packed cvt so
//      that the f16 pairs run along the contraction index): O^T += V^T P^T.
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
constexpr float MAX_SLACK = 8.0f;  // log2 of how far a score may exceed the running maximum before it moves
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
    uint32_t stages_bytes;  // whole stage area (also holds the query staging and the merge buffers)
};

__host__ __device__ constexpr bool fmt_is4(int m) { return m == B200_MXFP4 || m == B200_NVFP4 || m == B200_TURBO_MSE; }
__host__ __device__ constexpr bool fmt_is_mx(int m) { return m == B200_MXFP4 || m == B200_MXFP8; }
// f32 words of key metadata per key: one scale per 32-block (MX) or the row scale
__host__ __device__ constexpr int kmeta_words(int km, int hd) { return fmt_is_mx(km) ? (hd / 32 < 2 ? 2 : hd / 32) : 1; }
// f16 block scales of V per key
__host__ __device__ constexpr int vsc_blocks(int vm, int hd) { return fmt_is_mx(vm) ? hd / 32 : (vm == B200_NVFP4 ? hd / 16 : 0); }
__host__ __device__ constexpr int meta_bytes(int km, int vm, int hd) {
    return WK * (kmeta_words(km, hd) * 4 + 8 + vsc_blocks(vm, hd) * 2);
}
constexpr int FIXED_SMEM = 128 + 2048;  // barriers, pair tables

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts16(uint32_t a, uint32_t v) {
    asm volatile("{\n .reg .b16 t;\n cvt.u16.u32 t, %1;\n st.shared.u16 [%0], t;\n}" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// largest byte of a word
__device__ __forceinline__ uint32_t max_byte(uint32_t w) {
    const uint32_t m = __vmaxu4(w, w >> 16);
    return max(m & 0xffu, (m >> 8) & 0xffu);
}
// f16 bits of 2^d for d <= 0 (flushes to zero below 2^-14)
__device__ __forceinline__ uint32_t pow2_f16(int d) { return (uint32_t)max(d + 15, 0) << 10; }

// f16x2 pair table lookups (codebook format) or packed cvt of the four bytes of x
template <int M>
__device__ __forceinline__ void dq4(uint32_t x, uint32_t lut, uint32_t &h0, uint32_t &h1, uint32_t &h2, uint32_t &h3) {
    if constexpr (M == B200_TURBO_MSE) {
        h0 = lds32(lut + ((x & 0xffu) << 2));
        h1 = lds32(lut + ((x >> 6) & 0x3fcu));
        h2 = lds32(lut + ((x >> 14) & 0x3fcu));
        h3 = lds32(lut + ((x >> 22) & 0x3fcu));
    } else {
        cvt_e2m1x8_f16x2(x, h0, h1, h2, h3);
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

template <int KM, int VM, int HD>
__global__ void __launch_bounds__(DW * 32, 3) tq_decode_kernel(const DecodeParams p) {
    constexpr int STEPS = HD / 16;          // k-steps of K Q^T == m-tiles of the output
    constexpr bool K4 = fmt_is4(KM), V4 = fmt_is4(VM);
    constexpr bool KMX = fmt_is_mx(KM);     // block-wise accumulation, contraction order A
    constexpr int KMW = kmeta_words(KM, HD);
    constexpr int NBK = HD / 32;            // 32-blocks per row
    constexpr int NBV = vsc_blocks(VM, HD);
    constexpr int META = meta_bytes(KM, VM, HD);
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);  // [DW][NS_MAX]
    const int NS = (int)p.ns;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t lut_k = sbase + 128, lut_v = lut_k + 1024;
    uint8_t *stages = smem + FIXED_SMEM + DW * META;
    float *mbuf = reinterpret_cast<float *>(stages);  // [DW][PACK][HD], then M and L [DW][PACK]: used before / after the key loop
    const uint32_t stage_bytes = p.k_stage_bytes + p.v_stage_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const uint32_t split = blockIdx.x, y = blockIdx.y, b = blockIdx.z;
    const uint32_t hk = y / p.packs, pack = y % p.packs;
    const uint32_t G = p.group, R = p.rows_per_kv;
    const int lk_b = p.kv_len ? max(p.kv_len[b], 0) : (int)p.lk;

    // visible key range of query row r of this kv head (r = token * G + head in group)
    auto row_range = [&](uint32_t r, int &lo, int &hi, int &pos) {
        const long long i = r / G;
        const long long ps = i + (long long)lk_b - (long long)p.lq;
        long long l = p.wl >= 0 ? max(ps - p.wl, 0ll) : 0ll;
        long long h = p.wr >= 0 ? min(ps + p.wr + 1, (long long)lk_b) : (long long)lk_b;
        l = min(l, (long long)lk_b);
        h = max(h, l);
        lo = (int)l;
        hi = (int)h;
        pos = (int)max(min(ps, 2147483647ll), -2147483647ll);
    };
    int LO = lk_b, HI = 0, LOmax = 0, HImin = lk_b;
    for (uint32_t rr = 0; rr < PACK; ++rr) {
        const uint32_t r = pack * PACK + rr;
        if (r < R) {
            int lo, hi, pos;
            row_range(r, lo, hi, pos);
            if (lo < hi) {
                LO = min(LO, lo);
                HI = max(HI, hi);
            }
            LOmax = max(LOmax, lo);
            HImin = min(HImin, hi);
        }
    }
    if (HI < LO) HI = LO;
    const uint32_t nsplit = (uint32_t)(((long long)HI - LO + p.chunk - 1) / p.chunk);
    if (split == 0 && tid == 0 && p.meta) p.meta[(size_t)b * gridDim.y + y] = (int32_t)nsplit;
    if (split >= max(nsplit, 1u)) return;
    const int c_lo = LO + (int)(split * p.chunk);
    const int c_hi = (int)min((long long)c_lo + p.chunk, (long long)HI);
    const bool plain = p.softcap <= 0.0f && p.alibi == nullptr;  // tiles inside every row's range take the unmasked path

    // the two query rows whose scores this lane holds (columns 2c, 2c + 1 of the score fragments)
    int r_lo[2], r_hi[2], r_pos[2];
    float r_slope[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const uint32_t r = pack * PACK + 2 * c + e;
        r_lo[e] = r_hi[e] = r_pos[e] = 0;
        r_slope[e] = 0.0f;
        if (r < R) {
            row_range(r, r_lo[e], r_hi[e], r_pos[e]);
            r_hi[e] = min(r_hi[e], c_hi);
            if (p.alibi) r_slope[e] = p.alibi[(size_t)b * p.alibi_bs + hk * G + r % G];
        }
    }

    // ------------------------------------------------------------------ prologue
    if (tid == 0) {
        for (int i = 0; i < DW * NS_MAX; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    if constexpr (KM == B200_TURBO_MSE)
        for (int i = tid; i < 256; i += DW * 32) sts32(lut_k + 4 * i, pack_f16x2(p.k.tab[i & 15], p.k.tab[i >> 4]));
    if constexpr (VM == B200_TURBO_MSE)
        for (int i = tid; i < 256; i += DW * 32) sts32(lut_v + 4 * i, pack_f16x2(p.v.tab[i & 15], p.v.tab[i >> 4]));
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
    // power of two normalization of row g, then the f16 B fragments of K Q^T: per k-step the four
    // contraction slots of this lane are the consecutive dims dbase(s) ... dbase(s) + 3
    uint32_t qb0[STEPS], qb1[STEPS];
    float qs[2];  // softmax scale times the row's power of two, for the rows 2c and 2c + 1
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
        const float qscale = p.scale * up;
        qs[0] = __shfl_sync(0xffffffffu, qscale, (2 * c) * 4);
        qs[1] = __shfl_sync(0xffffffffu, qscale, (2 * c + 1) * 4);
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const int dbase = KMX ? 32 * (s >> 1) + 8 * c + 4 * (s & 1) : c * (HD / 4) + 4 * s;
            const float *q4 = qr + dbase;
            qb0[s] = pack_f16x2(q4[0] * down, q4[1] * down);
            qb1[s] = pack_f16x2(q4[2] * down, q4[3] * down);
        }
    }
    __syncthreads();  // qbuf lives in the stage area; barriers are initialized

    // ------------------------------------------------------------------ per-warp key loop
    const uint32_t *kbase = p.k_rows + (size_t)b * p.k_sb + (size_t)hk * p.k_sh;
    const uint32_t *vbase = p.v_rows + (size_t)b * p.v_sb + (size_t)hk * p.v_sh;
    const uint32_t krb = (uint32_t)p.k_ss * 4u, vrb = (uint32_t)p.v_ss * 4u;  // row bytes
    const int ntiles = (c_hi - c_lo + WK - 1) / WK;
    const int my_tiles = ntiles > warp ? (ntiles - warp + DW - 1) / DW : 0;
    uint8_t *wstage = stages + (size_t)warp * NS * stage_bytes;
    const uint32_t wstage_s = smem_u32(wstage);
    uint64_t *wbar = bars + warp * NS_MAX;
    const uint32_t meta_s = sbase + FIXED_SMEM + warp * META;    // [WK][KMW] f32
    const uint32_t vmeta_s = meta_s + WK * KMW * 4;              // [WK] (sigma, log2 sigma)
    const uint32_t vsc_s = vmeta_s + WK * 8;                     // [NBV][WK] f16
    const uint32_t k_cw4 = (uint32_t)p.k.code_words * 4u, k_rsc4 = (uint32_t)p.k.rsc_off * 4u;
    const uint32_t v_cw4 = (uint32_t)p.v.code_words * 4u, v_rsc4 = (uint32_t)p.v.rsc_off * 4u;
    bool wait_failed = false;

    // copies tile n of this warp into its stage n % NS
    auto issue = [&](int n) {
        const int key0 = c_lo + (warp + n * DW) * WK;
        const int nkeys = min(WK, c_hi - key0);
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

    // running maxima (log2 domain, value scale folded in) and partial normalizers of rows 2c, 2c + 1
    float M[2] = {-1e30f, -1e30f}, lsum[2] = {0.0f, 0.0f};
    float oacc[STEPS][4];
#pragma unroll
    for (int mt = 0; mt < STEPS; ++mt) oacc[mt][0] = oacc[mt][1] = oacc[mt][2] = oacc[mt][3] = 0.0f;

    // lane offsets inside a tile: K rows g (and g + 8), V rows 2c (and 2c + 1, 2c + 8, 2c + 9)
    const uint32_t k_lane = g * krb + (KMX ? (K4 ? 4u * c : 8u * c) : (K4 ? c * (HD / 8) : c * (HD / 4)));
    const uint32_t v_lane = 2 * c * vrb + (V4 ? g * (HD / 16) : g * (HD / 8));

    for (int n = 0; n < min(NS, my_tiles); ++n) issue(n);

    for (int n = 0; n < my_tiles; ++n) {
        if (!mbar_wait_bounded(&wbar[n % NS], (uint32_t)((n / NS) & 1))) {
            wait_failed = true;
            break;
        }
        const int key0 = c_lo + (warp + n * DW) * WK;
        const int nkeys = min(WK, c_hi - key0);
        const uint32_t st_s = wstage_s + (uint32_t)(n % NS) * stage_bytes;
        const uint32_t kt = st_s + (uint32_t)((reinterpret_cast<uintptr_t>(kbase) + (uintptr_t)key0 * krb) & 15u);
        const uint32_t vt = st_s + p.k_stage_bytes + (uint32_t)((reinterpret_cast<uintptr_t>(vbase) + (uintptr_t)key0 * vrb) & 15u);
        if (nkeys < WK) {
            // rows past the chunk hold stale bytes: clear them so that masked keys decode to finite values
            const uint32_t nround = (uint32_t)((nkeys + 15) & ~15);
            for (uint32_t w = nkeys * (krb >> 2) + lane; w < nround * (krb >> 2); w += 32) sts32(kt + 4 * w, 0u);
            for (uint32_t w = nkeys * (vrb >> 2) + lane; w < nround * (vrb >> 2); w += 32) sts32(vt + 4 * w, 0u);
            __syncwarp();
        }
        // ---- per-key scalars of the tile, lane = key
        {
            const bool have = lane < ((nkeys + 15) & ~15);
            const uint32_t kr = kt + lane * krb, vr = vt + lane * vrb;
            const float k0 = have ? u2f(lds32(kr + k_rsc4)) : 0.0f;
            if constexpr (KMX) {
#pragma unroll
                for (int w = 0; w < (NBK + 3) / 4; ++w) {
                    const uint32_t aux = have ? lds32(kr + k_cw4 + 4 * w) : 0u;
#pragma unroll
                    for (int i = 0; i < 4 && 4 * w + i < KMW; ++i) {
                        const uint32_t e = (aux >> (8 * i)) & 0xffu;
                        sts32(meta_s + (lane * KMW + 4 * w + i) * 4, f2u(e ? k0 * u2f(e << 23) : 0.0f));
                    }
                }
            } else {
                sts32(meta_s + lane * 4, f2u(k0));
            }
            const float v0 = have ? u2f(lds32(vr + v_rsc4)) : 0.0f;
            float sigma = v0;
            if constexpr (fmt_is_mx(VM)) {
                uint32_t aux[(NBV + 3) / 4];
                uint32_t em = 0;
#pragma unroll
                for (int w = 0; w < (NBV + 3) / 4; ++w) {
                    aux[w] = have ? lds32(vr + v_cw4 + 4 * w) : 0u;
                    em = w == 0 ? aux[w] : __vmaxu4(em, aux[w]);
                }
                const uint32_t emax = max_byte(em);
                sigma = emax ? v0 * u2f(emax << 23) : 0.0f;
#pragma unroll
                for (int bk = 0; bk < NBV; ++bk) {
                    const int e = (int)((aux[bk >> 2] >> (8 * (bk & 3))) & 0xffu);
                    sts16(vsc_s + (bk * WK + lane) * 2, pow2_f16(e - (int)emax));
                }
            } else if constexpr (VM == B200_NVFP4) {
#pragma unroll
                for (int w = 0; w < NBV / 4; ++w) {
                    const uint32_t aux = have ? lds32(vr + v_cw4 + 4 * w) : 0u;
                    const uint32_t lo = cvt_e4m3x2_f16x2(aux), hi = cvt_e4m3x2_hi_f16x2(aux);
                    sts16(vsc_s + ((4 * w) * WK + lane) * 2, lo & 0xffffu);
                    sts16(vsc_s + ((4 * w + 1) * WK + lane) * 2, lo >> 16);
                    sts16(vsc_s + ((4 * w + 2) * WK + lane) * 2, hi & 0xffffu);
                    sts16(vsc_s + ((4 * w + 3) * WK + lane) * 2, hi >> 16);
                }
            }
            const bool live = sigma > 0.0f && sigma < INFINITY;
            const float sc = live ? fminf(fmaxf(sigma, 7.8886091e-31f), 1.2676506e30f) : 0.0f;  // 2^-100 ... 2^100
            sts32(vmeta_s + lane * 8, f2u(sc));
            sts32(vmeta_s + lane * 8 + 4, f2u(live ? fast_log2(sc) : -100.0f));
            __syncwarp();
        }
        const bool full = plain && nkeys == WK && key0 >= LOmax && key0 + WK <= HImin;
#pragma unroll
        for (int u = 0; u < WK / 16; ++u) {
            if (u * 16 < nkeys) {
                // ---- scores of keys g and g + 8 of the 16 against the rows 2c, 2c + 1
                const uint32_t ka = kt + k_lane + u * 16 * krb, ka8 = ka + 8 * krb;
                float sr[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if constexpr (KMX) {
                    float ks0[KMW], ks8[KMW];
                    if constexpr (KMW == 2) {
                        const float2 a = lds64f(meta_s + (16 * u + g) * 8), b8 = lds64f(meta_s + (16 * u + 8 + g) * 8);
                        ks0[0] = a.x; ks0[1] = a.y; ks8[0] = b8.x; ks8[1] = b8.y;
                    } else {
#pragma unroll
                        for (int w = 0; w < KMW / 4; ++w) {
                            const float4 a = lds128f(meta_s + ((16 * u + g) * KMW + 4 * w) * 4);
                            const float4 b8 = lds128f(meta_s + ((16 * u + 8 + g) * KMW + 4 * w) * 4);
                            ks0[4 * w] = a.x; ks0[4 * w + 1] = a.y; ks0[4 * w + 2] = a.z; ks0[4 * w + 3] = a.w;
                            ks8[4 * w] = b8.x; ks8[4 * w + 1] = b8.y; ks8[4 * w + 2] = b8.z; ks8[4 * w + 3] = b8.w;
                        }
                    }
#pragma unroll
                    for (int bk = 0; bk < NBK; ++bk) {
                        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if constexpr (K4) {
                            const uint32_t x0 = lds32(ka + 16 * bk), x8 = lds32(ka8 + 16 * bk);
                            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                            cvt_e2m1x8_f16x2(x0, a0, a1, a2, a3);
                            cvt_e2m1x8_f16x2(x8, b0, b1, b2, b3);
                            mma_f16_16816(acc, a0, b0, a1, b1, qb0[2 * bk], qb1[2 * bk]);
                            mma_f16_16816(acc, a2, b2, a3, b3, qb0[2 * bk + 1], qb1[2 * bk + 1]);
                        } else {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const uint32_t x0 = lds32(ka + 32 * bk + 4 * h), x8 = lds32(ka8 + 32 * bk + 4 * h);
                                mma_f16_16816(acc, cvt_e4m3x2_f16x2(x0), cvt_e4m3x2_f16x2(x8), cvt_e4m3x2_hi_f16x2(x0),
                                              cvt_e4m3x2_hi_f16x2(x8), qb0[2 * bk + h], qb1[2 * bk + h]);
                            }
                        }
                        sr[0] = fmaf(acc[0], ks0[bk], sr[0]);
                        sr[1] = fmaf(acc[1], ks0[bk], sr[1]);
                        sr[2] = fmaf(acc[2], ks8[bk], sr[2]);
                        sr[3] = fmaf(acc[3], ks8[bk], sr[3]);
                    }
                } else {
                    if constexpr (K4) {
                        constexpr int WPL = HD / 32;  // words of this lane per key
                        uint32_t sg[WPL > 1 ? WPL / 2 : 1], sg8[WPL > 1 ? WPL / 2 : 1];
                        if constexpr (KM == B200_NVFP4) {
                            // E4M3 block scales of the lane's 16-blocks c * (HD / 64) ..., as f16x2 {s, s}
#pragma unroll
                            for (int i = 0; i < HD / 64; ++i) {
                                const int blk = c * (HD / 64) + i;
                                const uint32_t off = k_cw4 + (uint32_t)(blk & ~3) - c * (HD / 8);  // from the lane's first code byte
                                const uint32_t w0 = lds32(ka + off), w8 = lds32(ka8 + off);
                                const uint32_t b0 = (w0 >> (8 * (blk & 3))) & 0xffu, b8 = (w8 >> (8 * (blk & 3))) & 0xffu;
                                sg[i] = cvt_e4m3x2_f16x2(b0 | (b0 << 8));
                                sg8[i] = cvt_e4m3x2_f16x2(b8 | (b8 << 8));
                            }
                        }
#pragma unroll
                        for (int w = 0; w < WPL; ++w) {
                            const uint32_t x0 = lds32(ka + 4 * w), x8 = lds32(ka8 + 4 * w);
                            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                            dq4<KM>(x0, lut_k, a0, a1, a2, a3);
                            dq4<KM>(x8, lut_k, b0, b1, b2, b3);
                            if constexpr (KM == B200_NVFP4) {
                                const uint32_t s0 = sg[w / 2], s8 = sg8[w / 2];
                                a0 = hmul2_u32(a0, s0); a1 = hmul2_u32(a1, s0); a2 = hmul2_u32(a2, s0); a3 = hmul2_u32(a3, s0);
                                b0 = hmul2_u32(b0, s8); b1 = hmul2_u32(b1, s8); b2 = hmul2_u32(b2, s8); b3 = hmul2_u32(b3, s8);
                            }
                            mma_f16_16816(sr, a0, b0, a1, b1, qb0[2 * w], qb1[2 * w]);
                            mma_f16_16816(sr, a2, b2, a3, b3, qb0[2 * w + 1], qb1[2 * w + 1]);
                        }
                    } else {
#pragma unroll
                        for (int s = 0; s < STEPS; ++s) {
                            const uint32_t x0 = lds32(ka + 4 * s), x8 = lds32(ka8 + 4 * s);
                            mma_f16_16816(sr, cvt_e4m3x2_f16x2(x0), cvt_e4m3x2_f16x2(x8), cvt_e4m3x2_hi_f16x2(x0),
                                          cvt_e4m3x2_hi_f16x2(x8), qb0[s], qb1[s]);
                        }
                    }
                    const float kp0 = u2f(lds32(meta_s + (16 * u + g) * 4)), kp8 = u2f(lds32(meta_s + (16 * u + 8 + g) * 4));
                    sr[0] *= kp0; sr[1] *= kp0; sr[2] *= kp8; sr[3] *= kp8;
                }
                // ---- online softmax: sr[2 k + e] = key (g + 8 k), row 2c + e
                const float2 vm0 = lds64f(vmeta_s + (16 * u + g) * 8), vm8 = lds64f(vmeta_s + (16 * u + 8 + g) * 8);
                float s2[4];
                if (full) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) s2[i] = sr[i] * (qs[i & 1] * LOG2E);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int e = i & 1, j = key0 + 16 * u + g + 8 * (i >> 1);
                        float s = sr[i] * qs[e];
                        if (p.softcap > 0.0f) s = p.softcap * tanhf(s / p.softcap);
                        if (r_slope[e] != 0.0f) s -= r_slope[e] * fabsf((float)(r_pos[e] - j));
                        s2[i] = (j >= r_lo[e] && j < r_hi[e]) ? s * LOG2E : -INFINITY;
                    }
                }
                const float t0 = s2[0] + vm0.y, t1 = s2[1] + vm0.y, t2 = s2[2] + vm8.y, t3 = s2[3] + vm8.y;
                const bool grow = fmaxf(t0, t2) > M[0] + MAX_SLACK || fmaxf(t1, t3) > M[1] + MAX_SLACK;
                if (__any_sync(0xffffffffu, grow)) {
                    float c0 = fmaxf(t0, t2), c1 = fmaxf(t1, t3);
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) {
                        c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, o));
                        c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, o));
                    }
                    const float n0 = fmaxf(M[0], c0), n1 = fmaxf(M[1], c1);
                    const float al0 = fast_exp2(M[0] - n0), al1 = fast_exp2(M[1] - n1);
                    M[0] = n0;
                    M[1] = n1;
                    lsum[0] *= al0;
                    lsum[1] *= al1;
#pragma unroll
                    for (int mt = 0; mt < STEPS; ++mt) {
                        oacc[mt][0] *= al0;
                        oacc[mt][1] *= al1;
                        oacc[mt][2] *= al0;
                        oacc[mt][3] *= al1;
                    }
                }
                const float p0 = fast_exp2(s2[0] - M[0]), p1 = fast_exp2(s2[1] - M[1]);
                const float p2 = fast_exp2(s2[2] - M[0]), p3 = fast_exp2(s2[3] - M[1]);
                lsum[0] += p0 + p2;
                lsum[1] += p1 + p3;
                const uint32_t pb0 = movmatrix_trans(pack_f16x2(p0 * vm0.x, p1 * vm0.x));
                const uint32_t pb1 = movmatrix_trans(pack_f16x2(p2 * vm8.x, p3 * vm8.x));
                // ---- O^T += V^T P^T: keys 2c, 2c+1 | 2c+8, 2c+9 of the 16, dims [g HD/8, (g+1) HD/8)
                const uint32_t va = vt + v_lane + u * 16 * vrb;
#pragma unroll
                for (int w = 0; w < (V4 ? (HD / 64 > 0 ? HD / 64 : 1) : HD / 32); ++w) {
                    const uint32_t xa = lds32(va + 4 * w), xb = lds32(va + vrb + 4 * w);
                    const uint32_t xc = lds32(va + 8 * vrb + 4 * w), xd = lds32(va + 9 * vrb + 4 * w);
                    if constexpr (V4) {
                        // nibbles of two keys side by side: byte i = (a[2i], b[2i]) and (a[2i+1], b[2i+1])
                        const uint32_t tl0 = (xa & 0x0f0f0f0fu) | ((xb & 0x0f0f0f0fu) << 4);
                        const uint32_t th0 = ((xa >> 4) & 0x0f0f0f0fu) | (xb & 0xf0f0f0f0u);
                        const uint32_t tl1 = (xc & 0x0f0f0f0fu) | ((xd & 0x0f0f0f0fu) << 4);
                        const uint32_t th1 = ((xc >> 4) & 0x0f0f0f0fu) | (xd & 0xf0f0f0f0u);
                        uint32_t l0[4], h0[4], l1[4], h1[4];
                        dq4<VM>(tl0, lut_v, l0[0], l0[1], l0[2], l0[3]);
                        dq4<VM>(th0, lut_v, h0[0], h0[1], h0[2], h0[3]);
                        dq4<VM>(tl1, lut_v, l1[0], l1[1], l1[2], l1[3]);
                        dq4<VM>(th1, lut_v, h1[0], h1[1], h1[2], h1[3]);
                        if constexpr (NBV > 0) {
                            const int d0 = g * (HD / 8) + 8 * w;  // first dim of this word
                            const int blk = d0 / (HD / NBV);
                            const uint32_t sa = lds32(vsc_s + (blk * WK + 16 * u + 2 * c) * 2);
                            const uint32_t sb = lds32(vsc_s + (blk * WK + 16 * u + 8 + 2 * c) * 2);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                l0[i] = hmul2_u32(l0[i], sa); h0[i] = hmul2_u32(h0[i], sa);
                                l1[i] = hmul2_u32(l1[i], sb); h1[i] = hmul2_u32(h1[i], sb);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) mma_f16_16816(oacc[4 * w + i], l0[i], h0[i], l1[i], h1[i], pb0, pb1);
                    } else {
                        const uint32_t ta0 = __byte_perm(xa, xb, 0x5140), ta1 = __byte_perm(xa, xb, 0x7362);
                        const uint32_t tb0 = __byte_perm(xc, xd, 0x5140), tb1 = __byte_perm(xc, xd, 0x7362);
                        uint32_t l0 = cvt_e4m3x2_f16x2(ta0), h0 = cvt_e4m3x2_hi_f16x2(ta0);
                        uint32_t l1 = cvt_e4m3x2_f16x2(tb0), h1 = cvt_e4m3x2_hi_f16x2(tb0);
                        uint32_t l2 = cvt_e4m3x2_f16x2(ta1), h2 = cvt_e4m3x2_hi_f16x2(ta1);
                        uint32_t l3 = cvt_e4m3x2_f16x2(tb1), h3 = cvt_e4m3x2_hi_f16x2(tb1);
                        if constexpr (NBV > 0) {
                            const int blk = (g * (HD / 8) + 4 * w) / 32;
                            const uint32_t sa = lds32(vsc_s + (blk * WK + 16 * u + 2 * c) * 2);
                            const uint32_t sb = lds32(vsc_s + (blk * WK + 16 * u + 8 + 2 * c) * 2);
                            l0 = hmul2_u32(l0, sa); h0 = hmul2_u32(h0, sa); l2 = hmul2_u32(l2, sa); h2 = hmul2_u32(h2, sa);
                            l1 = hmul2_u32(l1, sb); h1 = hmul2_u32(h1, sb); l3 = hmul2_u32(l3, sb); h3 = hmul2_u32(h3, sb);
                        }
                        mma_f16_16816(oacc[2 * w], l0, h0, l1, h1, pb0, pb1);
                        mma_f16_16816(oacc[2 * w + 1], l2, h2, l3, h3, pb0, pb1);
                    }
                }
            }
        }
        // the stage was read (and possibly patched) through the generic proxy: order that before the
        // bulk copy of the next tile into it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (n + NS < my_tiles) issue(n + NS);
    }
    if (wait_failed && p.status) atomicExch(p.status, 1);

    // ------------------------------------------------------------------ merge the warps
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        lsum[0] += __shfl_xor_sync(0xffffffffu, lsum[0], o);
        lsum[1] += __shfl_xor_sync(0xffffffffu, lsum[1], o);
    }
    __syncthreads();  // every warp is done with its stages: the area becomes the merge buffer
    float *m_M = mbuf + DW * PACK * HD, *m_L = m_M + DW * PACK;
    if (g == 0) {
        m_M[warp * PACK + 2 * c] = M[0];
        m_M[warp * PACK + 2 * c + 1] = M[1];
        m_L[warp * PACK + 2 * c] = lsum[0];
        m_L[warp * PACK + 2 * c + 1] = lsum[1];
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
    // thread -> (row, slice of dims)
    constexpr int TPR = DW * 32 / PACK;  // threads per row
    constexpr int DPT = HD / TPR;        // dims per thread
    const int rr = tid / TPR, dsl = (tid % TPR) * DPT;
    float mstar = -1e30f;
#pragma unroll
    for (int w = 0; w < DW; ++w) mstar = fmaxf(mstar, m_M[w * PACK + rr]);
    float L = 0.0f, f[DW];
#pragma unroll
    for (int w = 0; w < DW; ++w) {
        f[w] = fast_exp2(m_M[w * PACK + rr] - mstar);
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
