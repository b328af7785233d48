// Attention over dense (uncompressed) K / V: b200_flash_attn and b200_fa_prefill_append.
//
// One kernel serves decode and prefill. The query rows that share a kv head are packed into one row
// space (row = token * group + head in group), so a tile of 64 rows reuses every K / V tile for all
// the heads of the group. Block = 4 warps x 16 rows; K and V tiles of 64 keys are double buffered
// in shared memory with cp.async (16-byte chunks, rows padded by 16 bytes so that ldmatrix reads are
// conflict free); S = Q K^T and O += P V run on mma.sync m16n8k16 (f16 or bf16 operands, f32
// accumulation) with the online softmax in registers. FP8 (E4M3) K / V are widened to the query
// dtype while they are stored to shared memory. Few row tiles (decode) are split along the keys
// into partial results that fa_combine_kernel merges.
//
// Semantics: candle-core/kernels/flash_attn_impl.h (fa_row*, fa2_*, fa3_*, fa_combine_*): bottom
// right aligned windows, softcap, ALiBi, k / v descale, varlen through cumulative offsets, zeros
// for rows without a visible key; output row (token, head) of d contiguous elements.
#include <algorithm>
#include <atomic>
#include <mutex>
#include <cuda_bf16.h>

#include "common.cuh"
#include "fa_params.cuh"

namespace b200 {

constexpr int FA_BM = 64, FA_BN = 64, FA_WARPS = 4;
constexpr float LOG2E_F = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool pred) {
    const int n = pred ? 16 : 0;  // zero fill when the row is outside the tile
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t d;
    if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <bool BF16>
__device__ __forceinline__ uint16_t to16(float f) {
    return BF16 ? f_to_bf16_bits(f) : f_to_f16_bits(f);
}

// HD: the head dim bucket (64, 128 or 256: the smallest one that holds p.d, like the dmax of the reference's tile
// kernels, candle-core/src/accel/attention.rs:428-435); the rows' elements d .. HD - 1 are zeros in shared memory and
// are not stored. BF16: the mma operand type (bf16, else f16). Queries, keys and values of another dtype (f32
// everywhere, E4M3 or f32 keys and values) are rounded to it on their way into shared memory.
// DEC (decode: the kv head's packed rows fit one 16-row group): the four warps share the keys of every tile instead of
// the tile's rows. Each takes 16 of its 64 keys for the same 16 rows, with a running maximum and partial sums of its
// own; the four partial results are merged through shared memory when the keys are done. Without it three of the four
// warps would run the products and the softmax of rows that do not exist.
template <int HD, bool BF16, bool DEC>
__global__ void __launch_bounds__(FA_WARPS * 32) fa_dense_kernel(const FaParams p) {
    constexpr int ROWB = HD * 2 + 16;          // padded row bytes in shared memory
    constexpr int KSTEPS = HD / 16, NT = HD / 8;
    constexpr int CH = HD / 8;                 // 16-byte chunks per row
    constexpr bool QREG = HD <= 128;           // the Q fragments stay in registers; at 256 they are re-read per k step
    constexpr int KG = DEC ? 1 : FA_BN / 16;   // groups of 16 keys of a tile that one warp takes
    constexpr int QROWS = DEC ? 16 : FA_BM;    // rows of the Q tile in shared memory
    const uint32_t D = p.d;                    // elements per row in memory (a multiple of 8, at most HD)
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sQ = smem_u32(smem);                       // [QROWS][ROWB]
    const uint32_t sK = sQ + QROWS * ROWB;                    // 2 x [FA_BN][ROWB]
    const uint32_t sV = sK + 2 * FA_BN * ROWB;                // 2 x [FA_BN][ROWB]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int wrow = DEC ? 0 : warp;           // the warp's group of 16 rows
    const int kg0 = DEC ? warp : 0;            // its first group of 16 keys
    const uint32_t hk = blockIdx.y;
    const uint32_t b = blockIdx.z / p.n_splits, split = blockIdx.z % p.n_splits;
    const uint32_t G = p.group;
    uint32_t lq = p.lq, lk = p.lk;
    uint64_t q0 = (uint64_t)b * p.lq, k0 = 0;
    if (p.varlen) {
        q0 = p.cu_q[b];
        lq = p.cu_q[b + 1] - p.cu_q[b];
        k0 = p.cu_k[b];
        lk = p.cu_k[b + 1] - p.cu_k[b];
    }
    if (p.pages) lk = min(lk, p.pg_keys[p.n_pages]);  // the keys of a paged call are the valid rows of its blocks
    const uint32_t R = lq * G;  // packed rows of this kv head
    const uint32_t row0 = blockIdx.x * FA_BM;
    if (row0 >= R) return;
    const char *qb = reinterpret_cast<const char *>(p.q);
    const uint64_t kv_esize = p.kv_kind == 0 ? 2 : (p.kv_kind == 1 ? 1 : 4);
    const char *kb = reinterpret_cast<const char *>(p.k) + (p.varlen ? k0 * p.k_ss + hk * p.k_sh : b * p.k_sb + hk * p.k_sh) * kv_esize;
    const char *vb = reinterpret_cast<const char *>(p.v) + (p.varlen ? k0 * p.v_ss + hk * p.v_sh : b * p.v_sb + hk * p.v_sh) * kv_esize;

    // key range of the tile: from the lowest lower bound (first row) to the highest upper bound (last row)
    auto range_of = [&](uint32_t r, long long &lo, long long &hi, long long &pos) {
        const long long i = r / G;
        pos = i + (long long)lk - (long long)lq;
        lo = p.wl >= 0 ? max(pos - p.wl, 0ll) : 0ll;
        hi = p.wr >= 0 ? min(pos + p.wr + 1, (long long)lk) : (long long)lk;
        lo = min(lo, (long long)lk);
        hi = max(hi, lo);
    };
    long long t_lo, t_hi, tmp0, tmp1, tmp2;
    range_of(row0, t_lo, tmp0, tmp1);
    range_of(min(row0 + FA_BM, R) - 1, tmp0, t_hi, tmp2);
    if (t_hi < t_lo) t_hi = t_lo;
    // this split's share of the range, in whole tiles
    const long long ntile_all = (t_hi - t_lo + FA_BN - 1) / FA_BN;
    const long long per = (ntile_all + p.n_splits - 1) / p.n_splits;
    const long long s_lo = t_lo + (long long)split * per * FA_BN;
    const long long s_hi = min(s_lo + per * FA_BN, t_hi);
    const int ntiles = s_hi > s_lo ? (int)((s_hi - s_lo + FA_BN - 1) / FA_BN) : 0;

    // ---- Q tile -> shared memory (any alignment), then A fragments in registers
    for (int idx = tid; idx < QROWS * HD; idx += FA_WARPS * 32) {
        const uint32_t rr = idx / HD, dd = idx % HD, r = row0 + rr;
        uint16_t v = 0;
        if (r < R) {
            const uint32_t i = r / G, h = hk * G + r % G;
            const uint64_t off = (p.varlen ? (q0 + i) * p.q_ss : b * p.q_sb + i * p.q_ss) + h * p.q_sh + dd;
            if (dd < D) v = (p.q_dtype == B200_F32) ? to16<BF16>(reinterpret_cast<const float *>(qb)[off]) : reinterpret_cast<const uint16_t *>(qb)[off];
        }
        *reinterpret_cast<uint16_t *>(smem + rr * ROWB + dd * 2) = v;
    }
    // Paged K / V: the addresses of a tile's 64 rows, found by its first 64 threads in the block table (block i holds
    // the keys pg_keys[i] .. pg_keys[i + 1] - 1 at rows 0 .. of its (batch entry, kv head) slab) and left in shared memory
    // behind the tiles; `cursor` is a block at or before the tile's first key (tiles are loaded in ascending order).
    const char **row_k = reinterpret_cast<const char **>(smem + QROWS * ROWB + 4 * FA_BN * ROWB);
    const char **row_v = row_k + FA_BN;
    uint32_t *cursor = reinterpret_cast<uint32_t *>(row_v + FA_BN);
    if (p.pages && tid == 0) {
        // the block that holds the split's first key: binary search over the prefix sums, once per block of threads
        uint32_t lo = 0, hi = p.n_pages;
        while (lo + 1 < hi) {
            const uint32_t mid = (lo + hi) / 2;
            if ((long long)p.pg_keys[mid] <= s_lo) lo = mid;
            else hi = mid;
        }
        *cursor = lo;
    }
    auto locate_rows = [&](long long j0) {
        __syncthreads();  // the table of the previous tile has been read, the cursor is visible
        if (tid < FA_BN) {
            const long long j = j0 + tid;
            const char *kr = nullptr, *vr = nullptr;
            uint32_t pg = *cursor;
            if (j < s_hi) {
                while (pg + 1 < p.n_pages && (long long)p.pg_keys[pg + 1] <= j) ++pg;
                const B200Page pd = p.pages[pg];
                const uint64_t row = (uint64_t)(j - p.pg_keys[pg]), slab = (uint64_t)b * p.hkv + hk;
                kr = reinterpret_cast<const char *>(pd.k) + ((slab * pd.k_cap + row) * p.k_ss) * kv_esize;
                vr = reinterpret_cast<const char *>(pd.v) + ((slab * pd.v_cap + row) * p.v_ss) * kv_esize;
            }
            row_k[tid] = kr;
            row_v[tid] = vr;
            __syncwarp();
            if (tid == FA_BN - 1 && j < s_hi) *cursor = pg;  // at or before the next tile's first key
        }
        __syncthreads();
    };
    // K / V tile loader: tile t of this split into buffer (t & 1)
    auto load_tile = [&](int t) {
        const long long j0 = s_lo + (long long)t * FA_BN;
        const uint32_t dk = sK + (t & 1) * FA_BN * ROWB, dv = sV + (t & 1) * FA_BN * ROWB;
        const bool paged = p.pages != nullptr;
        if (paged) locate_rows(j0);
        // row rr of the tile (key j): where its elements start
        auto k_row = [&](int rr, long long j) { return paged ? row_k[rr] : kb + ((uint64_t)j * p.k_ss) * kv_esize; };
        auto v_row = [&](int rr, long long j) { return paged ? row_v[rr] : vb + ((uint64_t)j * p.v_ss) * kv_esize; };
        if (p.kv_kind == 0) {
            for (int idx = tid; idx < FA_BN * CH; idx += FA_WARPS * 32) {
                const int rr = idx / CH, ch = idx % CH;
                const long long j = j0 + rr;
                const bool ok = j < s_hi && (uint32_t)ch * 8 < D;
                const long long jj = j < s_hi ? j : s_lo;
                const int rj = j < s_hi ? rr : 0;  // a row past the end copies nothing: any valid address will do
                cp_async16(dk + rr * ROWB + ch * 16, k_row(rj, jj) + ch * 16, ok);
                cp_async16(dv + rr * ROWB + ch * 16, v_row(rj, jj) + ch * 16, ok);
            }
        } else if (p.kv_kind == 2) {
            // f32 -> mma type: 8 elements per step
            for (int idx = tid; idx < FA_BN * CH; idx += FA_WARPS * 32) {
                const int rr = idx / CH, ch = idx % CH;
                const long long j = j0 + rr;
                uint32_t ko[4] = {0, 0, 0, 0}, vo[4] = {0, 0, 0, 0};
                if (j < s_hi && (uint32_t)ch * 8 < D) {
                    const float *ks = reinterpret_cast<const float *>(k_row(rr, j)) + ch * 8;
                    const float *vs = reinterpret_cast<const float *>(v_row(rr, j)) + ch * 8;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        ko[e] = pack2<BF16>(ks[2 * e], ks[2 * e + 1]);
                        vo[e] = pack2<BF16>(vs[2 * e], vs[2 * e + 1]);
                    }
                }
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dk + rr * ROWB + ch * 16), "r"(ko[0]), "r"(ko[1]), "r"(ko[2]), "r"(ko[3]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dv + rr * ROWB + ch * 16), "r"(vo[0]), "r"(vo[1]), "r"(vo[2]), "r"(vo[3]) : "memory");
            }
        } else {
            // E4M3 bytes -> mma type: 8 elements per step
            for (int idx = tid; idx < FA_BN * CH; idx += FA_WARPS * 32) {
                const int rr = idx / CH, ch = idx % CH;
                const long long j = j0 + rr;
                uint32_t ko[4] = {0, 0, 0, 0}, vo[4] = {0, 0, 0, 0};
                if (j < s_hi && (uint32_t)ch * 8 < D) {
                    const uint8_t *ks = reinterpret_cast<const uint8_t *>(k_row(rr, j)) + ch * 8;
                    const uint8_t *vs = reinterpret_cast<const uint8_t *>(v_row(rr, j)) + ch * 8;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        ko[e] = pack2<BF16>(e4m3_to_f(ks[2 * e]), e4m3_to_f(ks[2 * e + 1]));
                        vo[e] = pack2<BF16>(e4m3_to_f(vs[2 * e]), e4m3_to_f(vs[2 * e + 1]));
                    }
                }
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dk + rr * ROWB + ch * 16), "r"(ko[0]), "r"(ko[1]), "r"(ko[2]), "r"(ko[3]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dv + rr * ROWB + ch * 16), "r"(vo[0]), "r"(vo[1]), "r"(vo[2]), "r"(vo[3]) : "memory");
            }
        }
        cp_async_commit();
    };
    if (ntiles > 0) load_tile(0);
    __syncthreads();
    // ldmatrix x4: rows (lane & 15) of the warp's 16 rows, column halves by lane >> 4
    const uint32_t q_base = sQ + (wrow * 16 + (lane & 15)) * ROWB + (lane >> 4) * 16;
    uint32_t qa[QREG ? KSTEPS : 1][4];
    if (QREG) {
#pragma unroll
        for (int ks = 0; ks < (QREG ? KSTEPS : 1); ++ks) ldsm_x4(q_base + ks * 32, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    }

    // rows of this lane: warp * 16 + g and + 8
    long long r_lo[2], r_hi[2], r_pos[2];
    float slope[2] = {0.0f, 0.0f};
    bool r_ok[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const uint32_t r = row0 + wrow * 16 + g + 8 * e;
        r_ok[e] = r < R;
        r_lo[e] = r_hi[e] = r_pos[e] = 0;
        if (r_ok[e]) {
            range_of(r, r_lo[e], r_hi[e], r_pos[e]);
            if (p.alibi) slope[e] = p.alibi[(size_t)b * p.alibi_bs + hk * G + r % G];
        }
    }
    const float sc = p.scale * p.kd;
    const bool plain = p.softcap <= 0.0f && p.alibi == nullptr;
    // rows of the warp: the warp-wide tightest bounds decide whether a tile needs masks
    long long w_lomax = 0, w_himin = 0;
    {
        long long a, bq, cpos;
        const uint32_t rf = row0 + wrow * 16, rl = min(row0 + wrow * 16 + 16, R);
        if (rf < R) {
            range_of(rl - 1, w_lomax, a, cpos);
            range_of(rf, a, w_himin, cpos);
            if (rl - rf < 16) w_himin = -1;  // rows outside the sequence: always masked
            (void)bq;
        } else {
            w_himin = -1;
        }
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float oacc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.0f;

    for (int t = 0; t < ntiles; ++t) {
        if (t + 1 < ntiles) load_tile(t + 1);
        if (t + 1 < ntiles) cp_async_wait<1>();
        else cp_async_wait<0>();
        __syncthreads();
        const long long j0 = s_lo + (long long)t * FA_BN;
        const uint32_t tk = sK + (t & 1) * FA_BN * ROWB, tv = sV + (t & 1) * FA_BN * ROWB;
        // ---- S = Q K^T: the warp's key groups of 8 (all eight of the tile, or the two of its 16 keys)
        float s[2 * KG][4];
#pragma unroll
        for (int n = 0; n < 2 * KG; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a0, a1, a2, a3;
            if (QREG) a0 = qa[QREG ? ks : 0][0], a1 = qa[QREG ? ks : 0][1], a2 = qa[QREG ? ks : 0][2], a3 = qa[QREG ? ks : 0][3];
            else ldsm_x4(q_base + ks * 32, a0, a1, a2, a3);
#pragma unroll
            for (int np = 0; np < KG; ++np) {
                // matrices: keys (kg0 + np)*16 + (0..7 | 8..15), dims ks*16 + (0..7 | 8..15)
                uint32_t b0, b1, b2, b3;
                const uint32_t addr = tk + ((kg0 + np) * 16 + (lane & 7) + ((lane >> 4) << 3)) * ROWB + ks * 32 + ((lane >> 3) & 1) * 16;
                ldsm_x4(addr, b0, b1, b2, b3);
                mma16816<BF16>(s[2 * np], a0, a1, a2, a3, b0, b1);
                mma16816<BF16>(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- scale, masks, online softmax (rows g and g + 8; columns 8 n + 2 c, + 1)
        const bool full = plain && j0 >= w_lomax && j0 + FA_BN <= w_himin && j0 + FA_BN <= s_hi;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2 * KG; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int e = i >> 1;
                float x = s[n][i] * sc;
                if (!full) {
                    const long long j = j0 + 16 * kg0 + 8 * n + 2 * c + (i & 1);
                    if (p.softcap > 0.0f) x = p.softcap * tanhf(x / p.softcap);
                    if (slope[e] != 0.0f) x -= slope[e] * fabsf((float)(r_pos[e] - j));
                    if (!(r_ok[e] && j >= r_lo[e] && j < r_hi[e] && j < s_hi)) x = -INFINITY;
                }
                s[n][i] = x;
                mx[e] = fmaxf(mx[e], x);
            }
        }
        float alpha[2], msafe[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
            const float mn = fmaxf(m[e], mx[e]);
            msafe[e] = mn == -INFINITY ? 0.0f : mn;
            alpha[e] = fast_exp2((m[e] - msafe[e]) * LOG2E_F);
            m[e] = mn;
            l[e] *= alpha[e];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            oacc[n][0] *= alpha[0];
            oacc[n][1] *= alpha[0];
            oacc[n][2] *= alpha[1];
            oacc[n][3] *= alpha[1];
        }
        uint32_t pa[KG][4];
#pragma unroll
        for (int n = 0; n < 2 * KG; ++n) {
            const float p0 = fast_exp2((s[n][0] - msafe[0]) * LOG2E_F), p1 = fast_exp2((s[n][1] - msafe[0]) * LOG2E_F);
            const float p2 = fast_exp2((s[n][2] - msafe[1]) * LOG2E_F), p3 = fast_exp2((s[n][3] - msafe[1]) * LOG2E_F);
            l[0] += p0 + p1;
            l[1] += p2 + p3;
            pa[n >> 1][(n & 1) * 2] = pack2<BF16>(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack2<BF16>(p2, p3);
        }
        // ---- O += P V: contraction over the warp's keys in steps of 16
#pragma unroll
        for (int kk = 0; kk < KG; ++kk) {
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                // transposed matrices: keys (kg0 + kk)*16 + (0..7 | 8..15), dims np*16 + (0..7 | 8..15)
                uint32_t b0, b1, b2, b3;
                const uint32_t addr = tv + ((kg0 + kk) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + np * 32 + (lane >> 4) * 16;
                ldsm_x4_trans(addr, b0, b1, b2, b3);
                mma16816<BF16>(oacc[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                mma16816<BF16>(oacc[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
            }
        }
        __syncthreads();  // the buffer of tile t is free for tile t + 2
    }

    // ---- finish: normalize, write rows (token, head) or the split's partial
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
    }
    if constexpr (DEC) {
        // The four warps hold partial results of the same 16 rows over different keys: [warp][row][HD sums, maximum, sum
        // of weights] in the K / V buffers (every tile is consumed: the loop ends with a barrier), then eight threads
        // per row merge them.
        constexpr int MS = HD + 2;
        float *mg = reinterpret_cast<float *>(smem + QROWS * ROWB);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float *dst = mg + ((size_t)warp * 16 + g + 8 * e) * MS;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<float2 *>(dst + 8 * n + 2 * c) = make_float2(oacc[n][2 * e], oacc[n][2 * e + 1]);
            if (c == 0) dst[HD] = m[e], dst[HD + 1] = l[e];
        }
        __syncthreads();
        const uint32_t row = tid >> 3, ch = tid & 7, r = row0 + row;
        if (r >= R) return;
        float f[FA_WARPS], M = -INFINITY, L = 0.0f;
#pragma unroll
        for (int w = 0; w < FA_WARPS; ++w) M = fmaxf(M, mg[((size_t)w * 16 + row) * MS + HD]);
        const float msafe = M == -INFINITY ? 0.0f : M;
#pragma unroll
        for (int w = 0; w < FA_WARPS; ++w) {
            f[w] = fast_exp2((mg[((size_t)w * 16 + row) * MS + HD] - msafe) * LOG2E_F);
            L += f[w] * mg[((size_t)w * 16 + row) * MS + HD + 1];
        }
        const float inv = L > 0.0f ? p.vd / L : 0.0f;
        const uint32_t i = r / G, h = hk * G + r % G;
        const uint64_t orow = (q0 + i) * p.hq + h, prow = (uint64_t)split * p.rows_total + orow;
#pragma unroll 4
        for (uint32_t dd = ch * (HD / 8); dd < (ch + 1) * (HD / 8); ++dd) {
            if (dd >= D) break;
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < FA_WARPS; ++w) o = fmaf(f[w], mg[((size_t)w * 16 + row) * MS + dd], o);
            if (p.n_splits == 1) store_elem_rt(p.o, orow * D + dd, o * inv, p.q_dtype);
            else p.part_o[prow * D + dd] = o * inv;
        }
        if (p.n_splits > 1 && ch == 0) p.part_lse[prow] = L > 0.0f ? M + logf(L) : -INFINITY;
    } else {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const uint32_t r = row0 + warp * 16 + g + 8 * e;
        if (r >= R) continue;
        const uint32_t i = r / G, h = hk * G + r % G;
        const uint64_t orow = (q0 + i) * p.hq + h;
        if (p.n_splits == 1) {
            const float inv = l[e] > 0.0f ? p.vd / l[e] : 0.0f;
            if (p.q_dtype == B200_F32) {
                float *o = reinterpret_cast<float *>(p.o) + orow * D;
#pragma unroll
                for (int n = 0; n < NT; ++n)
                    if ((uint32_t)8 * n < D) *reinterpret_cast<float2 *>(o + 8 * n + 2 * c) = make_float2(oacc[n][2 * e] * inv, oacc[n][2 * e + 1] * inv);
            } else {
                uint16_t *o = reinterpret_cast<uint16_t *>(p.o) + orow * D;
#pragma unroll
                for (int n = 0; n < NT; ++n)
                    if ((uint32_t)8 * n < D) *reinterpret_cast<uint32_t *>(o + 8 * n + 2 * c) = pack2<BF16>(oacc[n][2 * e] * inv, oacc[n][2 * e + 1] * inv);
            }
        } else {
            const float inv = l[e] > 0.0f ? p.vd / l[e] : 0.0f;
            const uint64_t prow = (uint64_t)split * p.rows_total + orow;
            float *po = p.part_o + prow * D;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if ((uint32_t)8 * n < D) *reinterpret_cast<float2 *>(po + 8 * n + 2 * c) = make_float2(oacc[n][2 * e] * inv, oacc[n][2 * e + 1] * inv);
            if (c == 0) p.part_lse[prow] = l[e] > 0.0f ? m[e] + logf(l[e]) : -INFINITY;
        }
    }
    }
}

// candle-core/kernels/flash_attn_impl.h:445-473
__global__ void __launch_bounds__(128) fa_combine_kernel(const float *__restrict__ part_o, const float *__restrict__ part_lse,
                                                        void *__restrict__ o, int o_dtype, uint64_t rows, uint32_t D, uint32_t n_splits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint64_t row = (uint64_t)blockIdx.x * 4 + warp; row < rows; row += (uint64_t)gridDim.x * 4) {
        float mx = -INFINITY;
        for (uint32_t s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_lse[(uint64_t)s * rows + row]);
        float wsum = 0.0f;
        for (uint32_t s = 0; s < n_splits; ++s) {
            const float e = part_lse[(uint64_t)s * rows + row];
            wsum += e == -INFINITY ? 0.0f : expf(e - mx);
        }
        for (uint32_t d = lane; d < D; d += 32) {
            float acc = 0.0f;
            for (uint32_t s = 0; s < n_splits; ++s) {
                const float e = part_lse[(uint64_t)s * rows + row];
                const float w = e == -INFINITY ? 0.0f : expf(e - mx);
                if (w != 0.0f) acc += w * part_o[((uint64_t)s * rows + row) * D + d];
            }
            store_elem_rt(o, row * D + d, wsum > 0.0f ? acc / wsum : 0.0f, o_dtype);
        }
    }
}

struct FaPlan {
    FaParams p;
    dim3 grid;
    size_t smem, ws_bytes, off_lse;
    bool bf16;  // mma operand type
};

// keys before every block of a paged call, and their total behind them: one block of threads, a running sum over
// chunks of 256 blocks
__global__ void __launch_bounds__(256) fa_page_prefix_kernel(const B200Page *__restrict__ pages, uint32_t n_pages, uint32_t *__restrict__ pg_keys) {
    __shared__ uint32_t sk[256];
    uint32_t base = 0;
    for (uint32_t start = 0; start < n_pages; start += 256) {
        const uint32_t i = start + threadIdx.x;
        const uint32_t r = i < n_pages ? pages[i].rows : 0u;
        sk[threadIdx.x] = r;
        __syncthreads();
        for (int o = 1; o < 256; o <<= 1) {  // inclusive scan
            const uint32_t add = threadIdx.x >= (unsigned)o ? sk[threadIdx.x - o] : 0u;
            __syncthreads();
            sk[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < n_pages) pg_keys[i] = base + sk[threadIdx.x] - r;
        base += sk[255];
        __syncthreads();
    }
    if (threadIdx.x == 0) pg_keys[n_pages] = base;
}

static int fa_plan(const B200FaArgs *a, FaPlan &pl, bool paged = false) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "flash_attn: null args");
    if (a->hkv == 0 || a->hq % a->hkv != 0)
        return set_error(B200_ERR_BAD_ARG, "flash-attn: %u query heads are not a multiple of %u kv heads", a->hq, a->hkv);
    if (a->q_dtype != B200_F16 && a->q_dtype != B200_BF16 && a->q_dtype != B200_F32)
        return set_error(B200_ERR_BAD_ARG, "flash-attn: query dtype %d", a->q_dtype);
    // candle-core/src/cuda_backend/accel.rs: k / v share q's dtype, are E4M3, or are f16 / bf16 under f32 queries
    const bool kv16 = a->kv_dtype == B200_F16 || a->kv_dtype == B200_BF16;
    if (a->kv_dtype != a->q_dtype && a->kv_dtype != B200_FP8 && !(a->q_dtype == B200_F32 && kv16))
        return set_error(B200_ERR_BAD_ARG, "flash-attn: k/v dtype must match q or be F8E4M3");
    // the reference's kernels take any head dim up to 256 (candle-core/src/accel/attention.rs:283-290); the tensor core tiles
    // here take the multiples of 8 among them (16-byte chunks of 16-bit elements)
    if (a->d == 0 || a->d > 256 || a->d % 8) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "flash_attn: head dim %u (fused kernel: multiples of 8 up to 256)", a->d);
    if (a->varlen && (!a->cu_q || !a->cu_k)) return set_error(B200_ERR_BAD_ARG, "flash_attn: varlen needs cu_q and cu_k");
    const bool fp8 = a->kv_dtype == B200_FP8;
    if (paged && a->varlen) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "flash_attn_paged: cumulative lengths are not offered over paged blocks");
    if (kv16 && !paged) {
        // cp.async moves 16-byte chunks: rows must start on 16-byte boundaries
        const uint64_t al = reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v);
        if ((al & 15) || ((a->k_strides[0] | a->k_strides[1] | a->k_strides[2] | a->v_strides[0] | a->v_strides[1] | a->v_strides[2]) & 7))
            return set_error(B200_ERR_UNSUPPORTED_SHAPE, "flash_attn: k / v rows must be 16-byte aligned");
    }
    if (kv16 && paged && ((a->k_strides[1] | a->v_strides[1]) & 7))
        return set_error(B200_ERR_UNSUPPORTED_SHAPE, "flash_attn_paged: k / v rows must be 16-byte aligned");
    if (paged && (a->k_strides[1] < a->d || a->v_strides[1] < a->d))
        return set_error(B200_ERR_BAD_ARG, "flash_attn_paged: row strides below the head dim");
    FaParams &p = pl.p;
    memset(&p, 0, sizeof(p));
    p.q = a->q; p.k = a->k; p.v = a->v; p.o = a->o;
    p.cu_q = a->cu_q; p.cu_k = a->cu_k; p.alibi = a->alibi;
    p.b = a->b; p.lq = a->lq; p.lk = a->lk; p.hq = a->hq; p.hkv = a->hkv; p.d = a->d;
    p.group = a->hq / a->hkv;
    p.q_sb = a->q_strides[0]; p.q_ss = a->q_strides[1]; p.q_sh = a->q_strides[2];
    p.k_sb = a->k_strides[0]; p.k_ss = a->k_strides[1]; p.k_sh = a->k_strides[2];
    p.v_sb = a->v_strides[0]; p.v_ss = a->v_strides[1]; p.v_sh = a->v_strides[2];
    p.scale = a->scale; p.softcap = a->softcap; p.kd = a->k_descale; p.vd = a->v_descale;
    p.wl = a->wl; p.wr = a->wr;
    p.alibi_bs = a->alibi_bstride; p.varlen = a->varlen;
    p.q_dtype = a->q_dtype;
    p.kv_kind = kv16 ? 0 : (fp8 ? 1 : 2);
    pl.bf16 = kv16 ? a->kv_dtype == B200_BF16 : a->q_dtype == B200_BF16;
    p.rows_total = a->total_q * a->hq;
    const uint64_t rows = (uint64_t)a->lq * p.group;
    const uint32_t row_tiles = (uint32_t)std::max<uint64_t>((rows + FA_BM - 1) / FA_BM, 1);
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t ctas = (uint64_t)row_tiles * a->hkv * std::max<uint32_t>(a->b, 1);
    uint32_t splits = 1;
    if (ctas < 2ull * sms && a->lk > 2 * FA_BN) {
        const uint64_t by_occ = (2ull * sms + ctas - 1) / ctas, by_keys = (a->lk + 4 * FA_BN - 1) / (4 * FA_BN);
        splits = (uint32_t)std::min<uint64_t>(std::min(by_occ, by_keys), 64);
    } else if (rows <= 16 && a->lk >= 16 * FA_BN) {
        // decode with enough blocks to fill the device: up to four key splits where they make the blocks a better fit to
        // whole waves of resident blocks (four per SM up to head dim 64, three up to 128, one at 256)
        const uint64_t resident = (uint64_t)sms * (a->d > 128 ? 1 : (a->d > 64 ? 3 : 4));
        double best = 0.0;
        for (uint32_t sp = 1; sp <= 4; ++sp) {
            const uint64_t n = ctas * sp, waves = (n + resident - 1) / resident;
            const double fill = (double)n / (double)(waves * resident) - 0.02 * (sp - 1);  // a split costs a partial result
            if (fill > best) best = fill, splits = sp;
        }
    }
    p.n_splits = 1;
    // long chunks run as whole tiles on the tcgen05 kernel and are never split along the keys
    if (paged || !fa_prefill_sm100_supported(p, kv16)) p.n_splits = std::max(splits, 1u);
    if ((uint64_t)a->b * p.n_splits > 65535) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "flash_attn: batch x splits too large");
    pl.grid = dim3(row_tiles, a->hkv, a->b * p.n_splits);
    const size_t rowb = (a->d <= 64 ? 64 : (a->d <= 128 ? 128 : 256)) * 2 + 16;
    // a decode call keeps one group of 16 query rows in shared memory, which lets a third block share the SM
    pl.smem = ((rows <= 16 ? 16 : FA_BM) + 4 * FA_BN) * rowb;
    if (paged) pl.smem += 2 * FA_BN * sizeof(void *) + 16;  // the row addresses of a tile and the block cursor
    const size_t part_o = p.n_splits > 1 ? (size_t)p.n_splits * p.rows_total * a->d * 4 : 0;
    pl.off_lse = (part_o + 255) / 256 * 256;
    pl.ws_bytes = p.n_splits > 1 ? pl.off_lse + (size_t)p.n_splits * p.rows_total * 4 : 0;
    return B200_OK;
}

template <int HD, bool BF16, bool DEC>
static int fa_launch_as(const FaPlan &pl, cudaStream_t stream) {
    auto kern = fa_dense_kernel<HD, BF16, DEC>;
    static thread_local bool done[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !done[dev]) {
        // the most this instantiation ever asks for: its tiles plus the row addresses of a paged call
        const int most = ((DEC ? 16 : FA_BM) + 4 * FA_BN) * (HD * 2 + 16) + 2 * FA_BN * (int)sizeof(void *) + 16;
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "flash_attn: shared memory opt-in: %s", cudaGetErrorString(e));
        done[dev] = true;
    }
    kern<<<pl.grid, FA_WARPS * 32, pl.smem, stream>>>(pl.p);
    int rc = check_launch("flash_attn");
    if (rc) return rc;
    if (pl.p.n_splits > 1) {
        const unsigned gx = (unsigned)std::min<uint64_t>((pl.p.rows_total + 3) / 4, 148ull * 16);
        fa_combine_kernel<<<gx, 128, 0, stream>>>(pl.p.part_o, pl.p.part_lse, pl.p.o, pl.p.q_dtype, pl.p.rows_total, pl.p.d, pl.p.n_splits);
        rc = check_launch("fa_combine");
    }
    return rc;
}

// decode calls (the packed rows of a kv head fit one group of 16) share the keys of a tile among the warps
template <int HD, bool BF16>
static int fa_launch(const FaPlan &pl, cudaStream_t stream) {
    if ((uint64_t)pl.p.lq * pl.p.group <= 16) return fa_launch_as<HD, BF16, true>(pl, stream);
    return fa_launch_as<HD, BF16, false>(pl, stream);
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_flash_attn_workspace_bytes(const B200FaArgs *a) {
    FaPlan pl;
    if (fa_plan(a, pl)) return 0;
    return pl.ws_bytes;
}

extern "C" int b200_flash_attn(const B200FaArgs *a, b200_stream_t stream_) {
    FaPlan pl;
    const int rc = fa_plan(a, pl);
    if (rc) return rc;
    if (a->total_q * a->hq == 0 || a->b == 0) return B200_OK;
    if (!a->q || !a->k || !a->v || !a->o) return set_error(B200_ERR_BAD_ARG, "flash_attn: null pointer");
    if (pl.ws_bytes) {
        if (!a->workspace || a->workspace_bytes < pl.ws_bytes)
            return set_error(B200_ERR_WORKSPACE, "flash_attn: workspace of %zu bytes needed, %zu given", pl.ws_bytes,
                             a->workspace ? a->workspace_bytes : (size_t)0);
        pl.p.part_o = reinterpret_cast<float *>(a->workspace);
        pl.p.part_lse = reinterpret_cast<float *>(reinterpret_cast<char *>(a->workspace) + pl.off_lse);
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    const bool bf = pl.bf16;
    // long prefill chunks: tiles on the tcgen05 tensor cores
    if (fa_prefill_sm100_supported(pl.p, pl.p.kv_kind == 0)) return fa_prefill_sm100_launch(pl.p, bf, stream);
    if (a->d <= 64) return bf ? fa_launch<64, true>(pl, stream) : fa_launch<64, false>(pl, stream);
    if (a->d <= 128) return bf ? fa_launch<128, true>(pl, stream) : fa_launch<128, false>(pl, stream);
    return bf ? fa_launch<256, true>(pl, stream) : fa_launch<256, false>(pl, stream);
}

// Decoding attention over the dense K / V of paged cache blocks, read where they are (candle-core/src/cuda_backend/
// accel.rs:391-506, kernels fa_rowp* / fa_rowpg*). Workspace: the keys before every block, then the split buffers.
static size_t fa_paged_prefix_bytes(uint32_t n_pages) { return ((size_t)(n_pages + 1) * 4 + 255) / 256 * 256; }

extern "C" size_t b200_flash_attn_paged_workspace_bytes(const B200FaArgs *a, uint32_t n_pages) {
    FaPlan pl;
    if (n_pages == 0 || fa_plan(a, pl, true)) return 0;
    return fa_paged_prefix_bytes(n_pages) + pl.ws_bytes;
}

extern "C" int b200_flash_attn_paged(const B200FaArgs *a, const B200Page *pages, uint32_t n_pages, b200_stream_t stream_) {
    if (!pages || n_pages == 0) return set_error(B200_ERR_BAD_ARG, "flash_attn_paged: no blocks");
    FaPlan pl;
    const int rc = fa_plan(a, pl, true);
    if (rc) return rc;
    if (a->total_q * a->hq == 0 || a->b == 0) return B200_OK;
    if (!a->q || !a->o) return set_error(B200_ERR_BAD_ARG, "flash_attn_paged: null pointer");
    const size_t pre = fa_paged_prefix_bytes(n_pages);
    if (!a->workspace || a->workspace_bytes < pre + pl.ws_bytes)
        return set_error(B200_ERR_WORKSPACE, "flash_attn_paged: workspace of %zu bytes needed, %zu given", pre + pl.ws_bytes,
                         a->workspace ? a->workspace_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return set_error(B200_ERR_BAD_ARG, "flash_attn_paged: workspace must be 16-byte aligned");
    cudaStream_t stream = (cudaStream_t)stream_;
    char *ws = reinterpret_cast<char *>(a->workspace);
    uint32_t *pg_keys = reinterpret_cast<uint32_t *>(ws);
    fa_page_prefix_kernel<<<1, 256, 0, stream>>>(pages, n_pages, pg_keys);
    int lrc = check_launch("flash_attn_paged (prefix)");
    if (lrc) return lrc;
    pl.p.pages = pages;
    pl.p.pg_keys = pg_keys;
    pl.p.n_pages = n_pages;
    if (pl.ws_bytes) {
        pl.p.part_o = reinterpret_cast<float *>(ws + pre);
        pl.p.part_lse = reinterpret_cast<float *>(ws + pre + pl.off_lse);
    }
    const bool bf = pl.bf16;
    if (a->d <= 64) return bf ? fa_launch<64, true>(pl, stream) : fa_launch<64, false>(pl, stream);
    if (a->d <= 128) return bf ? fa_launch<128, true>(pl, stream) : fa_launch<128, false>(pl, stream);
    return bf ? fa_launch<256, true>(pl, stream) : fa_launch<256, false>(pl, stream);
}

// Auxiliary streams of b200_fa_prefill_append: a few per device, each with its fork / join events (created on first
// use, kept for the life of the process). A call holds one of them while it enqueues its work (event records and waits
// of two calls on one pair of events must not interleave), so calls from several host threads, on several streams,
// run side by side; with more concurrent callers than slots a caller waits for a slot.
struct PrefillFork {
    cudaStream_t aux = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    std::mutex busy;
};
constexpr int FORK_SLOTS = 4;
static PrefillFork g_fork[16][FORK_SLOTS];
static std::atomic<unsigned> g_fork_next{0};

extern "C" int b200_fa_prefill_append(const B200FaArgs *fa, const B200KvAppendArgs *append, b200_stream_t stream_) {
    // The attention reads the uncompressed k / v and is bound by the tensor core; the cache write reads the same
    // tensors once more and is bound by memory. They do not depend on one another, so the cache write runs on an
    // auxiliary stream beside the attention (its blocks fit into the registers and shared memory the attention blocks
    // leave free) and joins the caller's stream at the end. Both orderings are expressed with events, so the call
    // can be captured in a CUDA graph.
    cudaStream_t stream = (cudaStream_t)stream_;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
        const int rc = b200_flash_attn(fa, stream_);
        return rc ? rc : b200_kv_append(append, stream_);
    }
    // a free slot, or the next one in turn
    PrefillFork *f = nullptr;
    for (int i = 0; i < FORK_SLOTS && !f; ++i)
        if (g_fork[dev][i].busy.try_lock()) f = &g_fork[dev][i];
    if (!f) {
        f = &g_fork[dev][g_fork_next.fetch_add(1, std::memory_order_relaxed) % FORK_SLOTS];
        f->busy.lock();
    }
    std::lock_guard<std::mutex> held(f->busy, std::adopt_lock);
    if (!f->aux) {
        if (cudaStreamCreateWithFlags(&f->aux, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&f->fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&f->join, cudaEventDisableTiming) != cudaSuccess) {
            f->aux = nullptr;
            return set_error(B200_ERR_LAUNCH, "fa_prefill_append: cannot create the auxiliary stream");
        }
    }
    if (cudaEventRecord(f->fork, stream) != cudaSuccess || cudaStreamWaitEvent(f->aux, f->fork, 0) != cudaSuccess)
        return set_error(B200_ERR_LAUNCH, "fa_prefill_append: fork: %s", cudaGetErrorString(cudaGetLastError()));
    // the attention first: its blocks (one per SM) take their place, the blocks of the cache write fill in beside them
    const int rc_attn = b200_flash_attn(fa, stream_);
    const int rc_append = b200_kv_append(append, (b200_stream_t)f->aux);
    // join in any case, so that the auxiliary stream never outlives the call in the caller's ordering
    if (cudaEventRecord(f->join, f->aux) != cudaSuccess || cudaStreamWaitEvent(stream, f->join, 0) != cudaSuccess)
        return set_error(B200_ERR_LAUNCH, "fa_prefill_append: join: %s", cudaGetErrorString(cudaGetLastError()));
    return rc_attn ? rc_attn : rc_append;
}
