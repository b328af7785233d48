// Decode attention over packed K/V rows (FP8, MXFP8, MXFP4, NVFP4, TurboQuant 4-bit): kernel body.
//
// Work split: the visible keys of every column (batch entry, kv head, pack of up to 8 query rows that
// share that kv head) are cut into 32-key tiles; the tiles of all columns form one list that the
// warps of the persistent blocks share in cost order. Every warp is a worker of its own: it streams
// its tiles through a private ring of shared memory stages filled by bulk copies (cp.async.bulk +
// mbarrier, no multicast), so no block-wide barrier sits in the key loop. Per tile the warp first
// derives the per-key scalars once (lane = key): f32 key scales, the value scale sigma = rsc0_v *
// 2^(largest block exponent) with its log2, and the f16 block scales of V relative to that exponent.
// Then per 16 keys it
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
// A worker's piece of a column (a segment) ends in a normalized partial result and its log-sum-exp.
// A column that one worker covers alone is stored straight from the registers; otherwise the
// partial goes to the workspace and the worker counts itself on the column's arrival counter: the
// last of the column's workers to arrive merges the partials (in segment order, so the result does
// not depend on who arrives last), rotates back, casts and stores the rows. Columns with very many
// segments (few long sequences) are merged by a separate combine grid instead.
//
// Semantics: candle-core/kernels/turbo_quant_impl.h:232-401 (tq_attn): score = scale * rsc0_k *
// sum_d elem_k q_d, softcap, ALiBi, bottom-right aligned windows, value weight p * rsc0_v, zeros
// for rows without keys; merge of partials: turbo_quant_impl.h:659-685.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int DW = 4;         // warps per block
constexpr int WK = 32;        // keys per warp tile
#ifndef B200_DECODE_MIN_BLOCKS
#define B200_DECODE_MIN_BLOCKS 3
#endif
constexpr int NS_MAX = 3;     // stages per warp (fewer when the rows are large)
constexpr float MAX_SLACK = 8.0f;  // log2 of how far a score may exceed the running maximum before it moves
constexpr int PACK = 8;       // query rows per block
#ifndef B200_DECODE_COL_COST
#define B200_DECODE_COL_COST 4  // cost of starting a column, in tiles, in the split of the work between the workers
#endif
constexpr int CTR_SLABS = 32;    // arrival-counter slabs of the library (consecutive calls take them in turn)
constexpr int CTR_COLS = 8192;   // columns a call may have for the decode grid to merge them itself
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// branch hints: the rare side of a branch inside the tile loop is laid out behind the loop, which keeps the loop's
// instructions close together (the loop is larger than the instruction cache nearest to the schedulers)
#define B200_LIKELY(x) __builtin_expect(!!(x), 1)
#define B200_UNLIKELY(x) __builtin_expect(!!(x), 0)

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
    int32_t kv_len_add;     // added to every entry of kv_len
    uint32_t b, lq, lk, hq, hkv, d, group;
    uint32_t rows_per_kv, packs;
    DecodeSide k, v;
    float scale, softcap;
    int32_t wl, wr;
    const float *alibi;
    uint32_t alibi_bs;
    float *part_o;     // [slot][rows][d], slot = worker + column, rows = min(PACK, query rows per kv head)
    float *part_lse;   // [slot][rows]
    int32_t *meta;     // [column] (first slot, number of segments)
    int32_t *status;
    uint32_t k_stage_bytes, v_stage_bytes;
    uint32_t ns;       // stages per warp
    uint32_t rows_cap;      // rows that exist in every (batch, head) slab of both caches (0 = only the visible ones)
    uint32_t col_cost;      // cost of starting a column, in tiles, for the split of the work between the warps
    uint32_t qstage_bytes;  // query staging for the rotation (0 without it)
    uint32_t after_prev;    // launched as a programmatic dependent of the stream's previous kernel
    uint32_t prefetch;      // with after_prev: rows below kv_len - fresh_rows may be copied while that kernel still runs
    uint32_t out_free;      // with after_prev: the outputs and the workspace are not in that kernel's hands: stores do not wait for it
    uint32_t fresh_rows;
    // outputs gathered on every GPU by the combine kernel (world == 0: off)
    void *const *peer_bufs;
    uint32_t *const *peer_flags;
    uint32_t world, rank;
    uint32_t *step, *done_ctr;
    uint32_t gather_polls;  // polls of the wait for the other ranks' flags (0: 2^21)
    // arrival counters of the columns, one word each, zero between calls (the last arrival wraps its
    // counter back to zero): the last worker of a column merges it. Null: the combine grid merges.
    uint32_t *ctr;
    int32_t *lib_status;    // library-wide flag: set when a bounded wait of a kernel of this call runs out
    // paged rows (null: dense rows): the block table, and for every block the keys and the 32-key tiles of the
    // blocks before it (n_pages + 1 entries each, written by tq_page_prefix_kernel right before this grid)
    const B200Page *pages;
    uint32_t n_pages;
    const uint32_t *pg_keys, *pg_tiles;
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
constexpr int FIXED_SMEM = 128 + 2048 + 64;  // barriers, pair tables, byte-plane tables

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
// N consecutive words of shared memory at `a`, which is known to be a multiple of AL bytes: the widest loads that
// alignment and count allow. Rows of 72 or 80 bytes (an even number of words) put the 4-byte loads of a warp, eight
// rows x four chunks, four to a bank; a lane's whole chunk in one or two loads halves the trips through the banks.
template <int N, int AL>
__device__ __forceinline__ void lds_words(uint32_t a, uint32_t (&x)[N]) {
    if constexpr (AL >= 16 && N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N / 4; ++i)
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(x[4 * i]), "=r"(x[4 * i + 1]), "=r"(x[4 * i + 2]), "=r"(x[4 * i + 3]) : "r"(a + 16 * i));
    } else if constexpr (AL >= 8 && N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(x[2 * i]), "=r"(x[2 * i + 1]) : "r"(a + 8 * i));
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x[i]) : "r"(a + 4 * i));
    }
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

// The 16 f16 centroids of a codebook as byte planes: lo[i] holds the low bytes of entries 4i .. 4i+3,
// hi[i] the high bytes. A byte permute with four codes as its selector then looks four entries up at once,
// in registers: the pair table in shared memory costs one access per two codes, and codes are random, so
// those accesses collide on the banks (3 wavefronts per access measured) and bound the kernel on the
// load/store pipe.
struct Tab16 {
    uint32_t lo[4], hi[4];
};
__device__ __forceinline__ Tab16 load_tab16(uint32_t addr) {
    Tab16 t;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.lo[0]), "=r"(t.lo[1]), "=r"(t.lo[2]), "=r"(t.lo[3]) : "r"(addr));
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.hi[0]), "=r"(t.hi[1]), "=r"(t.hi[2]), "=r"(t.hi[3]) : "r"(addr + 16));
    return t;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// four codes (the nibbles of the low 16 bits of `sel`, bit 3 of each cleared) with `m` = 0xff in the bytes
// of the codes >= 8: f16x2 (codes 0, 1) and (codes 2, 3)
__device__ __forceinline__ void tab16_lookup4(const Tab16 &t, uint32_t sel, uint32_t m, uint32_t &h01, uint32_t &h23) {
    const uint32_t lo_a = prmt(t.lo[0], t.lo[1], sel), lo_b = prmt(t.lo[2], t.lo[3], sel);
    const uint32_t hi_a = prmt(t.hi[0], t.hi[1], sel), hi_b = prmt(t.hi[2], t.hi[3], sel);
    const uint32_t lo = (lo_a & ~m) | (lo_b & m), hi = (hi_a & ~m) | (hi_b & m);
    h01 = prmt(lo, hi, 0x5140u);
    h23 = prmt(lo, hi, 0x7362u);
}
// the eight codes of x -> four f16x2, in the order of the pair table (low nibble in the low half)
__device__ __forceinline__ void tab16_dq8(const Tab16 &t, uint32_t x, uint32_t &h0, uint32_t &h1, uint32_t &h2, uint32_t &h3) {
    const uint32_t x4 = x << 4;
    // sign-replicating selectors: bit 3 of every nibble, spread over its byte
    const uint32_t m_lo = prmt(x4, x, 0xd9c8u), m_hi = prmt(x4, x, 0xfbeau);
    tab16_lookup4(t, x & 0x7777u, m_lo, h0, h1);
    tab16_lookup4(t, (x >> 16) & 0x7777u, m_hi, h2, h3);
}

#ifndef B200_TURBO_PRMT
#define B200_TURBO_PRMT 2  // bit 0: keys, bit 1: values decode codebook rows in registers instead of by table loads (measured: the mix of both keeps either pipe from saturating)
#endif

// f16x2 pair table lookups (codebook format) or packed cvt of the four bytes of x
// WIDE: the pair table holds one copy of every entry per lane ([256][32] words, `lut` already points at the lane's
// column), so that the random look-ups of a warp never meet on a bank
template <int M, bool WIDE = false>
__device__ __forceinline__ void dq4(uint32_t x, uint32_t lut, uint32_t &h0, uint32_t &h1, uint32_t &h2, uint32_t &h3) {
    if constexpr (M == B200_TURBO_MSE && WIDE) {
        // byte k of x by a byte permute, then one shift-and-add: three instructions per look-up with the load
        h0 = lds32(lut + (prmt(x, 0u, 0x4440u) << 7));
        h1 = lds32(lut + (prmt(x, 0u, 0x4441u) << 7));
        h2 = lds32(lut + (prmt(x, 0u, 0x4442u) << 7));
        h3 = lds32(lut + (prmt(x, 0u, 0x4443u) << 7));
    } else if constexpr (M == B200_TURBO_MSE) {
        h0 = lds32(lut + (prmt(x, 0u, 0x4440u) << 2));
        h1 = lds32(lut + (prmt(x, 0u, 0x4441u) << 2));
        h2 = lds32(lut + (prmt(x, 0u, 0x4442u) << 2));
        h3 = lds32(lut + (prmt(x, 0u, 0x4443u) << 2));
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

// The rotation back (x = diag(s) H y / sqrt(n)) of an output row of n = 8 EL elements that eight lanes hold between them,
// lane part p (0..7) the elements [p EL, (p + 1) EL): the butterflies of the index bits inside a lane run on its
// registers, those of the three bits that the part carries across the lanes, where bit i of the part is bit `m[i]` of the
// lane number. All 32 lanes call it (lanes without a row carry zeros). No shared memory, no pass per row.
template <int EL>
__device__ __forceinline__ void hadamard_back_parts(float (&x)[EL], int lane, int m0, int m1, int m2, const float *signs, int d0) {
#pragma unroll
    for (int o = 1; o < EL; o <<= 1) {
#pragma unroll
        for (int e = 0; e < EL; ++e) {
            if (!(e & o)) {
                const float a = x[e], c2 = x[e | o];
                x[e] = a + c2;
                x[e | o] = a - c2;
            }
        }
    }
    const int masks[3] = {m0, m1, m2};
#pragma unroll
    for (int i = 0; i < 3; ++i) {
#pragma unroll
        for (int e = 0; e < EL; ++e) {
            const float y = __shfl_xor_sync(0xffffffffu, x[e], masks[i]);
            x[e] = (lane & masks[i]) ? y - x[e] : x[e] + y;
        }
    }
    const float sc = 1.0f / sqrtf((float)(8 * EL));
#pragma unroll
    for (int e = 0; e < EL; ++e) x[e] *= sc * __ldg(signs + d0 + e);
}

// One column = the keys of one (batch entry, kv head, pack of query rows). Its visible keys
// [lo, hi) are cut into tiles of WK keys; the tiles of all columns, in (batch, column, tile) order,
// form the work list that the warps of the persistent blocks share: every warp is a worker of
// its own, with its own copy ring, segments and partial results, so no block-wide barrier or merge
// sits between the warps.
struct Column {
    int lo, hi, lk, tiles;
    uint32_t t_lo;  // paged rows: index of the column's first tile in the block table's list of tiles
};

// Paged rows: tiles never straddle blocks (as the reference's windows never do, candle-core/kernels/
// flash_attn_impl.h:135-151): block g holds ceil(rows_g / WK) tiles, the last one short. The block that holds key
// position `key` (< the total number of keys): the last g with pg_keys[g] <= key.
__device__ __forceinline__ uint32_t page_of_key(const DecodeParams &p, uint32_t key) {
    uint32_t lo = 0, hi = p.n_pages;  // invariant: pg_keys[lo] <= key < pg_keys[hi]
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (p.pg_keys[mid] <= key) lo = mid;
        else hi = mid;
    }
    return lo;
}
// the block that holds tile T of the table's list (< the total number of tiles)
__device__ __forceinline__ uint32_t page_of_tile(const DecodeParams &p, uint32_t T) {
    uint32_t lo = 0, hi = p.n_pages;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (p.pg_tiles[mid] <= T) lo = mid;
        else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ Column make_column(const DecodeParams &p, uint32_t b) {
    Column c;
    c.lk = p.kv_len ? min(max(p.kv_len[b] + p.kv_len_add, 0), (int)p.lk) : (int)p.lk;
    if (p.pages) c.lk = (int)min((uint32_t)c.lk, p.pg_keys[p.n_pages]);  // never more keys than the blocks hold
    // union of the rows' ranges: first query token gives the lowest, the last the highest key
    const long long pos0 = (long long)c.lk - (long long)p.lq, pos1 = (long long)c.lk - 1;
    long long lo = p.wl >= 0 ? max(pos0 - p.wl, 0ll) : 0ll;
    long long hi = p.wr >= 0 ? min(pos1 + p.wr + 1, (long long)c.lk) : (long long)c.lk;
    lo = min(lo, (long long)c.lk);
    hi = max(hi, lo);
    c.lo = (int)lo;
    c.hi = (int)hi;
    c.t_lo = 0;
    if (p.pages == nullptr) {
        c.tiles = (c.hi - c.lo + WK - 1) / WK;
    } else if (c.hi > c.lo) {
        const uint32_t g0 = page_of_key(p, (uint32_t)c.lo), g1 = page_of_key(p, (uint32_t)c.hi - 1);
        c.t_lo = p.pg_tiles[g0] + ((uint32_t)c.lo - p.pg_keys[g0]) / WK;
        c.tiles = (int)(p.pg_tiles[g1] + ((uint32_t)c.hi - 1 - p.pg_keys[g1]) / WK + 1 - c.t_lo);
    } else {
        c.tiles = 0;
    }
    return c;
}

// worker that owns cost position x when `total` is shared by `nw` workers (worker i starts at floor(i total / nw))
__device__ __forceinline__ uint32_t owner_of(uint64_t x, uint64_t total, uint32_t nw) {
    return (uint32_t)(((x + 1) * nw - 1) / total);
}

// A worker's share is a list of segments: tiles [t0, t1) of column y of batch entry b.
// Cost space: every column takes col_cost (its set up and its partial result) plus one per tile, laid
// out in (batch, column) order; worker i takes the tiles whose cost position lies in
// [i total / nw, (i + 1) total / nw). Columns without tiles cost nothing.
struct Segment {
    uint32_t b, y, t0, t1;
    uint64_t x;  // cost position of tile t0
    Column col;
};

// next segment of the share that ends at x_end; false when the share is exhausted
__device__ __forceinline__ bool next_segment(Segment &s, const DecodeParams &p, uint32_t ny, uint64_t x_end) {
    if (s.t1 < (uint32_t)s.col.tiles) return false;  // the share ended inside the column
    const uint64_t x = s.x + (s.t1 - s.t0) + p.col_cost;
    if (x >= x_end) return false;
    if (++s.y == ny) {
        s.y = 0;
        do {
            if (++s.b >= p.b) return false;
            s.col = make_column(p, s.b);
        } while (s.col.tiles == 0);
    }
    s.x = x;
    s.t0 = 0;
    s.t1 = (uint32_t)min((uint64_t)s.col.tiles, x_end - x);
    return true;
}

// ---- row layout of a format at head dim HD (candle-core/src/accel/formats.rs:206-242), in bytes
__host__ __device__ constexpr int code_bytes(int m, int hd) { return fmt_is4(m) ? hd / 2 : hd; }
__host__ __device__ constexpr int aux_words_of(int m, int hd) {
    return fmt_is_mx(m) ? (hd / 32 + 3) / 4 : (m == B200_NVFP4 ? (hd / 16 + 3) / 4 : 0);
}
__host__ __device__ constexpr int rsc_byte_off(int m, int hd) { return code_bytes(m, hd) + 4 * aux_words_of(m, hd); }
__host__ __device__ constexpr int nat_row_bytes(int m, int hd) { return rsc_byte_off(m, hd) + 8; }
// what every native row's address is a multiple of when the first one's is a multiple of 16 (4, 8 or 16 bytes)
__host__ __device__ constexpr int nat_row_align(int m, int hd) { return nat_row_bytes(m, hd) % 16 == 0 ? 16 : (nat_row_bytes(m, hd) % 8 == 0 ? 8 : 4); }
__host__ __device__ constexpr int min_i(int a, int b) { return a < b ? a : b; }
// bytes of a stage's K (or V) part: WK rows plus the slack of a copy that starts below its first row
__host__ __device__ constexpr uint32_t stage_part_bytes(uint32_t row_bytes) { return (WK * row_bytes + 16u + 15u) / 16u * 16u; }

// Output offset (elements) of row rr of column (b, y), and its index among the rows of the call in
// (batch, head, token) order; false for a row that the pack does not have.
__device__ __forceinline__ bool row_addr(const DecodeParams &p, uint32_t b, uint32_t y, uint32_t rr, size_t &obase, size_t &grow) {
    const uint32_t hk = y / p.packs, pack = y % p.packs, r = pack * PACK + rr;
    if (r >= p.rows_per_kv) return false;
    const uint32_t i = p.lq == 1 ? 0u : r / p.group, h = hk * p.group + (p.lq == 1 ? r : r % p.group);
    obase = (size_t)b * p.o_sb + (size_t)h * p.o_sh + (size_t)i * p.o_ss;
    grow = ((size_t)b * p.hq + h) * p.lq + i;
    return true;
}

// EPL consecutive elements of a row, cast to the output type: one vector store for 16-bit types on an 8-byte boundary
template <int EPL>
__device__ __forceinline__ void store_row_piece(void *out, size_t off, const float (&v)[EPL], int dt) {
    if constexpr (EPL % 4 == 0) {
        if ((dt == B200_F16 || dt == B200_BF16) && ((reinterpret_cast<uintptr_t>(out) + 2 * off) & 7u) == 0) {
            uint16_t *o16 = reinterpret_cast<uint16_t *>(out) + off;
#pragma unroll
            for (int q = 0; q < EPL / 4; ++q) {
                uint32_t w[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t lo = dt == B200_F16 ? f_to_f16_bits(v[4 * q + 2 * h]) : f_to_bf16_bits(v[4 * q + 2 * h]);
                    const uint32_t hi = dt == B200_F16 ? f_to_f16_bits(v[4 * q + 2 * h + 1]) : f_to_bf16_bits(v[4 * q + 2 * h + 1]);
                    w[h] = lo | (hi << 16);
                }
                *reinterpret_cast<uint2 *>(o16 + 4 * q) = make_uint2(w[0], w[1]);
            }
            return;
        }
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k) store_elem_rt(out, off + k, v[k], dt);
}

// Merge of the `ns` partial results of one output row (candle-core/kernels/turbo_quant_impl.h:659-685) by one
// warp: lane l ends with the normalized elements [l HD/32, (l + 1) HD/32) of the row. `po` points at the lane's
// piece of the first segment's partial row, `pl` at its log-sum-exp; consecutive segments are seg_stride floats
// (lse_stride words) apart. Loads bypass L1: the partials were written by other SMs during this kernel.
template <int HD>
__device__ __forceinline__ void merge_row(const float *po, const float *pl, int ns, size_t seg_stride, size_t lse_stride, int lane,
                                          float (&acc)[HD / 32]) {
    constexpr int EPL = HD / 32;
#pragma unroll
    for (int k = 0; k < EPL; ++k) acc[k] = 0.0f;
    // the first four segments' rows are requested before the log-sum-exps are looked at
    float pre[4][EPL];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (j < ns) {
#pragma unroll
            for (int q = 0; q < EPL / 2; ++q) {
                const float2 v = __ldcg(reinterpret_cast<const float2 *>(po + (size_t)j * seg_stride + 2 * q));
                pre[j][2 * q] = v.x;
                pre[j][2 * q + 1] = v.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < EPL; ++k) pre[j][k] = 0.0f;
        }
    }
    float mx = -INFINITY;
    for (int s0 = lane; s0 < ns; s0 += 32) mx = fmaxf(mx, __ldcg(pl + (size_t)s0 * lse_stride));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float wsum = 0.0f;
    for (int base = 0; base < ns; base += 32) {  // lane l weighs segment base + l
        const int sl = base + lane;
        float wl = 0.0f;
        if (sl < ns) {
            const float e = __ldcg(pl + (size_t)sl * lse_stride);
            wl = e == -INFINITY ? 0.0f : expf(e - mx);
        }
        wsum += wl;
        const int cnt = min(32, ns - base);
        int j = 0;
        if (base == 0) {
            // the four rows in registers (segments past the last one weigh nothing)
#pragma unroll
            for (; j < 4; ++j) {
                const float w = __shfl_sync(0xffffffffu, wl, j);
#pragma unroll
                for (int k = 0; k < EPL; ++k) acc[k] = fmaf(w, pre[j][k], acc[k]);
            }
        }
#pragma unroll 4
        for (; j < cnt; ++j) {
            const float w = __shfl_sync(0xffffffffu, wl, j);
            const float *src = po + (size_t)(base + j) * seg_stride;
#pragma unroll
            for (int q = 0; q < EPL / 2; ++q) {
                const float2 v = __ldcg(reinterpret_cast<const float2 *>(src + 2 * q));
                acc[2 * q] = fmaf(w, v.x, acc[2 * q]);
                acc[2 * q + 1] = fmaf(w, v.y, acc[2 * q + 1]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
#pragma unroll
    for (int k = 0; k < EPL; ++k) acc[k] = wsum > 0.0f ? acc[k] / wsum : 0.0f;
}

// A finished output row (lane l holds its elements [l HD/32, (l + 1) HD/32) in the rotated domain of the values):
// rotated back through the warp's staging row `rb` (HD floats of shared memory; only touched when the values
// were rotated), cast and stored, also into every rank's gathered buffer when the outputs are gathered.
template <int HD>
__device__ __forceinline__ void finish_row(const DecodeParams &p, size_t obase, size_t grow, size_t g_base, float (&acc)[HD / 32], float *rb,
                                           int lane, bool rotate = true) {
    constexpr int EPL = HD / 32;
    if (rotate && p.v.rot == B200_ROT_HADAMARD) {
        __syncwarp();
#pragma unroll
        for (int k = 0; k < EPL; ++k) rb[lane * EPL + k] = acc[k];
        __syncwarp();
        warp_hadamard(rb, HD, p.v.signs, false, lane);
        __syncwarp();
#pragma unroll
        for (int k = 0; k < EPL; ++k) acc[k] = rb[lane * EPL + k];
    }
    store_row_piece<EPL>(p.out, obase + (size_t)lane * EPL, acc, p.out_dtype);
    // the same row into every rank's gathered buffer: plain stores through the peer mappings
    for (uint32_t pr = 0; pr < p.world; ++pr) store_row_piece<EPL>(p.peer_bufs[pr], g_base + grow * HD + (size_t)lane * EPL, acc, p.out_dtype);
}

// Merge of all rows of one column by one warp, inside the decode grid (the last worker of the column to arrive).
// Eight lanes share a row (lane l: row l / 8 of a group of four rows, elements [(l % 8) HD / 8, +HD / 8)), so four
// rows are merged side by side and the partial rows of two segments are in flight per lane: a group of rows costs two
// or three trips to L2 instead of a few per row. `slot0`: the first segment's slot; consecutive segments are
// consecutive slots. Rotated values are rotated back in registers.
template <int HD>
__device__ __forceinline__ void merge_column(const DecodeParams &p, uint32_t b, uint32_t y, size_t slot0, int ns, uint32_t prow, size_t g_base,
                                             int lane) {
    constexpr int LPR = 8, EL = HD / LPR;  // lanes per row, elements of a row per lane
    const uint32_t q = (uint32_t)lane % LPR;
    const size_t seg_stride = (size_t)prow * HD;
    for (uint32_t rbase = 0; rbase < prow; rbase += 32 / LPR) {
        const uint32_t rr = rbase + (uint32_t)lane / LPR;
        size_t obase = 0, grow = 0;
        const bool live = rr < prow && row_addr(p, b, y, rr, obase, grow);
        const float *pl = p.part_lse + slot0 * prow + rr;
        const float *po = p.part_o + (slot0 * prow + rr) * HD + q * EL;
        float acc[EL];
#pragma unroll
        for (int k = 0; k < EL; ++k) acc[k] = 0.0f;
        if (live) {
            // the first two segments' rows are requested before the log-sum-exps are looked at
            float4 pre[2][EL / 4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int k = 0; k < EL / 4; ++k)
                    pre[j][k] = j < ns ? __ldcg(reinterpret_cast<const float4 *>(po + (size_t)j * seg_stride) + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float mx = -INFINITY;
#pragma unroll 8
            for (int s0 = 0; s0 < ns; ++s0) mx = fmaxf(mx, __ldcg(pl + (size_t)s0 * prow));
            float wsum = 0.0f;
            for (int s0 = 0; s0 < ns; s0 += 2) {
                float w[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float e = s0 + j < ns ? __ldcg(pl + (size_t)(s0 + j) * prow) : -INFINITY;
                    w[j] = e == -INFINITY ? 0.0f : expf(e - mx);
                    wsum += w[j];
                }
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int k = 0; k < EL / 4; ++k) {
                        acc[4 * k] = fmaf(w[j], pre[j][k].x, acc[4 * k]);
                        acc[4 * k + 1] = fmaf(w[j], pre[j][k].y, acc[4 * k + 1]);
                        acc[4 * k + 2] = fmaf(w[j], pre[j][k].z, acc[4 * k + 2]);
                        acc[4 * k + 3] = fmaf(w[j], pre[j][k].w, acc[4 * k + 3]);
                    }
                // the next two segments
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int k = 0; k < EL / 4; ++k)
                        if (s0 + 2 + j < ns) pre[j][k] = __ldcg(reinterpret_cast<const float4 *>(po + (size_t)(s0 + 2 + j) * seg_stride) + k);
            }
            const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
#pragma unroll
            for (int k = 0; k < EL; ++k) acc[k] *= inv;
        }
        // rotate back: the eight lanes of a row are consecutive (part = lane % 8)
        if (p.v.rot == B200_ROT_HADAMARD) hadamard_back_parts<EL>(acc, lane, 1, 2, 4, p.v.signs, (int)(q * EL));
        if (live) {
            store_row_piece<EL>(p.out, obase + q * EL, acc, p.out_dtype);
            // the same row into every rank's gathered buffer: plain stores through the peer mappings
            for (uint32_t pr = 0; pr < p.world; ++pr) store_row_piece<EL>(p.peer_bufs[pr], g_base + grow * HD + q * EL, acc, p.out_dtype);
        }
    }
}

// Release / acquire fence at system scope (peer stores included): orders as much as the sequentially consistent
// `__threadfence_system()` does for the publish protocol below (rows, then a counter, then a flag), and costs less.
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Gathered outputs: one warp publishes this rank's step in every rank's flags and waits, with a bound, until all
// ranks have published it. The caller has made this rank's rows visible system-wide (fence) before. A wait that
// runs out sets the call's status word to 2 and the library-wide flag; the step is advanced all the same, so the
// next call does not reuse this step's slot.
__device__ __forceinline__ void gather_publish(uint32_t *const *peer_flags, uint32_t world, uint32_t rank, uint32_t *step, uint32_t g_step,
                                               uint32_t polls, int32_t *status, int32_t *lib_status, int lane) {
    bool ok = true;
    for (uint32_t pr = lane; pr < world; pr += 32)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flags[pr] + rank), "r"(g_step) : "memory");
    const uint32_t limit = polls ? polls : (1u << 21);
    for (uint32_t pr = lane; pr < world; pr += 32) {
        const uint32_t *flag = peer_flags[rank] + pr;
        uint32_t seen = 0;
        // steps only grow; a rank that is one step ahead has already passed this one
        for (uint32_t spin = 0; spin < limit; ++spin) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if ((int32_t)(seen - g_step) >= 0) break;
            __nanosleep(32);
        }
        if ((int32_t)(seen - g_step) < 0) ok = false;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
        if (!ok) {
            if (status) atomicExch(status, 2);
            if (lib_status) atomicExch(lib_status, 1);
        }
        *reinterpret_cast<volatile uint32_t *>(step) = g_step;
    }
}

// The end of a combine grid whose rows are gathered: every block makes its rows (local and peer stores) visible
// system-wide and counts itself on the call's counter (which wraps to zero); the warp 0 of the last block to arrive
// publishes the step to the other ranks and waits for theirs. Called by all threads of the block.
__device__ __forceinline__ void combine_publish(const DecodeParams &p, uint32_t g_step) {
    __shared__ uint32_t last_block;
    fence_sys();
    __syncthreads();
    if (threadIdx.x == 0) last_block = atomicInc(p.done_ctr, gridDim.x - 1u) == gridDim.x - 1u ? 1u : 0u;
    __syncthreads();
    if (last_block && threadIdx.x < 32) {
        fence_sys();
        gather_publish(p.peer_flags, p.world, p.rank, p.step, g_step, p.gather_polls, p.status, p.lib_status, (int)threadIdx.x);
    }
}

// Online softmax of a tile in the log2 domain, on the score fragments sr[u][2 k + e] = key 16 u + g + 8 k, row 2c + e.
// vm[k] = (sigma, log2 sigma) of key g + 8 k: the value scale is folded into the running maxima M (which track
// s_j + log2 sigma_j), so the f16 weights w_j = exp2(s_j - M) sigma_j stay in range for value scales of any
// magnitude while the normalizers lsum add exp2(s_j - M) in f32. M only moves when a score exceeds it by 2^MAX_SLACK
// (one warp vote per tile); the function then returns true with the factors al[e] = exp2(M_old - M_new) for
// everything accumulated so far (lsum is already scaled). pb: the weights as B fragments of the second product.
// Plain form: every key of the tile is visible to every row, no soft-capping, no ALiBi.
__device__ __forceinline__ bool softmax_plain(const float (&sr)[2][4], const float2 (&vm)[4], const float (&qs2)[2], float (&M)[2],
                                              float (&lsum)[2], uint32_t (&pb)[4], float (&al)[2]) {
    // scale, maximum check and exponent in fused multiply-adds
    float c0 = fmaxf(fmaxf(fmaf(sr[0][0], qs2[0], vm[0].y), fmaf(sr[0][2], qs2[0], vm[1].y)),
                     fmaxf(fmaf(sr[1][0], qs2[0], vm[2].y), fmaf(sr[1][2], qs2[0], vm[3].y)));
    float c1 = fmaxf(fmaxf(fmaf(sr[0][1], qs2[1], vm[0].y), fmaf(sr[0][3], qs2[1], vm[1].y)),
                     fmaxf(fmaf(sr[1][1], qs2[1], vm[2].y), fmaf(sr[1][3], qs2[1], vm[3].y)));
    const bool moved = __any_sync(0xffffffffu, c0 > M[0] + MAX_SLACK || c1 > M[1] + MAX_SLACK);
    if (B200_UNLIKELY(moved)) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, o));
            c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, o));
        }
        const float n0 = fmaxf(M[0], c0), n1 = fmaxf(M[1], c1);
        al[0] = fast_exp2(M[0] - n0);
        al[1] = fast_exp2(M[1] - n1);
        M[0] = n0;
        M[1] = n1;
        lsum[0] *= al[0];
        lsum[1] *= al[1];
    }
    const float nm0 = -M[0], nm1 = -M[1];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float pa = fast_exp2(fmaf(sr[k >> 1][2 * (k & 1)], qs2[0], nm0));
        const float pc = fast_exp2(fmaf(sr[k >> 1][2 * (k & 1) + 1], qs2[1], nm1));
        lsum[0] += pa;
        lsum[1] += pc;
        pb[k] = movmatrix_trans(pack_f16x2(pa * vm[k].x, pc * vm[k].x));
    }
    return moved;
}

// Visible keys [lo, hi), key position and ALiBi slope of the two query rows (2c, 2c + 1) whose scores a lane holds
struct RowMask {
    int lo[2], hi[2], pos[2];
    float slope[2];
};

// General form: masks, soft-capping, ALiBi. `key_g`: index of the tile's key g (the lane's keys are key_g + 8 k);
// qs[e]: score scale of row 2c + e.
template <bool PERM = false>
__device__ __forceinline__ bool softmax_masked(const float (&sr)[2][4], const float2 (&vm)[4], const float (&qs)[2], float softcap, int key_g,
                                               const RowMask &rm, float (&M)[2], float (&lsum)[2], uint32_t (&pb)[4], float (&al)[2]) {
    float s2[8];  // s2[2 k + e]
#pragma unroll
    for (int e = 0; e < 2; ++e) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int j = key_g + (PERM ? 2 * (k & 1) + 16 * (k >> 1) : 8 * k);  // the lane's keys: g + 8 k, or in the other order
            float sx = sr[k >> 1][2 * (k & 1) + e] * qs[e];
            if (softcap > 0.0f) sx = softcap * tanhf(sx / softcap);
            if (rm.slope[e] != 0.0f) sx -= rm.slope[e] * fabsf((float)(rm.pos[e] - j));
            s2[2 * k + e] = (j >= rm.lo[e] && j < rm.hi[e]) ? sx * LOG2E : -INFINITY;
        }
    }
    float c0 = fmaxf(fmaxf(s2[0] + vm[0].y, s2[2] + vm[1].y), fmaxf(s2[4] + vm[2].y, s2[6] + vm[3].y));
    float c1 = fmaxf(fmaxf(s2[1] + vm[0].y, s2[3] + vm[1].y), fmaxf(s2[5] + vm[2].y, s2[7] + vm[3].y));
    const bool moved = __any_sync(0xffffffffu, c0 > M[0] + MAX_SLACK || c1 > M[1] + MAX_SLACK);
    if (B200_UNLIKELY(moved)) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, o));
            c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, o));
        }
        const float n0 = fmaxf(M[0], c0), n1 = fmaxf(M[1], c1);
        al[0] = fast_exp2(M[0] - n0);
        al[1] = fast_exp2(M[1] - n1);
        M[0] = n0;
        M[1] = n1;
        lsum[0] *= al[0];
        lsum[1] *= al[1];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float pa = fast_exp2(s2[2 * k] - M[0]), pc = fast_exp2(s2[2 * k + 1] - M[1]);
        lsum[0] += pa;
        lsum[1] += pc;
        pb[k] = movmatrix_trans(pack_f16x2(pa * vm[k].x, pc * vm[k].x));
    }
    return moved;
}

// Query rows of pack `pack` of kv head `hk` of batch entry `b` as the B fragments of K Q^T: row g of the pack for the
// lanes of quad row g, rotated with the key signs when the cache is rotated (through the warp's staging rows), then
// normalized by a power of two and rounded to f16. Per k-step the four contraction slots of a lane are the
// consecutive dims dbase(s) ... + 3, so the four lanes of a quad hold the whole row between them. qs[e]: the score
// scale of row 2c + e (softmax scale times the power of two taken out), qs2[e] the same in the log2 domain.
template <int KM, int HD>
__device__ __forceinline__ void load_query(const DecodeParams &p, uint32_t b, uint32_t hk, uint32_t pack, float *qstage, int lane,
                                           uint32_t (&qb0)[HD / 16], uint32_t (&qb1)[HD / 16], float (&qs)[2], float (&qs2)[2]) {
    constexpr int STEPS = HD / 16;
    constexpr bool KMX = fmt_is_mx(KM);
    const int g = lane >> 2, c = lane & 3;
    const uint32_t G = p.group, R = p.rows_per_kv;
    const uint32_t r = pack * PACK + g;
    float qv[STEPS][4];
    if (HD <= 128 && p.k.rot == B200_ROT_HADAMARD) {
        // Rotation in registers. The four lanes of quad row g hold row g between them, each the HD / 4 elements that its
        // own fragments need: element e of the lane is dim d(e) = c HD/4 + e (the codebook, FP8 and NVFP4 orders) or
        // 32 (e / 8) + 8 c + e % 8 (the MX order), so that slot j of k-step s is element 4 s + j either way. The
        // butterflies of the index bits that e carries run inside the lane, those of the two bits that c carries
        // across the quad; no shared memory, no pass per row.
        constexpr int EPL = HD / 4;
        float x[EPL];
        const uint32_t i = p.lq == 1 ? 0u : r / G, h = hk * G + (p.lq == 1 ? r : r % G);
        const size_t qoff = b * p.q_sb + h * p.q_sh + i * p.q_ss;
        const bool q16 = p.q_dtype == B200_F16 || p.q_dtype == B200_BF16;
        if (r >= R) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) x[e] = 0.0f;
        } else if (q16 && ((reinterpret_cast<uintptr_t>(p.q) + 2 * qoff) & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.k.signs) & 15u) == 0) {
            // 16-bit rows on a 16-byte boundary: the lane's elements come as runs of eight (one 16-byte load each), all
            // loads issued before the first conversion
            const uint16_t *q16p = reinterpret_cast<const uint16_t *>(p.q) + qoff;
            uint4 raw[EPL / 8];
#pragma unroll
            for (int t = 0; t < EPL / 8; ++t) raw[t] = __ldg(reinterpret_cast<const uint4 *>(q16p + (KMX ? 32 * t + 8 * c : c * EPL + 8 * t)));
#pragma unroll
            for (int t = 0; t < EPL / 8; ++t) {
                const int d0 = KMX ? 32 * t + 8 * c : c * EPL + 8 * t;
                const float4 s0 = __ldg(reinterpret_cast<const float4 *>(p.k.signs + d0)), s1 = __ldg(reinterpret_cast<const float4 *>(p.k.signs + d0 + 4));
                const uint32_t w[4] = {raw[t].x, raw[t].y, raw[t].z, raw[t].w};
                const float sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = p.q_dtype == B200_BF16 ? u2f(w[j] << 16) : f16_bits_to_f((uint16_t)(w[j] & 0xffffu));
                    const float hi = p.q_dtype == B200_BF16 ? u2f(w[j] & 0xffff0000u) : f16_bits_to_f((uint16_t)(w[j] >> 16));
                    x[8 * t + 2 * j] = lo * sg[2 * j];
                    x[8 * t + 2 * j + 1] = hi * sg[2 * j + 1];
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const int dd = KMX ? 32 * (e / 8) + 8 * c + (e % 8) : c * EPL + e;
                x[e] = load_elem_rt(p.q, qoff + dd, p.q_dtype) * __ldg(p.k.signs + dd);
            }
        }
#pragma unroll
        for (int o = 1; o < EPL; o <<= 1) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                if (!(e & o)) {
                    const float a = x[e], d2 = x[e | o];
                    x[e] = a + d2;
                    x[e | o] = a - d2;
                }
            }
        }
#pragma unroll
        for (int o = 1; o < 4; o <<= 1) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const float y = __shfl_xor_sync(0xffffffffu, x[e], o);
                x[e] = (lane & o) ? y - x[e] : x[e] + y;
            }
        }
        const float hs = 1.0f / sqrtf((float)HD);
#pragma unroll
        for (int s2 = 0; s2 < STEPS; ++s2)
#pragma unroll
            for (int j = 0; j < 4; ++j) qv[s2][j] = x[4 * s2 + j] * hs;
    } else if (p.k.rot == B200_ROT_HADAMARD) {
        __syncwarp();
        for (int idx = lane; idx < PACK * HD; idx += 32) {
            const uint32_t rr = idx / HD, dd = idx % HD, r2 = pack * PACK + rr;
            float v = 0.0f;
            if (r2 < R) {
                const uint32_t i = p.lq == 1 ? 0u : r2 / G, h = hk * G + (p.lq == 1 ? r2 : r2 % G);
                v = load_elem_rt(p.q, b * p.q_sb + h * p.q_sh + i * p.q_ss + dd, p.q_dtype);
            }
            qstage[idx] = v;
        }
        __syncwarp();
        for (int rr = 0; rr < PACK; ++rr) warp_hadamard(qstage + rr * HD, HD, p.k.signs, true, lane);
        __syncwarp();
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const int dbase = KMX ? 32 * (s >> 1) + 8 * c + 4 * (s & 1) : c * (HD / 4) + 4 * s;
#pragma unroll
            for (int j = 0; j < 4; ++j) qv[s][j] = qstage[g * HD + dbase + j];
        }
    } else {
        const uint32_t i = p.lq == 1 ? 0u : r / G, h = hk * G + (p.lq == 1 ? r : r % G);
        const size_t qoff = b * p.q_sb + h * p.q_sh + i * p.q_ss;
        const bool q16 = p.q_dtype == B200_F16 || p.q_dtype == B200_BF16;
        if (q16 && r < R && ((reinterpret_cast<uintptr_t>(p.q) + 2 * qoff) & 7u) == 0) {
            // 16-bit rows on an 8-byte boundary: the four contraction slots of a k-step in one load, all
            // loads of the row issued before the first conversion
            const uint16_t *q16p = reinterpret_cast<const uint16_t *>(p.q) + qoff;
            uint2 raw[STEPS];
#pragma unroll
            for (int s = 0; s < STEPS; ++s) {
                const int dbase = KMX ? 32 * (s >> 1) + 8 * c + 4 * (s & 1) : c * (HD / 4) + 4 * s;
                raw[s] = __ldg(reinterpret_cast<const uint2 *>(q16p + dbase));
            }
            if (p.q_dtype == B200_BF16) {
#pragma unroll
                for (int s = 0; s < STEPS; ++s) {
                    qv[s][0] = u2f(raw[s].x << 16); qv[s][1] = u2f(raw[s].x & 0xffff0000u);
                    qv[s][2] = u2f(raw[s].y << 16); qv[s][3] = u2f(raw[s].y & 0xffff0000u);
                }
            } else {
#pragma unroll
                for (int s = 0; s < STEPS; ++s) {
                    qv[s][0] = f16_bits_to_f((uint16_t)(raw[s].x & 0xffffu)); qv[s][1] = f16_bits_to_f((uint16_t)(raw[s].x >> 16));
                    qv[s][2] = f16_bits_to_f((uint16_t)(raw[s].y & 0xffffu)); qv[s][3] = f16_bits_to_f((uint16_t)(raw[s].y >> 16));
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < STEPS; ++s) {
                const int dbase = KMX ? 32 * (s >> 1) + 8 * c + 4 * (s & 1) : c * (HD / 4) + 4 * s;
#pragma unroll
                for (int j = 0; j < 4; ++j) qv[s][j] = r < R ? load_elem_rt(p.q, qoff + dbase + j, p.q_dtype) : 0.0f;
            }
        }
    }
    float am = 0.0f;
#pragma unroll
    for (int s = 0; s < STEPS; ++s)
#pragma unroll
        for (int j = 0; j < 4; ++j) am = fmaxf(am, fabsf(qv[s][j]));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
    int e = 0;
    if (am > 0.0f && am < INFINITY) e = (int)((f2u(am) >> 23) & 0xffu) - 127 - 7;
    e = max(min(e, 100), -100);
    const float down = u2f((uint32_t)(127 - e) << 23), up = u2f((uint32_t)(127 + e) << 23);
    const float qscale = p.scale * up;
    qs[0] = __shfl_sync(0xffffffffu, qscale, (2 * c) * 4);
    qs[1] = __shfl_sync(0xffffffffu, qscale, (2 * c + 1) * 4);
    qs2[0] = qs[0] * LOG2E;
    qs2[1] = qs[1] * LOG2E;
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
        qb0[s] = pack_f16x2(qv[s][0] * down, qv[s][1] * down);
        qb1[s] = pack_f16x2(qv[s][2] * down, qv[s][3] * down);
    }
}

// Per-key scalars of a tile, lane = key. `kr` / `vr`: the lane's K and V row in the stage. Written for the tile's
// consumers: f32 key scales (rsc0 times the block scales of the MX formats) at meta_s [key][KMW], the value scale
// sigma = rsc0_v * 2^(largest block exponent) and its log2 at vmeta_s [key], f16 block scales of V relative to that
// exponent at vsc_s [block][key].
template <int KM, int VM, int HD>
__device__ __forceinline__ void tile_meta(uint32_t kr, uint32_t vr, uint32_t meta_s, uint32_t vmeta_s, uint32_t vsc_s, int lane) {
    constexpr bool KMX = fmt_is_mx(KM);
    constexpr int KMW = kmeta_words(KM, HD);
    constexpr int NBK = HD / 32;
    constexpr int NBV = vsc_blocks(VM, HD);
    constexpr uint32_t k_cw4 = code_bytes(KM, HD), k_rsc4 = rsc_byte_off(KM, HD);
    constexpr uint32_t v_cw4 = code_bytes(VM, HD), v_rsc4 = rsc_byte_off(VM, HD);
        const float k0 = u2f(lds32(kr + k_rsc4));
    if constexpr (KMX) {
#pragma unroll
        for (int w = 0; w < (NBK + 3) / 4; ++w) {
            const uint32_t aux = lds32(kr + k_cw4 + 4 * w);
            // rsc0 * 2^(e - 127); a zero code gives +0 (its block holds zero codes)
            float sc[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[i] = k0 * u2f(((aux >> (8 * i)) & 0xffu) << 23);
            if constexpr (KMW >= 4) {
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(meta_s + (lane * KMW + 4 * w) * 4), "f"(sc[0]), "f"(sc[1]),
                             "f"(sc[2]), "f"(sc[3])
                             : "memory");
            } else {
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(meta_s + lane * KMW * 4), "f"(sc[0]), "f"(sc[1]) : "memory");
            }
        }
    } else {
        sts32(meta_s + lane * 4, f2u(k0));
    }
    float sigma = u2f(lds32(vr + v_rsc4));
    if constexpr (fmt_is_mx(VM)) {
        uint32_t aux[(NBV + 3) / 4];
        uint32_t em = 0;
#pragma unroll
        for (int w = 0; w < (NBV + 3) / 4; ++w) {
            aux[w] = lds32(vr + v_cw4 + 4 * w);
            em = w == 0 ? aux[w] : __vmaxu4(em, aux[w]);
        }
        const uint32_t emax = max_byte(em);
        sigma *= u2f(emax << 23);
#pragma unroll
        for (int bk = 0; bk < NBV; ++bk) {
            const int e = (int)((aux[bk >> 2] >> (8 * (bk & 3))) & 0xffu);
            sts16(vsc_s + (bk * WK + lane) * 2, pow2_f16(e - (int)emax));
        }
    } else if constexpr (VM == B200_NVFP4) {
#pragma unroll
        for (int w = 0; w < NBV / 4; ++w) {
            const uint32_t aux = lds32(vr + v_cw4 + 4 * w);
            const uint32_t lo = cvt_e4m3x2_f16x2(aux), hi = cvt_e4m3x2_hi_f16x2(aux);
            sts16(vsc_s + ((4 * w) * WK + lane) * 2, lo & 0xffffu);
            sts16(vsc_s + ((4 * w + 1) * WK + lane) * 2, lo >> 16);
            sts16(vsc_s + ((4 * w + 2) * WK + lane) * 2, hi & 0xffffu);
            sts16(vsc_s + ((4 * w + 3) * WK + lane) * 2, hi >> 16);
        }
    }
    // sigma in [2^-100, 2^100], or 0 (then log2 = -inf: the key only counts in the normalizer)
    float sc = fminf(fmaxf(sigma, 7.8886091e-31f), 1.2676506e30f);
    sc = sigma > 0.0f ? sc : 0.0f;
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(vmeta_s + lane * 8), "f"(sc), "f"(fast_log2(sc)) : "memory");
    __syncwarp();
}

// Scores of keys g and g + 8 of the 16 keys at `ka` (the lane's first code byte of key g; rows krb bytes apart)
// against the query rows 2c, 2c + 1: sr[2 k + e] = key g + 8 k, row 2c + e. `mrow`: the f32 key scales of key g
// (per-key scalars of the tile), qb0 / qb1: the query fragments.
// AL: what the rows' addresses in shared memory are known to be multiples of (bytes).
// PERM: the tile's keys are dealt to the lanes in another order (perm_key below): the lane's second key is 2 rows
// after its first instead of 8.
template <int KM, int HD, bool WIDE = false, int AL = 4, bool PERM = false>
__device__ __forceinline__ void k_scores16(uint32_t ka, uint32_t krb, uint32_t mrow, const uint32_t (&qb0)[HD / 16], const uint32_t (&qb1)[HD / 16],
                                           uint32_t lut_k, uint32_t plane_k, int c, float (&sr)[4]) {
    constexpr int STEPS = HD / 16;
    constexpr bool K4 = fmt_is4(KM), KMX = fmt_is_mx(KM);
    constexpr int KMW = kmeta_words(KM, HD);
    constexpr int NBK = HD / 32;
    constexpr uint32_t k_cw4 = code_bytes(KM, HD);
    static_assert(!PERM || !fmt_is_mx(KM), "the other order of keys is for rows without block scales");
    const uint32_t ka8 = ka + (PERM ? 2 : 8) * krb;
    if constexpr (KMX) {
        float ks0[KMW], ks8[KMW];
        if constexpr (KMW == 2) {
            const float2 a = lds64f(mrow), b8 = lds64f(mrow + 8 * KMW * 4);
            ks0[0] = a.x; ks0[1] = a.y; ks8[0] = b8.x; ks8[1] = b8.y;
        } else {
#pragma unroll
            for (int w = 0; w < KMW / 4; ++w) {
                const float4 a = lds128f(mrow + 16 * w), b8 = lds128f(mrow + 8 * KMW * 4 + 16 * w);
                ks0[4 * w] = a.x; ks0[4 * w + 1] = a.y; ks0[4 * w + 2] = a.z; ks0[4 * w + 3] = a.w;
                ks8[4 * w] = b8.x; ks8[4 * w + 1] = b8.y; ks8[4 * w + 2] = b8.z; ks8[4 * w + 3] = b8.w;
            }
        }
#pragma unroll
        for (int bk = 0; bk < NBK; ++bk) {
            float acc[4];
            if constexpr (K4) {
                const uint32_t x0 = lds32(ka + 16 * bk), x8 = lds32(ka8 + 16 * bk);
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                cvt_e2m1x8_f16x2(x0, a0, a1, a2, a3);
                cvt_e2m1x8_f16x2(x8, b0, b1, b2, b3);
                mma_f16_16816_z(acc, a0, b0, a1, b1, qb0[2 * bk], qb1[2 * bk]);
                mma_f16_16816(acc, a2, b2, a3, b3, qb0[2 * bk + 1], qb1[2 * bk + 1]);
            } else {
                const uint32_t x0 = lds32(ka + 32 * bk), x8 = lds32(ka8 + 32 * bk);
                const uint32_t y0 = lds32(ka + 32 * bk + 4), y8 = lds32(ka8 + 32 * bk + 4);
                mma_f16_16816_z(acc, cvt_e4m3x2_f16x2(x0), cvt_e4m3x2_f16x2(x8), cvt_e4m3x2_hi_f16x2(x0),
                                cvt_e4m3x2_hi_f16x2(x8), qb0[2 * bk], qb1[2 * bk]);
                mma_f16_16816(acc, cvt_e4m3x2_f16x2(y0), cvt_e4m3x2_f16x2(y8), cvt_e4m3x2_hi_f16x2(y0),
                              cvt_e4m3x2_hi_f16x2(y8), qb0[2 * bk + 1], qb1[2 * bk + 1]);
            }
            if (bk == 0) {
                sr[0] = acc[0] * ks0[0]; sr[1] = acc[1] * ks0[0]; sr[2] = acc[2] * ks8[0]; sr[3] = acc[3] * ks8[0];
            } else {
                sr[0] = fmaf(acc[0], ks0[bk], sr[0]);
                sr[1] = fmaf(acc[1], ks0[bk], sr[1]);
                sr[2] = fmaf(acc[2], ks8[bk], sr[2]);
                sr[3] = fmaf(acc[3], ks8[bk], sr[3]);
            }
        }
    } else {
        if constexpr (K4) {
            constexpr int WPL = HD / 32;  // words of this lane per key
            uint32_t sg[HD / 64], sg8[HD / 64];
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
            constexpr bool KPL = KM == B200_TURBO_MSE && (B200_TURBO_PRMT & 1) && !WIDE;
            Tab16 kt;
            if constexpr (KPL) kt = load_tab16(plane_k);
            // the lane's chunk of a row: HD / 8 bytes at a multiple of HD / 8
            uint32_t xs0[WPL], xs8[WPL];
            lds_words<WPL, min_i(AL, HD / 8)>(ka, xs0);
            lds_words<WPL, min_i(AL, HD / 8)>(ka8, xs8);
#pragma unroll
            for (int w = 0; w < WPL; ++w) {
                const uint32_t x0 = xs0[w], x8 = xs8[w];
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                if constexpr (KPL) {
                    tab16_dq8(kt, x0, a0, a1, a2, a3);
                    tab16_dq8(kt, x8, b0, b1, b2, b3);
                } else {
                    dq4<KM, WIDE>(x0, lut_k, a0, a1, a2, a3);
                    dq4<KM, WIDE>(x8, lut_k, b0, b1, b2, b3);
                }
                if constexpr (KM == B200_NVFP4) {
                    const uint32_t s0 = sg[w / 2], s8 = sg8[w / 2];
                    a0 = hmul2_u32(a0, s0); a1 = hmul2_u32(a1, s0); a2 = hmul2_u32(a2, s0); a3 = hmul2_u32(a3, s0);
                    b0 = hmul2_u32(b0, s8); b1 = hmul2_u32(b1, s8); b2 = hmul2_u32(b2, s8); b3 = hmul2_u32(b3, s8);
                }
                if (w == 0) mma_f16_16816_z(sr, a0, b0, a1, b1, qb0[0], qb1[0]);
                else mma_f16_16816(sr, a0, b0, a1, b1, qb0[2 * w], qb1[2 * w]);
                mma_f16_16816(sr, a2, b2, a3, b3, qb0[2 * w + 1], qb1[2 * w + 1]);
            }
        } else {
            uint32_t xs0[STEPS], xs8[STEPS];  // the lane's chunk of a row: HD / 4 bytes at a multiple of HD / 4
            lds_words<STEPS, min_i(AL, HD / 4)>(ka, xs0);
            lds_words<STEPS, min_i(AL, HD / 4)>(ka8, xs8);
#pragma unroll
            for (int s = 0; s < STEPS; ++s) {
                const uint32_t x0 = xs0[s], x8 = xs8[s];
                if (s == 0)
                    mma_f16_16816_z(sr, cvt_e4m3x2_f16x2(x0), cvt_e4m3x2_f16x2(x8), cvt_e4m3x2_hi_f16x2(x0),
                                    cvt_e4m3x2_hi_f16x2(x8), qb0[0], qb1[0]);
                else
                    mma_f16_16816(sr, cvt_e4m3x2_f16x2(x0), cvt_e4m3x2_f16x2(x8), cvt_e4m3x2_hi_f16x2(x0),
                                  cvt_e4m3x2_hi_f16x2(x8), qb0[s], qb1[s]);
            }
        }
        const float kp0 = u2f(lds32(mrow)), kp8 = u2f(lds32(mrow + (PERM ? 2 : 8) * 4));
        sr[0] *= kp0; sr[1] *= kp0; sr[2] *= kp8; sr[3] *= kp8;
    }
}

// O^T += V^T P^T for the 16 keys at `va` (the lane's first code byte of key 2c; rows vrb bytes apart): keys 2c, 2c+1 |
// 2c+8, 2c+9, dims [g HD/8, (g+1) HD/8). `vsc_row`: the f16 block scales of the keys 2c, 2c + 1 (+ 16 bytes: 2c + 8,
// 2c + 9), pb0 / pb1: the weights as B fragments.
// PERM: the lane's four keys are four consecutive rows from `va` on (perm_key below) instead of 2c, 2c + 1, 2c + 8, 2c + 9.
template <int VM, int HD, bool WIDE = false, int AL = 4, bool PERM = false>
__device__ __forceinline__ void v_accum16(uint32_t va, uint32_t vrb, uint32_t vsc_row, uint32_t pb0, uint32_t pb1, float (&oacc)[HD / 16][4],
                                          uint32_t lut_v, uint32_t plane_v, int g) {
    constexpr bool V4 = fmt_is4(VM);
    constexpr int NBV = vsc_blocks(VM, HD);
    // the lane's chunk of each of its four rows: NW words at a multiple of 4 NW bytes
    constexpr int NW = V4 ? (HD / 64 > 0 ? HD / 64 : 1) : HD / 32;
    uint32_t xas[NW], xbs[NW], xcs[NW], xds[NW];
    lds_words<NW, min_i(AL, 4 * NW)>(va, xas);
    lds_words<NW, min_i(AL, 4 * NW)>(va + vrb, xbs);
    static_assert(!PERM || NBV == 0, "the other order of keys is for rows without block scales");
    lds_words<NW, min_i(AL, 4 * NW)>(va + (PERM ? 2 : 8) * vrb, xcs);
    lds_words<NW, min_i(AL, 4 * NW)>(va + (PERM ? 3 : 9) * vrb, xds);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        const uint32_t xa = xas[w], xb = xbs[w], xc = xcs[w], xd = xds[w];
        if constexpr (V4) {
            // nibbles of two keys side by side: byte i = (a[2i], b[2i]) and (a[2i+1], b[2i+1])
            const uint32_t tl0 = (xa & 0x0f0f0f0fu) | ((xb & 0x0f0f0f0fu) << 4);
            const uint32_t th0 = ((xa >> 4) & 0x0f0f0f0fu) | (xb & 0xf0f0f0f0u);
            const uint32_t tl1 = (xc & 0x0f0f0f0fu) | ((xd & 0x0f0f0f0fu) << 4);
            const uint32_t th1 = ((xc >> 4) & 0x0f0f0f0fu) | (xd & 0xf0f0f0f0u);
            uint32_t l0[4], h0[4], l1[4], h1[4];
            if constexpr (VM == B200_TURBO_MSE && (B200_TURBO_PRMT & 2) && !WIDE) {
                const Tab16 vt = load_tab16(plane_v);
                tab16_dq8(vt, tl0, l0[0], l0[1], l0[2], l0[3]);
                tab16_dq8(vt, th0, h0[0], h0[1], h0[2], h0[3]);
                tab16_dq8(vt, tl1, l1[0], l1[1], l1[2], l1[3]);
                tab16_dq8(vt, th1, h1[0], h1[1], h1[2], h1[3]);
            } else {
                dq4<VM, WIDE>(tl0, lut_v, l0[0], l0[1], l0[2], l0[3]);
                dq4<VM, WIDE>(th0, lut_v, h0[0], h0[1], h0[2], h0[3]);
                dq4<VM, WIDE>(tl1, lut_v, l1[0], l1[1], l1[2], l1[3]);
                dq4<VM, WIDE>(th1, lut_v, h1[0], h1[1], h1[2], h1[3]);
            }
            if constexpr (NBV > 0) {
                const int blk = (g * (HD / 8) + 8 * w) / (HD / NBV);
                const uint32_t sa = lds32(vsc_row + blk * WK * 2), sb = lds32(vsc_row + blk * WK * 2 + 16);
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
                const uint32_t sa = lds32(vsc_row + blk * WK * 2), sb = lds32(vsc_row + blk * WK * 2 + 16);
                l0 = hmul2_u32(l0, sa); h0 = hmul2_u32(h0, sa); l2 = hmul2_u32(l2, sa); h2 = hmul2_u32(h2, sa);
                l1 = hmul2_u32(l1, sb); h1 = hmul2_u32(h1, sb); l3 = hmul2_u32(l3, sb); h3 = hmul2_u32(h3, sb);
            }
            mma_f16_16816(oacc[2 * w], l0, h0, l1, h1, pb0, pb1);
            mma_f16_16816(oacc[2 * w + 1], l2, h2, l3, h3, pb0, pb1);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// A worker's share of the work
// ---------------------------------------------------------------------------------------------
struct Share {
    uint64_t total;   // cost of the whole call
    uint64_t x_end;   // end of this worker's range of cost positions
    uint32_t nw;      // workers that own cost positions (never more than there are positions)
    bool has_work;    // the worker owns at least one tile
    Segment seg;      // its first segment
};

// Computed by every worker (warp) from the lengths alone. Never more workers than cost positions: every worker
// between the owners of two tiles of a column then owns a tile of that column itself, so a column's segments are
// the consecutive workers first owner .. last owner.
__device__ __forceinline__ Share worker_share(const DecodeParams &p, uint32_t ny, uint32_t wid, uint32_t nw_grid, int lane) {
    Share sh;
    const uint32_t cc = p.col_cost;
    auto batch_cost = [&](uint32_t bb) -> uint32_t {
        const uint32_t t = (uint32_t)make_column(p, bb).tiles;
        return t ? (t + cc) * ny : 0u;
    };
    uint64_t total = 0;
    // up to 128 ragged entries: one round of loads (four entries per lane) serves the total and the search below
    const bool few = p.kv_len != nullptr && p.b <= 128;
    uint32_t fu[4], fincl[4];
    uint64_t fpre[4];
    if (p.kv_len == nullptr) {
        total = (uint64_t)batch_cost(0) * p.b;
    } else if (few) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t bb = 32 * k + lane;
            fu[k] = bb < p.b ? batch_cost(bb) : 0u;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint32_t incl = fu[k];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            fincl[k] = incl;
            fpre[k] = total;
            total += __shfl_sync(0xffffffffu, incl, 31);
        }
    } else {
        for (uint32_t base = 0; base < p.b; base += 32) {
            const uint32_t bb = base + lane;
            uint32_t u = bb < p.b ? batch_cost(bb) : 0u;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) u += __shfl_xor_sync(0xffffffffu, u, o);
            total += u;
        }
    }
    sh.total = total;
    sh.nw = (uint32_t)min((uint64_t)nw_grid, total);
    sh.has_work = wid < sh.nw;
    sh.x_end = 0;
    if (!sh.has_work) return sh;
    const uint64_t x_begin = total * wid / sh.nw;
    sh.x_end = total * (wid + 1) / sh.nw;
    // batch entry that holds cost position x_begin, and the position of its first column
    uint32_t b0 = 0;
    uint64_t b0_start = 0;
    if (p.kv_len == nullptr) {
        const uint64_t per_b = batch_cost(0);
        b0 = (uint32_t)(x_begin / per_b);
        b0_start = (uint64_t)b0 * per_b;
    } else if (few) {
        bool found = false;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t hit = __ballot_sync(0xffffffffu, fpre[k] + fincl[k] > x_begin);
            if (hit && !found) {
                const int l = __ffs(hit) - 1;
                b0 = 32 * k + l;
                b0_start = fpre[k] + __shfl_sync(0xffffffffu, fincl[k] - fu[k], l);
                found = true;
            }
        }
    } else {
        uint64_t carry = 0;
        for (uint32_t base = 0; base < p.b; base += 32) {
            const uint32_t bb = base + lane;
            const uint32_t u = bb < p.b ? batch_cost(bb) : 0u;
            uint32_t incl = u;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const uint32_t hit = __ballot_sync(0xffffffffu, carry + incl > x_begin);
            if (hit) {
                const int l = __ffs(hit) - 1;
                b0 = base + l;
                b0_start = carry + __shfl_sync(0xffffffffu, incl - u, l);
                break;
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    // first segment: the first tile at or after x_begin (a position inside a column's set up cost
    // snaps to the column's first tile)
    Segment &seg = sh.seg;
    seg.b = b0;
    seg.col = make_column(p, b0);
    const uint32_t tb = (uint32_t)seg.col.tiles;
    const uint64_t rem = x_begin - b0_start;
    seg.y = (uint32_t)(rem / (tb + cc));
    const uint32_t in_col = (uint32_t)(rem % (tb + cc));
    seg.t0 = in_col > cc ? in_col - cc : 0u;
    seg.x = b0_start + (uint64_t)seg.y * (tb + cc) + cc + seg.t0;
    if (seg.x >= sh.x_end) sh.has_work = false;  // the share lies inside a set up gap: no tile
    else seg.t1 = (uint32_t)min((uint64_t)tb, seg.t0 + (sh.x_end - seg.x));
    return sh;
}

// ---------------------------------------------------------------------------------------------
// What a worker does outside its tiles: the dependency on the stream's previous kernel, finished columns,
// gathered outputs
// ---------------------------------------------------------------------------------------------
// Launched as a programmatic dependent (after_prev), the grid runs, with nothing read but the lengths, while the
// stream's previous kernel is still running. What that kernel may still have in its hands (the outputs, the partial
// results, the gather's step word; without the caller's word that the inputs are final also the query and the rows)
// is not touched before prev_done() has returned: griddepcontrol.wait returns when the previous kernel has completed
// and its writes are visible, and is a no-op after a plain launch. With final inputs a worker gets through the tiles
// of its first segment before it has to ask: the step's first keys stream while the previous kernel's last blocks
// finish, and only the rows it must not read yet (the last fresh_rows of a sequence) and all stores wait.
struct Worker {
    const DecodeParams &p;
    int lane;
    uint32_t wid, nw_grid, ny, ncols, prow;
    uint64_t total;
    uint32_t nw;
    bool waited;
    uint32_t g_step;  // gathered outputs: this step's number, read once the previous kernel is done
    size_t g_base;    // and the offset of this rank's rows in the step's slot of every rank's buffer

    __device__ __forceinline__ Worker(const DecodeParams &p_, int lane_, uint32_t wid_, uint32_t nw_grid_, uint32_t ny_, const Share &sh)
        : p(p_), lane(lane_), wid(wid_), nw_grid(nw_grid_), ny(ny_), ncols(p_.b * ny_), prow(min((uint32_t)PACK, p_.rows_per_kv)),
          total(sh.total), nw(sh.nw), waited(false), g_step(0), g_base(0) {}

    __device__ __forceinline__ void prev_done() {
        if (waited) return;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
        if (p.ctr && p.world) {
            g_step = *reinterpret_cast<volatile uint32_t *>(p.step) + 1u;
            g_base = ((size_t)(g_step & 1u) * p.world + p.rank) * ((size_t)p.b * p.hq * p.lq) * p.d;
        }
    }

    // The last thing a worker does. A call whose stores did not wait for the previous kernel (out_free) still waits for
    // it here, in one block of the grid, when that block's work is done: a kernel of such a chain then never completes
    // before its predecessor, so whatever waits for one of them (a later call's prev_done(), an event, a plain launch)
    // has waited for all. One block, not all: every block waiting would make the fast places of the device wait for
    // the slow ones once per call (measured on 128 x 16384 MXFP8 keys: 696 us per call against 642 us).
    __device__ __forceinline__ void leave() {
        if (p.out_free && blockIdx.x == 0) prev_done();
    }

    // a column of this call is finished (its rows are stored): with gathered outputs the worker that finishes the
    // call's last column publishes the step to the other ranks
    __device__ __forceinline__ void column_done() {
        if (!p.world) return;
        fence_sys();
        __syncwarp();
        uint32_t last = 0;
        if (lane == 0) last = atomicInc(p.done_ctr, ncols - 1u) == ncols - 1u ? 1u : 0u;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            fence_sys();
            gather_publish(p.peer_flags, p.world, p.rank, p.step, g_step, p.gather_polls, p.status, p.lib_status, lane);
        }
    }

    // columns without a visible key get no worker: their rows are zeros, written once the previous kernel is done
    template <int HD>
    __device__ __forceinline__ void zero_columns(bool has_work) {
        if (!(p.ctr && (p.kv_len != nullptr || !has_work))) return;
        if (!p.out_free) prev_done();
        for (uint32_t col = wid; col < ncols; col += nw_grid) {
            const uint32_t b = col / ny, y = col - b * ny;
            if (make_column(p, b).tiles != 0) continue;
            float z[HD / 32];
#pragma unroll
            for (int k = 0; k < HD / 32; ++k) z[k] = 0.0f;
            for (uint32_t rr = 0; rr < prow; ++rr) {
                size_t obase, grow;
                if (!row_addr(p, b, y, rr, obase, grow)) break;
                store_row_piece<HD / 32>(p.out, obase + (size_t)lane * (HD / 32), z, p.out_dtype);
                for (uint32_t pr = 0; pr < p.world; ++pr)
                    store_row_piece<HD / 32>(p.peer_bufs[pr], g_base + grow * HD + (size_t)lane * (HD / 32), z, p.out_dtype);
            }
            column_done();
        }
    }

    // The end of a segment: oacc holds the unnormalized output rows 2c, 2c + 1 (dims [g HD/8, (g + 1) HD/8)) of the
    // segment's keys, M / lsum their running maxima (log2 domain) and normalizers, summed over the warp. A column
    // that this worker covers alone is stored straight from the registers; otherwise the normalized partial result
    // and its log-sum-exp go to the workspace and the worker counts itself on the column's arrival counter: the last
    // to arrive merges the column. Without arrival counters the combine grid merges. Rotated values are rotated back in
    // registers, wherever a row is finished.
    template <int HD>
    __device__ __forceinline__ void finish_segment(const Segment &seg, const float (&oacc)[HD / 16][4], const float (&M)[2], const float (&lsum)[2]) {
        constexpr int STEPS = HD / 16;
        const int g = lane >> 2, c = lane & 3;
        const uint32_t R = p.rows_per_kv, pack = seg.y % p.packs;
        if (!p.out_free) prev_done();
        const uint32_t colidx = seg.b * ny + seg.y;
        const float inv0 = lsum[0] > 0.0f ? 1.0f / lsum[0] : 0.0f, inv1 = lsum[1] > 0.0f ? 1.0f / lsum[1] : 0.0f;
        const uint32_t rr0 = 2 * c, rr1 = 2 * c + 1;
        const bool w0 = rr0 < prow && pack * PACK + rr0 < R, w1 = rr1 < prow && pack * PACK + rr1 < R;
        // the column's segments are the workers first .. last (consecutive, every one of them owns a tile of it)
        const uint64_t x_col = seg.x - seg.t0;  // cost position of the column's first tile
        const uint32_t first = seg.t0 == 0 ? wid : owner_of(x_col, total, nw);
        const uint32_t last = seg.t1 == (uint32_t)seg.col.tiles ? wid : owner_of(x_col + seg.col.tiles - 1, total, nw);
        const uint32_t nseg = last - first + 1;
        if (p.ctr && nseg == 1) {
            // the whole column in this worker's registers
            float o0[HD / 8], o1[HD / 8];
#pragma unroll
            for (int mt = 0; mt < STEPS; ++mt) {
                o0[2 * mt] = oacc[mt][0] * inv0; o0[2 * mt + 1] = oacc[mt][2] * inv0;
                o1[2 * mt] = oacc[mt][1] * inv1; o1[2 * mt + 1] = oacc[mt][3] * inv1;
            }
            if (p.v.rot == B200_ROT_HADAMARD) {
                // rows 2c and 2c + 1, each spread over the eight lanes g = 0..7 of this c (part = lane >> 2)
                hadamard_back_parts<HD / 8>(o0, lane, 4, 8, 16, p.v.signs, g * (HD / 8));
                hadamard_back_parts<HD / 8>(o1, lane, 4, 8, 16, p.v.signs, g * (HD / 8));
            }
            size_t obase, grow;
            if (w0 && row_addr(p, seg.b, seg.y, rr0, obase, grow)) {
                store_row_piece<HD / 8>(p.out, obase + g * (HD / 8), o0, p.out_dtype);
                for (uint32_t pr = 0; pr < p.world; ++pr) store_row_piece<HD / 8>(p.peer_bufs[pr], g_base + grow * HD + g * (HD / 8), o0, p.out_dtype);
            }
            if (w1 && row_addr(p, seg.b, seg.y, rr1, obase, grow)) {
                store_row_piece<HD / 8>(p.out, obase + g * (HD / 8), o1, p.out_dtype);
                for (uint32_t pr = 0; pr < p.world; ++pr) store_row_piece<HD / 8>(p.peer_bufs[pr], g_base + grow * HD + g * (HD / 8), o1, p.out_dtype);
            }
            column_done();
            return;
        }
        const size_t slot = (size_t)wid + colidx;
        float *po0 = p.part_o + (slot * prow + rr0) * HD + g * (HD / 8);
        float *po1 = p.part_o + (slot * prow + rr1) * HD + g * (HD / 8);
#pragma unroll
        for (int mt = 0; mt < STEPS; ++mt) {
            if (w0) *reinterpret_cast<float2 *>(po0 + 2 * mt) = make_float2(oacc[mt][0] * inv0, oacc[mt][2] * inv0);
            if (w1) *reinterpret_cast<float2 *>(po1 + 2 * mt) = make_float2(oacc[mt][1] * inv1, oacc[mt][3] * inv1);
        }
        if (g == 0) {
            if (w0) p.part_lse[slot * prow + rr0] = lsum[0] > 0.0f ? M[0] * LN2 + logf(lsum[0]) : -INFINITY;
            if (w1) p.part_lse[slot * prow + rr1] = lsum[1] > 0.0f ? M[1] * LN2 + logf(lsum[1]) : -INFINITY;
        }
        if (p.ctr) {
            // count this segment; the last of the column's workers to get here merges them all
            __threadfence();
            __syncwarp();
            uint32_t merge = 0;
            if (lane == 0) merge = atomicInc(p.ctr + colidx, nseg - 1u) == nseg - 1u ? 1u : 0u;
            merge = __shfl_sync(0xffffffffu, merge, 0);
            if (merge) {
                __threadfence();
                const size_t slot0 = (size_t)first + colidx;
                merge_column<HD>(p, seg.b, seg.y, slot0, (int)nseg, prow, g_base, lane);
                column_done();
            }
        } else if (seg.t0 == 0 && lane == 0) {
            // the worker that owns the first tile of a column publishes where its segments are (for the combine grid)
            p.meta[2 * (size_t)colidx] = (int32_t)(wid + colidx);
            p.meta[2 * (size_t)colidx + 1] = (int32_t)nseg;
        }
    }
};

// ---------------------------------------------------------------------------------------------
// The copy side of a worker: bulk copies of its tiles into the stages of its ring
// ---------------------------------------------------------------------------------------------
// Runs up to NS tiles ahead of the compute side through the same list of segments; tile t of the worker's list lives
// in stage t mod NS, so the copy issued after a tile is consumed goes into the stage just read. Rows are 72-140
// bytes: a copy starts at the 16-byte boundary below the tile's first row and ends at the one above its last.
struct CopySide {
    Segment iseg;
    int left;        // tiles still to copy in the copy side's segment
    int simple;      // of those, whole tiles that do not end their column: constant copy sizes, no tail handling
    bool more;       // the copy side has segments left
    uintptr_t k, v;  // 16-byte aligned global addresses of the next tile's copies
    uint32_t koff, voff;  // offset of the tile's first row inside its copy
    uint32_t kb, vb;      // bytes of a whole tile's copies
    int key;              // first key of the next tile
    // paged rows: the block of the next tile, the tile's first row in it, the block's rows and capacities, and the
    // addresses of the (batch entry, kv head) slabs of the block
    uint32_t pg, off, pg_rows, k_cap, v_cap;
    uintptr_t pk, pv;

    // per-segment constants
    __device__ __forceinline__ void enter(const DecodeParams &p, uint32_t krb, uint32_t vrb) {
        left = (int)(iseg.t1 - iseg.t0);
        simple = left - (iseg.t1 == (uint32_t)iseg.col.tiles ? 1 : 0);
        const uint32_t hk = iseg.y / p.packs;
        key = iseg.col.lo + (int)iseg.t0 * WK;
        const uintptr_t ka = reinterpret_cast<uintptr_t>(p.k_rows + (size_t)iseg.b * p.k_sb + (size_t)hk * p.k_sh) + (uintptr_t)(uint32_t)key * krb;
        const uintptr_t va = reinterpret_cast<uintptr_t>(p.v_rows + (size_t)iseg.b * p.v_sb + (size_t)hk * p.v_sh) + (uintptr_t)(uint32_t)key * vrb;
        koff = (uint32_t)(ka & 15u);
        voff = (uint32_t)(va & 15u);
        k = ka - koff;
        v = va - voff;
        kb = (koff + (uint32_t)WK * krb + 15u) & ~15u;
        vb = (voff + (uint32_t)WK * vrb + 15u) & ~15u;
    }

    __device__ __forceinline__ void start(const DecodeParams &p, const Segment &seg, uint32_t krb, uint32_t vrb) {
        iseg = seg;
        more = true;
        enter(p, krb, vrb);
    }

    // ---- paged rows: a tile's source is (block, row in the block) instead of rows + key * stride
    __device__ __forceinline__ void load_page(const DecodeParams &p, uint32_t krb, uint32_t vrb) {
        const B200Page pgd = p.pages[pg];
        const uint32_t hk = iseg.y / p.packs;
        pg_rows = pgd.rows;
        k_cap = pgd.k_cap;
        v_cap = pgd.v_cap;
        // block layout (batch entry, kv head, capacity, words): head stride = capacity rows, batch stride = hkv heads
        pk = reinterpret_cast<uintptr_t>(pgd.k) + ((uintptr_t)iseg.b * p.hkv + hk) * pgd.k_cap * krb;
        pv = reinterpret_cast<uintptr_t>(pgd.v) + ((uintptr_t)iseg.b * p.hkv + hk) * pgd.v_cap * vrb;
    }
    __device__ __forceinline__ void enter_paged(const DecodeParams &p, uint32_t krb, uint32_t vrb) {
        left = (int)(iseg.t1 - iseg.t0);
        const uint32_t T = iseg.col.t_lo + iseg.t0;
        pg = page_of_tile(p, T);
        off = (T - p.pg_tiles[pg]) * WK;
        load_page(p, krb, vrb);
    }
    __device__ __forceinline__ void start_paged(const DecodeParams &p, const Segment &seg, uint32_t krb, uint32_t vrb) {
        iseg = seg;
        more = true;
        enter_paged(p, krb, vrb);
    }
    // Copies the next tile into stage `st` and leaves its description (offsets of the first row inside the copies, first
    // key, number of keys) at `desc` for the compute side.
    __device__ __forceinline__ void tile_paged(Worker &w, uint32_t st, uint32_t bar, uint32_t desc, uint32_t krb, uint32_t vrb, uint32_t k_stage_bytes,
                                               uint64_t x_end) {
        const DecodeParams &p = w.p;
        const int lane = w.lane;
        const int key0 = (int)(p.pg_keys[pg] + off);
        const int nkeys = min(min(WK, (int)(pg_rows - off)), iseg.col.hi - key0);
        if (!w.waited && key0 + nkeys > iseg.col.lk - (int)p.fresh_rows) w.prev_done();
        const uintptr_t ka = pk + (uintptr_t)off * krb, va = pv + (uintptr_t)off * vrb;
        const uint32_t ko = (uint32_t)(ka & 15u), vo = (uint32_t)(va & 15u);
        const uintptr_t k0 = ka - ko, v0 = va - vo;
        const uint32_t ke = ko + (uint32_t)nkeys * krb, ve = vo + (uint32_t)nkeys * vrb;  // ends, from the copy start
        // A copy ends at the 16-byte boundary above its last row; where that may lie past the block's slab (the tile
        // reaches the slab's last row) it ends at the boundary below and the last words come by plain loads.
        const bool ktail = off + (uint32_t)nkeys >= k_cap, vtail = off + (uint32_t)nkeys >= v_cap;
        const uint32_t kbt = ktail ? (ke & ~15u) : ((ke + 15u) & ~15u), vbt = vtail ? (ve & ~15u) : ((ve + 15u) & ~15u);
        if (ktail && lane < 4) {
            const uint32_t o = kbt + 4u * lane;
            if (o >= ko && o < ke) sts32(st + o, *reinterpret_cast<const uint32_t *>(k0 + o));
        }
        if (vtail && lane >= 4 && lane < 8) {
            const uint32_t o = vbt + 4u * (lane - 4);
            if (o >= vo && o < ve) sts32(st + k_stage_bytes + o, *reinterpret_cast<const uint32_t *>(v0 + o));
        }
        if (lane == 0)
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(desc), "r"(ko), "r"(vo), "r"((uint32_t)key0), "r"((uint32_t)nkeys) : "memory");
        __syncwarp();
        if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kbt + vbt) : "memory");
            if (kbt)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(st), "l"(k0), "r"(kbt),
                             "r"(bar)
                             : "memory");
            if (vbt)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(st + k_stage_bytes),
                             "l"(v0), "r"(vbt), "r"(bar)
                             : "memory");
        }
        off += WK;
        if (--left == 0) {
            if (more) {
                more = next_segment(iseg, p, w.ny, x_end);
                if (more) enter_paged(p, krb, vrb);
            }
        } else if (off >= pg_rows) {
            // the next block that holds rows (there is one: tiles are left in this column)
            do ++pg; while (p.pages[pg].rows == 0);
            off = 0;
            load_page(p, krb, vrb);
        }
    }

    // copies the next tile into stage `st` with barrier `bar` (the caller checked left > 0) and moves on
    __device__ __forceinline__ void tile(Worker &w, uint32_t st, uint32_t bar, uint32_t krb, uint32_t vrb, uint32_t k_stage_bytes, uint64_t x_end) {
        const DecodeParams &p = w.p;
        const int lane = w.lane;
        // rows that the stream's previous kernel may still be writing are not copied before it is done
        if (B200_UNLIKELY(!w.waited && key + min(WK, iseg.col.hi - key) > iseg.col.lk - (int)p.fresh_rows)) w.prev_done();
        if (B200_LIKELY(simple > 0)) {
            --simple;
            if (lane == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kb + vb) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(st), "l"(k),
                             "r"(kb), "r"(bar)
                             : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(st + k_stage_bytes),
                             "l"(v), "r"(vb), "r"(bar)
                             : "memory");
            }
        } else {
            // the last tile of its column
            const int nkeys = min(WK, iseg.col.hi - key);
            // Rows below lk are readable, and so is the row after a tile when the cache has spare rows
            // (rows_cap): the 16-byte round up of a copy may then run into the next row. Otherwise the
            // last tile of a sequence copies the round down and fetches the few remaining words with
            // plain loads.
            const bool tail = key + nkeys >= iseg.col.lk && key + nkeys >= (int)p.rows_cap;
            uint32_t kbt = (koff + (uint32_t)nkeys * krb + 15u) & ~15u, vbt = (voff + (uint32_t)nkeys * vrb + 15u) & ~15u;
            if (tail) {
                const uint32_t ke = koff + (uint32_t)nkeys * krb, ve = voff + (uint32_t)nkeys * vrb;  // ends, from the copy start
                kbt = ke & ~15u;
                vbt = ve & ~15u;
                if (lane < 4) {
                    const uint32_t o = kbt + 4u * lane;
                    if (o >= koff && o < ke) sts32(st + o, *reinterpret_cast<const uint32_t *>(k + o));
                } else if (lane < 8) {
                    const uint32_t o = vbt + 4u * (lane - 4);
                    if (o >= voff && o < ve) sts32(st + k_stage_bytes + o, *reinterpret_cast<const uint32_t *>(v + o));
                }
                __syncwarp();
            }
            if (lane == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kbt + vbt) : "memory");
                if (kbt)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(st), "l"(k),
                                 "r"(kbt), "r"(bar)
                                 : "memory");
                if (vbt)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     st + k_stage_bytes),
                                 "l"(v), "r"(vbt), "r"(bar)
                                 : "memory");
            }
        }
        // WK rows are a multiple of 16 bytes: the next tile keeps its offset inside its copy
        k += (uintptr_t)WK * krb;
        v += (uintptr_t)WK * vrb;
        key += WK;
        if (B200_UNLIKELY(--left == 0 && more)) {
            more = next_segment(iseg, p, w.ny, x_end);
            if (more) enter(p, krb, vrb);
        }
    }

    __device__ __forceinline__ void stop() {
        left = 0;
        more = false;
    }
};

// Bounded wait for the phase of parity `par` of the mbarrier at `bar`: false when it did not complete in time
__device__ __forceinline__ bool stage_wait(uint32_t bar, uint32_t par) {
    uint32_t ok = 0;
    for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin)
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok)
                     : "r"(bar), "r"(par)
                     : "memory");
    return ok != 0;
}

// Visible keys of row r of a column's rows (ordered by token), bottom-right aligned masks
__device__ __forceinline__ void row_range(const DecodeParams &p, const Column &col, uint32_t r, int &lo, int &hi, int &pos) {
    const long long i = p.lq == 1 ? 0 : r / p.group;
    const long long ps = i + (long long)col.lk - (long long)p.lq;
    long long l = p.wl >= 0 ? max(ps - p.wl, 0ll) : 0ll;
    long long h = p.wr >= 0 ? min(ps + p.wr + 1, (long long)col.lk) : (long long)col.lk;
    l = min(l, (long long)col.lk);
    h = max(h, l);
    lo = (int)l;
    hi = (int)h;
    pos = (int)max(min(ps, 2147483647ll), -2147483647ll);
}

// Scores of a tile -> weights: vm from the tile's per-key scalars, plain or masked softmax. Returns whether the
// running maxima moved (al then holds the factors for what was accumulated before).
struct SegMask {
    int LOmax, HImin;  // every key in [LOmax, HImin) is visible to every row of the pack
    bool plain;        // no soft-capping, no ALiBi
};

// Which key of a 16-key half a lane's row g (0..7) stands for when the keys are dealt in the other order, for packed rows
// of 18 words: the four rows that a half warp reads together then start 0, 2, 16 and 18 banks apart (keys' side, 8-byte
// loads of four chunks per row) or 8 banks apart (values' side, eight lanes per row), so no load meets another on a
// bank. Row g + 8 of the product is the key 2 rows further; the values' lanes hold four consecutive keys.
__host__ __device__ constexpr int perm_key(int g) { return (g & 1) + 8 * ((g >> 1) & 1) + 4 * (g >> 2); }

template <bool PERM = false>
__device__ __forceinline__ bool tile_softmax(const DecodeParams &p, const Segment &seg, const SegMask &sm, int key0, int nkeys, uint32_t vmeta_g,
                                             const float (&sr)[2][4], const float (&qs)[2], const float (&qs2)[2], float (&M)[2], float (&lsum)[2],
                                             uint32_t (&pb)[4], float (&al)[2], int lane) {
    const int g = lane >> 2, c = lane & 3;
    float2 vm[4];  // (sigma, log2 sigma) of the keys g, g + 8, g + 16, g + 24 (the other order: vmeta_g is the key's, then + 2, + 16, + 18)
#pragma unroll
    for (int k = 0; k < 4; ++k) vm[k] = lds64f(vmeta_g + (PERM ? 16 * (k & 1) + 128 * (k >> 1) : k * 64));
    if (B200_LIKELY(sm.plain && nkeys == WK && key0 >= sm.LOmax && key0 + WK <= sm.HImin)) return softmax_plain(sr, vm, qs2, M, lsum, pb, al);
    // masks, soft-capping, ALiBi: the two query rows whose scores this lane holds (columns 2c, 2c + 1)
    const uint32_t hk = seg.y / p.packs, pack = seg.y % p.packs, G = p.group;
    RowMask rm;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const uint32_t r = pack * PACK + 2 * c + e;
        rm.lo[e] = rm.hi[e] = rm.pos[e] = 0;
        rm.slope[e] = 0.0f;
        if (r < p.rows_per_kv) {
            row_range(p, seg.col, r, rm.lo[e], rm.hi[e], rm.pos[e]);
            rm.hi[e] = min(rm.hi[e], key0 + nkeys);  // a short tile inside a column (the end of a cache block): its spare rows hold no keys
            if (p.alibi) rm.slope[e] = p.alibi[(size_t)seg.b * p.alibi_bs + hk * G + (p.lq == 1 ? r : r % G)];
        }
    }
    return softmax_masked<PERM>(sr, vm, qs, p.softcap, key0 + (PERM ? perm_key(g) : g), rm, M, lsum, pb, al);
}

__device__ __forceinline__ SegMask segment_mask(const DecodeParams &p, const Segment &seg) {
    // rows are ordered by token: the last row of the pack has the highest lower bound, the first the lowest upper bound
    SegMask sm;
    const uint32_t pack = seg.y % p.packs;
    int lo, hi, pos;
    row_range(p, seg.col, min(pack * PACK + PACK, p.rows_per_kv) - 1, lo, hi, pos);
    sm.LOmax = lo;
    row_range(p, seg.col, pack * PACK, lo, hi, pos);
    sm.HImin = hi;
    sm.plain = p.softcap <= 0.0f && p.alibi == nullptr;
    return sm;
}

// rows past the end of a column's last tile hold stale bytes: cleared so that masked keys decode to finite values
__device__ __forceinline__ void clear_stale_rows(uint32_t kt, uint32_t vt, int nkeys, uint32_t krb, uint32_t vrb, int lane) {
    for (uint32_t w = nkeys * (krb >> 2) + lane; w < WK * (krb >> 2); w += 32) sts32(kt + 4 * w, 0u);
    for (uint32_t w = nkeys * (vrb >> 2) + lane; w < WK * (vrb >> 2); w += 32) sts32(vt + 4 * w, 0u);
    __syncwarp();
}

// one time set up of a block: codebook tables of the TurboQuant formats in shared memory
template <int KM, int VM>
__device__ __forceinline__ void load_codebooks(const DecodeParams &p, uint32_t lut_k, uint32_t lut_v, uint32_t plane_k, int tid, int nthreads) {
    if constexpr (KM == B200_TURBO_MSE)
        for (int i = tid; i < 256; i += nthreads) sts32(lut_k + 4 * i, pack_f16x2(p.k.tab[i & 15], p.k.tab[i >> 4]));
    if constexpr (VM == B200_TURBO_MSE)
        for (int i = tid; i < 256; i += nthreads) sts32(lut_v + 4 * i, pack_f16x2(p.v.tab[i & 15], p.v.tab[i >> 4]));
    if (tid < 16 && ((tid < 8) ? KM == B200_TURBO_MSE : VM == B200_TURBO_MSE)) {
        // byte planes of the codebook: words 0..3 low bytes, 4..7 high bytes
        const float *tab = tid < 8 ? p.k.tab : p.v.tab;
        const int w = tid & 7, sh = w < 4 ? 0 : 8;
        uint32_t v = 0;
        for (int j = 0; j < 4; ++j) v |= ((pack_f16x2(tab[4 * (w & 3) + j], 0.0f) >> sh) & 0xffu) << (8 * j);
        sts32(plane_k + 4 * tid, v);
    }
}

// ---------------------------------------------------------------------------------------------
// Kernel 1: every warp a worker
// ---------------------------------------------------------------------------------------------
// PAGED: the rows live in the blocks of a page table; tiles are cut at the blocks' ends, the copy side leaves a
// description of every tile beside its stage, and the row strides are those of the call (NAT is not combined with it).
template <int KM, int VM, int HD, bool NAT, bool PAGED = false>
__global__ void __launch_bounds__(DW * 32, B200_DECODE_MIN_BLOCKS) tq_decode_kernel(const DecodeParams p) {
    constexpr int STEPS = HD / 16;          // k-steps of K Q^T == m-tiles of the output
    constexpr bool K4 = fmt_is4(KM), V4 = fmt_is4(VM);
    constexpr bool KMX = fmt_is_mx(KM);     // block-wise accumulation, contraction order A
    constexpr int KMW = kmeta_words(KM, HD);
    constexpr int META = meta_bytes(KM, VM, HD);
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);  // [DW][NS_MAX]
    const int NS = (int)p.ns;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t lut_k = sbase + 128, lut_v = lut_k + 1024, plane_k = lut_v + 1024, plane_v = plane_k + 32;
    // row strides and stage sizes: compile-time when the rows are packed back to back (NAT)
    const uint32_t krb = NAT ? (uint32_t)nat_row_bytes(KM, HD) : (uint32_t)p.k_ss * 4u;
    const uint32_t vrb = NAT ? (uint32_t)nat_row_bytes(VM, HD) : (uint32_t)p.v_ss * 4u;
    // native rows start at multiples of this many bytes (the host checks the base addresses and the slab strides)
    constexpr int KAL = NAT ? nat_row_align(KM, HD) : 4, VAL = NAT ? nat_row_align(VM, HD) : 4;
    const uint32_t k_stage_bytes = NAT ? stage_part_bytes((uint32_t)nat_row_bytes(KM, HD)) : p.k_stage_bytes;
    const uint32_t v_stage_bytes = NAT ? stage_part_bytes((uint32_t)nat_row_bytes(VM, HD)) : p.v_stage_bytes;
    const uint32_t stage_bytes = k_stage_bytes + v_stage_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const uint32_t ny = p.hkv * p.packs;
    const uint32_t nw_grid = gridDim.x * DW, wid = blockIdx.x * DW + warp;

    // ------------------------------------------------------------------ one time set up (the only block barrier)
    if (tid == 0) {
        for (int i = 0; i < DW * NS_MAX; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    load_codebooks<KM, VM>(p, lut_k, lut_v, plane_k, tid, DW * 32);
    __syncthreads();
    // the next kernel of the stream may be scheduled from here on (a combine grid, or the next attention launched as
    // a programmatic dependent); it waits for this grid's completion itself before it touches memory
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // paged rows: the kernel that wrote the table's prefix sums is the stream's previous kernel, and this grid was
    // launched as its programmatic dependent (its launch latency is hidden): the sums are read from here on
    if constexpr (PAGED) asm volatile("griddepcontrol.wait;" ::: "memory");
    const Share sh = worker_share(p, ny, wid, nw_grid, lane);
    Worker wk(p, lane, wid, nw_grid, ny, sh);
    if (PAGED || !p.prefetch) wk.prev_done();
    if (!sh.has_work) {
        wk.zero_columns<HD>(false);
        wk.leave();
        return;
    }

    const uint32_t meta_s = sbase + FIXED_SMEM + warp * META;    // [WK][KMW] f32
    const uint32_t vmeta_s = meta_s + WK * KMW * 4;              // [WK] (sigma, log2 sigma)
    const uint32_t vsc_s = vmeta_s + WK * 8;                     // [NBV][WK] f16
    float *qstage = reinterpret_cast<float *>(smem + FIXED_SMEM + DW * META) + (size_t)warp * PACK * HD;  // only with rotated keys of a head dim above 128
    const uint32_t wstage_s = sbase + FIXED_SMEM + DW * META + p.qstage_bytes + (uint32_t)warp * NS * stage_bytes;
    const uint32_t wbar_s = smem_u32(bars + warp * NS_MAX);
    // paged rows: one description per stage, behind the rings of all warps
    const uint32_t wdesc_s = sbase + FIXED_SMEM + DW * META + p.qstage_bytes + (uint32_t)DW * NS * stage_bytes + (uint32_t)warp * NS_MAX * 16;
    bool wait_failed = false;

    // Filling the ring. With the caller's word that the inputs are final (prefetch) all stages are asked for right away.
    // Otherwise the first tile alone, and the other stages once the first query rows are loaded: with every worker of
    // the grid asking for all its stages at once, the first tiles would arrive behind 26 MB of later ones.
    CopySide cs;
    if constexpr (PAGED) cs.start_paged(p, sh.seg, krb, vrb);
    else cs.start(p, sh.seg, krb, vrb);
    auto copy_tile = [&](uint32_t st, uint32_t bar, uint32_t desc) {
        if constexpr (PAGED) cs.tile_paged(wk, st, bar, desc, krb, vrb, k_stage_bytes, sh.x_end);
        else cs.tile(wk, st, bar, krb, vrb, k_stage_bytes, sh.x_end);
    };
    int primed = 0;
    auto prime = [&](int upto) {
        for (; primed < upto && cs.left > 0; ++primed)
            copy_tile(wstage_s + (uint32_t)primed * stage_bytes, wbar_s + 8u * (uint32_t)primed, wdesc_s + 16u * (uint32_t)primed);
    };
    prime(p.prefetch ? NS : 1);

    // ------------------------------------------------------------------ the compute side
    // lane offsets inside a tile: K rows g (and g + 8), V rows 2c (and 2c + 1, 2c + 8, 2c + 9)
    const uint32_t k_lane = g * krb + (KMX ? (K4 ? 4u * c : 8u * c) : (K4 ? c * (HD / 8) : c * (HD / 4)));
    const uint32_t v_lane = 2 * c * vrb + (V4 ? g * (HD / 16) : g * (HD / 8));
    const uint32_t mrow_g = meta_s + g * KMW * 4, vmeta_g = vmeta_s + g * 8, vsc_c = vsc_s + 4 * c;
    uint32_t c_st = wstage_s, c_bar = wbar_s;
    int c_stage = 0;
    uint32_t par = 0;  // parity to wait for on the current stage: flips every time the ring wraps

    uint32_t qb0[STEPS], qb1[STEPS];
    float qs[2], qs2[2];
    float oacc[STEPS][4];

    Segment seg = sh.seg;
    bool more = true;
    while (more) {
        // ================================================================ segment set up
        const uint32_t hk = seg.y / p.packs, pack = seg.y % p.packs;
        const Column &col = seg.col;
        const SegMask sm = segment_mask(p, seg);
        // running maxima (log2 domain, value scale folded in) and partial normalizers of rows 2c, 2c + 1
        float M[2] = {-1e30f, -1e30f}, lsum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int mt = 0; mt < STEPS; ++mt) oacc[mt][0] = oacc[mt][1] = oacc[mt][2] = oacc[mt][3] = 0.0f;

        if (!wait_failed) {
            load_query<KM, HD>(p, seg.b, hk, pack, qstage, lane, qb0, qb1, qs, qs2);
            // the other stages of the ring (first segment only)
            prime(NS);

            // ============================================================ the tiles of the segment
            const int n_t = (int)(seg.t1 - seg.t0);
            int key0 = col.lo + (int)seg.t0 * WK;
            // offsets of the tiles' first rows inside their copies (paged rows: per tile, from the tile's description)
            const uint32_t koff = PAGED ? 0u : (uint32_t)((reinterpret_cast<uintptr_t>(p.k_rows + (size_t)seg.b * p.k_sb + (size_t)hk * p.k_sh) + (uintptr_t)(uint32_t)key0 * krb) & 15u);
            const uint32_t voff = PAGED ? 0u : (uint32_t)((reinterpret_cast<uintptr_t>(p.v_rows + (size_t)seg.b * p.v_sb + (size_t)hk * p.v_sh) + (uintptr_t)(uint32_t)key0 * vrb) & 15u);
            uint32_t kt_off = koff + k_lane, vt_off = k_stage_bytes + voff + v_lane;
            uint32_t kr_off = koff + lane * krb, vr_off = k_stage_bytes + voff + lane * vrb;
            for (int n = 0; n < n_t; ++n, key0 += WK) {
                if (B200_UNLIKELY(!stage_wait(c_bar, par))) {
                    // the copy never landed: give up on the keys (the outputs are void, the status says so), stop
                    // copying, but keep counting this worker's segments so that no column waits for it
                    wait_failed = true;
                    cs.stop();
                    break;
                }
                const uint32_t st_s = c_st;
                int nkeys = min(WK, col.hi - key0);
                uint32_t tk_off = koff, tv_off = voff;
                if constexpr (PAGED) {
                    // the tile as the copy side described it
                    uint32_t dk, dv, d0, dn;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(dk), "=r"(dv), "=r"(d0), "=r"(dn) : "r"(wdesc_s + 16u * (uint32_t)c_stage));
                    tk_off = dk;
                    tv_off = dv;
                    key0 = (int)d0;
                    nkeys = (int)dn;
                    kt_off = dk + k_lane;
                    vt_off = k_stage_bytes + dv + v_lane;
                    kr_off = dk + lane * krb;
                    vr_off = k_stage_bytes + dv + lane * vrb;
                }
                if (B200_UNLIKELY(nkeys < WK)) clear_stale_rows(st_s + tk_off, st_s + k_stage_bytes + tv_off, nkeys, krb, vrb, lane);
                // ---- per-key scalars of the tile, lane = key
                tile_meta<KM, VM, HD>(st_s + kr_off, st_s + vr_off, meta_s, vmeta_s, vsc_s, lane);
                // ---- scores of the 32 keys: sr[u][2 k + e] = key 16 u + g + 8 k, row 2c + e
                float sr[2][4];
                k_scores16<KM, HD, false, KAL>(st_s + kt_off, krb, mrow_g, qb0, qb1, lut_k, plane_k, c, sr[0]);
                k_scores16<KM, HD, false, KAL>(st_s + kt_off + 16 * krb, krb, mrow_g + 16 * KMW * 4, qb0, qb1, lut_k, plane_k, c, sr[1]);
                // ---- online softmax
                uint32_t pb[4];
                float al[2];
                if (B200_UNLIKELY(tile_softmax(p, seg, sm, key0, nkeys, vmeta_g, sr, qs, qs2, M, lsum, pb, al, lane))) {
#pragma unroll
                    for (int mt = 0; mt < STEPS; ++mt) {
                        oacc[mt][0] *= al[0];
                        oacc[mt][1] *= al[1];
                        oacc[mt][2] *= al[0];
                        oacc[mt][3] *= al[1];
                    }
                }
                // ---- O^T += V^T P^T
                v_accum16<VM, HD, false, VAL>(st_s + vt_off, vrb, vsc_c, pb[0], pb[1], oacc, lut_v, plane_v, g);
                v_accum16<VM, HD, false, VAL>(st_s + vt_off + 16 * vrb, vrb, vsc_c + 32, pb[2], pb[3], oacc, lut_v, plane_v, g);
                // the stage was read (and possibly patched) through the generic proxy: order that before the
                // bulk copy of the next tile into it
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (B200_LIKELY(cs.left > 0)) copy_tile(c_st, c_bar, wdesc_s + 16u * (uint32_t)c_stage);
                c_st += stage_bytes;
                c_bar += 8;
                if (++c_stage == NS) {
                    c_stage = 0;
                    c_st = wstage_s;
                    c_bar = wbar_s;
                    par ^= 1u;
                }
            }
        }

        // ================================================================ this warp's partial result of the column
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            lsum[0] += __shfl_xor_sync(0xffffffffu, lsum[0], o);
            lsum[1] += __shfl_xor_sync(0xffffffffu, lsum[1], o);
        }
        wk.finish_segment<HD>(seg, oacc, M, lsum);
        more = next_segment(seg, p, ny, sh.x_end);
    }
    wk.zero_columns<HD>(true);
    if (wait_failed) {
        if (p.status) atomicExch(p.status, 1);
        if (p.lib_status) atomicExch(p.lib_status, 1);
    }
    wk.leave();
}

// ---------------------------------------------------------------------------------------------
// Kernel 2: a worker is a pair of warps (codebook formats, whose table look-ups bind the kernel to instruction issue)
// ---------------------------------------------------------------------------------------------
// The keys' warp computes the scores and the softmax of a tile and hands the weights (as B fragments), the value
// block scales and, when the running maxima moved, the rescale factors to the values' warp through a two-slot queue
// in shared memory; the values' warp accumulates the outputs, releases the stage and issues the copy of the tile
// that takes its place. Each warp holds half the state of a whole worker (query fragments and softmax state on one
// side, output accumulators and the copy side on the other), so twice as many warps fit on an SM at 128 registers
// each, and a pair works on two tiles at once: more instructions in flight for a kernel that is bound by their
// issue, with the same number of bytes in flight. The segment's last message carries the maxima and normalizers.
// Which format pairs take this kernel: 4-bit rows of which at least one side is a codebook format. Measured on B200:
// the table look-ups of the codebook formats gain 15 % from the split (TurboQuant-4 decode, 32768 keys per sequence),
// the packed conversions of MXFP4 / NVFP4 gain nothing (the extra warps make up for the messages' cost, no more).
__host__ __device__ constexpr bool pair_formats(int km, int vm) {
    return fmt_is4(km) && fmt_is4(vm) && (km == B200_TURBO_MSE || vm == B200_TURBO_MSE);
}
constexpr int PW = 4;        // pairs per block: warps 0..3 keys, 4..7 values
constexpr int PQ = 2;        // slots of a pair's queue
constexpr int PNS_MAX = 4;   // stages per pair
constexpr int PAIR_FIXED = 256 + 2048 + 128;  // barriers, pair tables, byte-plane tables
// Keys and values both in the 4-bit codebook format: one pair table with a copy of every entry per lane (32 KB) instead
// of two of 1 KB, so that the look-ups of a warp never collide on a bank; both sides are decoded from it.
#ifndef B200_WIDE_LUT
#define B200_WIDE_LUT 1
#endif
__host__ __device__ constexpr bool pair_wide_lut(int km, int vm) { return B200_WIDE_LUT && km == B200_TURBO_MSE && vm == B200_TURBO_MSE; }
__host__ __device__ constexpr int pair_fixed_bytes(int km, int vm) { return pair_wide_lut(km, vm) ? 256 + 32768 + 128 : PAIR_FIXED; }
// one message: weights [lane][4] u32, rescale factors [lane][2] f32, their flag, f16 block scales of V [block][key]
__host__ __device__ constexpr int pair_msg_bytes(int vm, int hd) { return 512 + 256 + 16 + vsc_blocks(vm, hd) * WK * 2; }
// per pair: key scales and (sigma, log2 sigma) of a tile (the keys' warp's own), then the queue
__host__ __device__ constexpr int pair_meta_bytes(int km, int vm, int hd) { return WK * kmeta_words(km, hd) * 4 + WK * 8 + PQ * pair_msg_bytes(vm, hd); }

template <int KM, int VM, int HD, bool NAT>
__global__ void __launch_bounds__(PW * 64, 2) tq_decode_pair_kernel(const DecodeParams p) {
    constexpr int STEPS = HD / 16;
    constexpr bool K4 = fmt_is4(KM), V4 = fmt_is4(VM);
    constexpr bool KMX = fmt_is_mx(KM);
    constexpr int KMW = kmeta_words(KM, HD);
    constexpr int MSG = pair_msg_bytes(VM, HD);
    constexpr int PMETA = pair_meta_bytes(KM, VM, HD);
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);  // [PW][8]: stages full 0..3, messages full 4..5, messages free 6..7
    const int NS = (int)p.ns;
    const uint32_t sbase = smem_u32(smem);
    constexpr bool WIDE = pair_wide_lut(KM, VM);
    // packed rows of 18 words (both sides 4-bit codebook rows): keys dealt to the lanes so that no code load meets another on a bank
    constexpr bool PERM = WIDE && NAT && nat_row_bytes(KM, HD) == 72 && nat_row_bytes(VM, HD) == 72;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    // WIDE: one table of [256][32] words for keys and values (both sides decode with the same codebook), every lane
    // reading its own column
    const uint32_t lut_base = sbase + 256;
    const uint32_t lut_k = WIDE ? lut_base + 4u * lane : lut_base, lut_v = WIDE ? lut_k : lut_k + 1024;
    const uint32_t plane_k = lut_base + (WIDE ? 32768u : 2048u), plane_v = plane_k + 32;
    const uint32_t krb = NAT ? (uint32_t)nat_row_bytes(KM, HD) : (uint32_t)p.k_ss * 4u;
    const uint32_t vrb = NAT ? (uint32_t)nat_row_bytes(VM, HD) : (uint32_t)p.v_ss * 4u;
    // native rows start at multiples of this many bytes (the host checks the base addresses and the slab strides)
    constexpr int KAL = NAT ? nat_row_align(KM, HD) : 4, VAL = NAT ? nat_row_align(VM, HD) : 4;
    const uint32_t k_stage_bytes = NAT ? stage_part_bytes((uint32_t)nat_row_bytes(KM, HD)) : p.k_stage_bytes;
    const uint32_t v_stage_bytes = NAT ? stage_part_bytes((uint32_t)nat_row_bytes(VM, HD)) : p.v_stage_bytes;
    const uint32_t stage_bytes = k_stage_bytes + v_stage_bytes;

    const int pair = warp & (PW - 1);
    const bool keys_side = warp < PW;
    const uint32_t ny = p.hkv * p.packs;
    const uint32_t nw_grid = gridDim.x * PW, wid = blockIdx.x * PW + pair;

    if (tid == 0) {
        for (int i = 0; i < PW * 8; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    if constexpr (WIDE) {
        // entry i (two codes) of the keys' codebook, once per lane; the values' codebook must be the same table
        for (int idx = tid; idx < 256 * 32; idx += PW * 64) sts32(lut_base + 4u * idx, pack_f16x2(p.k.tab[(idx >> 5) & 15], p.k.tab[idx >> 9]));
    } else {
        load_codebooks<KM, VM>(p, lut_k, lut_v, plane_k, tid, PW * 64);
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // both warps of a pair work out the pair's share
    const Share sh = worker_share(p, ny, wid, nw_grid, lane);
    Worker wk(p, lane, wid, nw_grid, ny, sh);
    if (!p.prefetch) wk.prev_done();
    if (!sh.has_work) {
        if (!keys_side) wk.zero_columns<HD>(false);
        wk.leave();
        return;
    }

    constexpr int PFIX = pair_fixed_bytes(KM, VM);
    const uint32_t pmeta_s = sbase + PFIX + pair * PMETA;
    const uint32_t meta_s = pmeta_s;                       // [WK][KMW] f32
    const uint32_t vmeta_s = meta_s + WK * KMW * 4;        // [WK] (sigma, log2 sigma)
    const uint32_t queue_s = vmeta_s + WK * 8;             // [PQ] messages
    // rotation staging of the keys' warp for the queries: head dims above 128 only (up to 128 the rotation runs in
    // registers, like the rotation back of the outputs at every head dim)
    float *qstage = reinterpret_cast<float *>(smem + PFIX + PW * PMETA) + (size_t)pair * PACK * HD;
    const uint32_t wstage_s = sbase + PFIX + PW * PMETA + p.qstage_bytes + (uint32_t)pair * NS * stage_bytes;
    const uint32_t wbar_s = smem_u32(bars + pair * 8);     // stages
    const uint32_t qfull_s = wbar_s + 32, qfree_s = wbar_s + 48;

    uint32_t c_st = wstage_s, c_bar = wbar_s;
    int c_stage = 0;
    uint32_t par = 0;      // parity of the current stage's barrier
    uint32_t msgs = 0;     // messages sent (keys' side) or taken (values' side) so far: slot = msgs % PQ
    bool wait_failed = false;
    Segment seg = sh.seg;
    bool more = true;

    if (keys_side) {
        // ============================================================== the keys' warp
        const uint32_t kg = PERM ? (uint32_t)perm_key(g) : (uint32_t)g;  // the key (of 16) behind the lane's row g
        const uint32_t k_lane = kg * krb + (KMX ? (K4 ? 4u * c : 8u * c) : (K4 ? c * (HD / 8) : c * (HD / 4)));
        const uint32_t mrow_g = meta_s + kg * KMW * 4, vmeta_g = vmeta_s + kg * 8;
        uint32_t qb0[STEPS], qb1[STEPS];
        float qs[2], qs2[2];
        // a free slot for message `msgs`: the values' warp has taken message msgs - PQ
        auto slot_wait = [&]() -> bool {
            if (msgs < (uint32_t)PQ) return true;
            return stage_wait(qfree_s + 8u * (msgs % PQ), ((msgs / PQ) - 1u) & 1u);
        };
        auto slot_send = [&]() {
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qfull_s + 8u * (msgs % PQ)) : "memory");
            ++msgs;
        };
        while (more && !wait_failed) {
            const uint32_t hk = seg.y / p.packs, pack = seg.y % p.packs;
            const Column &col = seg.col;
            const SegMask sm = segment_mask(p, seg);
            float M[2] = {-1e30f, -1e30f}, lsum[2] = {0.0f, 0.0f};
            load_query<KM, HD>(p, seg.b, hk, pack, qstage, lane, qb0, qb1, qs, qs2);
            const int n_t = (int)(seg.t1 - seg.t0);
            int key0 = col.lo + (int)seg.t0 * WK;
            const uint32_t koff = (uint32_t)((reinterpret_cast<uintptr_t>(p.k_rows + (size_t)seg.b * p.k_sb + (size_t)hk * p.k_sh) + (uintptr_t)(uint32_t)key0 * krb) & 15u);
            const uint32_t voff = (uint32_t)((reinterpret_cast<uintptr_t>(p.v_rows + (size_t)seg.b * p.v_sb + (size_t)hk * p.v_sh) + (uintptr_t)(uint32_t)key0 * vrb) & 15u);
            const uint32_t kt_off = koff + k_lane;
            const uint32_t kr_off = koff + lane * krb, vr_off = k_stage_bytes + voff + lane * vrb;
            for (int n = 0; n < n_t; ++n, key0 += WK) {
                if (!stage_wait(c_bar, par) || !slot_wait()) {
                    wait_failed = true;
                    break;
                }
                const uint32_t st_s = c_st, msg_s = queue_s + (msgs % PQ) * MSG;
                const int nkeys = min(WK, col.hi - key0);
                if (nkeys < WK) clear_stale_rows(st_s + koff, st_s + k_stage_bytes + voff, nkeys, krb, vrb, lane);
                tile_meta<KM, VM, HD>(st_s + kr_off, st_s + vr_off, meta_s, vmeta_s, msg_s + 784, lane);
                float sr[2][4];
                k_scores16<KM, HD, WIDE, KAL, PERM>(st_s + kt_off, krb, mrow_g, qb0, qb1, lut_k, plane_k, c, sr[0]);
                k_scores16<KM, HD, WIDE, KAL, PERM>(st_s + kt_off + 16 * krb, krb, mrow_g + 16 * KMW * 4, qb0, qb1, lut_k, plane_k, c, sr[1]);
                uint32_t pb[4];
                float al[2];
                const bool moved = tile_softmax<PERM>(p, seg, sm, key0, nkeys, vmeta_g, sr, qs, qs2, M, lsum, pb, al, lane);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(msg_s + lane * 16), "r"(pb[0]), "r"(pb[1]), "r"(pb[2]), "r"(pb[3]) : "memory");
                if (moved) asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(msg_s + 512 + lane * 8), "f"(al[0]), "f"(al[1]) : "memory");
                if (lane == 0) sts32(msg_s + 768, moved ? 1u : 0u);
                slot_send();
                c_st += stage_bytes;
                c_bar += 8;
                if (++c_stage == NS) {
                    c_stage = 0;
                    c_st = wstage_s;
                    c_bar = wbar_s;
                    par ^= 1u;
                }
            }
            if (wait_failed) break;
            // the segment's last message: maxima and normalizers (summed over the warp) of the rows 2c, 2c + 1
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                lsum[0] += __shfl_xor_sync(0xffffffffu, lsum[0], o);
                lsum[1] += __shfl_xor_sync(0xffffffffu, lsum[1], o);
            }
            if (!slot_wait()) {
                wait_failed = true;
                break;
            }
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(queue_s + (msgs % PQ) * MSG + lane * 16), "f"(M[0]), "f"(M[1]), "f"(lsum[0]),
                         "f"(lsum[1])
                         : "memory");
            slot_send();
            more = next_segment(seg, p, ny, sh.x_end);
        }
    } else {
        // ============================================================== the values' warp
        const uint32_t v_lane = (PERM ? (uint32_t)perm_key(2 * c) : 2u * c) * vrb + (V4 ? g * (HD / 16) : g * (HD / 8));
        float oacc[STEPS][4];
        CopySide cs;
        cs.start(p, sh.seg, krb, vrb);
        for (int i = 0; i < NS && cs.left > 0; ++i)
            cs.tile(wk, wstage_s + (uint32_t)i * stage_bytes, wbar_s + 8u * (uint32_t)i, krb, vrb, k_stage_bytes, sh.x_end);
        auto msg_wait = [&]() -> bool { return stage_wait(qfull_s + 8u * (msgs % PQ), (msgs / PQ) & 1u); };
        auto msg_done = [&]() {
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qfree_s + 8u * (msgs % PQ)) : "memory");
            ++msgs;
        };
        while (more) {
            const uint32_t hk = seg.y / p.packs;
            const Column &col = seg.col;
            float M[2] = {-1e30f, -1e30f}, lsum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int mt = 0; mt < STEPS; ++mt) oacc[mt][0] = oacc[mt][1] = oacc[mt][2] = oacc[mt][3] = 0.0f;
            if (!wait_failed) {
                const int n_t = (int)(seg.t1 - seg.t0);
                const int key0 = col.lo + (int)seg.t0 * WK;
                const uint32_t voff = (uint32_t)((reinterpret_cast<uintptr_t>(p.v_rows + (size_t)seg.b * p.v_sb + (size_t)hk * p.v_sh) + (uintptr_t)(uint32_t)key0 * vrb) & 15u);
                const uint32_t vt_off = k_stage_bytes + voff + v_lane;
                for (int n = 0; n < n_t; ++n) {
                    // the message implies the stage (the keys' warp waited for it); the wait on the stage's own barrier
                    // makes the copied bytes visible to this warp too
                    if (!msg_wait() || !stage_wait(c_bar, par)) {
                        wait_failed = true;
                        cs.stop();
                        break;
                    }
                    const uint32_t st_s = c_st, msg_s = queue_s + (msgs % PQ) * MSG;
                    if (lds32(msg_s + 768)) {
                        const float2 al = lds64f(msg_s + 512 + lane * 8);
#pragma unroll
                        for (int mt = 0; mt < STEPS; ++mt) {
                            oacc[mt][0] *= al.x;
                            oacc[mt][1] *= al.y;
                            oacc[mt][2] *= al.x;
                            oacc[mt][3] *= al.y;
                        }
                    }
                    uint32_t pb[4];
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pb[0]), "=r"(pb[1]), "=r"(pb[2]), "=r"(pb[3]) : "r"(msg_s + lane * 16));
                    const uint32_t vsc_c = msg_s + 784 + 4 * c;
                    v_accum16<VM, HD, WIDE, VAL, PERM>(st_s + vt_off, vrb, vsc_c, pb[0], pb[1], oacc, lut_v, plane_v, g);
                    v_accum16<VM, HD, WIDE, VAL, PERM>(st_s + vt_off + 16 * vrb, vrb, vsc_c + 32, pb[2], pb[3], oacc, lut_v, plane_v, g);
                    // the stage was read through the generic proxy (by both warps: the keys' warp before it sent the
                    // message): order that before the bulk copy of the next tile into it
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    msg_done();
                    if (cs.left > 0) cs.tile(wk, c_st, c_bar, krb, vrb, k_stage_bytes, sh.x_end);
                    c_st += stage_bytes;
                    c_bar += 8;
                    if (++c_stage == NS) {
                        c_stage = 0;
                        c_st = wstage_s;
                        c_bar = wbar_s;
                        par ^= 1u;
                    }
                }
                if (!wait_failed) {
                    if (msg_wait()) {
                        const float4 ml = lds128f(queue_s + (msgs % PQ) * MSG + lane * 16);
                        M[0] = ml.x; M[1] = ml.y; lsum[0] = ml.z; lsum[1] = ml.w;
                        msg_done();
                    } else {
                        wait_failed = true;
                        cs.stop();
                    }
                }
            }
            if (wait_failed) {
                // void outputs (the status says so); the segment is still counted, so that no column waits for it
                lsum[0] = lsum[1] = 0.0f;
            }
            wk.finish_segment<HD>(seg, oacc, M, lsum);
            more = next_segment(seg, p, ny, sh.x_end);
        }
        wk.zero_columns<HD>(true);
    }
    if (wait_failed) {
        if (p.status) atomicExch(p.status, 1);
        if (p.lib_status) atomicExch(p.lib_status, 1);
    }
    wk.leave();
}

// Merges the partial results of one output row (candle-core/kernels/turbo_quant_impl.h:659-685),
// rotates it back and casts it; rows of columns without any visible key are zeroed here.
// One block per output row: warp w merges the segments w, w + 4, ... with vector loads that do not
// depend on one another (a column of a short batch can have dozens of one-tile segments), then warp 0
// adds the four sums.
template <int HD>
__global__ void __launch_bounds__(128) tq_combine_kernel(const DecodeParams p) {
    constexpr int EPL = HD / 32;  // consecutive elements of a row per lane
    __shared__ __align__(16) float part[4][HD];
    __shared__ float wsums[4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rows = (size_t)p.b * p.hq * p.lq;
    const uint32_t ny = p.hkv * p.packs;
    const uint32_t prow = min((uint32_t)PACK, p.rows_per_kv);
    // launched with programmatic stream serialization: wait here until the decode grid has finished
    // and its partial results are visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // a grid launched as this one's programmatic dependent (the next attention) may be scheduled now; it waits for this
    // grid's completion itself
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // gathered outputs: this step's number (the same for all blocks: only the last block of the grid to finish
    // advances it, at its very end) selects one of the two slots of every rank's buffer
    const uint32_t g_step = p.world ? *reinterpret_cast<volatile uint32_t *>(p.step) + 1u : 0u;
    const size_t g_base = p.world ? ((size_t)(g_step & 1u) * p.world + p.rank) * rows * HD : 0;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint32_t i = (uint32_t)(row % p.lq);
        const uint32_t h = (uint32_t)((row / p.lq) % p.hq);
        const uint32_t b = (uint32_t)(row / ((size_t)p.lq * p.hq));
        const uint32_t hk = h / p.group, r = i * p.group + h % p.group;
        const uint32_t y = hk * p.packs + r / PACK, rr = r % PACK;
        const size_t obase = b * p.o_sb + h * p.o_sh + i * p.o_ss;
        if (make_column(p, b).tiles == 0) {  // the same for the whole block
            if (warp == 0) {
#pragma unroll
                for (int k = 0; k < EPL; ++k) store_elem_rt(p.out, obase + lane + 32 * k, 0.0f, p.out_dtype);
                for (uint32_t pr = 0; pr < p.world; ++pr)
#pragma unroll
                    for (int k = 0; k < EPL; ++k) store_elem_rt(p.peer_bufs[pr], g_base + row * HD + lane + 32 * k, 0.0f, p.out_dtype);
            }
            continue;
        }
        const size_t col = (size_t)b * ny + y;
        const int first = p.meta[2 * col], ns = p.meta[2 * col + 1];
        const size_t slot0 = (size_t)first * prow + rr;
        float mx = -INFINITY;
        for (int s = lane; s < ns; s += 32) mx = fmaxf(mx, p.part_lse[slot0 + (size_t)s * prow]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float acc[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) acc[k] = 0.0f;
        float wsum = 0.0f;
        for (int base = warp; base < ns; base += 128) {  // lane l of this warp weighs segment base + 4 l
            const int sl = base + 4 * lane;
            float wl = 0.0f;
            if (sl < ns) {
                const float e = p.part_lse[slot0 + (size_t)sl * prow];
                wl = e == -INFINITY ? 0.0f : expf(e - mx);
            }
            wsum += wl;
            const int cnt = min(32, (ns - base + 3) / 4);
            const float *po = p.part_o + (slot0 + (size_t)base * prow) * HD + lane * EPL;
#pragma unroll 8
            for (int j = 0; j < cnt; ++j) {
                const float w = __shfl_sync(0xffffffffu, wl, j);
                const float *src = po + (size_t)(4 * j) * prow * HD;
                if constexpr (EPL == 2) {
                    const float2 v = *reinterpret_cast<const float2 *>(src);
                    acc[0] = fmaf(w, v.x, acc[0]);
                    acc[1] = fmaf(w, v.y, acc[1]);
                } else {
#pragma unroll
                    for (int q = 0; q < EPL / 4; ++q) {
                        const float4 v = *reinterpret_cast<const float4 *>(src + 4 * q);
                        acc[4 * q] = fmaf(w, v.x, acc[4 * q]);
                        acc[4 * q + 1] = fmaf(w, v.y, acc[4 * q + 1]);
                        acc[4 * q + 2] = fmaf(w, v.z, acc[4 * q + 2]);
                        acc[4 * q + 3] = fmaf(w, v.w, acc[4 * q + 3]);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
#pragma unroll
        for (int k = 0; k < EPL; ++k) part[warp][lane * EPL + k] = acc[k];
        if (lane == 0) wsums[warp] = wsum;
        __syncthreads();
        if (warp == 0) {
            const float wt = wsums[0] + wsums[1] + wsums[2] + wsums[3];
            float *rb = part[0];
            float v[EPL];
#pragma unroll
            for (int k = 0; k < EPL; ++k) {
                const int d = lane + 32 * k;
                v[k] = part[0][d] + part[1][d] + part[2][d] + part[3][d];
            }
            __syncwarp();
#pragma unroll
            for (int k = 0; k < EPL; ++k) rb[lane + 32 * k] = wt > 0.0f ? v[k] / wt : 0.0f;
            __syncwarp();
            if (p.v.rot == B200_ROT_HADAMARD) {
                warp_hadamard(rb, HD, p.v.signs, false, lane);
                __syncwarp();
            }
#pragma unroll
            for (int k = 0; k < EPL; ++k) store_elem_rt(p.out, obase + lane + 32 * k, rb[lane + 32 * k], p.out_dtype);
            // the same row into every rank's gathered buffer: plain stores through the peer mappings
            for (uint32_t pr = 0; pr < p.world; ++pr)
#pragma unroll
                for (int k = 0; k < EPL; ++k) store_elem_rt(p.peer_bufs[pr], g_base + row * HD + lane + 32 * k, rb[lane + 32 * k], p.out_dtype);
        }
        __syncthreads();
    }
    if (p.world) combine_publish(p, g_step);
}

// The same merge for rows with few segments, as a grid of its own (the host picks it when the decode grid cannot
// merge in place: more columns than it has arrival counters for). One warp per output row, four rows per block:
// lane l owns the elements [l HD/32, (l + 1) HD/32) of the row, so a segment's partial row is one vector load per
// lane, the loads of the first segments are issued before the weights are known, and no barrier or shared memory
// sits between the warps. The grid fits on the device at once (rows beyond that are looped over): the blocks are
// resident, waiting, when the decode grid ends.
template <int HD>
__global__ void __launch_bounds__(128) tq_combine_rows_kernel(const DecodeParams p) {
    constexpr int EPL = HD / 32;  // consecutive elements of a row per lane
    constexpr int CW = 4;         // warps (rows) per block
    __shared__ __align__(16) float rot[CW][HD];  // used only when the values were rotated
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rows = (size_t)p.b * p.hq * p.lq;
    const uint32_t ny = p.hkv * p.packs;
    const uint32_t prow = min((uint32_t)PACK, p.rows_per_kv);
    // launched with programmatic stream serialization: wait here until the decode grid has finished
    // and its partial results are visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // a grid launched as this one's programmatic dependent (the next attention) may be scheduled now; it waits for this
    // grid's completion itself
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // gathered outputs: this step's number (the same for all blocks: only the last block of the grid to finish
    // advances it, at its very end) selects one of the two slots of every rank's buffer
    const uint32_t g_step = p.world ? *reinterpret_cast<volatile uint32_t *>(p.step) + 1u : 0u;
    const size_t g_base = p.world ? ((size_t)(g_step & 1u) * p.world + p.rank) * rows * HD : 0;
    for (size_t row = (size_t)blockIdx.x * CW + warp; row < rows; row += (size_t)gridDim.x * CW) {
        const uint32_t i = (uint32_t)(row % p.lq);
        const uint32_t h = (uint32_t)((row / p.lq) % p.hq);
        const uint32_t b = (uint32_t)(row / ((size_t)p.lq * p.hq));
        const uint32_t hk = h / p.group, r = i * p.group + h % p.group;
        const uint32_t y = hk * p.packs + r / PACK, rr = r % PACK;
        const size_t obase = b * p.o_sb + h * p.o_sh + i * p.o_ss;
        const size_t col = (size_t)b * ny + y;
        float acc[EPL];
        const bool any = make_column(p, b).tiles != 0;  // otherwise nothing was written for the row: zeros
        if (any) {
            const int2 fm = *reinterpret_cast<const int2 *>(p.meta + 2 * col);
            const size_t slot0 = (size_t)fm.x * prow + rr;
            merge_row<HD>(p.part_o + slot0 * HD + lane * EPL, p.part_lse + slot0, fm.y, (size_t)prow * HD, prow, lane, acc);
        } else {
#pragma unroll
            for (int k = 0; k < EPL; ++k) acc[k] = 0.0f;
        }
        finish_row<HD>(p, obase, row, g_base, acc, rot[warp], lane, any);
    }
    if (p.world) combine_publish(p, g_step);
}

}  // namespace b200
