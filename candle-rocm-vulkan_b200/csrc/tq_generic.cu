// Attention over packed rows for the shapes outside the tensor-core kernel: codebook formats with 1-3 bit
// codes, head dims that are multiples of 32 other than 64 / 128 / 256 (up to 256), and paged rows (a table of
// cache blocks in device memory, read in place: candle-core/src/accel/attention.rs:296-366,
// candle-core/kernels/turbo_quant_impl.h tq_attnp*). Same semantics as
// tq_decode.cuh (candle-core/kernels/turbo_quant_impl.h:232-619), plain f32 arithmetic: one block per output
// row, its 8 warps take every 8th key, a lane holds the dims lane, lane + 32, ...; scores by warp reduction,
// one online softmax per warp, the 8 partial results merged in shared memory. Calls with few output rows are
// split along the keys (grid y): every split leaves an unnormalised partial row with its maximum and sum in the
// workspace and tq_generic_merge_kernel finishes the rows. Not a fast path: it exists so that every row format
// the quantizer can write can also be attended over.
#include <algorithm>

#include "common.cuh"
#include "tq_decode.cuh"

namespace b200 {

constexpr int GW = 8;       // warps per block
constexpr int GMAX = 8;     // dims per lane: head dim <= 256

struct GenericSide {
    int32_t mode, bits, code_words, rsc_off;
};

// element j of a packed row without its row scale (candle-core/kernels/turbo_quant_impl.h:44-53)
__device__ __forceinline__ float tq_elem(const uint32_t *r, uint32_t j, const GenericSide &s, const float *tab) {
    const uint32_t pos = j * s.bits, wi = pos >> 5, sh = pos & 31u;
    uint32_t c = r[wi] >> sh;
    if (sh + s.bits > 32u) c |= r[wi + 1] << (32u - sh);
    c &= (1u << s.bits) - 1u;
    const uint32_t *aux = r + s.code_words;
    if (s.mode <= B200_TURBO_PROD) return tab[c];
    if (s.mode == B200_MXFP4) return __fmul_rn(fp4_to_f(c), e8m0_to_f((aux[j >> 7] >> (((j >> 5) & 3u) * 8u)) & 0xffu));
    if (s.mode == B200_NVFP4) return __fmul_rn(fp4_to_f(c), e4m3_to_f((aux[j >> 6] >> (((j >> 4) & 3u) * 8u)) & 0xffu));
    if (s.mode == B200_MXFP8) return __fmul_rn(e4m3_to_f(c), e8m0_to_f((aux[j >> 7] >> (((j >> 5) & 3u) * 8u)) & 0xffu));
    return e4m3_to_f(c);
}

// normalise, rotate back and store one output row held as o[k] = dims lane + 32 k of a warp (row: scratch of D floats)
__device__ __forceinline__ void generic_store_row(const DecodeParams &p, float *row, const float (&o)[GMAX], float inv, uint32_t b,
                                                  uint32_t h, uint32_t i, int lane) {
    const uint32_t D = p.d, nk = D / 32;
    for (uint32_t k = 0; k < nk; ++k) row[lane + 32 * k] = o[k] * inv;
    __syncwarp();
    if (p.v.rot == B200_ROT_HADAMARD) {
        warp_hadamard(row, (int)D, p.v.signs, false, lane);
        __syncwarp();
    }
    const size_t obase = b * p.o_sb + h * p.o_sh + i * p.o_ss;
    for (uint32_t k = 0; k < nk; ++k) store_elem_rt(p.out, obase + lane + 32 * k, row[lane + 32 * k], p.out_dtype);
}

// partial rows of the key splits: [row][split][D + 2] floats (the D sums, then the maximum and the sum of weights)
__global__ void __launch_bounds__(GW * 32) tq_generic_kernel(const DecodeParams p, const GenericSide ks, const GenericSide vs,
                                                             const B200Page *__restrict__ pages, const uint32_t n_pages,
                                                             float *__restrict__ partial) {
    __shared__ float qrow[GMAX * 32];
    __shared__ float qsrow[GMAX * 32];  // prod keys: S q
    __shared__ float part[GW][GMAX * 32 + 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t D = p.d, nk = D / 32;
    const size_t row = blockIdx.x;
    const uint32_t i = (uint32_t)(row % p.lq), h = (uint32_t)((row / p.lq) % p.hq), b = (uint32_t)(row / ((size_t)p.lq * p.hq));
    const uint32_t hk = h / p.group;
    int lk = p.kv_len ? min(max(p.kv_len[b] + p.kv_len_add, 0), (int)p.lk) : (int)p.lk;
    if (pages) {  // the keys of a paged call are the valid rows of all blocks, one after the other
        long long total = 0;
        for (uint32_t pg = 0; pg < n_pages; ++pg) total += pages[pg].rows;
        lk = (int)min(total, 2147483647ll);
    }
    // the row's visible keys (bottom right aligned)
    const long long pos = (long long)i + lk - (long long)p.lq;
    long long lo = p.wl >= 0 ? max(pos - p.wl, 0ll) : 0ll, hi = p.wr >= 0 ? min(pos + p.wr + 1, (long long)lk) : (long long)lk;
    lo = min(lo, (long long)lk);
    hi = max(hi, lo);
    if (gridDim.y > 1) {  // this split's share of the visible keys
        const long long chunk = (hi - lo + gridDim.y - 1) / gridDim.y;
        lo = min(lo + (long long)blockIdx.y * chunk, hi);
        hi = min(lo + chunk, hi);
    }
    // query row, rotated like the keys (prod keys: the caller's rotated query, followed by S q)
    const bool prod = ks.mode == B200_TURBO_PROD;
    if (warp == 0) {
        for (uint32_t k = 0; k < nk; ++k) {
            qrow[lane + 32 * k] = load_elem_rt(p.q, b * p.q_sb + h * p.q_sh + i * p.q_ss + lane + 32 * k, p.q_dtype);
            qsrow[lane + 32 * k] = prod ? load_elem_rt(p.q, b * p.q_sb + h * p.q_sh + i * p.q_ss + D + lane + 32 * k, p.q_dtype) : 0.0f;
        }
        __syncwarp();
        if (p.k.rot == B200_ROT_HADAMARD) warp_hadamard(qrow, (int)D, p.k.signs, true, lane);
    }
    __syncthreads();
    float q[GMAX], qs[GMAX];
#pragma unroll
    for (int k = 0; k < GMAX; ++k) {
        q[k] = (uint32_t)k < nk ? qrow[lane + 32 * k] * p.scale : 0.0f;
        // sqrt(pi / 2) / d of the sketch's term folded into S q (candle-core/kernels/turbo_quant_impl.h:268-277)
        qs[k] = (uint32_t)k < nk ? qsrow[lane + 32 * k] * (p.scale * 1.2533141f / (float)D) : 0.0f;
    }
    const float slope = p.alibi ? p.alibi[(size_t)b * p.alibi_bs + h] : 0.0f;
    float m = -INFINITY, l = 0.0f, acc[GMAX];
#pragma unroll
    for (int k = 0; k < GMAX; ++k) acc[k] = 0.0f;
    // blocks of keys: the whole dense cache, or one cache block after the other
    const uint32_t n_blk = pages ? n_pages : 1u;
    long long blk0 = 0;  // key index of the block's first row
    for (uint32_t pg = 0; pg < n_blk; ++pg) {
    const uint32_t *kbase, *vbase;
    long long blk_rows;
    if (pages) {
        const B200Page pgd = pages[pg];
        blk_rows = pgd.rows;
        // block layout (batch, kv head, capacity, words): head stride = capacity rows, batch stride = hkv heads
        kbase = reinterpret_cast<const uint32_t *>(pgd.k) + ((size_t)b * p.hkv + hk) * pgd.k_cap * p.k_ss;
        vbase = reinterpret_cast<const uint32_t *>(pgd.v) + ((size_t)b * p.hkv + hk) * pgd.v_cap * p.v_ss;
    } else {
        blk_rows = lk;
        kbase = p.k_rows + (size_t)b * p.k_sb + (size_t)hk * p.k_sh;
        vbase = p.v_rows + (size_t)b * p.v_sb + (size_t)hk * p.v_sh;
    }
    const long long j_lo = max(lo, blk0), j_hi = min(hi, blk0 + blk_rows);
    // every warp keeps its residue class of the global key index, so results do not depend on the paging
    long long j_first = j_lo + ((warp - j_lo) % GW + GW) % GW;
    for (long long j = j_first; j < j_hi; j += GW) {
        const uint32_t *kr = kbase + (size_t)(j - blk0) * p.k_ss, *vr = vbase + (size_t)(j - blk0) * p.v_ss;
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < GMAX; ++k)
            if ((uint32_t)k < nk) s = fmaf(tq_elem(kr, lane + 32 * k, ks, p.k.tab), q[k], s);
        if (prod) {
            // + rsc1 * signed sum of S q over the key's sign bits (word k of the sketch holds the lane's dims lane + 32 k)
            float sd = 0.0f;
#pragma unroll
            for (int k = 0; k < GMAX; ++k)
                if ((uint32_t)k < nk) sd += ((kr[ks.code_words + k] >> lane) & 1u) ? qs[k] : -qs[k];
            s = fmaf(u2f(kr[ks.rsc_off + 1]), sd, s);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= u2f(kr[ks.rsc_off]);
        if (p.softcap > 0.0f) s = p.softcap * tanhf(s / p.softcap);
        if (slope != 0.0f) s -= slope * fabsf((float)(pos - j));
        const float mn = fmaxf(m, s);
        const float al = m == -INFINITY ? 0.0f : expf(m - mn), pj = expf(s - mn);
        m = mn;
        l = l * al + pj;
        const float pv = pj * u2f(vr[vs.rsc_off]);
#pragma unroll
        for (int k = 0; k < GMAX; ++k)
            if ((uint32_t)k < nk) acc[k] = fmaf(pv, tq_elem(vr, lane + 32 * k, vs, p.v.tab), acc[k] * al);
    }
    blk0 += blk_rows;
    }
    // merge the warps
#pragma unroll
    for (int k = 0; k < GMAX; ++k)
        if ((uint32_t)k < nk) part[warp][lane + 32 * k] = acc[k];
    if (lane == 0) {
        part[warp][GMAX * 32] = m;
        part[warp][GMAX * 32 + 1] = l;
    }
    __syncthreads();
    if (warp == 0) {
        float mx = -INFINITY;
        for (int w = 0; w < GW; ++w) mx = fmaxf(mx, part[w][GMAX * 32]);
        float lt = 0.0f, o[GMAX];
#pragma unroll
        for (int k = 0; k < GMAX; ++k) o[k] = 0.0f;
        for (int w = 0; w < GW; ++w) {
            const float mw = part[w][GMAX * 32];
            const float f = mw == -INFINITY ? 0.0f : expf(mw - mx);
            lt += f * part[w][GMAX * 32 + 1];
#pragma unroll
            for (int k = 0; k < GMAX; ++k)
                if ((uint32_t)k < nk) o[k] = fmaf(f, part[w][lane + 32 * k], o[k]);
        }
        if (gridDim.y > 1) {
            float *dst = partial + (row * gridDim.y + blockIdx.y) * (size_t)(D + 2);
            for (uint32_t k = 0; k < nk; ++k) dst[lane + 32 * k] = o[k];
            if (lane == 0) dst[D] = mx, dst[D + 1] = lt;
            return;
        }
        generic_store_row(p, qrow, o, lt > 0.0f ? 1.0f / lt : 0.0f, b, h, i, lane);
    }
}

// one warp per output row: the splits' partial rows weighted by exp(max_s - max), normalised, rotated back, stored
__global__ void __launch_bounds__(GW * 32) tq_generic_merge_kernel(const DecodeParams p, const float *__restrict__ partial,
                                                                   const uint32_t nsplit, const uint64_t rows) {
    __shared__ float scratch[GW][GMAX * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint64_t row = (uint64_t)blockIdx.x * GW + warp;
    if (row >= rows) return;
    const uint32_t D = p.d, nk = D / 32;
    const uint32_t i = (uint32_t)(row % p.lq), h = (uint32_t)((row / p.lq) % p.hq), b = (uint32_t)(row / ((size_t)p.lq * p.hq));
    const float *src = partial + row * nsplit * (size_t)(D + 2);
    float mx = -INFINITY;
    for (uint32_t s = 0; s < nsplit; ++s) mx = fmaxf(mx, src[s * (size_t)(D + 2) + D]);
    float lt = 0.0f, o[GMAX];
#pragma unroll
    for (int k = 0; k < GMAX; ++k) o[k] = 0.0f;
    for (uint32_t s = 0; s < nsplit; ++s) {
        const float *ps = src + s * (size_t)(D + 2);
        const float ms = ps[D];
        const float f = ms == -INFINITY ? 0.0f : expf(ms - mx);
        lt += f * ps[D + 1];
#pragma unroll
        for (int k = 0; k < GMAX; ++k)
            if ((uint32_t)k < nk) o[k] = fmaf(f, ps[lane + 32 * k], o[k]);
    }
    generic_store_row(p, scratch[warp], o, lt > 0.0f ? 1.0f / lt : 0.0f, b, h, i, lane);
}

// 0 when the call is one this kernel takes (and the tensor-core kernel does not)
int tq_generic_plan(const B200TqAttnArgs *a, DecodeParams &p, GenericSide &ks, GenericSide &vs) {
    if (!a || a->hkv == 0 || a->hq % a->hkv != 0) return 1;
    if (a->pages && (a->n_pages == 0 || a->kv_len_dev)) return 1;
    if (a->d == 0 || a->d % 32 != 0 || a->d > GMAX * 32) return 1;
    const B200QuantSide *sides[2] = {&a->kq, &a->vq};
    GenericSide *gs[2] = {&ks, &vs};
    bool needed = (a->d != 64 && a->d != 128 && a->d != 256) || a->pages != nullptr;
    for (int s = 0; s < 2; ++s) {
        const B200QuantSide &q = *sides[s];
        if (q.mode == B200_TURBO_PROD && (s == 1 || q.rotation != B200_ROT_NONE)) return 1;  // keys only; the caller rotates and projects the query
        if (q.mode == B200_TURBO_PROD) needed = true;
        B200RowLayout lay;
        if (b200_row_layout(q.mode, q.bits, (int)a->d, &lay)) return 1;
        if (q.mode <= B200_TURBO_PROD && !q.tab) return 1;
        if (q.rotation == B200_ROT_HADAMARD ? (!q.signs || (a->d & (a->d - 1))) : q.rotation != B200_ROT_NONE) return 1;
        if (q.mode == B200_TURBO_MSE && q.bits != 4) needed = true;
        gs[s]->mode = q.mode;
        gs[s]->bits = lay.code_bits;
        gs[s]->code_words = lay.code_words;
        gs[s]->rsc_off = lay.rsc_offset;
    }
    if (!needed) return 1;
    memset(&p, 0, sizeof(p));
    p.q = a->q; p.out = a->out; p.q_dtype = a->q_dtype; p.out_dtype = a->out_dtype;
    p.q_sb = a->q_strides[0]; p.q_sh = a->q_strides[1]; p.q_ss = a->q_strides[2];
    p.o_sb = a->out_strides[0]; p.o_sh = a->out_strides[1]; p.o_ss = a->out_strides[2];
    p.k_rows = a->k_rows; p.v_rows = a->v_rows;
    p.k_sb = a->k_strides[0]; p.k_sh = a->k_strides[1]; p.k_ss = a->k_strides[2];
    p.v_sb = a->v_strides[0]; p.v_sh = a->v_strides[1]; p.v_ss = a->v_strides[2];
    p.kv_len = a->kv_len_dev;
    p.kv_len_add = a->kv_len_dev ? a->kv_len_add : 0;
    p.b = a->b; p.lq = a->lq; p.lk = a->lk; p.hq = a->hq; p.hkv = a->hkv; p.d = a->d; p.group = a->hq / a->hkv;
    p.k.rot = a->kq.rotation; p.k.tab = a->kq.tab; p.k.signs = a->kq.signs;
    p.v.rot = a->vq.rotation; p.v.tab = a->vq.tab; p.v.signs = a->vq.signs;
    p.scale = a->scale; p.softcap = a->softcap; p.wl = a->wl; p.wr = a->wr;
    p.alibi = a->alibi; p.alibi_bs = a->alibi_bstride;
    return 0;
}

// Key splits of a call: enough blocks for four per SM, at least 256 keys per split (a->lk: the capacity bound of a
// ragged call, the sum of the blocks' rows of a paged one), at most 64. Depends on the shape only, so a paged call and
// the dense call over the same rows split alike.
static uint32_t generic_splits(const B200TqAttnArgs *a) {
    const uint64_t rows = (uint64_t)a->b * a->hq * a->lq;
    if (rows == 0 || rows >= 4ull * 148) return 1;
    const uint64_t by_blocks = (4ull * 148 + rows - 1) / rows, by_keys = std::max<uint64_t>(a->lk / 256, 1);
    return (uint32_t)std::min<uint64_t>(std::min(by_blocks, by_keys), 64);
}

size_t tq_generic_workspace_bytes(const B200TqAttnArgs *a) {
    const uint32_t ns = generic_splits(a);
    // 16: the general kernel needs no scratch without splits; 0 is reserved for "cannot be planned"
    return ns > 1 ? (size_t)a->b * a->hq * a->lq * ns * (a->d + 2) * sizeof(float) : 16;
}

int tq_generic_launch(const B200TqAttnArgs *a, cudaStream_t stream) {
    DecodeParams p;
    GenericSide ks, vs;
    if (tq_generic_plan(a, p, ks, vs)) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: shape outside both kernels");
    const uint64_t rows = (uint64_t)a->b * a->hq * a->lq;
    if (rows == 0) return B200_OK;
    if (!a->q || !a->out || (!a->pages && (!a->k_rows || !a->v_rows))) return set_error(B200_ERR_BAD_ARG, "tq_attention: null pointer");
    if (rows > 0x7fffffffull) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: too many output rows");
    uint32_t ns = generic_splits(a);
    // a caller that sized its workspace for no splits (or passed none) still gets its result, from one block per row
    if (ns > 1 && (!a->workspace || a->workspace_bytes < tq_generic_workspace_bytes(a))) ns = 1;
    float *partial = ns > 1 ? reinterpret_cast<float *>(a->workspace) : nullptr;
    tq_generic_kernel<<<dim3((unsigned)rows, ns), GW * 32, 0, stream>>>(p, ks, vs, a->pages, a->n_pages, partial);
    int rc = check_launch("tq_attention (general kernel)");
    if (rc || ns == 1) return rc;
    tq_generic_merge_kernel<<<(unsigned)((rows + GW - 1) / GW), GW * 32, 0, stream>>>(p, partial, ns, rows);
    return check_launch("tq_attention (general kernel, merge)");
}

bool tq_generic_takes(const B200TqAttnArgs *a) {
    DecodeParams p;
    GenericSide ks, vs;
    return tq_generic_plan(a, p, ks, vs) == 0;
}

}  // namespace b200
