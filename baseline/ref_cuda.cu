// The reference's own GPU kernels on the same B200: a second baseline beside the CPU one.
//
// This file holds no kernel code. It includes the reference's kernel headers from where they lie
// (-I <reference>/candle-core/kernels), instantiates the entry points exactly as the reference's
// run-time compilation does (candle-core/src/accel/sources.rs:89-105: the concatenated headers
// followed by the TQ_QUANT_KERNELS / TQ_COMMON_KERNELS / FA_TILE_KERNEL lines), and replays the
// reference's launch plan from C: grid, block and shared memory of
// candle-core/src/cuda_backend/accel.rs:716-860 (tq_attention_impl), :202-233 (launch_combine),
// :254-388 (flash_attn) and candle-core/src/accel/attention.rs:390-411 (launch_dims).
// Test and bench infrastructure only: nothing of the product links or loads it.
#include <cuda_runtime.h>
#include <stdint.h>

#include "accel_common.h"
#include "flash_attn_impl.h"
#include "turbo_quant_impl.h"

TQ_QUANT_KERNELS(f32, float)
TQ_QUANT_KERNELS(f16, ax_f16)
TQ_QUANT_KERNELS(bf16, ax_bf16)
TQ_COMMON_KERNELS
FA_TILE_KERNEL(fa3_d128_bf16_bf16, ax_bf16, ax_bf16, 32, 64, 128)

namespace {

typedef void (*TqAttnFn)(TQ_ATTN_PARAMS);

TqAttnFn pick(unsigned group, int fp8) {
    switch (group) {
    case 8: return fp8 ? tq_attng8_fp8 : tq_attng8;
    case 4: return fp8 ? tq_attng4_fp8 : tq_attng4;
    case 2: return fp8 ? tq_attng2_fp8 : tq_attng2;
    default: return fp8 ? tq_attn_fp8 : tq_attn;
    }
}

} // namespace

extern "C" {

struct RefTqCall {
    const float *q;       // (B, Hq, Lq, D) f32, contiguous
    const uint32_t *kd;   // (B, Hkv, cap, row_words)
    const uint32_t *vd;
    const float *tab;     // [k table 32][v table 32]
    float *out;           // (B, Hq, Lq, D) f32
    float *part_o;        // splits * rows * D
    float *part_lse;      // splits * rows
    uint32_t b, lq, lk, hq, hkv, d;
    uint64_t k_strides[3], v_strides[3];          // (batch, head, row) in words
    uint32_t k_side[4], v_side[4];                // mode, code bits, code words, rsc offset
    float scale;
    uint32_t splits, group, fp8, pad;
};

// One tq_attn* launch and, with more than one split, the tq_combine launch that follows it.
int refcu_tq_attention(const RefTqCall *c, cudaStream_t s) {
    const uint64_t rows = (uint64_t)c->b * c->hq * c->lq;
    if (rows == 0 || c->d == 0) return 0;
    const unsigned g = c->group ? c->group : 1;
    const size_t smem = (size_t)(2 * g * c->d + 2 * g * TQ_NT + 32) * 4;
    TqAttnFn fn = pick(g, (int)c->fp8);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return -2;
    const dim3 grid((unsigned)(c->lq * c->hq / g ? c->lq * c->hq / g : 1), c->splits, c->b);
    const uint64_t w = c->d;
    fn<<<grid, TQ_NT, smem, s>>>(c->q, c->kd, c->vd, c->tab, nullptr, c->out, c->part_o, c->part_lse, c->lq, c->lk, c->hq,
                                 c->hkv, c->d, (uint64_t)c->hq * c->lq * w, (uint64_t)c->lq * w, w, c->k_strides[0],
                                 c->k_strides[1], c->k_strides[2], c->v_strides[0], c->v_strides[1], c->v_strides[2],
                                 c->k_side[0], c->k_side[1], c->k_side[2], c->k_side[3], c->v_side[0], c->v_side[1],
                                 c->v_side[2], c->v_side[3], c->scale, 0.0f, -1, -1, c->splits, 0u, rows);
    if (c->splits > 1) {
        const unsigned gx = (unsigned)(rows < 0x7fffffffull ? rows : 0x7fffffffull);
        tq_combine<<<gx, TQ_NT, c->splits * 4, s>>>(c->part_o, c->part_lse, c->out, rows, c->d, c->splits);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// `n` calls back to back on one stream: a ragged batch is one call per sequence for the reference,
// whose compressed cache has a single length (candle-nn/src/turbo_quant.rs:895-897).
int refcu_tq_attention_many(const RefTqCall *calls, int n, cudaStream_t s) {
    for (int i = 0; i < n; ++i) {
        const int rc = refcu_tq_attention(&calls[i], s);
        if (rc) return rc;
    }
    return 0;
}

// tq_quant_<dtype> as the reference launches it (accel.rs:509-553): one workgroup per row up to the grid limit,
// shared memory of candle-core/src/accel/turbo.rs:474-476.
int refcu_tq_quant(const void *src, int src_dtype, uint32_t *out, const float *tab, uint64_t rows, uint32_t d,
                   uint64_t src_stride, uint32_t mode, uint32_t cb, uint32_t code_words, uint32_t aux_words,
                   uint32_t row_words, cudaStream_t s) {
    if (rows == 0) return 0;
    const unsigned gx = (unsigned)(rows < 0x7fffffffull ? rows : 0x7fffffffull);
    const size_t smem = (size_t)(2 * d + TQ_NT + d / 16 + 1) * 4;
    if (src_dtype == 0)
        tq_quant_f32<<<gx, TQ_NT, smem, s>>>((const float *)src, out, tab, rows, d, src_stride, mode, cb, code_words, aux_words, row_words);
    else if (src_dtype == 1)
        tq_quant_f16<<<gx, TQ_NT, smem, s>>>((const ax_f16 *)src, out, tab, rows, d, src_stride, mode, cb, code_words, aux_words, row_words);
    else
        tq_quant_bf16<<<gx, TQ_NT, smem, s>>>((const ax_bf16 *)src, out, tab, rows, d, src_stride, mode, cb, code_words, aux_words, row_words);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Causal prefill on bf16 (B, S, H, D) tensors with the tile kernel of the V3 tier, the one a B200 (cc 10.0)
// selects (candle-core/src/accel/profile.rs:67-94): BR 32, BC 64, grid (ceil(S/32), Hq, B), 57 728 bytes.
int refcu_fa_prefill_bf16(const void *q, const void *k, const void *v, void *o, uint32_t b, uint32_t s_len, uint32_t hq,
                          uint32_t hkv, float scale, cudaStream_t s) {
    const uint32_t d = 128, br = 32, bc = 64;
    const size_t smem = (size_t)((br + bc) * (d + 1) + br * bc) * 4;
    if (cudaFuncSetAttribute((const void *)fa3_d128_bf16_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return -2;
    const dim3 grid((s_len + br - 1) / br, hq, b);
    const uint64_t q_ss = (uint64_t)hq * d, k_ss = (uint64_t)hkv * d;
    fa3_d128_bf16_bf16<<<grid, FA_NT, smem, s>>>((const ax_bf16 *)q, (const ax_bf16 *)k, (const ax_bf16 *)v, (ax_bf16 *)o, nullptr, nullptr,
                                                 nullptr, nullptr, nullptr, s_len, s_len, hq, hkv, d, q_ss * s_len, q_ss, (uint64_t)d,
                                                 k_ss * s_len, k_ss, (uint64_t)d, k_ss * s_len, k_ss, (uint64_t)d, scale, 0.0f, -1, 0,
                                                 1.0f, 1.0f, 1u, 0u, 0u, (uint64_t)b * hq * s_len);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

} // extern "C"
