// Parameters shared by the dense attention kernels (fa_dense.cu: mma.sync rows and tiles for every
// shape; fa_prefill_sm100.cu: tcgen05 tiles for long prefill chunks).
#pragma once
#include "common.cuh"

namespace b200 {

struct FaParams {
    const void *q, *k, *v;
    void *o;
    float *part_o, *part_lse;
    const uint32_t *cu_q, *cu_k;
    const float *alibi;
    uint32_t b, lq, lk, hq, hkv, d, group;
    uint64_t q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
    float scale, softcap, kd, vd;
    int32_t wl, wr;
    uint32_t alibi_bs, varlen, n_splits;
    int32_t q_dtype;  // dtype of q and o
    int32_t kv_kind;  // 0: 16-bit elements of the mma type, 1: E4M3 bytes, 2: f32
    uint64_t rows_total;  // total_q * hq
    // paged K / V (b200_flash_attn_paged): the blocks, and the keys before every block (n_pages + 1 entries, the last one
    // the total), written by a prefix kernel in front of the attention; null for dense tensors
    const B200Page *pages;
    const uint32_t *pg_keys;
    uint32_t n_pages;
};

// prefill tiles on the 5th generation tensor cores (fa_prefill_sm100.cu)
bool fa_prefill_sm100_supported(const FaParams &p, bool kv16);
int fa_prefill_sm100_launch(const FaParams &p, bool bf16, cudaStream_t stream);

}  // namespace b200
