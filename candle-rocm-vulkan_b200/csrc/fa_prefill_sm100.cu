// Prefill attention tiles on the 5th generation tensor cores (tcgen05, accumulators in tensor memory).
//
// One block = 128 packed query rows (row = token * group + head in group, so the heads that share a
// kv head also share every K / V tile) of one (batch entry, kv head), head dim 128, f16 or bf16.
//   warps 0-3  softmax: thread = row. Reads its row of S from tensor memory, keeps the running
//              maximum and sum in registers, writes P (16-bit pairs) back to tensor memory and, when the
//              maximum moved by more than 2^8, rescales its row of O in tensor memory.
//   warp 4     loader: K / V tiles of 64 keys, cp.async 16-byte chunks laid out as the 8 x 16 byte
//              core matrices the tensor core reads without swizzling; two stages.
//   warp 5     issues S = Q K^T (M 128, N 64, 8 k-steps; both operands from shared memory) and
//              O += P V (M 128, N 128, 4 k-steps; P from tensor memory, V from shared memory, N-major),
//              and owns the tensor memory allocation (256 columns: S 64, P 32, O 128).
// Two blocks fit one SM (96 KB of shared memory and 256 of the 512 columns each): while one runs its
// softmax the other runs its matrix products.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises a flag that ends all roles, the
// block frees its tensor memory and the host can read the flag (b200_device_wait_status).
//
// Semantics as fa_dense.cu (candle-core/kernels/flash_attn_impl.h:330-443: FA2-order tiles, bottom
// right aligned windows, zeros for rows without a visible key).
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "fa_params.cuh"

namespace b200 {

constexpr int PF_BM = 128, PF_BN = 64, PF_D = 128, PF_THREADS = 192;
constexpr uint32_t PF_TMEM_COLS = 256, PF_S_COL = 0, PF_P_COL = 64, PF_O_COL = 128;
// shared memory, bytes. K-major operands (Q, K): addr(row, chunk) = (row / 8) * 2048 + chunk * 128 + (row % 8) * 16
// (chunk = 8 elements of the head dim); N-major operand (V): addr(key, chunk) = chunk * 1024 + (key / 8) * 128 + (key % 8) * 16
constexpr uint32_t PF_Q_BYTES = 32768, PF_KT_BYTES = 16384, PF_VT_BYTES = 16384;
constexpr uint32_t PF_SM_Q = 0, PF_SM_K = PF_Q_BYTES, PF_SM_V = PF_SM_K + 2 * PF_KT_BYTES, PF_SM_BAR = PF_SM_V + 2 * PF_VT_BYTES;
constexpr uint32_t PF_SMEM = PF_SM_BAR + 128;
constexpr float PF_LOG2E = 1.4426950408889634f, PF_SLACK = 8.0f;

__device__ int g_wait_failed = 0;  // set when a bounded wait ran out in any kernel of this file

// ---- tcgen05 wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// shared memory matrix descriptor, no swizzle: start address, K-direction stride (between core
// matrices that follow one another along the contraction), M/N-direction stride, all in 16-byte units
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t k_stride, uint32_t mn_stride) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((k_stride >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((mn_stride >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;  // descriptor version of this architecture
    return d;
}
// The same for tiles that a tensor copy wrote with the 128-byte swizzle (rows of 128 bytes, 8-row atoms of 1024 bytes,
// tile base aligned to 1024 bytes): `lbo` is the distance between the two 64-element halves of an M/N-major operand
// (unused for a K-major one), `sbo` the distance between 8-row atoms.
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;  // layout type: 128-byte swizzle
    return d;
}
// one box of a tiled tensor map -> shared memory, completion counted in bytes on `bar`; one destination block
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
                 : "memory");
}
// instruction descriptor, kind::f16: f32 accumulator, A and B of one 16-bit type, B N-major or K-major
__host__ __device__ constexpr uint32_t tc_idesc(bool bf16, bool b_n_major, uint32_t m, uint32_t n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_n_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem), "l"(a),
                 "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// 32 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
                 "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void pf_cp16(uint32_t dst, const void *src, bool pred) {
    const int n = pred ? 16 : 0;  // zero fill for rows outside the tile
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
template <bool BF16>
__device__ __forceinline__ uint32_t pf_pack2(float lo, float hi) {
    uint32_t d;
    if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// ---- packed f32 pairs (fma.rn.f32x2 / add.rn.f32x2) and the three-input maximum ----------------------
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// One row's 64 scores of a tile (raw dot products in sa, sb; the softmax scale sl2 > 0 carries log2 e):
// masks, the row maximum, the decision to move the reference maximum (`need`, with the factor `f` that
// takes O and the running sum to the new reference) and P as 16-bit pairs. Three instructions per score
// besides the exponential: a shared three-input maximum, a packed multiply-add and a packed sum.
template <bool BF16>
__device__ __forceinline__ void pf_softmax_row(uint32_t (&sa)[32], uint32_t (&sb)[32], bool full, int lo_rel, int hi_rel, float sl2, bool first,
                                               float &mref, float &l, bool &need, float &f, uint32_t (&pr)[32]) {
    if (!full) {
        // keys lo_rel <= i < hi_rel of the tile are visible to this row (sa: keys 0-31, sb: keys 32-63)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (!(i >= lo_rel && i < hi_rel)) sa[i] = 0xff800000u;
            if (!(i + 32 >= lo_rel && i + 32 < hi_rel)) sb[i] = 0xff800000u;
        }
    }
    float m0 = fmax3(u2f(sa[0]), u2f(sa[1]), u2f(sb[0])), m1 = u2f(sb[1]);
#pragma unroll
    for (int i = 2; i < 32; i += 2) {
        m0 = fmax3(m0, u2f(sa[i]), u2f(sa[i + 1]));
        m1 = fmax3(m1, u2f(sb[i]), u2f(sb[i + 1]));
    }
    const float mx = fmaxf(m0, m1) * sl2;  // sl2 > 0: the maximum commutes with the scale
    need = false;
    if (first) mref = mx;
    else need = mx > mref + PF_SLACK;
    f = need ? fast_exp2(mref - mx) : 1.0f;
    if (need) {
        mref = mx;
        l *= f;
    }
    const float ms = mref == -INFINITY ? 0.0f : mref;
    const uint64_t sc2 = pk2(sl2, sl2), nm2 = pk2(-ms, -ms);
    uint64_t acc_a = pk2(0.0f, 0.0f), acc_b = acc_a;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float a0, a1, b0, b1;
        upk2(ffma2(pk2(u2f(sa[2 * i]), u2f(sa[2 * i + 1])), sc2, nm2), a0, a1);
        upk2(ffma2(pk2(u2f(sb[2 * i]), u2f(sb[2 * i + 1])), sc2, nm2), b0, b1);
        a0 = fast_exp2(a0);
        a1 = fast_exp2(a1);
        b0 = fast_exp2(b0);
        b1 = fast_exp2(b1);
        acc_a = fadd2(acc_a, pk2(a0, a1));
        acc_b = fadd2(acc_b, pk2(b0, b1));
        pr[i] = pf_pack2<BF16>(a0, a1);
        pr[16 + i] = pf_pack2<BF16>(b0, b1);
    }
    float s0, s1, s2, s3;
    upk2(acc_a, s0, s1);
    upk2(acc_b, s2, s3);
    l += (s0 + s1) + (s2 + s3);
}

// The same for the 128 scores of a tile of 128 keys (four chunks of 32 columns), in pieces: the maximum
// over all four chunks first, then the exponentials of two chunks at a time, so that the first half of P
// is on its way to tensor memory while the second is computed.
__device__ __forceinline__ void pf_mask32(uint32_t (&s)[32], int base, int lo_rel, int hi_rel) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (!(base + i >= lo_rel && base + i < hi_rel)) s[i] = 0xff800000u;
}
__device__ __forceinline__ float pf_max64(const uint32_t (&sa)[32], const uint32_t (&sb)[32]) {
    float m0 = fmax3(u2f(sa[0]), u2f(sa[1]), u2f(sb[0])), m1 = u2f(sb[1]);
#pragma unroll
    for (int i = 2; i < 32; i += 2) {
        m0 = fmax3(m0, u2f(sa[i]), u2f(sa[i + 1]));
        m1 = fmax3(m1, u2f(sb[i]), u2f(sb[i + 1]));
    }
    return fmaxf(m0, m1);
}
__device__ __forceinline__ float pf_max32(const uint32_t (&s)[32]) {
    float m0 = fmax3(u2f(s[0]), u2f(s[1]), u2f(s[2])), m1 = fmax3(u2f(s[3]), u2f(s[4]), u2f(s[5]));
#pragma unroll
    for (int i = 6; i < 30; i += 4) {
        m0 = fmax3(m0, u2f(s[i]), u2f(s[i + 1]));
        m1 = fmax3(m1, u2f(s[i + 2]), u2f(s[i + 3]));
    }
    return fmax3(m0, m1, fmaxf(u2f(s[30]), u2f(s[31])));
}
// 32 scores -> 16 columns of P (16-bit pairs), sums into acc
template <bool BF16>
__device__ __forceinline__ void pf_exp32(const uint32_t (&s)[32], uint64_t sc2, uint64_t nm2, uint64_t &acc, uint32_t (&pr)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float a0, a1;
        upk2(ffma2(pk2(u2f(s[2 * i]), u2f(s[2 * i + 1])), sc2, nm2), a0, a1);
        a0 = fast_exp2(a0);
        a1 = fast_exp2(a1);
        acc = fadd2(acc, pk2(a0, a1));
        pr[i] = pf_pack2<BF16>(a0, a1);
    }
}
template <bool BF16>
__device__ __forceinline__ void pf_exp64(const uint32_t (&sa)[32], const uint32_t (&sb)[32], uint64_t sc2, uint64_t nm2, uint64_t &acc_a,
                                         uint64_t &acc_b, uint32_t (&pr)[32]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float a0, a1, b0, b1;
        upk2(ffma2(pk2(u2f(sa[2 * i]), u2f(sa[2 * i + 1])), sc2, nm2), a0, a1);
        upk2(ffma2(pk2(u2f(sb[2 * i]), u2f(sb[2 * i + 1])), sc2, nm2), b0, b1);
        a0 = fast_exp2(a0);
        a1 = fast_exp2(a1);
        b0 = fast_exp2(b0);
        b1 = fast_exp2(b1);
        acc_a = fadd2(acc_a, pk2(a0, a1));
        acc_b = fadd2(acc_b, pk2(b0, b1));
        pr[i] = pf_pack2<BF16>(a0, a1);
        pr[16 + i] = pf_pack2<BF16>(b0, b1);
    }
}

// bounded wait that also ends when another role gave up; false = give up
__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
// bounded wait that ignores the abort flag: for copies in flight that must land before the block leaves
__device__ __forceinline__ void pf_wait_landed(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 16); ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return;
    }
}

template <bool BF16>
__global__ void __launch_bounds__(PF_THREADS, 2) fa_prefill_sm100_kernel(const FaParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + PF_SM_BAR);
    // barriers: 0,1 kv_full; 2,3 kv_empty; 4 s_full; 5 p_full; 6 o_full; 7 drain
    const uint32_t bar0 = sbase + PF_SM_BAR;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + PF_SM_BAR + 64);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + PF_SM_BAR + 72);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t hk = blockIdx.y, b = blockIdx.z, G = p.group;
    uint32_t lq = p.lq, lk = p.lk;
    uint64_t q0 = (uint64_t)b * p.lq, k0 = 0;
    if (p.varlen) {
        q0 = p.cu_q[b];
        lq = p.cu_q[b + 1] - p.cu_q[b];
        k0 = p.cu_k[b];
        lk = p.cu_k[b + 1] - p.cu_k[b];
    }
    const uint32_t R = lq * G;
    // the row tiles with the most keys first
    const uint32_t row0 = (gridDim.x - 1 - blockIdx.x) * PF_BM;
    if (row0 >= R) return;
    // a wait that ran out in an earlier block means something is wrong with the device or this build:
    // later blocks leave at once instead of each waiting out its own limit
    if (*reinterpret_cast<volatile int *>(&g_wait_failed)) return;
    const char *qb = reinterpret_cast<const char *>(p.q);
    const char *kb = reinterpret_cast<const char *>(p.k) + (p.varlen ? k0 * p.k_ss + hk * p.k_sh : b * p.k_sb + hk * p.k_sh) * 2;
    const char *vb = reinterpret_cast<const char *>(p.v) + (p.varlen ? k0 * p.v_ss + hk * p.v_sh : b * p.v_sb + hk * p.v_sh) * 2;
    auto range_of = [&](uint32_t r, long long &lo, long long &hi) {
        const long long i = r / G;
        const long long pos = i + (long long)lk - (long long)lq;
        lo = p.wl >= 0 ? max(pos - p.wl, 0ll) : 0ll;
        hi = p.wr >= 0 ? min(pos + p.wr + 1, (long long)lk) : (long long)lk;
        lo = min(lo, (long long)lk);
        hi = max(hi, lo);
    };
    long long t_lo, t_hi, tmp;
    range_of(row0, t_lo, tmp);
    range_of(min(row0 + PF_BM, R) - 1, tmp, t_hi);
    if (t_hi < t_lo) t_hi = t_lo;
    const int ntiles = (int)((t_hi - t_lo + PF_BN - 1) / PF_BN);

    // ---- set up: barriers, tensor memory, the Q tile
    if (tid == 0) {
        mbar_init(&bars[0], 32);
        mbar_init(&bars[1], 32);
        mbar_init(&bars[2], 1);
        mbar_init(&bars[3], 1);
        mbar_init(&bars[4], 1);
        mbar_init(&bars[5], 128);
        mbar_init(&bars[6], 1);
        mbar_init(&bars[7], 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(PF_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Q: 128 rows x 16 chunks; lanes 0-7 take the 8 rows of one core matrix, lane / 8 four chunks in a row
    for (int idx = tid; idx < PF_BM * 16; idx += PF_THREADS) {
        const int blk = idx >> 5, l = idx & 31;          // 32 chunks = 4 core matrices per step
        const int grp = blk >> 2, kc = (blk & 3) * 4 + (l >> 3), rr = grp * 8 + (l & 7);
        const uint32_t r = row0 + rr;
        const bool ok = r < R;
        const uint32_t i = ok ? r / G : 0, h = hk * G + (ok ? r % G : 0);
        const uint64_t off = (p.varlen ? (q0 + i) * p.q_ss : b * p.q_sb + i * p.q_ss) + h * p.q_sh;
        pf_cp16(sbase + PF_SM_Q + grp * 2048 + kc * 128 + (rr & 7) * 16, qb + off * 2 + kc * 16, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ================================================================ loader
        auto load_tile = [&](int t) {
            const long long j0 = t_lo + (long long)t * PF_BN;
            const uint32_t dk = sbase + PF_SM_K + (t & 1) * PF_KT_BYTES, dv = sbase + PF_SM_V + (t & 1) * PF_VT_BYTES;
            // K: 64 keys x 16 chunks, as Q
#pragma unroll 4
            for (int blk = 0; blk < 32; ++blk) {
                const int grp = blk >> 2, kc = (blk & 3) * 4 + (lane >> 3), rr = grp * 8 + (lane & 7);
                const long long j = j0 + rr;
                const bool ok = j < t_hi;
                pf_cp16(dk + grp * 2048 + kc * 128 + (rr & 7) * 16, kb + (uint64_t)(ok ? j : t_lo) * p.k_ss * 2 + kc * 16, ok);
            }
            // V: per chunk of 8 head dims, 64 keys = 8 core matrices of 8 keys; 32 lanes take 32 keys
#pragma unroll 4
            for (int blk = 0; blk < 32; ++blk) {
                // two neighbouring chunks of 16 keys each per step: every key row gives a whole 32-byte sector
                const int dc = (blk >> 2) * 2 + (lane & 1), key = (blk & 3) * 16 + (lane >> 1);
                const long long j = j0 + key;
                const bool ok = j < t_hi;
                pf_cp16(dv + dc * 1024 + (key >> 3) * 128 + (key & 7) * 16, vb + (uint64_t)(ok ? j : t_lo) * p.v_ss * 2 + dc * 16, ok);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // Two tiles in flight. A tile is announced as soon as it has landed; only then does the loader
        // wait for the products that free the stage it refills (the issuing warp, in turn, waits for a
        // tile only after it has issued the products of the tile before).
        bool ok = true;
        if (ntiles > 0) load_tile(0);
        if (ntiles > 1) load_tile(1);
        for (int t = 0; t < ntiles && ok; ++t) {
            if (t + 1 < ntiles) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&bars[t & 1]);
            if (t + 2 < ntiles) {
                ok = pf_wait(bar0 + 8 * (2 + (t & 1)), (t >> 1) & 1, abort_flag);  // O += P(t) V(t) has read the stage
                ok = __all_sync(0xffffffffu, ok);
                if (ok) load_tile(t + 2);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok) *abort_flag = 1;
    } else if (warp == 5) {
        // ================================================================ matrix products (one lane issues)
        if (lane == 0) {
            constexpr uint32_t IQK = tc_idesc(BF16, false, PF_BM, PF_BN), IPV = tc_idesc(BF16, true, PF_BM, PF_D);
            bool ok = true;
            auto issue_pv = [&](int t) {  // O += P(t) V(t)
                const uint32_t vs = sbase + PF_SM_V + (t & 1) * PF_VT_BYTES;
#pragma unroll
                for (int ks = 0; ks < PF_BN / 16; ++ks)
                    tc_mma_ts(tmem + PF_O_COL, tmem + PF_P_COL + ks * 8, tc_desc(vs + ks * 256, 128, 1024), IPV, (t > 0 || ks > 0) ? 1u : 0u);
                tc_commit(bar0 + 8 * (2 + (t & 1)));  // the stage is free once these have read it
            };
            for (int t = 0; t < ntiles && ok; ++t) {
                if (t > 0) {
                    ok = pf_wait(bar0 + 8 * 5, (t - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(t - 1);
                }
                ok = pf_wait(bar0 + 8 * (t & 1), (t >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t ks_ = sbase + PF_SM_K + (t & 1) * PF_KT_BYTES;
#pragma unroll
                for (int ks = 0; ks < PF_D / 16; ++ks)
                    tc_mma_ss(tmem + PF_S_COL, tc_desc(sbase + PF_SM_Q + ks * 256, 128, 2048), tc_desc(ks_ + ks * 256, 128, 2048), IQK, ks > 0 ? 1u : 0u);
                tc_commit(bar0 + 8 * 4);
            }
            if (ok && ntiles > 0) {
                ok = pf_wait(bar0 + 8 * 5, (ntiles - 1) & 1, abort_flag);
                if (ok) {
                    tc_fence_after();
                    issue_pv(ntiles - 1);
                    tc_commit(bar0 + 8 * 6);
                }
            }
            if (!ok) {
                *abort_flag = 1;
                // let the products already issued finish before the tensor memory goes
                tc_commit(bar0 + 8 * 7);
                for (uint32_t i = 0; i < (1u << 20); ++i) {
                    uint32_t done;
                    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                                 : "=r"(done)
                                 : "r"(bar0 + 8 * 7), "r"(0u)
                                 : "memory");
                    if (done) break;
                }
            }
        }
        __syncwarp();
    } else {
        // ================================================================ softmax, thread = row
        const uint32_t rr = warp * 32 + lane, r = row0 + rr;
        const bool r_ok = r < R;
        long long r_lo = 0, r_hi = 0;
        if (r_ok) range_of(r, r_lo, r_hi);
        // the tightest bounds over the block's rows decide which tiles need masks
        long long lomax, himin;
        {
            long long a, c2;
            range_of(min(row0 + PF_BM, R) - 1, lomax, a);
            range_of(row0, c2, himin);
            if (row0 + PF_BM > R) himin = -1;  // rows past the sequence: always masked
        }
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const float sl2 = p.scale * p.kd * PF_LOG2E;
        float mref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int t = 0; t < ntiles; ++t) {
            ok = pf_wait(bar0 + 8 * 4, t & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t sa[32], sb[32];
            tc_ld32(lane_base + PF_S_COL, sa);
            tc_ld32(lane_base + PF_S_COL + 32, sb);
            tc_wait_ld();
            const long long j0 = t_lo + (long long)t * PF_BN;
            const bool full = j0 >= lomax && j0 + PF_BN <= himin && j0 + PF_BN <= t_hi;
            const int lo_rel = r_ok ? (int)max(min(r_lo - j0, (long long)PF_BN), 0ll) : PF_BN;
            const int hi_rel = r_ok ? (int)max(min(min(r_hi, t_hi) - j0, (long long)PF_BN), 0ll) : 0;
            bool need;
            float f;
            uint32_t pr[32];
            pf_softmax_row<BF16>(sa, sb, full, lo_rel, hi_rel, sl2, t == 0, mref, l, need, f, pr);
            if (__any_sync(0xffffffffu, need)) {
                // rows whose maximum moved: O goes to the new reference
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t o[32];
                    tc_ld32(lane_base + PF_O_COL + 32 * ch, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = f2u(u2f(o[i]) * f);
                    tc_st32(lane_base + PF_O_COL + 32 * ch, o);
                }
                tc_wait_st();
            }
            tc_st32(lane_base + PF_P_COL, pr);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[5]);
        }
        if (ok && ntiles > 0) {
            ok = pf_wait(bar0 + 8 * 6, 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok) *abort_flag = 1;
        // ---- the row of the output: O / l, or zeros
        const float inv = (ok && ntiles > 0 && l > 0.0f) ? p.vd / l : 0.0f;
        const uint32_t i_tok = r_ok ? r / G : 0, h = hk * G + (r_ok ? r % G : 0);
        uint16_t *orow = reinterpret_cast<uint16_t *>(p.o) + ((q0 + i_tok) * p.hq + h) * PF_D;
        if (ok && ntiles > 0) tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            if (ok && ntiles > 0) {
                tc_ld32(lane_base + PF_O_COL + 32 * ch, o);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
            if (r_ok) {
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                    uint4 w;
                    w.x = pf_pack2<BF16>(u2f(o[8 * v4]) * inv, u2f(o[8 * v4 + 1]) * inv);
                    w.y = pf_pack2<BF16>(u2f(o[8 * v4 + 2]) * inv, u2f(o[8 * v4 + 3]) * inv);
                    w.z = pf_pack2<BF16>(u2f(o[8 * v4 + 4]) * inv, u2f(o[8 * v4 + 5]) * inv);
                    w.w = pf_pack2<BF16>(u2f(o[8 * v4 + 6]) * inv, u2f(o[8 * v4 + 7]) * inv);
                    *reinterpret_cast<uint4 *>(orow + 32 * ch + 8 * v4) = w;
                }
            }
        }
    }
    // ---- tear down
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(PF_TMEM_COLS) : "memory");
    if (tid == 0 && *abort_flag) atomicExch(&g_wait_failed, 1);
}

// ---------------------------------------------------------------------------------------------
// Two row tiles per block: 256 packed rows share every K / V tile, and the two softmax groups take
// turns with the tensor core (while group A runs its softmax the products of group B execute).
//   16 softmax warps: two threads per row, each with 64 of the 128 scores of a key tile (warps 0-3 / 8-11: rows
//   0-127 (A), first / second half of the tile; warps 4-7 / 12-15: rows 128-255 (B)); the halves exchange their
//   maxima through shared memory once per tile. Twice the warps to hide the latency of the exponentials and of
//   the tensor memory round trips: with one thread per row the softmax of a tile took 3300-4800 cycles and the
//   tensor core sat idle three quarters of the time. Warp 16 loader (two stages of 128 keys), warp 17 issues the
//   products and owns the tensor memory: 512 columns = S_A 128, S_B 128 (P_g overwrites the first 64 columns of
//   S_g once the scores are in registers), O_A 128, O_B 128.
//   Tiles of 128 keys: a tcgen05.mma costs the issuing thread about 90 cycles whatever its shape
//   (measured), so S = Q K^T runs as 8 products of N = 128 instead of 16 of N = 64. One block per SM.
// ---------------------------------------------------------------------------------------------
constexpr int P2_THREADS = 576, P2_ROWS = 256, P2_STAGES = 2, P2_BN = 128, P2_LOADER = 16, P2_ISSUER = 17;
constexpr uint32_t P2_KT_BYTES = 32768, P2_VT_BYTES = 32768;  // 128 keys x 128 dims x 2 bytes
constexpr uint32_t P2_TMEM_COLS = 512;
constexpr uint32_t P2_SM_Q = 0, P2_SM_K = 2 * PF_Q_BYTES, P2_SM_V = P2_SM_K + P2_STAGES * P2_KT_BYTES;
constexpr uint32_t P2_SM_BAR = P2_SM_V + P2_STAGES * P2_VT_BYTES, P2_SM_X = P2_SM_BAR + 256;  // exchange: [2][2][2][128] maxima, [2][2][128] sums
constexpr uint32_t P2_SMEM = P2_SM_X + 6144;
__host__ __device__ constexpr uint32_t p2_s_col(int g) { return 128u * g; }
__host__ __device__ constexpr uint32_t p2_p_col(int g) { return 128u * g; }  // over S_g
__host__ __device__ constexpr uint32_t p2_o_col(int g) { return 256u + 128u * g; }
// barriers
constexpr int B_KF = 0, B_VF = P2_STAGES, B_KE = 2 * P2_STAGES, B_VE = 3 * P2_STAGES, B_S = 4 * P2_STAGES, B_P = B_S + 2, B_O = B_P + 2, B_DRAIN = B_O + 1,
              B_X = B_DRAIN + 1,  // per group: both halves of the rows have published their maxima (or sums)
              B_Q = B_X + 2;      // the Q tile has landed

// TMA: K / V tiles arrive through two tensor copies each (boxes of 64 head-dim elements x 128 keys, 128-byte swizzle)
// that one lane issues, instead of 8192 16-byte cp.async chunks per tile from the whole loader warp.
template <bool BF16, bool TMA>
__global__ void __launch_bounds__(P2_THREADS, 1) fa_prefill_sm100_kernel2(const FaParams p, const __grid_constant__ CUtensorMap tm_k,
                                                                           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_q,
                                                                           const uint32_t tm_order) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + P2_SM_BAR);
    // barriers: k_full, v_full, k_empty, v_empty per stage, s_full and p_full per group, o_full, drain (B_* above)
    const uint32_t bar0 = sbase + P2_SM_BAR;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + P2_SM_BAR + 192);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + P2_SM_BAR + 200);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool q_tma = TMA && (tm_order >> 16) != 0;  // the Q tile comes by tensor copies too (bit 16)

    const uint32_t hk = blockIdx.y, b = blockIdx.z, G = p.group;
    uint32_t lq = p.lq, lk = p.lk;
    uint64_t q0 = (uint64_t)b * p.lq, k0 = 0;
    if (p.varlen) {
        q0 = p.cu_q[b];
        lq = p.cu_q[b + 1] - p.cu_q[b];
        k0 = p.cu_k[b];
        lk = p.cu_k[b + 1] - p.cu_k[b];
    }
    const uint32_t R = lq * G;
    const uint32_t row0 = (gridDim.x - 1 - blockIdx.x) * P2_ROWS;  // the row tiles with the most keys first
    if (row0 >= R) return;
    if (*reinterpret_cast<volatile int *>(&g_wait_failed)) return;
    const char *qb = reinterpret_cast<const char *>(p.q);
    const char *kb = reinterpret_cast<const char *>(p.k) + (p.varlen ? k0 * p.k_ss + hk * p.k_sh : b * p.k_sb + hk * p.k_sh) * 2;
    const char *vb = reinterpret_cast<const char *>(p.v) + (p.varlen ? k0 * p.v_ss + hk * p.v_sh : b * p.v_sb + hk * p.v_sh) * 2;
    auto range_of = [&](uint32_t r, long long &lo, long long &hi) {
        const long long i = r / G;
        const long long pos = i + (long long)lk - (long long)lq;
        lo = p.wl >= 0 ? max(pos - p.wl, 0ll) : 0ll;
        hi = p.wr >= 0 ? min(pos + p.wr + 1, (long long)lk) : (long long)lk;
        lo = min(lo, (long long)lk);
        hi = max(hi, lo);
    };
    long long t_lo, t_hi, tmp;
    range_of(row0, t_lo, tmp);
    range_of(min(row0 + P2_ROWS, R) - 1, tmp, t_hi);
    if (t_hi < t_lo) t_hi = t_lo;
    const int ntiles = (int)((t_hi - t_lo + P2_BN - 1) / P2_BN);

    if (tid == 0) {
        for (int i = 0; i < P2_STAGES; ++i) {
            mbar_init(&bars[B_KF + i], TMA ? 1 : 32);
            mbar_init(&bars[B_VF + i], TMA ? 1 : 32);
            mbar_init(&bars[B_KE + i], 1);
            mbar_init(&bars[B_VE + i], 1);
        }
        mbar_init(&bars[B_S], 1);
        mbar_init(&bars[B_S + 1], 1);
        mbar_init(&bars[B_P], 256);
        mbar_init(&bars[B_P + 1], 256);
        mbar_init(&bars[B_X], 256);
        mbar_init(&bars[B_X + 1], 256);
        mbar_init(&bars[B_O], 1);
        mbar_init(&bars[B_DRAIN], 1);
        mbar_init(&bars[B_Q], q_tma ? 1 : P2_THREADS);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == P2_ISSUER) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(P2_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Q: 256 rows x 16 chunks (two K-major operands of 128 rows). Nobody waits for it here: every thread leaves an
    // asynchronous arrival on the Q barrier, which the issuing thread waits for before its first product, so the first
    // K / V tiles load at the same time.
    for (int idx = tid; idx < P2_ROWS * 16 && !q_tma; idx += P2_THREADS) {
        const int blk = idx >> 5, l = idx & 31;
        const int grp = blk >> 2, kc = (blk & 3) * 4 + (l >> 3), rr = grp * 8 + (l & 7);
        const uint32_t r = row0 + rr;
        const bool ok = r < R;
        const uint32_t i = ok ? r / G : 0, h = hk * G + (ok ? r % G : 0);
        const uint64_t off = (p.varlen ? (q0 + i) * p.q_ss : b * p.q_sb + i * p.q_ss) + h * p.q_sh;
        pf_cp16(sbase + P2_SM_Q + grp * 2048 + kc * 128 + (rr & 7) * 16, qb + off * 2 + kc * 16, ok);
    }
    if (!q_tma) asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar0 + 8 * B_Q) : "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == P2_LOADER && TMA) {
        // ================================================================ loader (tensor copies)
        // coordinates: the head-dim element, then kv head, key and batch entry in the order of their strides (tm_order: two
        // bits each for the places of head, key and batch entry; K in bits 0-5, V in bits 8-13); keys past the end of the
        // tensor read as zeros
        if (lane == 0) {
            auto load = [&](const CUtensorMap *map, uint32_t ord, uint32_t dst, int j0, uint32_t bar) {
                const uint32_t ph = ord & 3u, pk = (ord >> 2) & 3u;
                const int c1 = ph == 0 ? (int)hk : (pk == 0 ? j0 : (int)b), c2 = ph == 1 ? (int)hk : (pk == 1 ? j0 : (int)b),
                          c3 = ph == 2 ? (int)hk : (pk == 2 ? j0 : (int)b);
                tma_load_4d(dst, map, 0, c1, c2, c3, bar);
                tma_load_4d(dst + P2_KT_BYTES / 2, map, 64, c1, c2, c3, bar);
            };
            bool ok = true;
            int issued_k = 0, issued_v = 0;
            if (q_tma && ntiles > 0) {
                // Q: coordinates (element, head in group, kv head, token, batch entry); a box is 64 elements of all heads
                // of the group for 256 / G tokens = 256 packed rows (row = token * G + head), one box per half of the
                // head dim: [half][row tile of 128][row][128 bytes, swizzled]
                mbar_expect_tx(&bars[B_Q], 2 * PF_Q_BYTES);
                tma_load_5d(sbase + P2_SM_Q, &tm_q, 0, 0, (int)hk, (int)(row0 / G), (int)b, bar0 + 8 * B_Q);
                tma_load_5d(sbase + P2_SM_Q + PF_Q_BYTES, &tm_q, 64, 0, (int)hk, (int)(row0 / G), (int)b, bar0 + 8 * B_Q);
            }
            for (int t = 0; t < ntiles; ++t) {
                const int st = t % P2_STAGES, j0 = (int)(t_lo + (long long)t * P2_BN);
                if (t >= P2_STAGES && !(ok = pf_wait(bar0 + 8 * (B_KE + st), ((t / P2_STAGES) - 1) & 1, abort_flag))) break;
                const uint32_t dk = sbase + P2_SM_K + st * P2_KT_BYTES, dv = sbase + P2_SM_V + st * P2_VT_BYTES;
                mbar_expect_tx(&bars[B_KF + st], P2_KT_BYTES);
                load(&tm_k, tm_order & 0x3fu, dk, j0, bar0 + 8 * (B_KF + st));
                issued_k = t + 1;
                if (t >= P2_STAGES && !(ok = pf_wait(bar0 + 8 * (B_VE + st), ((t / P2_STAGES) - 1) & 1, abort_flag))) break;
                mbar_expect_tx(&bars[B_VF + st], P2_VT_BYTES);
                load(&tm_v, (tm_order >> 8) & 0x3fu, dv, j0, bar0 + 8 * (B_VF + st));
                issued_v = t + 1;
            }
            if (!ok) {
                // gave up: the copies already issued must land before the block may leave (bounded)
                *abort_flag = 1;
                if (q_tma) pf_wait_landed(bar0 + 8 * B_Q, 0);
                for (int t = max(issued_k - P2_STAGES, 0); t < issued_k; ++t) pf_wait_landed(bar0 + 8 * (B_KF + t % P2_STAGES), (t / P2_STAGES) & 1);
                for (int t = max(issued_v - P2_STAGES, 0); t < issued_v; ++t) pf_wait_landed(bar0 + 8 * (B_VF + t % P2_STAGES), (t / P2_STAGES) & 1);
            }
        }
    } else if (warp == P2_LOADER) {
        // ================================================================ loader (16-byte chunks)
        // Per lane constants: the lane's row and chunk inside a step of 32 chunks (K: 8 rows x 4 chunks of one
        // core-matrix row group; V: 16 keys x 2 chunks), so that a copy costs an add or two besides itself.
        const uint64_t k_row8 = 8ull * p.k_ss * 2, v_row16 = 16ull * p.v_ss * 2;           // bytes between steps
        const uint64_t k_lane = (uint64_t)(lane & 7) * p.k_ss * 2 + (uint64_t)(lane >> 3) * 16;
        const uint64_t v_lane = (uint64_t)(lane >> 1) * p.v_ss * 2 + (uint64_t)(lane & 1) * 16;
        const uint32_t k_dst_lane = (uint32_t)(lane >> 3) * 128 + (uint32_t)(lane & 7) * 16;
        const uint32_t v_key = (uint32_t)(lane >> 1);
        const uint32_t v_dst_lane = (uint32_t)(lane & 1) * 2048 + (v_key >> 3) * 128 + (v_key & 7) * 16;
        auto load_k = [&](int t) {
            const long long j0 = t_lo + (long long)t * P2_BN;
            const uint32_t dk = sbase + P2_SM_K + (t % P2_STAGES) * P2_KT_BYTES + k_dst_lane;
            const char *ks = kb + (uint64_t)j0 * p.k_ss * 2 + k_lane;
            if (j0 + P2_BN <= t_hi) {
                // whole tile: step = row group g (8 keys) x chunks 4 q .. 4 q + 3
#pragma unroll 4
                for (int g8 = 0; g8 < 16; ++g8) {
                    const char *src = ks + g8 * k_row8;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) pf_cp16(dk + g8 * 2048 + q4 * 512, src + q4 * 64, true);
                }
            } else {
                // ragged last tile: rows past the end are zero filled
#pragma unroll 4
                for (int blk = 0; blk < 64; ++blk) {
                    const int g8 = blk >> 2, q4 = blk & 3;
                    const bool ok = j0 + g8 * 8 + (lane & 7) < t_hi;
                    pf_cp16(dk + g8 * 2048 + q4 * 512, ok ? ks + g8 * k_row8 + q4 * 64 : kb, ok);
                }
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar0 + 8 * (B_KF + t % P2_STAGES)) : "memory");
        };
        auto load_v = [&](int t) {
            const long long j0 = t_lo + (long long)t * P2_BN;
            const uint32_t dv = sbase + P2_SM_V + (t % P2_STAGES) * P2_VT_BYTES + v_dst_lane;
            const char *vs = vb + (uint64_t)j0 * p.v_ss * 2 + v_lane;
            if (j0 + P2_BN <= t_hi) {
                // whole tile: step = keys 16 q .. 16 q + 15 x chunks 2 c, 2 c + 1
#pragma unroll 2
                for (int q8 = 0; q8 < 8; ++q8) {
                    const char *src = vs + q8 * v_row16;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) pf_cp16(dv + c8 * 4096 + q8 * 256, src + c8 * 32, true);
                }
            } else {
#pragma unroll 4
                for (int blk = 0; blk < 64; ++blk) {
                    const int q8 = blk >> 3, c8 = blk & 7;
                    const bool ok = j0 + q8 * 16 + (lane >> 1) < t_hi;
                    pf_cp16(dv + c8 * 4096 + q8 * 256, ok ? vs + q8 * v_row16 + c8 * 32 : vb, ok);
                }
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar0 + 8 * (B_VF + t % P2_STAGES)) : "memory");
        };
        // K and V tiles of 128 keys, two stages each, released separately: the K stage of tile t is free as soon as
        // both S = Q K^T of that tile are done (early in the tile's life), the V stage after both O += P V. Nothing
        // here waits for a copy: every lane leaves an asynchronous arrival on the tile's barrier that fires when its
        // copies have landed.
        bool ok = true;
        for (int t = 0; t < ntiles && ok; ++t) {
            if (t >= P2_STAGES) {
                ok = pf_wait(bar0 + 8 * (B_KE + t % P2_STAGES), ((t / P2_STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            load_k(t);
            if (t >= P2_STAGES) {
                ok = pf_wait(bar0 + 8 * (B_VE + t % P2_STAGES), ((t / P2_STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            load_v(t);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok) *abort_flag = 1;
    } else if (warp == P2_ISSUER) {
        // ================================================================ matrix products (one lane issues)
        if (lane == 0) {
            constexpr uint32_t IQK = tc_idesc(BF16, false, PF_BM, P2_BN), IPV = tc_idesc(BF16, true, PF_BM, PF_D);
            bool ok = true;
            auto issue_qk = [&](int g, int t) {  // S_g = Q_g K(t)^T
                const uint32_t ks_ = sbase + P2_SM_K + (t % P2_STAGES) * P2_KT_BYTES, qs_ = sbase + P2_SM_Q + g * PF_Q_BYTES;
#pragma unroll
                for (int ks = 0; ks < PF_D / 16; ++ks)
                    tc_mma_ss(tmem + p2_s_col(g),
                              q_tma ? tc_desc_sw128(sbase + P2_SM_Q + (ks >> 2) * PF_Q_BYTES + g * (PF_Q_BYTES / 2) + (ks & 3) * 32, 16, 1024)
                                    : tc_desc(qs_ + ks * 256, 128, 2048),
                              TMA ? tc_desc_sw128(ks_ + (ks >> 2) * (P2_KT_BYTES / 2) + (ks & 3) * 32, 16, 1024) : tc_desc(ks_ + ks * 256, 128, 2048), IQK,
                              ks > 0 ? 1u : 0u);
                tc_commit(bar0 + 8 * (B_S + g));
            };
            auto issue_pv = [&](int g, int t) {  // O_g += P_g(t) V(t)
                const uint32_t vs = sbase + P2_SM_V + (t % P2_STAGES) * P2_VT_BYTES;
#pragma unroll
                for (int ks = 0; ks < P2_BN / 16; ++ks)
                    tc_mma_ts(tmem + p2_o_col(g), tmem + p2_s_col(g) + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8), TMA ? tc_desc_sw128(vs + ks * 2048, P2_VT_BYTES / 2, 1024) : tc_desc(vs + ks * 256, 128, 2048), IPV,
                              (t > 0 || ks > 0) ? 1u : 0u);  // P of keys 0-63 / 64-127 sits in the first columns of each half of S
            };
            if (ntiles > 0) {
                ok = pf_wait(bar0 + 8 * B_Q, 0, abort_flag) && pf_wait(bar0 + 8 * B_KF, 0, abort_flag);
                if (ok) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copies wrote through the generic proxy
                    tc_fence_after();
                    issue_qk(0, 0);
                    issue_qk(1, 0);
                    tc_commit(bar0 + 8 * B_KE);
                }
            }
            for (int t = 0; t < ntiles && ok; ++t) {
                ok = pf_wait(bar0 + 8 * B_P, t & 1, abort_flag) &&  // P_A(t) is in tensor memory, S_A is free
                     pf_wait(bar0 + 8 * (B_VF + t % P2_STAGES), (t / P2_STAGES) & 1, abort_flag);
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_after();
                issue_pv(0, t);
                if (t + 1 < ntiles) {
                    ok = pf_wait(bar0 + 8 * (B_KF + (t + 1) % P2_STAGES), ((t + 1) / P2_STAGES) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    tc_fence_after();
                    issue_qk(0, t + 1);
                }
                ok = pf_wait(bar0 + 8 * (B_P + 1), t & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                issue_pv(1, t);
                tc_commit(bar0 + 8 * (B_VE + t % P2_STAGES));  // the V stage is free once both have read it
                if (t + 1 < ntiles) {
                    issue_qk(1, t + 1);
                    tc_commit(bar0 + 8 * (B_KE + (t + 1) % P2_STAGES));  // and the K stage of the next tile
                }
            }
            if (ok && ntiles > 0) tc_commit(bar0 + 8 * B_O);
            if (!ok) {
                *abort_flag = 1;
                tc_commit(bar0 + 8 * B_DRAIN);
                for (uint32_t i = 0; i < (1u << 20); ++i) {
                    uint32_t done;
                    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                                 : "=r"(done)
                                 : "r"(bar0 + 8 * B_DRAIN), "r"(0u)
                                 : "memory");
                    if (done) break;
                }
            }
        }
        __syncwarp();
    } else {
        // ================================================================ softmax, two threads per row
        const int half = warp >> 3, g = (warp >> 2) & 1, w4 = warp & 3;
        const uint32_t g_row0 = row0 + g * PF_BM, rr = w4 * 32 + lane;
        const uint32_t r = g_row0 + rr;
        const bool r_ok = r < R;
        long long r_lo = 0, r_hi = 0;
        if (r_ok) range_of(r, r_lo, r_hi);
        long long lomax = 0, himin = -1;  // a group without rows: every tile masked
        if (g_row0 < R) {
            long long a, c2;
            range_of(min(g_row0 + PF_BM, R) - 1, lomax, a);
            range_of(g_row0, c2, himin);
            if (g_row0 + PF_BM > R) himin = -1;
        }
        const uint32_t lane_base = tmem + ((uint32_t)(w4 * 32) << 16);
        // each half keeps its P inside its own 64 columns of S (first 32 of them), so no half overwrites scores the other still reads
        const uint32_t s_col = p2_s_col(g) + 64 * half, p_col = s_col, o_col = p2_o_col(g) + 64 * half;
        float *xmax = reinterpret_cast<float *>(smem + P2_SM_X);           // [tile & 1][group][half][row]
        float *xsum = reinterpret_cast<float *>(smem + P2_SM_X + 4096);    // [group][half][row]
        const float sl2 = p.scale * p.kd * PF_LOG2E;
        float mref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int t = 0; t < ntiles; ++t) {
            ok = pf_wait(bar0 + 8 * (B_S + g), t & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long j0 = t_lo + (long long)t * P2_BN;
            const bool full = j0 >= lomax && j0 + P2_BN <= himin && j0 + P2_BN <= t_hi;
            int lo_rel = 0, hi_rel = P2_BN;
            if (!full) {
                lo_rel = r_ok ? (int)max(min(r_lo - j0, (long long)P2_BN), 0ll) : P2_BN;
                hi_rel = r_ok ? (int)max(min(min(r_hi, t_hi) - j0, (long long)P2_BN), 0ll) : 0;
            }
            // pass 1: this half's maximum, 32 columns at a time (the scores are read again below: a second
            // tensor memory load is cheaper than 64 registers held across the exchange)
            float hmax;
            {
                uint32_t sa[32];
                tc_ld32(lane_base + s_col, sa);
                tc_wait_ld();
                if (!full) pf_mask32(sa, 64 * half, lo_rel, hi_rel);
                hmax = pf_max32(sa);
                tc_ld32(lane_base + s_col + 32, sa);
                tc_wait_ld();
                if (!full) pf_mask32(sa, 64 * half + 32, lo_rel, hi_rel);
                hmax = fmaxf(hmax, pf_max32(sa));
            }
            // the row's maximum over both halves: through shared memory and the group's exchange barrier
            xmax[(((t & 1) * 2 + g) * 2 + half) * PF_BM + rr] = hmax;
            mbar_arrive(&bars[B_X + g]);
            ok = pf_wait(bar0 + 8 * (B_X + g), t & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float mx = fmaxf(hmax, xmax[(((t & 1) * 2 + g) * 2 + (half ^ 1)) * PF_BM + rr]) * sl2;  // sl2 > 0
            bool need = false;
            if (t == 0) mref = mx;
            else need = mx > mref + PF_SLACK;
            const float f = need ? fast_exp2(mref - mx) : 1.0f;
            if (need) {
                mref = mx;
                l *= f;
            }
            if (__any_sync(0xffffffffu, need)) {
                // rows whose maximum moved: this half's 64 columns of O go to the new reference
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t o[32];
                    tc_ld32(lane_base + o_col + 32 * ch, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = f2u(u2f(o[i]) * f);
                    tc_st32(lane_base + o_col + 32 * ch, o);
                }
                tc_wait_st();
            }
            // pass 2: exponentials, 32 scores -> 16 columns of P at a time
            const float ms = mref == -INFINITY ? 0.0f : mref;
            const uint64_t sc2 = pk2(sl2, sl2), nm2 = pk2(-ms, -ms);
            uint64_t acc = pk2(0.0f, 0.0f);
            {
                // P goes over columns 0-31 of this half's scores; columns 32-63 are read after the first store, which
                // does not touch them
                uint32_t sa[32], pr[16];
                tc_ld32(lane_base + s_col, sa);
                tc_wait_ld();
                if (!full) pf_mask32(sa, 64 * half, lo_rel, hi_rel);
                pf_exp32<BF16>(sa, sc2, nm2, acc, pr);
                tc_st16(lane_base + p_col, pr);
                tc_ld32(lane_base + s_col + 32, sa);
                tc_wait_ld();
                if (!full) pf_mask32(sa, 64 * half + 32, lo_rel, hi_rel);
                pf_exp32<BF16>(sa, sc2, nm2, acc, pr);
                tc_st16(lane_base + p_col + 16, pr);
            }
            {
                float a0, a1;
                upk2(acc, a0, a1);
                l += a0 + a1;
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[B_P + g]);
        }
        if (ok && ntiles > 0) {
            ok = pf_wait(bar0 + 8 * B_O, 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        // the row's sum over both halves
        float ltot = l;
        if (ok) {
            xsum[(g * 2 + half) * PF_BM + rr] = l;
            mbar_arrive(&bars[B_X + g]);
            ok = pf_wait(bar0 + 8 * (B_X + g), ntiles & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) ltot = l + xsum[(g * 2 + (half ^ 1)) * PF_BM + rr];
        }
        if (!ok) *abort_flag = 1;
        const float inv = (ok && ntiles > 0 && ltot > 0.0f) ? p.vd / ltot : 0.0f;
        const uint32_t i_tok = r_ok ? r / G : 0, h = hk * G + (r_ok ? r % G : 0);
        uint16_t *orow = reinterpret_cast<uint16_t *>(p.o) + ((q0 + i_tok) * p.hq + h) * PF_D + 64 * half;
        if (ok && ntiles > 0) tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
            uint32_t o[32];
            if (ok && ntiles > 0) {
                tc_ld32(lane_base + o_col + 32 * ch, o);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
            if (r_ok) {
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                    uint4 w;
                    w.x = pf_pack2<BF16>(u2f(o[8 * v4]) * inv, u2f(o[8 * v4 + 1]) * inv);
                    w.y = pf_pack2<BF16>(u2f(o[8 * v4 + 2]) * inv, u2f(o[8 * v4 + 3]) * inv);
                    w.z = pf_pack2<BF16>(u2f(o[8 * v4 + 4]) * inv, u2f(o[8 * v4 + 5]) * inv);
                    w.w = pf_pack2<BF16>(u2f(o[8 * v4 + 6]) * inv, u2f(o[8 * v4 + 7]) * inv);
                    *reinterpret_cast<uint4 *>(orow + 32 * ch + 8 * v4) = w;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == P2_ISSUER) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P2_TMEM_COLS) : "memory");
    if (tid == 0 && *abort_flag) atomicExch(&g_wait_failed, 1);
}


bool fa_prefill_sm100_supported(const FaParams &p, bool kv16) {
    if (!kv16 || p.kv_kind != 0 || p.d != PF_D || p.n_splits != 1) return false;
    if (p.q_dtype != B200_F16 && p.q_dtype != B200_BF16) return false;
    if (p.softcap > 0.0f || p.alibi != nullptr) return false;
    if (!(p.scale * p.kd > 0.0f)) return false;  // the row maximum is taken before the scale is applied
    if ((uint64_t)p.lq * p.group < 4 * PF_BM) return false;  // short chunks and decode stay on the mma.sync kernel
    // 16-byte chunks of q rows
    if ((reinterpret_cast<uintptr_t>(p.q) & 15) || ((p.q_sb | p.q_ss | p.q_sh) & 7)) return false;
    static const bool off = [] { const char *e = diag_env("B200_FA_NO_TCGEN05"); return e && *e == '1'; }();
    return !off;
}

// ---- tensor maps of K / V for the tensor-copy loader -------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static const EncodeTiledFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}
// A (batch, kv head, key, 128) tensor of 16-bit elements with element strides s_b, s_h, s_s and contiguous head dim as
// a rank-4 map: head dim first, the other three in ascending order of stride (entries of extent 1 last). Boxes of
// 64 x 128 keys, 128-byte swizzle. `order` gets the places of head, key and batch (two bits each). False when the tensor
// cannot be described (alignment, strides) or the driver refuses.
static bool make_kv_map(CUtensorMap *m, uint32_t *order, const void *base, bool bf16, uint64_t nb, uint64_t hkv, uint64_t lk, uint64_t s_b, uint64_t s_h,
                        uint64_t s_s) {
    const EncodeTiledFn enc = encode_tiled_fn();
    if (!enc || (reinterpret_cast<uintptr_t>(base) & 15)) return false;
    struct Dim {
        uint64_t size, stride;
        int role;
    } d[3] = {{hkv, s_h * 2, 0}, {lk, s_s * 2, 1}, {nb, s_b * 2, 2}};
    std::stable_sort(d, d + 3, [](const Dim &a, const Dim &c) {
        if ((a.size == 1) != (c.size == 1)) return c.size == 1;  // entries of extent 1 go last
        return a.size > 1 && a.stride < c.stride;
    });
    uint64_t prev = PF_D * 2;
    for (int i = 0; i < 3; ++i) {
        if (d[i].size == 1) d[i].stride = prev;  // any legal value: the coordinate is always 0
        if ((d[i].stride & 15) || d[i].stride < prev || d[i].stride >= (1ull << 40) || d[i].size > (1ull << 31)) return false;
        prev = d[i].stride * d[i].size;
    }
    uint32_t ord = 0;
    for (int i = 0; i < 3; ++i) ord |= (uint32_t)i << (2 * d[i].role);
    const cuuint64_t dims[4] = {(cuuint64_t)PF_D, d[0].size, d[1].size, d[2].size};
    const cuuint64_t strides[3] = {d[0].stride, d[1].stride, d[2].stride};
    cuuint32_t box[4] = {64, 1, 1, 1};
    box[1 + ((ord >> 2) & 3u)] = P2_BN;
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    *order = ord;
    return r == CUDA_SUCCESS;
}

// The (batch, token, head, 128) query tensor as a rank-5 map (element, head in group, kv head, token, batch entry) whose
// box of 64 x G x 1 x 256 / G lands as 256 packed rows (row = token * G + head in group).
static bool make_q_map(CUtensorMap *m, const FaParams &p, bool bf16) {
    const EncodeTiledFn enc = encode_tiled_fn();
    const uint64_t G = p.group;
    if (!enc || G == 0 || G > 256 || (G & (G - 1)) || (reinterpret_cast<uintptr_t>(p.q) & 15)) return false;
    const cuuint64_t dims[5] = {(cuuint64_t)PF_D, G, p.hkv, p.lq, p.b};
    cuuint64_t strides[4] = {p.q_sh * 2, G * p.q_sh * 2, p.q_ss * 2, p.q_sb * 2};
    if (G == 1) strides[0] = PF_D * 2;
    if (p.hkv == 1) strides[1] = strides[0] * G;
    if (p.b == 1) strides[3] = strides[2] * p.lq;
    for (int i = 0; i < 4; ++i)
        if ((strides[i] & 15) || strides[i] < PF_D * 2 || strides[i] >= (1ull << 40)) return false;
    const cuuint32_t box[5] = {64, (cuuint32_t)G, 1, (cuuint32_t)(P2_ROWS / G), 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void *>(p.q), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int fa_prefill_sm100_launch(const FaParams &p, bool bf16, cudaStream_t stream) {
    static thread_local bool done[16][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !done[dev][bf16]) {
        cudaError_t e = bf16 ? cudaFuncSetAttribute(fa_prefill_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM)
                             : cudaFuncSetAttribute(fa_prefill_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM);
        if (e == cudaSuccess)
            e = bf16 ? cudaFuncSetAttribute(fa_prefill_sm100_kernel2<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM)
                     : cudaFuncSetAttribute(fa_prefill_sm100_kernel2<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM);
        if (e == cudaSuccess)
            e = bf16 ? cudaFuncSetAttribute(fa_prefill_sm100_kernel2<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM)
                     : cudaFuncSetAttribute(fa_prefill_sm100_kernel2<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM);
        if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "flash_attn (tcgen05 tiles): shared memory opt-in: %s", cudaGetErrorString(e));
        done[dev][bf16] = true;
    }
    const uint64_t rows = (uint64_t)p.lq * p.group;
    static const long force = [] { const char *e = diag_env("B200_FA_TC_ROWS"); return e ? atol(e) : 0l; }();  // 128 or 256: tile height
    // 256-row blocks halve the K / V traffic per product and overlap softmax with products inside the block; they
    // need enough blocks to fill the device
    bool two = rows >= 1024;
    if (force == 128) two = false;
    if (force == 256) two = true;
    if (two) {
        const dim3 grid((unsigned)((rows + P2_ROWS - 1) / P2_ROWS), p.hkv, p.b);
        // K / V through tensor copies when the tensors can be described by a map (fixed-length batches, 16-byte aligned
        // strides); otherwise 16-byte chunks
        static const bool no_tma = [] { const char *e = diag_env("B200_FA_NO_TMA"); return e && *e == '1'; }();
        static const bool no_qtma = [] { const char *e = diag_env("B200_FA_NO_QTMA"); return e && *e == '1'; }();
        CUtensorMap tm_k, tm_v, tm_q;
        uint32_t ok_ = 0, ov_ = 0;
        const bool tma = !no_tma && !p.varlen && make_kv_map(&tm_k, &ok_, p.k, bf16, p.b, p.hkv, p.lk, p.k_sb, p.k_sh, p.k_ss) &&
                         make_kv_map(&tm_v, &ov_, p.v, bf16, p.b, p.hkv, p.lk, p.v_sb, p.v_sh, p.v_ss);
        const bool qtma = tma && !no_qtma && make_q_map(&tm_q, p, bf16);
        const uint32_t order = ok_ | (ov_ << 8) | (qtma ? 1u << 16 : 0u);
        if (!tma) memset(&tm_k, 0, sizeof(tm_k)), memset(&tm_v, 0, sizeof(tm_v));
        if (!qtma) memset(&tm_q, 0, sizeof(tm_q));
        if (tma && bf16) fa_prefill_sm100_kernel2<true, true><<<grid, P2_THREADS, P2_SMEM, stream>>>(p, tm_k, tm_v, tm_q, order);
        else if (tma) fa_prefill_sm100_kernel2<false, true><<<grid, P2_THREADS, P2_SMEM, stream>>>(p, tm_k, tm_v, tm_q, order);
        else if (bf16) fa_prefill_sm100_kernel2<true, false><<<grid, P2_THREADS, P2_SMEM, stream>>>(p, tm_k, tm_v, tm_q, order);
        else fa_prefill_sm100_kernel2<false, false><<<grid, P2_THREADS, P2_SMEM, stream>>>(p, tm_k, tm_v, tm_q, order);
    } else {
        const dim3 grid((unsigned)((rows + PF_BM - 1) / PF_BM), p.hkv, p.b);
        if (bf16) fa_prefill_sm100_kernel<true><<<grid, PF_THREADS, PF_SMEM, stream>>>(p);
        else fa_prefill_sm100_kernel<false><<<grid, PF_THREADS, PF_SMEM, stream>>>(p);
    }
    return check_launch("flash_attn (tcgen05 tiles)");
}

}  // namespace b200

using namespace b200;

// 1 when a bounded device-side wait of the attention kernels has run out since the library was
// loaded (the call that met it wrote zeros or partial rows); synchronizes the device.
namespace b200 {
int decode_wait_status();  // tq_decode.cu: the same flag of the kernels over packed rows
int decode_wait_clear();
}
extern "C" int b200_device_wait_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    const int d = b200::decode_wait_status();
    if (d < 0) return -1;
    return (v != 0 || d != 0) ? 1 : 0;
}

// B200_ERR_DEVICE_WAIT when a bounded device-side wait has run out on the current device since the library was loaded
// (or since the flag was last cleared), B200_OK otherwise; clear != 0 resets the flag, after which the tensor-core
// prefill kernels run again (they return at once, writing nothing, while it is set).
extern "C" int b200_device_wait_check(int clear) {
    const int st = b200_device_wait_status();
    if (st < 0) return set_error(B200_ERR_LAUNCH, "device_wait_check: the flag cannot be read (%s)", cudaGetErrorString(cudaGetLastError()));
    if (clear) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_wait_failed, &zero, sizeof(int)) != cudaSuccess || b200::decode_wait_clear() != 0)
            return set_error(B200_ERR_LAUNCH, "device_wait_check: the flag cannot be cleared");
    }
    if (st) return set_error(B200_ERR_DEVICE_WAIT, "a bounded device-side wait ran out: the outputs of the call that met it are incomplete");
    return B200_OK;
}
