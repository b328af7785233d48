// Host side of the attention over packed rows: argument checks, chunk planning, workspace layout,
// format dispatch and the combine launch.
#include <algorithm>
#include <cstdlib>
#include <atomic>
#include <mutex>

#include "tq_decode.cuh"

namespace b200 {

template <int KM, int VM, int HD, bool NAT, bool PAGED>
int launch_decode(const DecodeParams &p, dim3 grid, size_t smem, cudaStream_t stream);
template <int KM, int VM, int HD, bool NAT>
int launch_decode_pair(const DecodeParams &p, dim3 grid, size_t smem, cudaStream_t stream);

struct DecodePlan {
    DecodeParams p;
    uint32_t ny;
    size_t smem;
    size_t off_lse, off_meta, ws_bytes;
    uint32_t blocks;
    int hd_idx;
    uint32_t workers;  // warps (or pairs of warps) that share the tiles
    bool pair;       // the kernel whose workers are pairs of warps (4-bit formats)
    bool nat;        // rows packed back to back on both sides: the instantiation with compile-time row strides
    bool in_kernel;  // the decode grid merges the segments itself (arrival counters), no combine grid
};

static int sm_count_cached() {
    static thread_local int sms[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) return 148;
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

static int fill_decode_side(DecodeSide &s, const B200QuantSide &q, uint32_t d, const char *which) {
    B200RowLayout l;
    const int rc = b200_row_layout(q.mode, q.bits, (int)d, &l);
    if (rc) return rc;
    if (q.mode == B200_TURBO_PROD || (q.mode == B200_TURBO_MSE && q.bits != 4))
        return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: %s format %d with %d bits is outside the fused kernel", which,
                         q.mode, q.bits);
    if (q.mode == B200_TURBO_MSE && !q.tab) return set_error(B200_ERR_BAD_ARG, "tq_attention: %s codebook table missing", which);
    if (q.rotation == B200_ROT_HADAMARD) {
        if (!q.signs) return set_error(B200_ERR_BAD_ARG, "tq_attention: %s hadamard signs missing", which);
    } else if (q.rotation != B200_ROT_NONE) {
        return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: only none / hadamard rotations are fused");
    }
    s.mode = q.mode;
    s.code_words = l.code_words;
    s.rsc_off = l.rsc_offset;
    s.rot = q.rotation;
    s.tab = q.tab;
    s.signs = q.signs;
    return B200_OK;
}

// paged: the plan of a call whose rows are read in the blocks of its page table (the tensor-core kernel walks the table)
static int make_plan(const B200TqAttnArgs *a, DecodePlan &pl, bool paged = false) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "tq_attention: null args");
    if (a->hkv == 0 || a->hq % a->hkv != 0)
        return set_error(B200_ERR_BAD_ARG, "tq_attention: %u query heads are not a multiple of %u kv heads", a->hq, a->hkv);
    if (a->d != 64 && a->d != 128 && a->d != 256)
        return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: head dim %u (fused kernel: 64, 128, 256)", a->d);
    if ((a->pages != nullptr) != paged || (paged && (a->n_pages == 0 || a->kq.mode != a->vq.mode)))
        return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: paged rows without blocks, or with per-sequence lengths on a path that cannot take them");
    DecodeParams &p = pl.p;
    memset(&p, 0, sizeof(p));
    int rc = fill_decode_side(p.k, a->kq, a->d, "key");
    if (rc) return rc;
    rc = fill_decode_side(p.v, a->vq, a->d, "value");
    if (rc) return rc;
    for (int dt : {a->q_dtype, a->out_dtype})
        if (dt != B200_F32 && dt != B200_F16 && dt != B200_BF16)
            return set_error(B200_ERR_BAD_ARG, "tq_attention: q / out dtype must be f32, f16 or bf16");
    p.q = a->q;
    p.out = a->out;
    p.q_dtype = a->q_dtype;
    p.out_dtype = a->out_dtype;
    p.q_sb = a->q_strides[0]; p.q_sh = a->q_strides[1]; p.q_ss = a->q_strides[2];
    p.o_sb = a->out_strides[0]; p.o_sh = a->out_strides[1]; p.o_ss = a->out_strides[2];
    p.k_rows = a->k_rows;
    p.v_rows = a->v_rows;
    p.k_sb = a->k_strides[0]; p.k_sh = a->k_strides[1]; p.k_ss = a->k_strides[2];
    p.v_sb = a->v_strides[0]; p.v_sh = a->v_strides[1]; p.v_ss = a->v_strides[2];
    B200RowLayout kl, vl;
    b200_row_layout(a->kq.mode, a->kq.bits, (int)a->d, &kl);
    b200_row_layout(a->vq.mode, a->vq.bits, (int)a->d, &vl);
    if (p.k_ss < (uint64_t)kl.row_words || p.v_ss < (uint64_t)vl.row_words)
        return set_error(B200_ERR_BAD_ARG, "tq_attention: row strides %llu / %llu below the row sizes %d / %d",
                         (unsigned long long)p.k_ss, (unsigned long long)p.v_ss, kl.row_words, vl.row_words);
    if (p.k_ss > 512 || p.v_ss > 512) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: row stride above 512 words");
    p.kv_len = a->kv_len_dev;
    p.kv_len_add = a->kv_len_dev ? a->kv_len_add : 0;
    p.b = a->b; p.lq = a->lq; p.lk = a->lk; p.hq = a->hq; p.hkv = a->hkv; p.d = a->d;
    p.group = a->hq / a->hkv;
    p.rows_per_kv = p.group * a->lq;
    p.packs = (p.rows_per_kv + PACK - 1) / PACK;
    p.scale = a->scale;
    p.softcap = a->softcap;
    p.wl = a->wl;
    p.wr = a->wr;
    p.alibi = a->alibi;
    p.alibi_bs = a->alibi_bstride;
    p.status = a->status;
    pl.ny = a->hkv * p.packs;

    p.k_stage_bytes = (uint32_t)((WK * p.k_ss * 4 + 16 + 15) / 16 * 16);
    p.v_stage_bytes = (uint32_t)((WK * p.v_ss * 4 + 16 + 15) / 16 * 16);
    // shared memory: barriers and pair tables, per-warp key metadata, per-warp query staging (rotated
    // caches only), then the stage rings
    // staging rows for the rotation of the queries: head dims above 128 only (up to 128 it runs in registers, like the
    // rotation back of the outputs at every head dim)
    p.qstage_bytes = (a->kq.rotation == B200_ROT_HADAMARD && a->d > 128) ? (uint32_t)(DW * PACK * a->d * 4) : 0u;
    const size_t fixed = FIXED_SMEM + (size_t)DW * meta_bytes(a->kq.mode, a->vq.mode, (int)a->d) + p.qstage_bytes;
    const size_t stage = (size_t)p.k_stage_bytes + p.v_stage_bytes;
    // stages per warp and blocks per SM: as many bytes in flight as possible (a warp computes on one
    // stage while the others load), more blocks on a tie
    int bps = 1;
    p.ns = 2;
    size_t best = 0;
    for (int ns = 2; ns <= NS_MAX; ++ns) {
        const size_t sm = fixed + DW * ns * stage;
        if (sm > 227 * 1024) break;
        const int fit = (int)std::min<size_t>(B200_DECODE_MIN_BLOCKS, (228 * 1024) / (sm + 1024));
        if (fit < 1) break;
        const size_t flight = (size_t)fit * DW * (ns - 1) * stage;
        if (flight > best || (flight == best && fit > bps)) {
            best = flight;
            p.ns = (uint32_t)ns;
            bps = fit;
        }
    }
    bps = std::max(bps, 1);
    pl.smem = fixed + DW * p.ns * stage + DW * NS_MAX * 16;  // + the tile descriptions of paged rows
    pl.pair = false;
    int wpb = DW;  // workers per block
    // persistent blocks of independent workers: as many as fit on the device at once, at most one worker per tile of keys
    const uint64_t lk = std::max<uint32_t>(a->lk, 1);
    // paged rows: every block may end in a short tile
    const uint64_t max_tiles = (uint64_t)a->b * pl.ny * ((lk + WK - 1) / WK + (paged ? a->n_pages : 0u));
    const size_t ncols = (size_t)a->b * pl.ny;
    auto blocks_for = [&](int per_sm, int workers_per_block) {
        uint64_t nblocks = (uint64_t)sm_count_cached() * per_sm;
        if (a->splits > 0) nblocks = std::min<uint64_t>(nblocks, ((uint64_t)a->b * pl.ny * a->splits + workers_per_block - 1) / workers_per_block);
        return (uint32_t)std::max<uint64_t>(std::min(nblocks, (max_tiles + workers_per_block - 1) / workers_per_block), 1);
    };
    // Few segments per column (the workers outnumber the columns by less than eight to one): the last worker of a
    // column merges it inside the decode grid. Many segments per column (a few long sequences), or more columns
    // than there are arrival counters: a combine grid, whose blocks share a row's segments, follows. Calls that the
    // caller declared independent of the call before on both sides (inputs final with no fresh rows, outputs and
    // workspace its own) merge inside the grid up to 128 workers per column: a combine grid would be the one point
    // where such a call waits for all of its workers, and the calls behind it with it (measured on 32 sequences of
    // 32768 TurboQuant-4 keys: 51.5 against 58.8 us per call; a lone sequence of 2048 FP8 keys: 7.1 against 14.3 us). A
    // call that follows an append (fresh rows) keeps the combine grid: there the one warp that merges a long column is
    // on the step's critical path (69.1 against 62.4 us and 35.4 against 19.6 us per step for the same two).
    auto merges_itself = [&](uint32_t blocks, int workers_per_block) {
#ifdef B200_FORCE_COMBINE  // measurement builds only: always the separate combine grid
        return false;
#else
        const size_t per_col = (p.out_free && p.prefetch && p.fresh_rows == 0) ? 128 : 8;
        return (size_t)blocks * workers_per_block < per_col * ncols && ncols <= (size_t)CTR_COLS;
#endif
    };
    if (!paged && pair_formats(a->kq.mode, a->vq.mode)) {
        // codebook formats: a worker is a pair of warps, two blocks of four pairs per SM; as many stages as fit
        const size_t pq = p.qstage_bytes ? (size_t)PW * PACK * a->d * 4 : 0;  // staging rows of the keys' warps
        const size_t pfixed = pair_fixed_bytes(a->kq.mode, a->vq.mode) + (size_t)PW * pair_meta_bytes(a->kq.mode, a->vq.mode, (int)a->d) + pq;
        const size_t per_block = (228 * 1024) / 2 - 1024;
        int ns = 0;
        for (int n = 2; n <= PNS_MAX; ++n)
            if (pfixed + PW * n * stage <= per_block) ns = n;
        if (ns) {
            pl.pair = true;
            p.ns = (uint32_t)ns;
            p.qstage_bytes = (uint32_t)pq;
            pl.smem = pfixed + PW * ns * stage;
            bps = 2;
            wpb = PW;
        }
    }
    // rows that certainly exist after the visible ones: the head stride spans them
    p.rows_cap = 0;
    if (p.k_ss && p.v_ss && p.k_sh % p.k_ss == 0 && p.v_sh % p.v_ss == 0 && (a->hkv > 1 || a->b > 1))
        p.rows_cap = (uint32_t)std::min<uint64_t>(std::min(p.k_sh / p.k_ss, p.v_sh / p.v_ss), 0x7fffffffu);

    p.col_cost = B200_DECODE_COL_COST;
    pl.blocks = blocks_for(bps, wpb);
    pl.workers = pl.blocks * (uint32_t)wpb;

    p.after_prev = (a->flags & B200_TQ_AFTER_PREV) ? 1u : 0u;
    p.prefetch = (p.after_prev && (a->flags & B200_TQ_INPUTS_FINAL)) ? 1u : 0u;
    p.out_free = (p.after_prev && (a->flags & B200_TQ_OUTPUTS_FREE)) ? 1u : 0u;
    p.fresh_rows = std::min<uint32_t>(a->fresh_rows, 0x7fffffffu);
    pl.nat = !paged && p.k_ss == (uint64_t)kl.row_words && p.v_ss == (uint64_t)vl.row_words && a->kq.mode == a->vq.mode && a->d == 128;
    if (pl.nat) {
        // the native-row kernels read a lane's codes with 8- or 16-byte loads where the row length allows: every
        // (batch entry, kv head) slab must then start at such a multiple (caches allocated as whole rows do)
        const uint64_t al = (uint64_t)nat_row_align((int)a->kq.mode, 128);
        auto aligned = [&](const void *ptr, uint64_t sb, uint64_t sh) { return reinterpret_cast<uintptr_t>(ptr) % al == 0 && (sb * 4) % al == 0 && (sh * 4) % al == 0; };
        pl.nat = aligned(a->k_rows, p.k_sb, p.k_sh) && aligned(a->v_rows, p.v_sb, p.v_sh);
    }
    p.pages = paged ? a->pages : nullptr;
    p.n_pages = paged ? a->n_pages : 0u;
    pl.in_kernel = merges_itself(pl.blocks, wpb);
    const size_t prow = std::min<size_t>(PACK, p.rows_per_kv);
    const size_t slots = ((size_t)pl.workers + ncols) * prow;
    const size_t part_o = slots * a->d * 4;
    const size_t part_l = slots * 4;
    pl.off_lse = (part_o + 255) / 256 * 256;
    pl.off_meta = (pl.off_lse + part_l + 255) / 256 * 256;
    pl.ws_bytes = pl.off_meta + ncols * 8;
    pl.hd_idx = a->d == 64 ? 0 : (a->d == 128 ? 1 : 2);
    return B200_OK;
}

template <int KM, int VM>
static int dispatch_hd(const DecodePlan &pl, dim3 grid, cudaStream_t stream) {
    if constexpr (pair_formats(KM, VM)) {
        if (pl.pair) {
            if constexpr (KM == VM)
                if (pl.nat && pl.hd_idx == 1) return launch_decode_pair<KM, VM, 128, true>(pl.p, grid, pl.smem, stream);
            switch (pl.hd_idx) {
            case 0: return launch_decode_pair<KM, VM, 64, false>(pl.p, grid, pl.smem, stream);
            case 1: return launch_decode_pair<KM, VM, 128, false>(pl.p, grid, pl.smem, stream);
            default: return launch_decode_pair<KM, VM, 256, false>(pl.p, grid, pl.smem, stream);
            }
        }
    }
    if constexpr (KM == VM)
        if (pl.nat && pl.hd_idx == 1) return launch_decode<KM, VM, 128, true, false>(pl.p, grid, pl.smem, stream);
    switch (pl.hd_idx) {
    case 0: return launch_decode<KM, VM, 64, false, false>(pl.p, grid, pl.smem, stream);
    case 1: return launch_decode<KM, VM, 128, false, false>(pl.p, grid, pl.smem, stream);
    default: return launch_decode<KM, VM, 256, false, false>(pl.p, grid, pl.smem, stream);
    }
}

template <int KM>
static int dispatch_paged(const DecodePlan &pl, dim3 grid, cudaStream_t stream) {
    switch (pl.hd_idx) {
    case 0: return launch_decode<KM, KM, 64, false, true>(pl.p, grid, pl.smem, stream);
    case 1: return launch_decode<KM, KM, 128, false, true>(pl.p, grid, pl.smem, stream);
    default: return launch_decode<KM, KM, 256, false, true>(pl.p, grid, pl.smem, stream);
    }
}

template <int KM>
static int dispatch_v(const DecodePlan &pl, dim3 grid, cudaStream_t stream) {
    if (pl.p.pages) return dispatch_paged<KM>(pl, grid, stream);
#ifdef B200_ONLY_SAME_FORMAT  // measurement builds only: keys and values in one format, the other pairs are left out
    if (pl.p.v.mode != KM || pl.hd_idx != 1 || !pl.nat) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "measurement build");
    if constexpr (pair_formats(KM, KM)) {
        if (pl.pair) return launch_decode_pair<KM, KM, 128, true>(pl.p, grid, pl.smem, stream);
    }
    return launch_decode<KM, KM, 128, true, false>(pl.p, grid, pl.smem, stream);
#else
    switch (pl.p.v.mode) {
    case B200_TURBO_MSE: return dispatch_hd<KM, B200_TURBO_MSE>(pl, grid, stream);
    case B200_MXFP4: return dispatch_hd<KM, B200_MXFP4>(pl, grid, stream);
    case B200_NVFP4: return dispatch_hd<KM, B200_NVFP4>(pl, grid, stream);
    case B200_MXFP8: return dispatch_hd<KM, B200_MXFP8>(pl, grid, stream);
    default: return dispatch_hd<KM, B200_FP8_ROW>(pl, grid, stream);
    }
#endif
}

// Library-owned device words. g_col_ctr: arrival counters of the columns of the calls in flight, one slab per
// call, taken in turn; every counter is back at zero when its call ends (the last arrival wraps it), so the slabs
// need no clearing between calls. g_decode_wait_failed: set when a bounded wait of a decode kernel ran out.
static __device__ uint32_t g_col_ctr[CTR_SLABS][CTR_COLS];
static __device__ int32_t g_decode_wait_failed;

struct DeviceWords {
    uint32_t *ctr;
    int32_t *wait_failed;
};
static DeviceWords g_device_words[64];
static bool g_device_words_ok[64];
static std::mutex g_device_words_mutex;
static std::atomic<uint32_t> g_next_slab{0};

// Device addresses of the words above on the current device. In host code the arrays' names are handles for the
// runtime, not addresses a kernel can use: cudaGetSymbolAddress, once per device, with that device current.
static int device_words(DeviceWords &w) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return set_error(B200_ERR_LAUNCH, "tq_attention: no usable current device (%s)", cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(g_device_words_mutex);
    if (!g_device_words_ok[dev]) {
        void *c = nullptr, *f = nullptr;
        e = cudaGetSymbolAddress(&c, g_col_ctr);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&f, g_decode_wait_failed);
        if (e != cudaSuccess || !c || !f) return set_error(B200_ERR_LAUNCH, "tq_attention: address of the library's device words: %s", cudaGetErrorString(e));
        g_device_words[dev].ctr = reinterpret_cast<uint32_t *>(c);
        g_device_words[dev].wait_failed = reinterpret_cast<int32_t *>(f);
        g_device_words_ok[dev] = true;
    }
    w = g_device_words[dev];
    return B200_OK;
}

int decode_wait_clear() {
    DeviceWords w;
    if (device_words(w)) return -1;
    return cudaMemset(w.wait_failed, 0, sizeof(int32_t)) == cudaSuccess ? 0 : -1;
}

// 1 when a bounded wait of a decode kernel has run out on the current device since the library was loaded
int decode_wait_status() {
    DeviceWords w;
    if (device_words(w)) return -1;
    int32_t v = 0;
    if (cudaMemcpy(&v, w.wait_failed, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return v != 0;
}

// Keys and tiles before every block of a page table (n_pages + 1 entries each): one block of 256 threads.
__global__ void __launch_bounds__(256) tq_page_prefix_kernel(const B200Page *__restrict__ pages, uint32_t n_pages, uint32_t *__restrict__ pg_keys,
                                                              uint32_t *__restrict__ pg_tiles) {
    __shared__ uint32_t sk[256], st[256];
    // the attention that follows is launched as this kernel's programmatic dependent: its blocks may take their places
    // now (they wait for this kernel's completion before they read the sums)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t base_k = 0, base_t = 0;
    for (uint32_t start = 0; start < n_pages; start += 256) {
        const uint32_t i = start + threadIdx.x;
        const uint32_t r = i < n_pages ? pages[i].rows : 0u;
        sk[threadIdx.x] = r;
        st[threadIdx.x] = (r + WK - 1) / WK;
        __syncthreads();
        for (int o = 1; o < 256; o <<= 1) {  // inclusive scans
            const uint32_t ak = threadIdx.x >= (unsigned)o ? sk[threadIdx.x - o] : 0u, at = threadIdx.x >= (unsigned)o ? st[threadIdx.x - o] : 0u;
            __syncthreads();
            sk[threadIdx.x] += ak;
            st[threadIdx.x] += at;
            __syncthreads();
        }
        if (i < n_pages) {
            pg_keys[i] = base_k + sk[threadIdx.x] - r;
            pg_tiles[i] = base_t + st[threadIdx.x] - (r + WK - 1) / WK;
        }
        base_k += sk[255];
        base_t += st[255];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        pg_keys[n_pages] = base_k;
        pg_tiles[n_pages] = base_t;
    }
}

// n words from src to dst by the 256 threads of a block: 16-byte vectors where both sides sit at the same offset inside
// a 16-byte line, words at the ragged ends and everywhere else
__device__ __forceinline__ void copy_words(uint32_t *__restrict__ dst, const uint32_t *__restrict__ src, uint32_t n, uint32_t tid) {
    const uint32_t ph = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15u);
    if (ph != (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u)) {
        for (uint32_t w = tid; w < n; w += 256) dst[w] = src[w];
        return;
    }
    const uint32_t head = min(n, ((16u - ph) & 15u) >> 2), body = (n - head) >> 2;
    if (tid < head) dst[tid] = src[tid];
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src + head);
    uint4 *d4 = reinterpret_cast<uint4 *>(dst + head);
    for (uint32_t i = tid; i < body; i += 256) d4[i] = s4[i];
    for (uint32_t w = head + 4 * body + tid; w < n; w += 256) dst[w] = src[w];
}

// Paged rows -> dense rows: block (page, batch entry * kv heads + kv head) copies the valid rows of its page behind the
// rows of the pages before it, into slabs of `cap` rows per (batch entry, kv head). Block (0, 0) also writes the total
// number of keys (at most lk) once per batch entry: the attention that follows reads its lengths from there, so a
// table whose rows do not add up to lk cannot make it read rows that were never written.
__global__ void __launch_bounds__(256) tq_gather_pages_kernel(const B200Page *__restrict__ pages, uint32_t n_pages, uint32_t nb, uint32_t lk,
                                                               uint32_t cap, uint32_t kw, uint32_t vw, uint32_t *__restrict__ k_dst,
                                                               uint32_t *__restrict__ v_dst, int32_t *__restrict__ kv_len) {
    __shared__ uint32_t red[256];
    const uint32_t pg = blockIdx.x, bh = blockIdx.y, tid = threadIdx.x;
    const bool totals = pg == 0 && bh == 0;
    uint32_t acc = 0;
    for (uint32_t i = tid; i < pg; i += 256) acc += pages[i].rows;
    // rows before this page; block (0, 0) needs the sum over all pages too
    uint32_t all = 0;
    if (totals)
        for (uint32_t i = tid; i < n_pages; i += 256) all += pages[i].rows;
    __syncthreads();
    red[tid] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) red[tid] += red[tid + o];
        __syncthreads();
    }
    const uint32_t start = red[0];
    __syncthreads();
    if (totals) {
        red[tid] = all;
        __syncthreads();
        for (int o = 128; o > 0; o >>= 1) {
            if (tid < o) red[tid] += red[tid + o];
            __syncthreads();
        }
        const uint32_t total = min(red[0], lk);
        for (uint32_t i = tid; i < nb; i += 256) kv_len[i] = (int32_t)total;
    }
    const B200Page pgd = pages[pg];
    if (start >= lk) return;
    const uint32_t rows = min(pgd.rows, lk - start);
    const uint32_t *ks = reinterpret_cast<const uint32_t *>(pgd.k) + (size_t)bh * pgd.k_cap * kw;
    const uint32_t *vs = reinterpret_cast<const uint32_t *>(pgd.v) + (size_t)bh * pgd.v_cap * vw;
    uint32_t *kd = k_dst + ((size_t)bh * cap + start) * kw, *vd = v_dst + ((size_t)bh * cap + start) * vw;
    copy_words(kd, ks, rows * kw, tid);
    copy_words(vd, vs, rows * vw, tid);
}

}  // namespace b200

using namespace b200;

namespace b200 {
// tq_generic.cu: formats and head dims outside the tensor-core kernel
int tq_generic_launch(const B200TqAttnArgs *a, cudaStream_t stream);
bool tq_generic_takes(const B200TqAttnArgs *a);
size_t tq_generic_workspace_bytes(const B200TqAttnArgs *a);
}  // namespace b200

// A paged call that the tensor-core kernel can serve once the blocks are compacted: the dense twin of the call (rows in
// the workspace, lengths from device memory), the bytes of the compacted rows and the whole workspace need. False when
// the shape belongs to the general kernel anyway.
struct PagedFast {
    B200TqAttnArgs dense;
    size_t k_bytes, v_bytes, len_bytes, gather_bytes, need;
    uint32_t cap, kw, vw;
};
static bool paged_fast_plan(const B200TqAttnArgs *a, PagedFast &f) {
    static const bool off = diag_env("B200_PAGED_IN_PLACE") != nullptr;
    if (off || !a || !a->pages || a->n_pages == 0 || a->kv_len_dev || a->lk == 0 || a->b == 0 || a->hkv == 0) return false;
    if (a->flags & B200_TQ_IN_PLACE) return false;
    B200RowLayout kl, vl;
    if (b200_row_layout(a->kq.mode, a->kq.bits, (int)a->d, &kl) || b200_row_layout(a->vq.mode, a->vq.bits, (int)a->d, &vl)) return false;
    f.kw = (uint32_t)kl.row_words;
    f.vw = (uint32_t)vl.row_words;
    // at least one spare row per slab (the 16-byte round up of the last tile's copy stays inside the slab), and a
    // multiple of four rows, so that every slab starts on a 16-byte line
    f.cap = (a->lk + 4) & ~3u;
    const size_t slabs = (size_t)a->b * a->hkv;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    f.k_bytes = up(slabs * f.cap * f.kw * 4);
    f.v_bytes = up(slabs * f.cap * f.vw * 4);
    f.len_bytes = up((size_t)a->b * 4);
    f.gather_bytes = f.k_bytes + f.v_bytes + f.len_bytes;
    f.dense = *a;
    f.dense.pages = nullptr;
    f.dense.n_pages = 0;
    f.dense.k_rows = f.dense.v_rows = reinterpret_cast<const uint32_t *>(a->q);  // placeholders, set at launch
    f.dense.k_strides[0] = (uint64_t)a->hkv * f.cap * f.kw, f.dense.k_strides[1] = (uint64_t)f.cap * f.kw, f.dense.k_strides[2] = f.kw;
    f.dense.v_strides[0] = (uint64_t)a->hkv * f.cap * f.vw, f.dense.v_strides[1] = (uint64_t)f.cap * f.vw, f.dense.v_strides[2] = f.vw;
    f.dense.kv_len_dev = reinterpret_cast<const int32_t *>(a->q);
    f.dense.workspace = nullptr;
    f.dense.workspace_bytes = 0;
    // the compaction kernel of the call writes the rows and the lengths right before the attention: the attention
    // must not start as that kernel's programmatic dependent
    f.dense.flags &= ~(B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL);
    if (tq_generic_takes(&f.dense)) return false;
    DecodePlan pl;
    if (make_plan(&f.dense, pl)) return false;
    f.need = f.gather_bytes + pl.ws_bytes;
    return true;
}

// A paged call that the tensor-core kernel serves by walking the page table itself: keys and values in one format of
// that kernel. Workspace: the keys and tiles before every block (written by a one-block kernel in front of the
// attention), then the attention's own.
static size_t paged_prefix_bytes(uint32_t n_pages) { return ((size_t)(n_pages + 1) * 8 + 255) / 256 * 256; }
static bool paged_direct_plan(const B200TqAttnArgs *a, DecodePlan &pl) {
    static const bool off = diag_env("B200_PAGED_NO_WALK") != nullptr;  // diagnostic: paged rows on the compaction / general paths
    if (off || !a || !a->pages || a->n_pages == 0 || a->lk == 0 || a->b == 0 || a->kq.mode != a->vq.mode) return false;
    if (a->flags & B200_TQ_IN_PLACE) return false;  // the caller asked for the general kernel
    B200TqAttnArgs t = *a;
    t.flags &= ~(B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL);  // the prefix kernel of the call runs right before the attention
    if (tq_generic_takes(&t) && (a->d != 64 && a->d != 128 && a->d != 256)) return false;
    if (a->kq.mode == B200_TURBO_MSE && (a->kq.bits != 4 || a->vq.bits != 4)) return false;
    return make_plan(&t, pl, true) == B200_OK;
}

extern "C" size_t b200_tq_attention_workspace_bytes(const B200TqAttnArgs *a) {
    {
        DecodePlan pl;
        if (paged_direct_plan(a, pl)) return paged_prefix_bytes(a->n_pages) + pl.ws_bytes;
    }
    {
        // paged rows: with this much workspace the blocks are compacted into it and the tensor-core kernel runs; with
        // less (16 bytes are enough) the general kernel reads the blocks in place
        PagedFast f;
        if (paged_fast_plan(a, f)) return f.need;
    }
    if (tq_generic_takes(a)) return tq_generic_workspace_bytes(a);
    DecodePlan pl;
    if (make_plan(a, pl)) return 0;
    return pl.ws_bytes;
}

// set by b200_tq_attention_gather around its call of b200_tq_attention (same thread)
static thread_local const B200PeerGather *tl_gather = nullptr;

static int run_plan(const B200TqAttnArgs *a, DecodePlan &pl, char *ws, size_t ws_bytes, cudaStream_t stream);

extern "C" int b200_tq_attention(const B200TqAttnArgs *a, b200_stream_t stream_) {
    {
        // paged rows, keys and values in one format of the tensor-core kernel: that kernel walks the page table
        DecodePlan pl;
        if (paged_direct_plan(a, pl)) {
            const size_t pre = paged_prefix_bytes(a->n_pages);
            if (a->workspace && a->workspace_bytes >= pre + pl.ws_bytes && !(reinterpret_cast<uintptr_t>(a->workspace) & 15) &&
                (uint64_t)a->b * a->hq * a->lq != 0 && a->q && a->out) {
                char *ws = reinterpret_cast<char *>(a->workspace);
                uint32_t *pg_keys = reinterpret_cast<uint32_t *>(ws), *pg_tiles = pg_keys + (a->n_pages + 1);
                tq_page_prefix_kernel<<<1, 256, 0, (cudaStream_t)stream_>>>(a->pages, a->n_pages, pg_keys, pg_tiles);
                const int rc = check_launch("tq_page_prefix");
                if (rc) return rc;
                pl.p.pg_keys = pg_keys;
                pl.p.pg_tiles = pg_tiles;
                pl.p.after_prev = 1;  // launched as the prefix kernel's programmatic dependent (the paged kernel waits at its start)
                return run_plan(a, pl, ws + pre, a->workspace_bytes - pre, (cudaStream_t)stream_);
            }
        }
    }
    {
        PagedFast f;
        if (paged_fast_plan(a, f) && a->workspace && a->workspace_bytes >= f.need && !(reinterpret_cast<uintptr_t>(a->workspace) & 255) &&
            (uint64_t)a->b * a->hq * a->lq != 0 && a->q && a->out) {
            char *ws = reinterpret_cast<char *>(a->workspace);
            uint32_t *kd = reinterpret_cast<uint32_t *>(ws), *vd = reinterpret_cast<uint32_t *>(ws + f.k_bytes);
            int32_t *len = reinterpret_cast<int32_t *>(ws + f.k_bytes + f.v_bytes);
            const dim3 grid(a->n_pages, a->b * a->hkv);
            if (grid.y > 65535u) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention: too many (batch, kv head) slabs for the page gather");
            tq_gather_pages_kernel<<<grid, 256, 0, (cudaStream_t)stream_>>>(a->pages, a->n_pages, a->b, a->lk, f.cap, f.kw, f.vw, kd, vd, len);
            const int rc = check_launch("tq_gather_pages");
            if (rc) return rc;
            f.dense.k_rows = kd;
            f.dense.v_rows = vd;
            f.dense.kv_len_dev = len;
            f.dense.workspace = ws + f.gather_bytes;
            f.dense.workspace_bytes = a->workspace_bytes - f.gather_bytes;
            return b200_tq_attention(&f.dense, stream_);
        }
    }
    if (tq_generic_takes(a)) {
        if (tl_gather) return set_error(B200_ERR_UNSUPPORTED_SHAPE, "tq_attention_gather: not available for shapes of the general kernel");
        return tq_generic_launch(a, (cudaStream_t)stream_);
    }
    DecodePlan pl;
    const int rc = make_plan(a, pl);
    if (rc) return rc;
    if ((uint64_t)a->b * a->hq * a->lq == 0) return B200_OK;
    if (!a->k_rows || !a->v_rows) return set_error(B200_ERR_BAD_ARG, "tq_attention: null pointer");
    return run_plan(a, pl, reinterpret_cast<char *>(a->workspace), a->workspace ? a->workspace_bytes : 0, (cudaStream_t)stream_);
}

// The launches of a planned call: the decode grid, and the combine (and publish) grids where that grid does not merge
// its segments itself. `ws`: the attention's own part of the workspace.
static int run_plan(const B200TqAttnArgs *a, DecodePlan &pl, char *ws, size_t ws_bytes, cudaStream_t stream) {
    if (tl_gather) {
        pl.p.peer_bufs = tl_gather->peer_bufs;
        pl.p.peer_flags = tl_gather->peer_flags;
        pl.p.world = tl_gather->world;
        pl.p.rank = tl_gather->rank;
        pl.p.step = tl_gather->step;
        pl.p.done_ctr = tl_gather->done_ctr;
        pl.p.gather_polls = tl_gather->max_polls;
        pl.p.out_free = 0;  // the step word of the gather is the previous call's to write: stores wait for that call
    }
    if ((uint64_t)a->b * a->hq * a->lq == 0) return B200_OK;
    if (!a->q || !a->out) return set_error(B200_ERR_BAD_ARG, "tq_attention: null pointer");
    if (!ws || ws_bytes < pl.ws_bytes)
        return set_error(B200_ERR_WORKSPACE, "tq_attention: workspace of %zu bytes needed, %zu given", pl.ws_bytes, ws ? ws_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(ws) & 15) return set_error(B200_ERR_BAD_ARG, "tq_attention: workspace must be 16-byte aligned");
    DecodeParams &p = pl.p;
    p.part_o = reinterpret_cast<float *>(ws);
    p.part_lse = reinterpret_cast<float *>(ws + pl.off_lse);
    p.meta = reinterpret_cast<int32_t *>(ws + pl.off_meta);
    DeviceWords dw;
    const int wrc = device_words(dw);
    if (wrc) return wrc;
    p.lib_status = dw.wait_failed;
    // calls in flight at the same time must not share a slab: 32 slabs taken in turn
    p.ctr = pl.in_kernel ? dw.ctr + (size_t)(g_next_slab.fetch_add(1, std::memory_order_relaxed) % CTR_SLABS) * CTR_COLS : nullptr;
    const dim3 grid(pl.blocks);
    int lrc;
    switch (p.k.mode) {
    case B200_TURBO_MSE: lrc = dispatch_v<B200_TURBO_MSE>(pl, grid, stream); break;
    case B200_MXFP4: lrc = dispatch_v<B200_MXFP4>(pl, grid, stream); break;
    case B200_NVFP4: lrc = dispatch_v<B200_NVFP4>(pl, grid, stream); break;
    case B200_MXFP8: lrc = dispatch_v<B200_MXFP8>(pl, grid, stream); break;
    default: lrc = dispatch_v<B200_FP8_ROW>(pl, grid, stream); break;
    }
    if (lrc || pl.in_kernel) return lrc;
    {
        const size_t rows = (size_t)a->b * a->hq * a->lq;
        // Few segments per row: one warp per row, four rows per block, a grid that is resident at once (further rows
        // are looped over). Many segments per row: one block per row, its warps share the segments.
        const bool per_row = (size_t)pl.workers < 8 * (size_t)a->b * pl.ny;
        const unsigned gx = per_row ? (unsigned)std::max<size_t>(std::min<size_t>((rows + 3) / 4, (size_t)sm_count_cached() * 6), 1)
                                    : (unsigned)std::max<size_t>(std::min<size_t>(rows, (size_t)sm_count_cached() * 16), 1);
        // the combine grid is launched while the decode grid still runs and waits on the device for
        // its completion (programmatic dependent launch): its launch latency is off the critical path
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(gx);
        cfg.blockDim = dim3(128);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e;
        if (per_row) {
            if (a->d == 64) e = cudaLaunchKernelEx(&cfg, tq_combine_rows_kernel<64>, p);
            else if (a->d == 128) e = cudaLaunchKernelEx(&cfg, tq_combine_rows_kernel<128>, p);
            else e = cudaLaunchKernelEx(&cfg, tq_combine_rows_kernel<256>, p);
        } else if (a->d == 64) e = cudaLaunchKernelEx(&cfg, tq_combine_kernel<64>, p);
        else if (a->d == 128) e = cudaLaunchKernelEx(&cfg, tq_combine_kernel<128>, p);
        else e = cudaLaunchKernelEx(&cfg, tq_combine_kernel<256>, p);
        if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "tq_combine: %s", cudaGetErrorString(e));
        return check_launch("tq_combine");
    }
}

extern "C" int b200_tq_attention_gather(const B200TqAttnArgs *a, const B200PeerGather *g, b200_stream_t stream) {
    if (!a || !g) return set_error(B200_ERR_BAD_ARG, "tq_attention_gather: null args");
    if (g->world == 0 || g->world > 64 || g->rank >= g->world || !g->peer_bufs || !g->peer_flags || !g->step || !g->done_ctr)
        return set_error(B200_ERR_BAD_ARG, "tq_attention_gather: world %u, rank %u, or a null pointer", g->world, g->rank);
    if ((uint64_t)a->b * a->hq * a->lq == 0) return set_error(B200_ERR_BAD_ARG, "tq_attention_gather: no output rows to gather");
    tl_gather = g;
    const int rc = b200_tq_attention(a, stream);
    tl_gather = nullptr;
    return rc;
}

// ---------------------------------------------------------------------------------------------
// Attention over packed rows for callers that must not allocate device memory
// ---------------------------------------------------------------------------------------------
// Scratch of b200_tq_attention_static: lives in the library image, so every GPU that loads the
// library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[B200_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch per device ordinal. In host code the array's name is only a
// handle for the runtime, never a pointer a kernel can use: the address comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
static void *g_static_scratch_ptr[64] = {nullptr};
static std::mutex g_static_scratch_mutex;

extern "C" int b200_tq_attention_static(const B200TqAttnArgs *a, b200_stream_t stream) {
    if (!a) return set_error(B200_ERR_BAD_ARG, "tq_attention_static: null args");
    B200TqAttnArgs args = *a;
    args.flags &= ~B200_TQ_OUTPUTS_FREE;  // every call of a device shares the built-in buffer: stores keep waiting for the call before
    args.workspace = nullptr;
    args.workspace_bytes = 0;
    size_t need = b200_tq_attention_workspace_bytes(&args);
    const bool in_place = args.pages != nullptr && need > (size_t)B200_STATIC_SCRATCH_BYTES;  // too large to compact: read in place
    if (in_place) need = 16;
    if (need > (size_t)B200_STATIC_SCRATCH_BYTES)
        return set_error(B200_ERR_WORKSPACE,
                         "tq_attention_static: this call needs %zu bytes of scratch, the built-in buffer holds %zu; use "
                         "b200_tq_attention with a caller-provided workspace",
                         need, (size_t)B200_STATIC_SCRATCH_BYTES);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64)
        return set_error(B200_ERR_LAUNCH, "tq_attention_static: no usable current device (%s)", cudaGetErrorString(e));
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_ptr[dev]) {
            void *sym = nullptr;
            e = cudaGetSymbolAddress(&sym, g_static_scratch);
            if (e != cudaSuccess || !sym)
                return set_error(B200_ERR_LAUNCH, "tq_attention_static: address of the built-in scratch: %s", cudaGetErrorString(e));
            g_static_scratch_ptr[dev] = sym;
        }
        args.workspace = g_static_scratch_ptr[dev];
    }
    args.workspace_bytes = in_place ? (size_t)16 : (size_t)B200_STATIC_SCRATCH_BYTES;
    return b200_tq_attention(&args, stream);
}
