/*
 * b200attn: fused attention over a compressed KV cache for NVIDIA B200 (sm_100a).
 *
 * C ABI of libb200attn.so. Every entry point takes plain pointers and sizes, a CUDA stream
 * (0 = the legacy default stream, which is what candle's shared device uses:
 * candle-core/src/cuda_backend/device.rs:191-197), returns 0 or a negative B200_ERR_* code and
 * never aborts. The calls are re-entrant and keep no per-call global state; device pointers are
 * borrowed for the duration of the stream-ordered call and must already include any start offset
 * (the reference passes storage + element offset, candle-core/src/cuda_backend/accel.rs:103-130).
 * Outputs are written completely: the caller may hand in uninitialised memory
 * (accel.rs:132-144).
 *
 * Each declaration cites the interface of the reference (Qntology/candle-rocm-vulkan) that it
 * replaces. Format ids, the packed row layout and all scalar arguments have the reference's
 * meaning, so the reference's Rust host code can bind these symbols one to one.
 */
#ifndef B200ATTN_H
#define B200ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* CUDA stream handle (cudaStream_t / CUstream) without including the CUDA headers. */
typedef void *b200_stream_t;

/* ---- status codes ------------------------------------------------------------------------ */
#define B200_OK 0
#define B200_ERR_BAD_ARG (-1)            /* null pointer, zero dim, inconsistent sizes */
#define B200_ERR_UNSUPPORTED_SHAPE (-2)  /* shape / format outside the kernels (caller may fall back) */
#define B200_ERR_LAUNCH (-3)             /* CUDA reported an error; see b200_last_error() */
#define B200_ERR_WORKSPACE (-4)          /* workspace missing or smaller than *_workspace_bytes() */
#define B200_ERR_DEVICE_WAIT (-5)        /* a bounded device-side wait ran out (status word set) */

/* ---- element dtypes ---------------------------------------------------------------------- */
#define B200_F32 0
#define B200_F16 1
#define B200_BF16 2
#define B200_FP8 3 /* OCP E4M3FN */

/* ---- quantization formats: ids of candle-core/src/accel/formats.rs:41-48 ------------------- */
#define B200_TURBO_MSE 0
#define B200_TURBO_PROD 1
#define B200_MXFP4 2
#define B200_NVFP4 3
#define B200_MXFP8 4
#define B200_FP8_ROW 5

/* ---- rotations: candle-core/src/accel/config.rs RotationKind -------------------------------- */
#define B200_ROT_NONE 0
#define B200_ROT_HADAMARD 1

/* Word layout of one packed row: [codes][aux][rsc0 f32][rsc1 f32], little-endian u32 words.
 * Replaces RowLayout / row_layout (candle-core/src/accel/formats.rs:206-242). */
typedef struct B200RowLayout {
    int32_t dim;
    int32_t code_bits;
    int32_t code_words;
    int32_t aux_words;
    int32_t row_words;
    int32_t rsc_offset;
} B200RowLayout;

/* `bits`: width of the TurboQuant formats (mse 1-4, prod 2-5), ignored by the float formats.
 * Errors like QuantFormat::validate (formats.rs:166-187): dim in 1..=1024, dim % block == 0. */
int b200_row_layout(int mode, int bits, int dim, B200RowLayout *out);

/* Lloyd-Max table [16 centroids | 16 boundaries padded with +inf] of `bits` bits for unit
 * vectors of length dim. Host memory. Replaces accel::turbo::codebook + Codebook::table
 * (candle-core/src/accel/turbo.rs:46-55,58-146). */
int b200_codebook(int dim, int bits, float tab[32]);

/* Column signs (+1 / -1) of the randomized Hadamard rotation of `seed`, host memory, dim floats.
 * Replaces the sign draw of accel::turbo::rotation_matrix (turbo.rs:188-195). Keys use the
 * cache seed, values seed + 2 (candle-nn/src/turbo_quant.rs:148-153,868). */
int b200_hadamard_signs(int dim, uint64_t seed, float *signs);

/* Row-major dim x dim matrix S of i.i.d. standard normals: the projection of the prod format's 1-bit sketch of the
 * residual (QJL). Host memory. Replaces accel::turbo::qjl_matrix (turbo.rs:236-239). */
int b200_qjl_matrix(int dim, uint64_t seed, float *s);

/* Query heads that share one kv head per work group (8, 4, 2 or 1) and the reference's key split
 * count for a device of `compute_units` SMs. Replace accel::attention::row_group and
 * split_count_grouped with SplitKv::Auto (candle-core/src/accel/attention.rs:486-506,586-592). */
int b200_row_group(int hq, int hkv);
int b200_split_count_grouped(int64_t rows, int group, int64_t lk, int compute_units);

/* ---- device report ------------------------------------------------------------------------- */
typedef struct B200Profile {
    int32_t cc_major, cc_minor;
    int32_t sm_count;
    int32_t max_smem_optin; /* bytes of dynamic shared memory a block may opt into */
    int64_t total_mem;
    char name[64];
} B200Profile;

/* Replaces CudaDevice::accel_profile (candle-core/src/cuda_backend/accel.rs:40-60). */
int b200_describe(int device, B200Profile *out);

/* Message of the last failing call of this thread ("" if none). Replaces the `candle::Error`
 * strings of the launchers. */
const char *b200_last_error(void);

/* ---- one side (keys or values) of a compressed cache ------------------------------------------ */
typedef struct B200QuantSide {
    int32_t mode;       /* B200_TURBO_MSE ... B200_FP8_ROW */
    int32_t bits;       /* TurboQuant width, else ignored */
    const float *tab;   /* device, 32 floats (b200_codebook layout); may be NULL for float formats */
    int32_t rotation;   /* B200_ROT_NONE / B200_ROT_HADAMARD */
    const float *signs; /* device, dim floats (+1 / -1) when rotation is Hadamard */
} B200QuantSide;

/* ---- row quantizer --------------------------------------------------------------------------- */
/* Replaces CudaStorage::tq_quantize (candle-core/src/cuda_backend/accel.rs:509-552) and the
 * kernels tq_quant_{f32,f16,bf16} (candle-core/kernels/turbo_quant_impl.h:71-159,687-694): rows of
 * `dim` values -> packed rows. Codes, block scales and rsc0 are bit-exact with those kernels.
 * The rows must already be in the rotated domain (the reference rotates with a matmul before
 * this call, candle-nn/src/turbo_quant.rs:199-212). */
typedef struct B200TqQuantArgs {
    const void *src;     /* device, (rows, dim) of src_dtype, row stride src_stride elements */
    uint32_t *out;       /* device, (rows, out_stride) u32 */
    const float *tab;    /* device, 32 floats; NULL allowed for the float formats */
    uint64_t rows;
    uint32_t dim;
    uint64_t src_stride; /* elements */
    uint64_t out_stride; /* words between output rows; 0 = row_words */
    int32_t src_dtype;   /* B200_F32 / B200_F16 / B200_BF16 */
    int32_t mode, bits;
} B200TqQuantArgs;
int b200_tq_quantize(const B200TqQuantArgs *args, b200_stream_t stream);

/* Replaces CudaStorage::tq_dequantize without the QJL part (accel.rs:639-684) and the kernel
 * tq_dequant (turbo_quant_impl.h:208-224): out[r][j] = rsc0 * element j, f32, rotated domain. */
typedef struct B200TqDequantArgs {
    const uint32_t *data; /* device, (rows, data_stride) */
    float *out;           /* device, (rows, dim) contiguous */
    const float *tab;     /* device, 32 floats (TurboQuant formats) */
    uint64_t rows;
    uint32_t dim;
    uint64_t data_stride; /* words; 0 = row_words */
    int32_t mode, bits;
    float *zs;            /* optional, prod rows only: (rows, dim) QJL coefficients +-(rsc0 rsc1 sqrt(pi/2) / dim) by sign bit
                           * (the second part of the reference's output, accel.rs:639-684 with_qjl) */
} B200TqDequantArgs;
int b200_tq_dequantize(const B200TqDequantArgs *args, b200_stream_t stream);

/* ---- prod (QJL) rows, stage two ------------------------------------------------------------------ */
/* b200_tq_quantize with mode B200_TURBO_PROD writes stage one: codes of bits - 1 bits, rsc0 = norm, an empty
 * sketch and rsc1 = 0 (turbo_quant_impl.h:71-159). The two calls below finish the rows as the reference does
 * (candle-nn/src/turbo_quant.rs:214-236): residual -> (the host's matmul with S^T) -> sign bits.
 *
 * Replaces CudaStorage::tq_residual (accel.rs:555-598) and the kernel tq_resid (turbo_quant_impl.h:161-177):
 * resid[r][j] = src[r][j] / rsc0 - centroid[code j], f32, rows in the rotated domain. */
typedef struct B200TqResidArgs {
    const void *src;      /* device, (rows, dim) of src_dtype, row stride src_stride elements */
    const uint32_t *data; /* device, stage-one rows, (rows, data_stride) u32 */
    const float *tab;     /* device, 32 floats: the codebook of bits - 1 bits */
    float *resid;         /* device, (rows, dim) contiguous */
    uint64_t rows;
    uint32_t dim;
    uint64_t src_stride;  /* elements */
    uint64_t data_stride; /* words; 0 = row_words */
    int32_t src_dtype;    /* B200_F32 / B200_F16 / B200_BF16 */
    int32_t bits;         /* width of the prod format (2-5) */
} B200TqResidArgs;
int b200_tq_residual(const B200TqResidArgs *args, b200_stream_t stream);

/* Replaces CudaStorage::tq_signs (accel.rs:600-636) and the kernel tq_signs (turbo_quant_impl.h:179-206): copies
 * the rows and fills in the sketch (bit j set when proj[r][j] >= 0, proj = resid S^T) and rsc1 = |resid| (sum of
 * squares in the order of the reference kernel's 128-lane tree: bit-exact). in == out is allowed. */
typedef struct B200TqSignsArgs {
    const uint32_t *in;   /* device, (rows, row_words) stage-one rows */
    const float *proj;    /* device, (rows, dim) */
    const float *resid;   /* device, (rows, dim) */
    uint32_t *out;        /* device, (rows, row_words) */
    uint64_t rows;
    uint32_t dim;
    int32_t bits;
} B200TqSignsArgs;
int b200_tq_signs(const B200TqSignsArgs *args, b200_stream_t stream);

/* Rows into (inverse = 0: y = x Pi^T) or out of (inverse = 1: x = y Pi) the rotated domain of the
 * randomized Hadamard rotation Pi = H diag(signs) / sqrt(dim), f32, in place allowed. Replaces the
 * matmuls of TurboQuantizer::rotate / unrotate (candle-nn/src/turbo_quant.rs:182-196) for the
 * Hadamard kind; the sums run as butterflies, so values agree with the matmul to rounding. */
int b200_tq_rotate(const float *in, float *out, const float *signs, uint64_t rows, uint32_t dim, int inverse,
                   b200_stream_t stream);

/* The rotation of lengths that are not powers of two (RotationKind::Dense, candle-core/src/accel/turbo.rs:204-229;
 * RotationKind::Auto resolves to it for such lengths, accel/config.rs:131-138). b200_rotation_matrix: the row-major
 * dim x dim matrix Pi of a seed (host). b200_tq_rotate_dense: out = in Pi^T (inverse: in Pi) for rows of dim floats on
 * the device (the reference's matmul, candle-nn/src/turbo_quant.rs:182-196); pi: device, dim x dim. The fused kernels
 * take rotation none / Hadamard only: a dense-rotated cache is quantized and attended over with rotation none on rows
 * and queries rotated by this call, and the outputs rotated back by it, as the reference does for every rotation. */
int b200_rotation_matrix(int dim, uint64_t seed, float *pi);
int b200_tq_rotate_dense(const float *in, float *out, const float *pi, uint64_t rows, uint32_t dim, int inverse,
                         b200_stream_t stream);

/* ---- fused quantize-on-append ------------------------------------------------------------------ */
/* Replaces TurboKvCache::append (candle-nn/src/turbo_quant.rs:916-945), i.e. per tensor the chain
 * to_dtype(F32) -> matmul with the rotation -> tq_quant -> Cache::append / slice_set
 * (candle-nn/src/kv_cache.rs:68-96), by one launch that reads K and V (b, hkv, t, d), rotates in
 * registers (Hadamard) and writes the packed rows at positions [pos, pos + t) of the capacity
 * buffers (b, hkv, cap, row_words). Without rotation the rows are bit-exact with tq_quant.
 * The reference's cache grows or fails before it writes (kv_cache.rs:60-96); here the caller owns the
 * buffers, so the call is told their capacity: with host positions a write past `cap` is refused
 * (B200_ERR_BAD_ARG); with device positions a row whose position lies outside [0, cap) is skipped
 * by the kernel and `status` (if given) is set to 3. cap = 0: positions are not checked. */
typedef struct B200KvAppendArgs {
    const void *k, *v;        /* device, element strides below, last dim contiguous */
    uint64_t k_strides[3];    /* (batch, head, token) in elements */
    uint64_t v_strides[3];
    uint32_t *k_cache, *v_cache;
    uint64_t k_cache_strides[3]; /* (batch, head, row) in words */
    uint64_t v_cache_strides[3];
    const int32_t *pos;       /* device, one write position per batch entry, or NULL: pos0 for all */
    int32_t pos0;             /* with pos: added to every entry (tokens appended since pos was written) */
    uint32_t b, hkv, t, d;
    int32_t src_dtype;
    B200QuantSide kq, vq;
    uint32_t cap;             /* rows per (batch entry, head) of both caches; 0 = unchecked */
    int32_t *status;          /* optional device word, set to 3 when a device position was out of range */
    uint32_t flags;           /* B200_KV_* below; 0 = none */
    uint32_t pad;
} B200KvAppendArgs;
/* The append may run while the stream's previous kernel is still running (programmatic dependent launch): the caller
 * states that this kernel neither reads the rows written here nor writes k, v or pos. True for the decode loop, where
 * the previous kernel is the attention of the step before: it reads the rows below the position this call writes (and
 * at most the first bytes of that row, which it ignores). The append's own completion still waits for that kernel, so
 * whatever follows in the stream is ordered behind both; an attention that follows with B200_TQ_AFTER_PREV |
 * B200_TQ_INPUTS_FINAL and fresh_rows = t then streams its old rows while the previous attention drains. */
#define B200_KV_AFTER_PREV 1u
int b200_kv_append(const B200KvAppendArgs *args, b200_stream_t stream);

/* ---- paged rows --------------------------------------------------------------------------------- */
/* One block of a paged cache, device memory. Block i holds `rows` valid keys; k / v point at its
 * (batch 0, kv head 0, row 0); head stride = k_cap (v_cap) rows, batch stride = hkv head strides.
 * Same meaning as ax_pages / PageTable (candle-core/kernels/accel_common.h:109-123,
 * candle-core/src/accel/attention.rs:296-366), but the table is an array in device memory
 * instead of a 3 592-byte kernel argument, so it is not limited to 128 blocks. */
typedef struct B200Page {
    const void *k, *v;
    uint32_t rows, k_cap, v_cap, pad;
} B200Page;

/* ---- attention over packed rows ------------------------------------------------------------------ */
/* Replaces CudaStorage::tq_attention / tq_attention_paged (accel.rs:687-857), the kernels
 * tq_attn* / tq_combine (turbo_quant_impl.h:232-747) and the host chain around them in
 * fused_attention_rows / tq_prepare (candle-nn/src/turbo_quant.rs:1143-1264): query cast, query
 * rotation, attention, split combine, output rotation back and cast, in one or two launches.
 *
 * q (b, hq, lq, d) -> out (b, hq, lq, d), both with (batch, head, token) element strides.
 * Keys are the rows [0, kv_len) of k_rows / v_rows (b, hkv, cap, words); masks are aligned to the
 * bottom right (query i sits at key position i + kv_len - lq; key j visible when
 * pos - wl <= j <= pos + wr, negative = unbounded, wr = 0 causal). score = scale * rsc0_k *
 * sum_d elem_k * q_d, then softcap (> 0) and ALiBi; value weight p * rsc0_v. Rows without a
 * visible key give zeros. With kq.rotation / vq.rotation = Hadamard the query is rotated with the
 * key signs and the output rotated back with the value signs; with B200_ROT_NONE, q_dtype =
 * out_dtype = B200_F32 the call is exactly the reference's tq_attention.
 *
 * Any word-aligned row address and any row stride are accepted. Rows packed back to back (stride = the format's row
 * words) whose slabs start at multiples of 16 bytes, as a cache allocated in whole rows has them, take the
 * instantiations with constant row geometry and, for rows of 72, 80 or 136 bytes, wider shared-memory loads.
 *
 * Extension for ragged batches (the reference has one seq_len per cache, turbo_quant.rs:895-897):
 * kv_len_dev, one length per batch entry in device memory; lk is then the maximum length.
 *
 * Prod keys (kq.mode = B200_TURBO_PROD; turbo_quant_impl.h:268-277): every query row holds 2 d values, the query in
 * the rotated domain followed by S times it (the caller rotates and projects, as the reference's tq_prepare does,
 * candle-nn/src/turbo_quant.rs:1161-1168), kq.rotation must be B200_ROT_NONE, and every score gains
 * rsc0 rsc1 sqrt(pi / 2) / d times the signed sum of S q over the key's sign bits. Served by the general kernel. */
typedef struct B200TqAttnArgs {
    const void *q;
    void *out;
    int32_t q_dtype, out_dtype;
    uint64_t q_strides[3], out_strides[3]; /* (batch, head, token) in elements */
    const uint32_t *k_rows, *v_rows;       /* dense rows, or NULL when pages is set */
    uint64_t k_strides[3], v_strides[3];   /* (batch, head, row) in words */
    const B200Page *pages;                 /* device array of n_pages blocks, or NULL */
    uint32_t n_pages;
    const int32_t *kv_len_dev;             /* device, b entries, or NULL */
    uint32_t b, lq, lk, hq, hkv, d;
    B200QuantSide kq, vq;
    float scale, softcap;
    int32_t wl, wr;
    const float *alibi;                    /* device f32 slopes or NULL */
    uint32_t alibi_bstride;                /* 0 or hq */
    int32_t splits;                        /* key splits per sequence; 0 = chosen by the library */
    void *workspace;                       /* device, b200_tq_attention_workspace_bytes() */
    size_t workspace_bytes;
    int32_t *status;                       /* optional device word, set non-zero if a device wait ran out */
    uint32_t flags;                        /* B200_TQ_* below; 0 = none */
    int32_t kv_len_add;                    /* added to every kv_len_dev entry: the tokens appended since the device
                                            * lengths were written (a serving loop updates them once per graph of
                                            * steps, not per token); sums must not exceed lk; unused without kv_len_dev */
    uint32_t fresh_rows;                   /* with B200_TQ_INPUTS_FINAL: rows at the end of every sequence that the stream's
                                            * previous kernel may still be writing (1 after the append of a decode step) */
} B200TqAttnArgs;
/* The attention may start while the stream's previous kernel is still running (programmatic dependent launch): its
 * blocks take their places and work out their shares of the keys from kv_len_dev during that kernel's last
 * microseconds, and wait for its completion before they touch q, the rows, alibi or the workspace. For the layers of
 * one decode step, whose lengths were final before the step began. Do not set it when the previous kernel in the
 * stream writes kv_len_dev (or the page table: paged calls ignore the flag). The reference has no counterpart: it
 * launches every kernel after the previous one has finished (candle-core/src/cuda_backend/accel.rs:190-252). */
#define B200_TQ_AFTER_PREV 1u
/* Together with B200_TQ_AFTER_PREV: the stream's previous kernel writes none of this call's inputs (q, alibi, the
 * codebooks and signs, kv_len_dev) except the last `fresh_rows` rows of every sequence (rows kv_len - fresh_rows ..
 * kv_len - 1); everything else was final before that kernel started. The attention then does not wait for that kernel
 * before it reads: its first keys stream, and its first scores are computed, while the previous kernel's last blocks
 * still run; it waits before it copies a tile that reaches into the fresh rows and before it stores anything (outputs,
 * workspace). True for a decode step, whose previous kernel is the quantize-on-append of the step's one new token
 * (fresh_rows = 1: q was produced before that kernel), and for attention calls that follow one another over caches
 * nobody writes (fresh_rows = 0). The outputs are those of the plain call. */
#define B200_TQ_INPUTS_FINAL 2u
/* Together with B200_TQ_AFTER_PREV: this call's `out` and its workspace are touched by no kernel launched on the stream
 * since the last kernel that was launched without B200_TQ_AFTER_PREV (an attention without the flag, or any other plain
 * launch: it starts when all earlier work has completed). A caller that runs several attentions back to back gives
 * each run of flagged calls outputs and workspaces of their own and starts every run with a call without
 * B200_TQ_AFTER_PREV. The attention then stores partial results and finished rows without waiting for the previous
 * kernel, so that consecutive calls overlap for as long as the device has room for both (a worker that finishes its
 * first column early no longer sits on its place until the whole previous grid has gone); a tile that reaches into the
 * fresh rows still waits, and one block of the grid waits for the previous kernel before it leaves, so that a kernel of
 * such a run never completes before its predecessor. With no fresh rows either (fresh_rows = 0), a call whose columns are
 * split over many workers merges them inside its grid rather than in a combine grid behind it, so that nothing between two
 * calls waits for all workers. Ignored by calls with gathered outputs (their step word is the previous call's to write)
 * and by b200_tq_attention_static (its buffer is shared). The outputs are those of the plain call up to the order of the
 * merge's sums. */
#define B200_TQ_OUTPUTS_FREE 8u
/* Paged calls (pages != NULL): the blocks are read where they are, without a copy, by the general kernel; by the
 * tensor-core kernel too when keys and values share one of its formats (it walks the block table). Other format pairs
 * of the tensor-core kernel are compacted into the workspace by one copy kernel first, unless this flag is set: then
 * the general kernel serves the call (split along the keys when the output rows are few) and the workspace asked
 * for is only that of its partial rows. */
#define B200_TQ_IN_PLACE 4u
/* Paged calls: the size returned covers what the route above needs (the block prefix table of the walking kernel, or a
 * compacted copy of all valid rows, or the general kernel's partial rows); with less the call still runs, on the general
 * kernel with one block per output row (16 bytes are enough). lk is an upper bound of the sum of the blocks' rows. */
size_t b200_tq_attention_workspace_bytes(const B200TqAttnArgs *args);
int b200_tq_attention(const B200TqAttnArgs *args, b200_stream_t stream);

/* Same call as b200_tq_attention for hosts that cannot give the library a workspace. It has no
 * counterpart in the reference, whose launcher allocates its split buffers on every call
 * (candle-core/src/cuda_backend/accel.rs:190-199 is the behaviour this avoids, not an interface it
 * replaces).
 *
 * Who needs it: a serving process that handed all of HBM to its own pool at start-up and has no
 * allocator handle to pass down through an FFI layer; a decode loop in which a cudaMalloc or
 * cudaFree is forbidden because both synchronize the whole device; a binding that runs while
 * another thread holds the host allocator's lock. For those, the split partials, their
 * log-sum-exps and the column table live in a buffer of B200_STATIC_SCRATCH_BYTES that is part
 * of the library image: every GPU that loads libb200attn.so holds that many bytes until the
 * process exits, whether or not this entry point is ever called. The call itself allocates
 * nothing: no cudaMalloc, cudaFree or allocating library routine.
 *
 * args->workspace and args->workspace_bytes are ignored; inputs and outputs are passed as usual.
 * A call whose b200_tq_attention_workspace_bytes() exceeds B200_STATIC_SCRATCH_BYTES is refused
 * with B200_ERR_WORKSPACE and a message that names both sizes (use b200_tq_attention then).
 * The first call on each device looks up the buffer's device address (with that device current)
 * and keeps it; make that first call before any stream capture begins on that device.
 * Every call on a device shares the one buffer, which keeps the previous call's contents. Nothing
 * in it has to start at zero (each call writes every word it later reads), but two calls that
 * overlap on the GPU, from different streams or threads, race on it: keep calls to this entry
 * point ordered on one stream per device. */
#define B200_STATIC_SCRATCH_BYTES (8u << 20)
int b200_tq_attention_static(const B200TqAttnArgs *args, b200_stream_t stream);

/* ---- attention over packed rows, outputs gathered on every GPU ---------------------------------- */
/* The all-gather of the outputs that follows a sharded decode step (every rank holds its own batch
 * entries or kv heads, and the layer's outputs are assembled on every rank: one all-gather per
 * layer when done with NCCL), fused into the epilogue of the attention: the warp that finishes an
 * output row (the one that merges its key splits) stores it into the gathered buffer of every rank
 * (plain peer stores over NVLink, no multicast); the warp that finishes the call's last row publishes
 * this rank's step number in every rank's flag array and waits, with a bound, until every rank has
 * published the same step. One launch when the attention merges its splits itself, else the
 * combine grid stores the rows and its last block to finish publishes.
 * When the call has completed in stream order, slot (step & 1) of this rank's gathered buffer
 * holds the rows of all ranks: [world][b * hq * lq][d] elements of out_dtype, rank r's rows in
 * block r, each in (batch, head, token) order. Two slots, because a rank may run one step ahead.
 *   peer_bufs   device array of `world` pointers: the gathered buffers (2 slots each) of all ranks,
 *               mapped into this process (symmetric memory / IPC); peer_bufs[rank] is the local one
 *   peer_flags  device array of `world` pointers: each rank's `world` flag words, zeroed once
 *   step        device word of this rank, zero before the first call: steps completed so far
 *   done_ctr    device word of this rank, zero before the first call: counts the finished columns of
 *               the call in flight and is back at zero when the call ends
 *   max_polls   polls of every flag before the wait for the other ranks gives up (0 = 2^21, about a
 *               tenth of a second)
 * All ranks must make the same sequence of calls. The wait for the other ranks is bounded; if it
 * runs out, args->status (if given) is set to 2, b200_device_wait_status() reports 1 from then on
 * and the buffer is incomplete for that step; the call still completes and later calls work. */
typedef struct B200PeerGather {
    void *const *peer_bufs;
    uint32_t *const *peer_flags;
    uint32_t world, rank;
    uint32_t *step;
    uint32_t *done_ctr;
    uint32_t max_polls;
    uint32_t pad;
} B200PeerGather;
int b200_tq_attention_gather(const B200TqAttnArgs *args, const B200PeerGather *gather, b200_stream_t stream);

/* ---- attention over dense K / V ------------------------------------------------------------------- */
/* Replaces CudaStorage::flash_attn / flash_attn_paged (accel.rs:254-506), the kernels fa_row*,
 * fa2_*, fa3_*, fa_combine_* (candle-core/kernels/flash_attn_impl.h) and therefore the device
 * side of candle_flash_attn::flash_attn / flash_attn_varlen (candle-flash-attn/src/lib.rs:149-345).
 * Arguments are the kernel parameter list FA_PARAMS (flash_attn_impl.h:29-35): q (b, lq, hq, d),
 * k / v (b, lk, hkv, d) with (batch, seq, head) element strides; varlen: q (total_q, hq, d) with
 * cu_q / cu_k u32 offsets (b + 1 entries), lq / lk the maxima. o: (token, head, d) contiguous.
 * Head dims: every multiple of 8 up to 256 (kernel_supported of candle-core/src/accel/attention.rs:283-290 takes any
 * d <= 256; others return B200_ERR_UNSUPPORTED_SHAPE and the caller's unfused path serves them). */
typedef struct B200FaArgs {
    const void *q, *k, *v;
    void *o;
    int32_t q_dtype;  /* B200_F16 / B200_BF16 / B200_F32; o has the same dtype */
    int32_t kv_dtype; /* q_dtype or B200_FP8 */
    const uint32_t *cu_q, *cu_k; /* device, varlen only */
    uint32_t b, lq, lk, hq, hkv, d;
    uint64_t q_strides[3], k_strides[3], v_strides[3]; /* (batch, seq, head) in elements */
    float scale, softcap;
    int32_t wl, wr;
    float k_descale, v_descale;
    const float *alibi;
    uint32_t alibi_bstride;
    uint32_t varlen;
    uint64_t total_q; /* output tokens: b * lq, or the varlen total */
    void *workspace;
    size_t workspace_bytes;
} B200FaArgs;
size_t b200_flash_attn_workspace_bytes(const B200FaArgs *args);
int b200_flash_attn(const B200FaArgs *args, b200_stream_t stream);

/* Replaces CudaStorage::flash_attn_paged (accel.rs:391-506; kernels fa_rowp*, fa_rowpg*): attention over the dense K / V
 * of paged cache blocks, read where they are (no limit on the number of blocks or of query tokens). Block i (B200Page)
 * holds rows[i] keys at rows 0 .. of its (batch entry, kv head) slabs, laid out (batch, kv head, capacity, row) with
 * k_cap[i] / v_cap[i] rows per slab; the keys of the call are the blocks' valid rows in order (candle-nn/src/
 * flash_attn.rs:608-646). args: q, o, dtypes, masks as for b200_flash_attn; k and v are ignored; k_strides[1] /
 * v_strides[1] are the row strides of every block in elements (16-byte multiples for 16-bit elements, block pointers
 * 16-byte aligned); lk bounds the number of keys (the blocks' total if smaller); varlen must be 0. `pages`: device array.
 * The workspace holds the keys before every block (written by a one-block kernel in front) and the split buffers. */
size_t b200_flash_attn_paged_workspace_bytes(const B200FaArgs *args, uint32_t n_pages);
int b200_flash_attn_paged(const B200FaArgs *args, const B200Page *pages, uint32_t n_pages, b200_stream_t stream);

/* Causal / windowed prefill with the new keys and values written into the compressed cache in
 * the same call. Replaces the pair flash_attn(q, k, v, scale, causal) + TurboKvCache::append(k, v)
 * (candle-flash-attn/src/lib.rs:149-157, candle-nn/src/turbo_quant.rs:916-945). `fa` describes the
 * attention over the uncompressed k / v (b, lk, hkv, d); `append` the cache write, whose k / v
 * pointers and strides must describe the same tensors viewed as (b, hkv, t, d). */
int b200_fa_prefill_append(const B200FaArgs *fa, const B200KvAppendArgs *append, b200_stream_t stream);

/* Health check: 1 when a bounded device-side wait of the attention kernels (an mbarrier that a copy or
 * a tensor core commit should have completed, the flag of another rank in the gathered attention) has run out
 * on the current device since the library was loaded or the flag was last cleared, 0 otherwise, -1 when the
 * device cannot be read. Synchronizes the device. The flag is sticky: while it is set, the tensor-core prefill
 * kernels return at once without writing their outputs (b200_flash_attn / b200_fa_prefill_append still return
 * B200_OK: the launch itself succeeded), so a caller of those polls this after a step whose results matter. The
 * reference has no counterpart: its kernels hold no device-side waits (candle-core/kernels/flash_attn_impl.h
 * uses block barriers only). */
int b200_device_wait_status(void);

/* The same as a status code: B200_ERR_DEVICE_WAIT (with a message for b200_last_error) when the flag is set,
 * B200_OK otherwise; clear != 0 also resets it, after which all kernels run normally again. */
int b200_device_wait_check(int clear);

/* ---- offloaded KV blocks: pinned host buffers and the device's copy stream ------------------------------------ */
/* Replaces candle-core/src/cuda_backend/offload.rs:122-441 (PinnedHostBuffer, CopyStream, CopyEvent;
 * CudaDevice::alloc_pinned / copy_stream), which the reference offers for packed KV blocks that live in host memory
 * or on disk and are uploaded per step (candle-nn/src/turbo_quant.rs:999-1004). One non-blocking copy stream per
 * device, shared by all callers. A copy starts after the work queued so far on `compute` and yields an event:
 * b200_copy_event_wait_on_compute before kernels that read uploaded bytes (or overwrite / free the source of a
 * download), b200_copy_event_synchronize before the host reads downloaded bytes. The device buffer must stay alive
 * until the event was waited on or freed. b200_pinned_ptr waits for the copies queued on the buffer first, so a
 * reused staging buffer is never rewritten while the DMA engine still reads it. */
typedef struct B200PinnedBuffer B200PinnedBuffer; /* page-locked host memory, usable with every device */
typedef struct B200CopyEvent B200CopyEvent;       /* completion of one queued copy */
int b200_pinned_alloc(size_t bytes, B200PinnedBuffer **out);
int b200_pinned_free(B200PinnedBuffer *buf);          /* waits for the copies queued on it */
size_t b200_pinned_len(const B200PinnedBuffer *buf);
int b200_pinned_wait_idle(B200PinnedBuffer *buf);
void *b200_pinned_ptr(B200PinnedBuffer *buf);         /* the bytes, after the queued copies completed; NULL on error */
/* src[src_off .. src_off + bytes) -> dst (device, dst_len bytes) at byte offset dst_off (offload.rs:345-379) */
int b200_copy_upload(B200PinnedBuffer *src, size_t src_off, void *dst, size_t dst_len, size_t dst_off, size_t bytes,
                     b200_stream_t compute, B200CopyEvent **event);
/* src (device, src_len bytes) from byte offset src_off -> dst[dst_off .. dst_off + bytes) (offload.rs:385-419) */
int b200_copy_download(const void *src, size_t src_len, size_t src_off, B200PinnedBuffer *dst, size_t dst_off, size_t bytes,
                       b200_stream_t compute, B200CopyEvent **event);
int b200_copy_event_wait_on_compute(B200CopyEvent *event, b200_stream_t compute); /* on the GPU; the host does not block */
int b200_copy_event_synchronize(B200CopyEvent *event);                            /* blocks the calling thread */
int b200_copy_event_is_complete(B200CopyEvent *event);                            /* 1 / 0, does not block */
/* Releases the event; one that was never waited on first makes `compute` wait for the copy (offload.rs:259-266). */
int b200_copy_event_free(B200CopyEvent *event, b200_stream_t compute);
int b200_copy_stream_synchronize(void); /* every copy queued so far on the current device's copy stream */

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H */
