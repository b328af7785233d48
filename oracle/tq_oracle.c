/*
 * CPU oracle for the quantized-KV attention path. TEST INFRASTRUCTURE ONLY: this file is the
 * checker that the CUDA kernels are compared with (tests, the smoke check and the CPU baseline
 * leg of the benchmark); the product never calls it.
 *
 * It restates, in plain C, the algorithm of the reference (Qntology/candle-rocm-vulkan):
 *   element codecs / row layout      candle-core/src/accel/formats.rs:224-407,
 *                                    candle-core/kernels/accel_common.h:131-236
 *   row codec (quantize/dequantize)  candle-core/src/accel/turbo.rs:293-424,
 *                                    candle-core/kernels/turbo_quant_impl.h:71-159,208-224
 *   SplitMix64, rotations, codebook  candle-core/src/accel/turbo.rs:58-239
 *   attention semantics              candle-core/src/accel/attention.rs:82-92,671-734,
 *                                    candle-core/kernels/turbo_quant_impl.h:232-401
 *   unfused CPU path (the baseline)  candle-nn/src/flash_attn.rs:930-1000,
 *                                    candle-nn/src/turbo_quant.rs:916-991
 *   split combine                    candle-core/kernels/turbo_quant_impl.h:659-685
 *
 * Parity is pinned: tests/test_oracle_pins.py checks these functions against the reference's own
 * kernel sources compiled as plain C++ (oracle/_ref, built by oracle/Makefile from the
 * reference tree) through the committed fixtures in tests/golden/, and against the
 * known-answer values of the reference's unit tests. The one unpinned piece is the Lloyd-Max
 * codebook (the reference computes it in Rust, which cannot run here): it is only checked
 * against the approximations asserted in candle-core/src/accel/turbo.rs:585-597.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no fused multiply-add, like the
 * reference's host build, candle-core/tests/accel_kernels_host.rs:24-28).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MSE 0
#define ORC_PROD 1
#define ORC_QJL 1.2533141f /* sqrt(pi / 2): turbo_quant_impl.h:26 */
#define ORC_MXFP4 2
#define ORC_NVFP4 3
#define ORC_MXFP8 4
#define ORC_FP8 5

static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* ------------------------------------------------------------------ element codecs */

/* accel_common.h:131-138 */
float orc_h2f(uint16_t h) {
    const uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    const float sub = (float)m * 5.9604644775390625e-8f;
    const uint32_t big = (e == 31u ? 0x7f800000u : ((e + 112u) << 23)) | (m << 13);
    const float v = e == 0u ? sub : u2f(big);
    return (h & 0x8000u) ? -v : v;
}

/* accel_common.h:140-152 */
uint16_t orc_f2h(float f) {
    const uint32_t x = f2u(f), s = (x >> 16) & 0x8000u, ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return (uint16_t)(s | 0x7e00u);
    if (ax >= 0x477ff000u) return (uint16_t)(s | 0x7c00u);
    if (ax < 0x38800000u) {
        const float v = rintf(u2f(ax) * 16777216.0f);
        return (uint16_t)(s | (uint32_t)v);
    }
    const uint32_t r = ax + 0xfffu + ((ax >> 13) & 1u);
    return (uint16_t)(s | ((r >> 13) - (112u << 10)));
}

float orc_bf2f(uint16_t b) { return u2f(((uint32_t)b) << 16); }

/* accel_common.h:156-161 */
uint16_t orc_f2bf(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* formats.rs:267-284 */
float orc_e4m3_to_f32(uint32_t c) {
    const uint32_t e = (c >> 3) & 0xfu, m = c & 7u;
    if (e == 15u && m == 7u) return u2f(0x7fc00000u);
    const float v = e == 0 ? (float)m * 0.001953125f : u2f(((e + 120u) << 23) | (m << 20));
    return (c & 0x80u) ? -v : v;
}

/* formats.rs:288-308 */
uint32_t orc_f32_to_e4m3(float f) {
    const uint32_t x = f2u(f), s = (x >> 24) & 0x80u, ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return s | 0x7fu;
    const float a = u2f(ax);
    if (a >= 448.0f) return s | 0x7eu;
    if (a < 0.015625f) return s | (uint32_t)rintf(a * 512.0f);
    const uint32_t r = ax + 0x7ffffu + ((ax >> 20) & 1u);
    uint32_t code = (((r >> 23) - 120u) << 3) | ((r >> 20) & 7u);
    if (code > 0x7eu) code = 0x7eu;
    return s | code;
}

/* formats.rs:312-325 */
float orc_fp4_to_f32(uint32_t c) {
    const uint32_t e = (c >> 1) & 3u, m = c & 1u;
    const float v = e == 0 ? 0.5f * (float)m : u2f(((e + 126u) << 23) | (m << 22));
    return (c & 8u) ? -v : v;
}

/* formats.rs:329-350 */
uint32_t orc_f32_to_fp4(float f) {
    const uint32_t s = (f2u(f) >> 28) & 8u;
    const float a = fabsf(f);
    uint32_t c;
    if (!(a > 0.25f)) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return s | c;
}

/* formats.rs:354-360 */
float orc_e8m0_to_f32(uint32_t c) { return c == 0 ? u2f(0x00400000u) : u2f(c << 23); }

/* formats.rs:365-372, accel_common.h:228-236 */
uint32_t orc_mx_scale_code(float amax, int emax_elem) {
    int e = -127;
    const uint32_t bits = f2u(amax);
    const int be = (int)((bits >> 23) & 0xffu);
    if (amax > 0.0f && be != 0xff && be != 0) e = be - 127 - emax_elem;
    if (e < -127) e = -127;
    if (e > 127) e = 127;
    return (uint32_t)(e + 127);
}

static inline uint32_t get_bits(const uint32_t *w, size_t pos, uint32_t nb) {
    const size_t wi = pos >> 5;
    const uint32_t sh = (uint32_t)(pos & 31);
    uint32_t v = w[wi] >> sh;
    if (sh + nb > 32u) v |= w[wi + 1] << (32u - sh);
    return v & ((1u << nb) - 1u);
}

static inline void put_bits(uint32_t *w, size_t pos, uint32_t nb, uint32_t v) {
    const size_t wi = pos >> 5;
    const uint32_t sh = (uint32_t)(pos & 31);
    v &= (1u << nb) - 1u;
    w[wi] |= v << sh;
    if (sh + nb > 32u) w[wi + 1] |= v >> (32u - sh);
}

static inline uint32_t get_byte(const uint32_t *w, size_t k) { return (w[k >> 2] >> ((k & 3) * 8)) & 0xffu; }
static inline void put_byte(uint32_t *w, size_t k, uint32_t b) { w[k >> 2] |= (b & 0xffu) << ((k & 3) * 8); }

/* ------------------------------------------------------------------ row layout */

/* formats.rs:138-145,224-242. `bits` is the format width (TurboMse 1-4, TurboProd 2-5), ignored
 * by the float formats. out = {code_bits, code_words, aux_words, row_words, rsc_offset}.
 * Returns 0, or -1 when the format does not fit the vector length (formats.rs:166-187). */
int orc_row_layout(int mode, int bits, int dim, int out[5]) {
    int cb, block = 0;
    switch (mode) {
    case ORC_MSE: if (bits < 1 || bits > 4) return -1; cb = bits; break;
    case ORC_PROD: if (bits < 2 || bits > 5) return -1; cb = bits - 1; break;
    case ORC_MXFP4: cb = 4; block = 32; break;
    case ORC_NVFP4: cb = 4; block = 16; break;
    case ORC_MXFP8: cb = 8; block = 32; break;
    case ORC_FP8: cb = 8; break;
    default: return -1;
    }
    if (dim <= 0 || dim > 1024) return -1;
    if (block && dim % block) return -1;
    const int code_words = (dim * cb + 31) / 32;
    int aux = 0;
    if (mode == ORC_PROD) aux = (dim + 31) / 32;
    else if (block) aux = (dim / block + 3) / 4;
    out[0] = cb; out[1] = code_words; out[2] = aux; out[3] = code_words + aux + 2; out[4] = code_words + aux;
    return 0;
}

/* ------------------------------------------------------------------ SplitMix64 */

typedef struct { uint64_t s; } orc_rng;

/* turbo.rs:157-163 */
static inline uint64_t rng_next(orc_rng *r) {
    r->s += 0x9e3779b97f4a7c15ull;
    uint64_t z = r->s;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
/* turbo.rs:166-168 */
static inline double rng_f64(orc_rng *r) { return ((double)(rng_next(r) >> 11) + 0.5) / 9007199254740992.0; }
/* turbo.rs:171-175 */
static inline double rng_normal(orc_rng *r) {
    const double u1 = rng_f64(r), u2 = rng_f64(r);
    return sqrt(-2.0 * log(u1)) * cos(2.0 * 3.14159265358979323846 * u2);
}

void orc_u64_fill(uint64_t seed, uint64_t *out, size_t n) {
    orc_rng r = {seed};
    for (size_t i = 0; i < n; ++i) out[i] = rng_next(&r);
}

/* n standard normals as f32, the sequence of the reference's test generator
 * (candle-nn/src/turbo_quant.rs:1391-1396). The state advances by a constant, so value i only
 * depends on (seed, i): filled in parallel. */
void orc_normal_fill(uint64_t seed, float scale, float *out, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        orc_rng r = {seed + (uint64_t)(2 * i) * 0x9e3779b97f4a7c15ull};
        out[i] = (float)rng_normal(&r) * scale;
    }
}

/* ------------------------------------------------------------------ tables */

/* turbo.rs:58-129: Lloyd-Max codebook of one coordinate of a random unit vector.
 * tab = [16 centroids | 16 boundaries padded with +inf] (turbo.rs:47-55). */
int orc_codebook(int dim, int bits, float tab[32]) {
    if (bits < 1 || bits > 4 || dim < 2) return -1;
    const int k = 1 << bits;
    double lim = 12.0 / sqrt((double)dim);
    if (lim > 1.0) lim = 1.0;
    const int n = 1 << 16;
    const double h = 2.0 * lim / (double)n;
    const double expo = ((double)dim - 3.0) / 2.0;
    double *xs = malloc(sizeof(double) * n), *w = malloc(sizeof(double) * n);
    double *cw = malloc(sizeof(double) * (n + 1)), *cx = malloc(sizeof(double) * (n + 1));
    double total = 0.0;
    for (int i = 0; i < n; ++i) {
        xs[i] = -lim + ((double)i + 0.5) * h;
        double t = 1.0 - xs[i] * xs[i];
        if (t < 1e-300) t = 1e-300;
        w[i] = exp(expo * log(t));
        total += w[i];
    }
    cw[0] = cx[0] = 0.0;
    for (int i = 0; i < n; ++i) {
        w[i] /= total;
        cw[i + 1] = cw[i] + w[i];
        cx[i + 1] = cx[i] + w[i] * xs[i];
    }
    double c[16], bnd[16];
    for (int i = 0; i < k; ++i) {
        const double p = ((double)i + 0.5) / (double)k;
        int j = 0; /* partition_point(cw, v < p) over n + 1 entries */
        int lo = 0, hi = n + 1;
        while (lo < hi) { int mid = (lo + hi) / 2; if (cw[mid] < p) lo = mid + 1; else hi = mid; }
        j = lo;
        if (j < 1) j = 1;
        if (j > n) j = n;
        c[i] = xs[j - 1];
    }
    for (int it = 0; it < 2000; ++it) {
        for (int i = 0; i + 1 < k; ++i) bnd[i] = 0.5 * (c[i] + c[i + 1]);
        double delta = 0.0;
        int lo = 0;
        for (int i = 0; i < k; ++i) {
            int hi = n;
            if (i + 1 < k) { /* first grid index with x >= b */
                int a = 0, b = n;
                while (a < b) { int mid = (a + b) / 2; if (xs[mid] < bnd[i]) a = mid + 1; else b = mid; }
                hi = a;
            }
            const double mass = cw[hi] - cw[lo];
            if (mass > 0.0) {
                const double m = (cx[hi] - cx[lo]) / mass;
                const double dd = fabs(m - c[i]);
                if (dd > delta) delta = dd;
                c[i] = m;
            }
            lo = hi;
        }
        if (delta < 1e-12) break;
    }
    for (int i = 0; i < k / 2; ++i) {
        const double v = 0.5 * (c[k - 1 - i] - c[i]);
        c[i] = -v;
        c[k - 1 - i] = v;
    }
    for (int i = 0; i < 32; ++i) tab[i] = 0.0f;
    for (int i = 0; i < k; ++i) tab[i] = (float)c[i];
    for (int i = 0; i + 1 < k; ++i) tab[16 + i] = (float)(0.5 * (c[i] + c[i + 1]));
    for (int i = 16 + k - 1; i < 32; ++i) tab[i] = INFINITY;
    free(xs); free(w); free(cw); free(cx);
    return 0;
}

/* turbo.rs:192-195: signs of the randomized Hadamard rotation, +1 / -1 per column. */
int orc_hadamard_signs(int dim, uint64_t seed, float *signs) {
    if (dim <= 0 || (dim & (dim - 1))) return -1;
    orc_rng r = {seed ^ 0x484144414d415244ull};
    for (int j = 0; j < dim; ++j) signs[j] = (rng_next(&r) & 1) == 0 ? 1.0f : -1.0f;
    return 0;
}

/* turbo.rs:180-233: row-major dim x dim rotation, kind 0 none / 1 hadamard / 2 dense. */
int orc_rotation_matrix(int dim, int kind, uint64_t seed, float *m) {
    memset(m, 0, sizeof(float) * (size_t)dim * dim);
    if (kind == 0) {
        for (int i = 0; i < dim; ++i) m[(size_t)i * dim + i] = 1.0f;
        return 0;
    }
    if (kind == 1) {
        float *signs = malloc(sizeof(float) * dim);
        if (orc_hadamard_signs(dim, seed, signs)) { free(signs); return -1; }
        const float s = 1.0f / sqrtf((float)dim);
        for (int i = 0; i < dim; ++i)
            for (int j = 0; j < dim; ++j) {
                const float hv = (__builtin_popcount((unsigned)(i & j)) % 2 == 0) ? s : -s;
                m[(size_t)i * dim + j] = hv * signs[j];
            }
        free(signs);
        return 0;
    }
    orc_rng r = {seed ^ 0x524f544154452121ull};
    double *rows = malloc(sizeof(double) * (size_t)dim * dim);
    for (size_t i = 0; i < (size_t)dim * dim; ++i) rows[i] = rng_normal(&r);
    for (int pass = 0; pass < 2; ++pass)
        for (int i = 0; i < dim; ++i) {
            double *ri = rows + (size_t)i * dim;
            for (int j = 0; j < i; ++j) {
                const double *rj = rows + (size_t)j * dim;
                double dot = 0.0;
                for (int t = 0; t < dim; ++t) dot += ri[t] * rj[t];
                for (int t = 0; t < dim; ++t) ri[t] -= dot * rj[t];
            }
            double n = 0.0;
            for (int t = 0; t < dim; ++t) n += ri[t] * ri[t];
            n = sqrt(n);
            for (int t = 0; t < dim; ++t) ri[t] /= n;
        }
    for (size_t i = 0; i < (size_t)dim * dim; ++i) m[i] = (float)rows[i];
    free(rows);
    return 0;
}

/* y = x Pi^T (candle-nn/src/turbo_quant.rs:182-188) / x = y Pi (:191-196), plain f32 sums in
 * index order. The reference uses a library GEMM whose summation order is unspecified. */
void orc_rotate_rows(const float *x, size_t rows, int dim, const float *pi, int transpose, float *y) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const float *xr = x + r * dim;
        float *yr = y + r * dim;
        for (int i = 0; i < dim; ++i) {
            float acc = 0.0f;
            if (!transpose) for (int j = 0; j < dim; ++j) acc += pi[(size_t)i * dim + j] * xr[j];
            else for (int j = 0; j < dim; ++j) acc += pi[(size_t)j * dim + i] * xr[j];
            yr[i] = acc;
        }
    }
}

/* ------------------------------------------------------------------ row codec */

/* Sum of squares in the order of the kernel (turbo_quant_impl.h:84-94 with
 * accel_common.h:255-267): lane t of 128 adds j = t, t + 128, ... then the halving tree. */
static float sumsq_tree(const float *y, int d) {
    float red[128];
    for (int t = 0; t < 128; ++t) {
        float ss = 0.0f;
        for (int j = t; j < d; j += 128) ss += y[j] * y[j];
        red[t] = ss;
    }
    for (int s = 64; s > 0; s >>= 1)
        for (int t = 0; t < s; ++t) red[t] = red[t] + red[t + s];
    return red[0];
}

/* One row: turbo.rs:293-379 (norm_order 0: sequential sum of the CPU codec) or
 * turbo_quant_impl.h:71-159 (norm_order 1: the kernel's tree). Prod rows get stage one only
 * (codes and norm, empty sketch, rsc1 = 0), like tq_quant. */
static void quantize_row(const float *y, int d, int mode, const int lay[5], const float *tab,
                         int norm_order, uint32_t *out) {
    const int cb = lay[0], cw = lay[1];
    for (int i = 0; i < lay[3]; ++i) out[i] = 0;
    float rsc0 = 1.0f;
    if (mode <= ORC_PROD) {
        float ss = 0.0f;
        if (norm_order) ss = sumsq_tree(y, d);
        else for (int j = 0; j < d; ++j) ss += y[j] * y[j];
        const float norm = sqrtf(ss);
        const float inv = norm > 0.0f ? 1.0f / norm : 0.0f;
        const int nb = (1 << cb) - 1;
        for (int j = 0; j < d; ++j) {
            const float u = y[j] * inv;
            uint32_t idx = 0;
            for (int bi = 0; bi < nb; ++bi) idx += u >= tab[16 + bi] ? 1u : 0u;
            put_bits(out, (size_t)j * cb, cb, idx);
        }
        rsc0 = norm;
    } else if (mode == ORC_MXFP4 || mode == ORC_MXFP8) {
        const int fp4 = mode == ORC_MXFP4;
        for (int b = 0; b < d / 32; ++b) {
            float amax = 0.0f;
            for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(y[b * 32 + e]));
            const uint32_t code = orc_mx_scale_code(amax, fp4 ? 2 : 8);
            const float scale = orc_e8m0_to_f32(code);
            put_byte(out + cw, b, code);
            for (int e = 0; e < 32; ++e) {
                const float v = y[b * 32 + e];
                const uint32_t c = code == 0 ? 0u : (fp4 ? orc_f32_to_fp4(v / scale) : orc_f32_to_e4m3(v / scale));
                put_bits(out, (size_t)(b * 32 + e) * cb, cb, c);
            }
        }
    } else if (mode == ORC_NVFP4) {
        float amax = 0.0f;
        for (int j = 0; j < d; ++j) amax = fmaxf(amax, fabsf(y[j]));
        const float g = amax > 0.0f ? amax / 2688.0f : 1.0f;
        for (int b = 0; b < d / 16; ++b) {
            float bmax = 0.0f;
            for (int e = 0; e < 16; ++e) bmax = fmaxf(bmax, fabsf(y[b * 16 + e]));
            const uint32_t cs = orc_f32_to_e4m3(bmax / 6.0f / g);
            const float eff = orc_e4m3_to_f32(cs) * g;
            put_byte(out + cw, b, cs);
            for (int e = 0; e < 16; ++e) {
                const uint32_t c = eff > 0.0f ? orc_f32_to_fp4(y[b * 16 + e] / eff) : 0u;
                put_bits(out, (size_t)(b * 16 + e) * 4, 4, c);
            }
        }
        rsc0 = g;
    } else {
        float amax = 0.0f;
        for (int j = 0; j < d; ++j) amax = fmaxf(amax, fabsf(y[j]));
        const float s = amax > 0.0f ? amax / 448.0f : 1.0f;
        for (int j = 0; j < d; ++j) put_bits(out, (size_t)j * 8, 8, orc_f32_to_e4m3(y[j] / s));
        rsc0 = s;
    }
    out[lay[4]] = f2u(rsc0);
    out[lay[4] + 1] = 0u;
}

int orc_quantize_rows(const float *y, size_t rows, int dim, int mode, int bits, const float *tab,
                      int norm_order, uint32_t *out) {
    int lay[5];
    if (orc_row_layout(mode, bits, dim, lay)) return -1;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r)
        quantize_row(y + r * dim, dim, mode, lay, tab, norm_order, out + r * lay[3]);
    return 0;
}

/* Element j without rsc0: turbo.rs:383-396, turbo_quant_impl.h:44-53. */
static inline float row_elem(const uint32_t *row, int j, int mode, int cb, int cw, const float *cent) {
    const uint32_t c = get_bits(row, (size_t)j * cb, cb);
    const uint32_t *aux = row + cw;
    if (mode <= ORC_PROD) return cent[c];
    if (mode == ORC_MXFP4) return orc_fp4_to_f32(c) * orc_e8m0_to_f32(get_byte(aux, j >> 5));
    if (mode == ORC_NVFP4) return orc_fp4_to_f32(c) * orc_e4m3_to_f32(get_byte(aux, j >> 4));
    if (mode == ORC_MXFP8) return orc_e4m3_to_f32(c) * orc_e8m0_to_f32(get_byte(aux, j >> 5));
    return orc_e4m3_to_f32(c);
}

/* turbo.rs:404-409 without the QJL part, turbo_quant_impl.h:208-218: rsc0 * element. */
int orc_dequantize_rows(const uint32_t *data, size_t rows, size_t row_stride_words, int dim, int mode,
                        int bits, const float *tab, float *out) {
    int lay[5];
    if (orc_row_layout(mode, bits, dim, lay)) return -1;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const uint32_t *row = data + r * row_stride_words;
        const float r0 = u2f(row[lay[4]]);
        for (int j = 0; j < dim; ++j) out[r * dim + j] = r0 * row_elem(row, j, mode, lay[0], lay[1], tab);
    }
    return 0;
}

/* Prod rows, stage two (turbo_quant_impl.h:161-206; CPU twin turbo.rs:320-345).
 * Residual of the unit vector to its codebook value: resid = x / rsc0 - centroid[code]. */
int orc_tq_residual(const float *y, const uint32_t *data, size_t rows, int dim, int bits, const float *tab, float *resid) {
    int lay[5];
    if (orc_row_layout(ORC_PROD, bits, dim, lay)) return -1;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const uint32_t *row = data + r * lay[3];
        const float norm = u2f(row[lay[4]]);
        const float inv = norm > 0.0f ? 1.0f / norm : 0.0f;
        for (int j = 0; j < dim; ++j) {
            const float u = y[r * dim + j] * inv;
            resid[r * dim + j] = u - tab[get_bits(row, (size_t)j * lay[0], lay[0])];
        }
    }
    return 0;
}

/* Copies packed rows and fills in the QJL sign bits (bit j: proj_j >= 0, proj = S resid) and rsc1 = |resid|, the sum of
 * squares in the order of the kernel's 128-lane tree. */
int orc_tq_signs(const uint32_t *in, const float *proj, const float *resid, size_t rows, int dim, int bits, uint32_t *out) {
    int lay[5];
    if (orc_row_layout(ORC_PROD, bits, dim, lay)) return -1;
    const int sign_words = (dim + 31) / 32;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const uint32_t *ir = in + r * lay[3];
        uint32_t *orow = out + r * lay[3];
        for (int w = 0; w < lay[3]; ++w) orow[w] = ir[w];
        for (int w = 0; w < sign_words; ++w) {
            uint32_t word = 0;
            for (int e = 0; e < 32 && w * 32 + e < dim; ++e)
                if (proj[r * dim + w * 32 + e] >= 0.0f) word |= 1u << e;
            orow[lay[1] + w] = word;
        }
        orow[lay[1] + sign_words + 1] = f2u(sqrtf(sumsq_tree(resid + r * dim, dim)));
    }
    return 0;
}

/* turbo.rs:236-239: row-major dim x dim matrix of standard normals, the QJL projection S. */
void orc_qjl_matrix(int dim, uint64_t seed, float *s) {
    orc_rng r = {(seed + 1) ^ 0x514a4c5f534b4554ull};
    for (size_t i = 0; i < (size_t)dim * dim; ++i) s[i] = (float)rng_normal(&r);
}

/* QJL coefficients of prod rows (turbo_quant_impl.h:219-222): +-c with c = rsc0 rsc1 sqrt(pi / 2) / d. */
int orc_dequantize_qjl(const uint32_t *data, size_t rows, int dim, int bits, float *zs) {
    int lay[5];
    if (orc_row_layout(ORC_PROD, bits, dim, lay)) return -1;
    for (size_t r = 0; r < rows; ++r) {
        const uint32_t *row = data + r * lay[3];
        const float c = u2f(row[lay[4]]) * u2f(row[lay[4] + 1]) * ORC_QJL / (float)dim;
        for (int j = 0; j < dim; ++j) zs[r * dim + j] = ((row[lay[1] + (j >> 5)] >> (j & 31)) & 1u) ? c : -c;
    }
    return 0;
}

/* ------------------------------------------------------------------ attention */

/* attention.rs:82-92 */
static void key_range(long long i, long long lq, long long lk, int wl, int wr, long long *lo, long long *hi) {
    const long long pos = i + lk - lq;
    long long l = wl >= 0 ? (pos - wl > 0 ? pos - wl : 0) : 0;
    long long h = wr >= 0 ? (pos + wr + 1 < lk ? pos + wr + 1 : lk) : lk;
    if (l > lk) l = lk;
    if (h < l) h = l;
    *lo = l;
    *hi = h;
}

typedef struct {
    int b, lq, lk, hq, hkv, d;
    float scale, softcap;
    int wl, wr;
    float k_descale, v_descale;
} orc_attn_params;

/* attention.rs:671-734: contiguous f32 q (b, lq, hq, d) / (total_q, hq, d), k and v
 * (b, lk, hkv, d) / (total_k, hkv, d); cu_q / cu_k (b + 1 entries) or NULL; alibi slopes with
 * batch stride alibi_bs or NULL. out: (total_q * hq, d). */
void orc_reference_attention(const float *q, const float *k, const float *v, const uint32_t *cu_q,
                             const uint32_t *cu_k, const float *alibi, int alibi_bs,
                             const orc_attn_params *p, float *out) {
    const int hq = p->hq, hkv = p->hkv, d = p->d, group = hq / hkv;
    const size_t total_q = cu_q ? cu_q[p->b] : (size_t)p->b * p->lq;
    const size_t rows = total_q * hq;
#pragma omp parallel for schedule(dynamic, 4)
    for (size_t row = 0; row < rows; ++row) {
        float *o = out + row * d;
        for (int t = 0; t < d; ++t) o[t] = 0.0f;
        const size_t tok = row / hq;
        const int h = (int)(row % hq);
        size_t b, k0;
        long long i, lq_b, lk_b;
        if (cu_q && cu_k) {
            b = 0;
            while (b + 1 < (size_t)p->b && cu_q[b + 1] <= tok) ++b;
            lq_b = cu_q[b + 1] - cu_q[b];
            lk_b = cu_k[b + 1] - cu_k[b];
            i = (long long)tok - cu_q[b];
            k0 = cu_k[b];
        } else {
            b = tok / p->lq;
            i = tok % p->lq;
            lq_b = p->lq;
            lk_b = p->lk;
            k0 = b * p->lk;
        }
        const int hk = h / group;
        const float *qv = q + (tok * hq + h) * d;
        long long lo, hi;
        key_range(i, lq_b, lk_b, p->wl, p->wr, &lo, &hi);
        if (lo >= hi) continue;
        const float slope = alibi ? alibi[b * alibi_bs + h] : 0.0f;
        const long long pos = i + lk_b - lq_b;
        float *s = malloc(sizeof(float) * (size_t)(hi - lo));
        float m = -INFINITY;
        for (long long j = lo; j < hi; ++j) {
            const float *kv = k + ((k0 + j) * hkv + hk) * d;
            float dot = 0.0f;
            for (int t = 0; t < d; ++t) dot += qv[t] * kv[t];
            dot *= p->k_descale;
            float l = dot * p->scale;
            if (p->softcap > 0.0f) l = p->softcap * tanhf(l / p->softcap);
            if (slope != 0.0f) l -= slope * (float)llabs(pos - j);
            if (l > m) m = l;
            s[j - lo] = l;
        }
        float sum = 0.0f;
        for (long long j = 0; j < hi - lo; ++j) { s[j] = expf(s[j] - m); sum += s[j]; }
        for (long long j = lo; j < hi; ++j) {
            const float w = s[j - lo] / sum * p->v_descale;
            const float *vv = v + ((k0 + j) * hkv + hk) * d;
            for (int t = 0; t < d; ++t) o[t] += w * vv[t];
        }
        free(s);
    }
}

typedef struct {
    int k_mode, k_bits, v_mode, v_bits;
    /* word strides (batch, head, row) of the packed K / V rows */
    size_t k_sb, k_sh, k_ss, v_sb, v_sh, v_ss;
} orc_packed_sides;


/* Attention of (rotated) f32 queries (b, hq, lq, d) over packed K / V rows with the arithmetic
 * of tq_attn (turbo_quant_impl.h:232-401): score = scale * rsc0_k * sum_d elem_k * q_d, softcap,
 * ALiBi, softmax, value weight p * rsc0_v, value element without rsc0. One pass per row in key
 * order (no windows of 128, no splits: those only change the summation order). kv_len: NULL
 * (every sequence has p->lk keys) or one length per batch entry (ragged batch: sequence b
 * attends keys [0, kv_len[b]) with its queries as the last lq positions). tab: 64 floats, key
 * centroids at [0, 16), value centroids at [32, 48). out: (b, hq, lq, d) f32. Prod keys
 * (turbo_quant_impl.h:268-277): the query rows are 2 d wide, the rotated query followed by S q, and
 * every score gains rsc0 rsc1 sqrt(pi / 2) / d times the signed sum of S q over the key's sign bits. */
int orc_tq_attention(const float *q, const uint32_t *kd, const uint32_t *vd, const int32_t *kv_len,
                     const float *tab, const float *alibi, int alibi_bs, const orc_attn_params *p,
                     const orc_packed_sides *sd, float *out) {
    int kl[5], vl[5];
    if (orc_row_layout(sd->k_mode, sd->k_bits, p->d, kl) || orc_row_layout(sd->v_mode, sd->v_bits, p->d, vl)) return -1;
    const int hq = p->hq, hkv = p->hkv, d = p->d, group = hq / hkv, lq = p->lq;
    const size_t rows = (size_t)p->b * hq * lq;
    const float *kc = tab, *vc = tab + 32;
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t row = 0; row < rows; ++row) {
        const size_t b = row / ((size_t)hq * lq);
        const int h = (int)((row / lq) % hq), i = (int)(row % lq);
        const int hk = h / group;
        const long long lk = kv_len ? kv_len[b] : p->lk;
        float *o = out + row * d;
        for (int t = 0; t < d; ++t) o[t] = 0.0f;
        long long lo, hi;
        key_range(i, lq, lk, p->wl, p->wr, &lo, &hi);
        if (lo >= hi) continue;
        const int prod = sd->k_mode == ORC_PROD;
        const float *qr = q + row * (prod ? 2 * d : d), *qs = qr + d;
        const float slope = alibi ? alibi[b * alibi_bs + h] : 0.0f;
        const long long pos = (long long)i + lk - lq;
        const uint32_t *kbase = kd + b * sd->k_sb + (size_t)hk * sd->k_sh;
        const uint32_t *vbase = vd + b * sd->v_sb + (size_t)hk * sd->v_sh;
        float *s = malloc(sizeof(float) * (size_t)(hi - lo));
        float m = -INFINITY;
        for (long long j = lo; j < hi; ++j) {
            const uint32_t *kr = kbase + (size_t)j * sd->k_ss;
            float dot = 0.0f;
            for (int t = 0; t < d; ++t) dot += row_elem(kr, t, sd->k_mode, kl[0], kl[1], kc) * qr[t];
            float sc = u2f(kr[kl[4]]) * dot;
            if (prod) {
                float sdot = 0.0f;
                for (int t = 0; t < d; ++t) sdot += ((kr[kl[1] + (t >> 5)] >> (t & 31)) & 1u) ? qs[t] : -qs[t];
                sc += u2f(kr[kl[4]]) * u2f(kr[kl[4] + 1]) * ORC_QJL / (float)d * sdot;
            }
            sc *= p->scale;
            if (p->softcap > 0.0f) sc = p->softcap * tanhf(sc / p->softcap);
            if (slope != 0.0f) sc -= slope * (float)llabs(pos - j);
            if (sc > m) m = sc;
            s[j - lo] = sc;
        }
        float l = 0.0f;
        float *vrow = malloc(sizeof(float) * d);
        for (long long j = lo; j < hi; ++j) {
            const float pj = expf(s[j - lo] - m);
            l += pj;
            const uint32_t *vr = vbase + (size_t)j * sd->v_ss;
            const float w = pj * u2f(vr[vl[4]]);
            if (w != 0.0f) {
                for (int t = 0; t < d; ++t) vrow[t] = row_elem(vr, t, sd->v_mode, vl[0], vl[1], vc);
                for (int t = 0; t < d; ++t) o[t] += w * vrow[t];
            }
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        for (int t = 0; t < d; ++t) o[t] *= inv;
        free(vrow);
        free(s);
    }
    return 0;
}

/* The reference's unfused CPU path on one (b, lq, hq, d) / (b, lk, hkv, d) f32 problem
 * (candle-nn/src/flash_attn.rs:930-1000): scores = q k^T * scale, additive -1e30 mask,
 * softmax over the whole key axis, p v, fully masked rows multiplied by zero. The full
 * (lq, lk) score matrix is materialized per head, as the matmul path does. */
void orc_unfused_attention(const float *q, const float *k, const float *v, const orc_attn_params *p, float *out) {
    const int hq = p->hq, hkv = p->hkv, d = p->d, group = hq / hkv, lq = p->lq, lk = p->lk;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < p->b; ++b)
        for (int h = 0; h < hq; ++h) {
            const int hk = h / group;
            float *s = malloc(sizeof(float) * (size_t)lq * lk);
            for (int i = 0; i < lq; ++i) {
                const float *qv = q + (((size_t)b * lq + i) * hq + h) * d;
                long long lo, hi;
                key_range(i, lq, lk, p->wl, p->wr, &lo, &hi);
                float *si = s + (size_t)i * lk;
                float m = -INFINITY;
                for (int j = 0; j < lk; ++j) {
                    const float *kv = k + (((size_t)b * lk + j) * hkv + hk) * d;
                    float dot = 0.0f;
                    for (int t = 0; t < d; ++t) dot += qv[t] * (kv[t] * p->k_descale);
                    float x = dot * p->scale;
                    if (p->softcap > 0.0f) x = tanhf(x / p->softcap) * p->softcap;
                    if (j < lo || j >= hi) x += -1e30f;
                    si[j] = x;
                    if (x > m) m = x;
                }
                float sum = 0.0f;
                for (int j = 0; j < lk; ++j) { si[j] = expf(si[j] - m); sum += si[j]; }
                float *o = out + (((size_t)b * lq + i) * hq + h) * d;
                for (int t = 0; t < d; ++t) o[t] = 0.0f;
                for (int j = 0; j < lk; ++j) {
                    const float w = si[j] / sum;
                    const float *vv = v + (((size_t)b * lk + j) * hkv + hk) * d;
                    for (int t = 0; t < d; ++t) o[t] += w * (vv[t] * p->v_descale);
                }
                if (lo >= hi) for (int t = 0; t < d; ++t) o[t] *= 0.0f;
            }
            free(s);
        }
}

/* One decode step of the reference's CPU path over a compressed cache, for the timed CPU baseline: dequantize every
 * cached row and cast it to the cache dtype (TurboKvCache::keys_values, candle-nn/src/turbo_quant.rs:947-966), then the
 * unfused attention of the single query token (candle-nn/src/flash_attn.rs:930-1000: all scores, softmax over the whole
 * key axis, p v). k_rows / v_rows: (hkv, L, row words) packed rows of one sequence, q: (hq, d) f32, out: (hq, d) f32.
 * cache_dtype: 0 f32, 1 f16, 2 bf16. Scratch of 2 hkv L d floats is allocated inside (as the reference materializes K
 * and V). Returns 0, or -1 for an unknown format / no memory. */
static inline float round_cache(float x, int dt) {
    if (dt == 1) return (float)(_Float16)x;
    if (dt == 2) {
        uint32_t u = f2u(x);
        if ((u & 0x7fffffffu) > 0x7f800000u) return u2f(u | 0x00400000u);
        u += 0x7fffu + ((u >> 16) & 1u);
        return u2f(u & 0xffff0000u);
    }
    return x;
}

int orc_cpu_decode_step(const uint32_t *k_rows, const uint32_t *v_rows, size_t L, int hkv, int hq, int d, int mode, int bits,
                        const float *k_tab, const float *v_tab, int cache_dtype, const float *q, float scale, float *out) {
    int lay[5];
    if (orc_row_layout(mode, bits, d, lay)) return -1;
    const size_t rw = (size_t)lay[3], n = (size_t)hkv * L;
    float *kd = malloc(sizeof(float) * n * d), *vd = malloc(sizeof(float) * n * d);
    if (!kd || !vd) { free(kd); free(vd); return -1; }
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n; ++r) {
        const uint32_t *kr = k_rows + r * rw, *vr = v_rows + r * rw;
        const float k0 = u2f(kr[lay[4]]), v0 = u2f(vr[lay[4]]);
        for (int j = 0; j < d; ++j) {
            kd[r * d + j] = round_cache(k0 * row_elem(kr, j, mode, lay[0], lay[1], k_tab), cache_dtype);
            vd[r * d + j] = round_cache(v0 * row_elem(vr, j, mode, lay[0], lay[1], v_tab), cache_dtype);
        }
    }
    const int group = hq / hkv;
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < hq; ++h) {
        const float *kb = kd + (size_t)(h / group) * L * d, *vb = vd + (size_t)(h / group) * L * d, *qv = q + (size_t)h * d;
        float *s = malloc(sizeof(float) * (L ? L : 1)), *o = out + (size_t)h * d;
        if (!s) { bad = 1; continue; }
        float m = -INFINITY;
        for (size_t j = 0; j < L; ++j) {
            float dot = 0.0f;  /* the order of this sum is the matmul library's in the reference: vector lanes here */
#pragma omp simd reduction(+ : dot)
            for (int t = 0; t < d; ++t) dot += qv[t] * kb[j * d + t];
            s[j] = dot * scale;
            if (s[j] > m) m = s[j];
        }
        float sum = 0.0f;
        for (size_t j = 0; j < L; ++j) { s[j] = expf(s[j] - m); sum += s[j]; }
        for (int t = 0; t < d; ++t) o[t] = 0.0f;
        for (size_t j = 0; j < L; ++j) {
            const float w = s[j] / sum;
#pragma omp simd
            for (int t = 0; t < d; ++t) o[t] += w * vb[j * d + t];
        }
        if (L == 0) for (int t = 0; t < d; ++t) o[t] = 0.0f;
        free(s);
    }
    free(kd);
    free(vd);
    return bad ? -1 : 0;
}

/* turbo_quant_impl.h:659-685 / flash_attn_impl.h:445-473 */
void orc_combine(const float *part_o, const float *part_lse, size_t rows, int d, int n_splits, float *o) {
    for (size_t row = 0; row < rows; ++row) {
        float mx = -INFINITY;
        for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_lse[(size_t)s * rows + row]);
        float w[64], wsum = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float e = part_lse[(size_t)s * rows + row];
            w[s] = e == -INFINITY ? 0.0f : expf(e - mx);
        }
        for (int s = 0; s < n_splits; ++s) wsum += w[s];
        for (int t = 0; t < d; ++t) {
            float acc = 0.0f;
            for (int s = 0; s < n_splits; ++s)
                if (w[s] != 0.0f) acc += w[s] * part_o[((size_t)s * rows + row) * d + t];
            o[row * d + t] = wsum > 0.0f ? acc / wsum : 0.0f;
        }
    }
}

/* attention.rs:486-506 (policy Auto) and :586-592 */
int orc_row_group(int hq, int hkv) {
    const int group = hq / (hkv > 0 ? hkv : 1);
    const int gs[3] = {8, 4, 2};
    for (int i = 0; i < 3; ++i) if (group >= gs[i] && group % gs[i] == 0) return gs[i];
    return 1;
}

int orc_split_count_grouped(long long rows, int group, long long lk, int compute_units) {
    if (group < 1) group = 1;
    long long wg = rows / group;
    if (wg < 1) wg = 1;
    const long long cu = compute_units > 0 ? compute_units : 1;
    const long long by_occ = (64 * cu + wg - 1) / wg;
    const long long keys = group > 1 ? 64 : 128;
    long long by_keys = (lk + keys - 1) / keys;
    if (by_keys < 1) by_keys = 1;
    long long n = by_occ < by_keys ? by_occ : by_keys;
    if (n < 1) n = 1;
    if (n > 64) n = 64;
    return (int)n;
}

/* test / benchmark infrastructure: threads of the OpenMP loops (launchers may export OMP_NUM_THREADS=1) */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    n = omp_get_max_threads();
#endif
    return n;
}
