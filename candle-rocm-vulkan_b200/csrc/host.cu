// Host side of libb200attn that needs no kernel: error strings, row layouts, the Lloyd-Max
// codebook, rotation signs, the reference's launch heuristics and the device report.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[512] = "";

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" const char *b200_last_error(void) { return g_err; }

// candle-core/src/accel/formats.rs:138-145,166-187,224-242
extern "C" int b200_row_layout(int mode, int bits, int dim, B200RowLayout *out) {
    if (!out) return set_error(B200_ERR_BAD_ARG, "row_layout: null output");
    int cb = 0, block = 0;
    switch (mode) {
    case B200_TURBO_MSE:
        if (bits < 1 || bits > 4) return set_error(B200_ERR_BAD_ARG, "turbo (mse) supports 1-4 bits, got %d", bits);
        cb = bits;
        break;
    case B200_TURBO_PROD:
        if (bits < 2 || bits > 5) return set_error(B200_ERR_BAD_ARG, "turbo prod supports 2-5 bits, got %d", bits);
        cb = bits - 1;
        break;
    case B200_MXFP4: cb = 4; block = 32; break;
    case B200_NVFP4: cb = 4; block = 16; break;
    case B200_MXFP8: cb = 8; block = 32; break;
    case B200_FP8_ROW: cb = 8; break;
    default: return set_error(B200_ERR_BAD_ARG, "unknown quantization format %d", mode);
    }
    if (dim <= 0 || dim > 1024) return set_error(B200_ERR_BAD_ARG, "vector length %d not in 1..=1024", dim);
    if (block && dim % block)
        return set_error(B200_ERR_BAD_ARG, "vector length %d must be a multiple of the %d element block", dim, block);
    out->dim = dim;
    out->code_bits = cb;
    out->code_words = (dim * cb + 31) / 32;
    out->aux_words = mode == B200_TURBO_PROD ? (dim + 31) / 32 : (block ? (dim / block + 3) / 4 : 0);
    out->row_words = out->code_words + out->aux_words + 2;
    out->rsc_offset = out->code_words + out->aux_words;
    return B200_OK;
}

// candle-core/src/accel/turbo.rs:58-129: density of one coordinate of a random unit vector,
// 65 536 midpoint cells on |x| < min(12 / sqrt(dim), 1), quantile start, Lloyd iterations in f64.
extern "C" int b200_codebook(int dim, int bits, float tab[32]) {
    if (!tab) return set_error(B200_ERR_BAD_ARG, "codebook: null table");
    if (bits < 1 || bits > 4) return set_error(B200_ERR_BAD_ARG, "turbo-quant codebooks have 1 to 4 bits, got %d", bits);
    if (dim < 2) return set_error(B200_ERR_BAD_ARG, "turbo-quant needs vectors of length >= 2, got %d", dim);
    const int k = 1 << bits, n = 1 << 16;
    const double lim = std::min(12.0 / std::sqrt((double)dim), 1.0);
    const double h = 2.0 * lim / n, expo = (dim - 3.0) / 2.0;
    std::vector<double> xs(n), w(n), cw(n + 1, 0.0), cx(n + 1, 0.0);
    double total = 0.0;
    for (int i = 0; i < n; ++i) {
        xs[i] = -lim + (i + 0.5) * h;
        w[i] = std::exp(expo * std::log(std::max(1.0 - xs[i] * xs[i], 1e-300)));
        total += w[i];
    }
    for (int i = 0; i < n; ++i) {
        w[i] /= total;
        cw[i + 1] = cw[i] + w[i];
        cx[i + 1] = cx[i] + w[i] * xs[i];
    }
    std::vector<double> c(k), bnd(k);
    for (int i = 0; i < k; ++i) {
        const double p = (i + 0.5) / k;
        int j = (int)(std::lower_bound(cw.begin(), cw.end(), p) - cw.begin());
        j = std::min(std::max(j, 1), n);
        c[i] = xs[j - 1];
    }
    for (int it = 0; it < 2000; ++it) {
        for (int i = 0; i + 1 < k; ++i) bnd[i] = 0.5 * (c[i] + c[i + 1]);
        double delta = 0.0;
        int lo = 0;
        for (int i = 0; i < k; ++i) {
            const int hi = i + 1 < k ? (int)(std::lower_bound(xs.begin(), xs.end(), bnd[i]) - xs.begin()) : n;
            const double mass = cw[hi] - cw[lo];
            if (mass > 0.0) {
                const double m = (cx[hi] - cx[lo]) / mass;
                delta = std::max(delta, std::fabs(m - c[i]));
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
    return B200_OK;
}

// candle-core/src/accel/turbo.rs:148-163,188-195
extern "C" int b200_hadamard_signs(int dim, uint64_t seed, float *signs) {
    if (!signs) return set_error(B200_ERR_BAD_ARG, "hadamard_signs: null output");
    if (dim <= 0 || (dim & (dim - 1)))
        return set_error(B200_ERR_BAD_ARG, "hadamard rotation needs a power of two length, got %d", dim);
    uint64_t s = seed ^ 0x484144414d415244ull;
    for (int j = 0; j < dim; ++j) {
        s += 0x9e3779b97f4a7c15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        z ^= z >> 31;
        signs[j] = (z & 1) == 0 ? 1.0f : -1.0f;
    }
    return B200_OK;
}

// candle-core/src/accel/turbo.rs:148-176,236-239: row-major dim x dim standard normals (Box-Muller in f64 over
// SplitMix64(seed + 1 ^ "QJL_SKET")), the projection S of the prod format's sketch
extern "C" int b200_qjl_matrix(int dim, uint64_t seed, float *s_out) {
    if (!s_out) return set_error(B200_ERR_BAD_ARG, "qjl_matrix: null output");
    if (dim <= 0 || dim > 1024) return set_error(B200_ERR_BAD_ARG, "qjl_matrix: dim %d outside 1..1024", dim);
    uint64_t s = (seed + 1) ^ 0x514a4c5f534b4554ull;
    auto next_f64 = [&]() {
        s += 0x9e3779b97f4a7c15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        z ^= z >> 31;
        return ((double)(z >> 11) + 0.5) / 9007199254740992.0;
    };
    for (size_t i = 0; i < (size_t)dim * dim; ++i) {
        const double u1 = next_f64(), u2 = next_f64();
        s_out[i] = (float)(sqrt(-2.0 * log(u1)) * cos(2.0 * 3.14159265358979323846 * u2));
    }
    return B200_OK;
}

// candle-core/src/accel/turbo.rs:204-229: the dense rotation for lengths that are not powers of two. Row-major
// dim x dim: standard normals (Box-Muller in f64 over SplitMix64(seed ^ "ROTATE!!")), made orthonormal by two passes
// of modified Gram-Schmidt in f64, rounded to f32.
extern "C" int b200_rotation_matrix(int dim, uint64_t seed, float *m_out) {
    if (!m_out) return set_error(B200_ERR_BAD_ARG, "rotation_matrix: null output");
    if (dim <= 0 || dim > 1024) return set_error(B200_ERR_BAD_ARG, "rotation_matrix: dim %d outside 1..1024", dim);
    uint64_t s = seed ^ 0x524f544154452121ull;
    auto next_f64 = [&]() {
        s += 0x9e3779b97f4a7c15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        z ^= z >> 31;
        return ((double)(z >> 11) + 0.5) / 9007199254740992.0;
    };
    const size_t d = (size_t)dim;
    std::vector<double> rows(d * d);
    for (size_t i = 0; i < d * d; ++i) {
        const double u1 = next_f64(), u2 = next_f64();
        rows[i] = sqrt(-2.0 * log(u1)) * cos(2.0 * 3.14159265358979323846 * u2);
    }
    for (int pass = 0; pass < 2; ++pass)
        for (size_t i = 0; i < d; ++i) {
            double *ri = &rows[i * d];
            for (size_t j = 0; j < i; ++j) {
                const double *rj = &rows[j * d];
                double dot = 0.0;
                for (size_t t = 0; t < d; ++t) dot += ri[t] * rj[t];
                for (size_t t = 0; t < d; ++t) ri[t] -= dot * rj[t];
            }
            double n = 0.0;
            for (size_t t = 0; t < d; ++t) n += ri[t] * ri[t];
            n = sqrt(n);
            for (size_t t = 0; t < d; ++t) ri[t] /= n;
        }
    for (size_t i = 0; i < d * d; ++i) m_out[i] = (float)rows[i];
    return B200_OK;
}

// candle-core/src/accel/attention.rs:586-592
extern "C" int b200_row_group(int hq, int hkv) {
    const int group = hq / (hkv > 0 ? hkv : 1);
    for (int g : {8, 4, 2})
        if (group >= g && group % g == 0) return g;
    return 1;
}

// candle-core/src/accel/attention.rs:486-506 with SplitKv::Auto
extern "C" int b200_split_count_grouped(int64_t rows, int group, int64_t lk, int compute_units) {
    group = std::max(group, 1);
    const int64_t wg = std::max<int64_t>(rows / group, 1);
    const int64_t by_occ = (64 * (int64_t)std::max(compute_units, 1) + wg - 1) / wg;
    const int64_t keys = group > 1 ? 64 : 128;
    const int64_t by_keys = std::max<int64_t>((lk + keys - 1) / keys, 1);
    return (int)std::min<int64_t>(std::max<int64_t>(std::min(by_occ, by_keys), 1), 64);
}

extern "C" int b200_describe(int device, B200Profile *out) {
    if (!out) return set_error(B200_ERR_BAD_ARG, "describe: null output");
    cudaDeviceProp p;
    const cudaError_t e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "describe: %s", cudaGetErrorString(e));
    memset(out, 0, sizeof(*out));
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    out->sm_count = p.multiProcessorCount;
    out->max_smem_optin = (int32_t)p.sharedMemPerBlockOptin;
    out->total_mem = (int64_t)p.totalGlobalMem;
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    return B200_OK;
}
