// Host-side weight quantization pass of the backend library (compile time, not a kernel).
//
// Mirrors fastnn's `quantize_weights` / `quantize_weights_fp`
// (src/compiler/passes/quantization.rs:36-273, 281-495): the [K,N] graph constant is
// transposed to [N,K] and packed per output channel with the quantizers of
// src/packed_tensor.rs.  Built with -ffp-contract=off: every f32 rounding of the reference is
// reproduced, so the packed bytes and scales are identical to what the Rust pass emits.
// Rows are independent and are quantized in parallel.
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <vector>

#include "../../include/fastnn_cuda.h"

namespace {

constexpr size_t kMargin = 16;  // packed_tensor.rs:981 SIMD_MARGIN
constexpr size_t kBlock = 32;   // quantization.rs:375

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// f32::round (half away from zero) followed by a saturating `as i8`, NaN -> 0.
inline int round_to_i8(float clamped) {
    if (std::isnan(clamped)) return 0;
    float r = std::round(clamped);
    return (int)std::max(-128.0f, std::min(127.0f, r));
}
inline unsigned round_to_u8(float x) {
    if (std::isnan(x)) return 0;
    float r = std::round(x);
    return (unsigned)std::max(0.0f, std::min(255.0f, r));
}

// ---- lane encoders: f32 lane value -> code ---------------------------------------------------

struct EncI8 {  // src/dtypes/i8x4.rs:33-41
    static constexpr int bits = 8;
    static uint32_t code(float v) {
        float c = v < -128.0f ? -128.0f : (v > 127.0f ? 127.0f : v);
        return (uint32_t)(uint8_t)(int8_t)round_to_i8(c);
    }
};
struct EncI4 {  // src/dtypes/i4x8.rs:33-40
    static constexpr int bits = 4;
    static uint32_t code(float v) {
        float c = v < -8.0f ? -8.0f : (v > 7.0f ? 7.0f : v);
        return (uint32_t)(uint8_t)(int8_t)round_to_i8(c) & 0xFu;
    }
};
struct EncE4M3 {  // src/dtypes/f8x4.rs:41-77
    static constexpr int bits = 8;
    static uint32_t code(float v) {
        if (std::isnan(v)) return 0x7F;
        uint32_t sign = v < 0.0f ? 0x80u : 0u;
        float a = std::fabs(v);
        if (a == 0.0f) return std::signbit(v) ? 0x80u : 0u;
        a = std::min(a, 240.0f);
        if (a < 0.015625f) {
            unsigned m = round_to_u8(a * 512.0f);
            if (m >= 8) return sign | 0x08u;
            return sign | m;
        }
        int e = (int)std::floor(std::log2(a));
        unsigned biased = (unsigned)(e + 7) & 0xFFu;
        float norm = a / std::ldexp(1.0f, e);
        unsigned mant = round_to_u8((norm - 1.0f) * 8.0f);
        if (mant >= 8) {
            unsigned nb = biased + 1;
            return nb >= 15 ? (sign | 0x7Bu) : (sign | (nb << 3));
        }
        if (biased >= 15) return sign | 0x7Bu;
        return sign | (biased << 3) | mant;
    }
};
struct EncE2M1 {  // src/dtypes/f4x8.rs:49-70
    static constexpr int bits = 4;
    static uint32_t code(float v) {
        static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
        if (std::isnan(v)) return 0;
        float a = std::fabs(v);
        unsigned best = 0;
        float best_d = a;
        for (unsigned i = 0; i < 8; ++i) {
            float d = std::fabs(a - mag[i]);
            if (d < best_d) {
                best_d = d;
                best = i;
            }
        }
        return (std::signbit(v) && best != 0) ? (best | 8u) : best;
    }
};

// Pack one row; lanes past `K` stay 0.0 and are encoded as such (packed_tensor.rs:993-1004).
template <class Enc, class Lane>
void pack_row(const float *row, size_t K, uint32_t *dst, Lane lane) {
    constexpr size_t items = 32 / Enc::bits;
    size_t kp = ceil_div(K, items);
    for (size_t w = 0; w < kp; ++w) {
        uint32_t word = 0;
        for (size_t i = 0; i < items; ++i) {
            size_t c = w * items + i;
            float v = c < K ? lane(row[c]) : 0.0f;
            word |= Enc::code(v) << (i * Enc::bits);
        }
        dst[w] = word;
    }
}

// Calls fn(n, row) for every output channel n with `row` = column n of the [K,N] constant.
// Columns are transposed 16 at a time so each 64-byte line of the constant is read once.
template <class Fn>
void for_each_channel(const float *w_kn, size_t K, size_t N, Fn fn) {
    constexpr size_t kCols = 16;
    const long nblocks = (long)ceil_div(N, kCols);
#pragma omp parallel
    {
        std::vector<float> buf(kCols * K);
#pragma omp for schedule(dynamic, 4)
        for (long b = 0; b < nblocks; ++b) {
            size_t n0 = (size_t)b * kCols, nc = std::min(kCols, N - n0);
            for (size_t k = 0; k < K; ++k)
                for (size_t j = 0; j < nc; ++j) buf[j * K + k] = w_kn[k * N + n0 + j];
            for (size_t j = 0; j < nc; ++j) fn(n0 + j, &buf[j * K]);
        }
    }
}

// src/packed_tensor.rs:852-1049 (group_size 0): integer branch :966-974, fp4 branch :950-965.
template <class Enc, bool kFp4>
void quantize_asym(const float *w_kn, size_t K, size_t N, uint32_t *words, float *scales,
                   float *zeros) {
    constexpr size_t items = 32 / Enc::bits;
    const size_t kp = ceil_div(K, items);
    const float umax = (float)((1u << Enc::bits) - 1u);
    const float sbias = (float)(1u << (Enc::bits - 1));
    for_each_channel(w_kn, K, N, [&](size_t n, const float *row) {
        {
            float mn = FLT_MAX, mx = -FLT_MAX;
            for (size_t k = 0; k < K; ++k) {
                mn = std::fmin(mn, row[k]);
                mx = std::fmax(mx, row[k]);
            }
            float range = mx - mn, scale, zp;
            if (range == 0.0f) {
                scale = 1.0f;
                zp = 0.0f;
            } else if (kFp4) {
                float sum = 0.0f;
                for (size_t k = 0; k < K; ++k) sum += row[k];  // sequential, as `iter().sum()`
                float mean = sum / (float)K;
                float dev = std::fmax(std::fabs(mean - mn), std::fabs(mx - mean));
                scale = (dev == 0.0f ? 1e-10f : dev) / 4.0f;
                zp = mean;
            } else {
                float init = range / umax;
                float lo = mn - init, hi = mx + init;
                scale = (hi - lo) / umax;
                zp = lo + sbias * scale;
            }
            scales[n] = scale;
            zeros[n] = zp;
            const float inv = scale != 0.0f ? 1.0f / scale : 0.0f;
            pack_row<Enc>(row, K, words + n * kp, [=](float x) { return (x - zp) * inv; });
        }
    });
}

// src/packed_tensor.rs:661-742
void quantize_sym_e4m3(const float *w_kn, size_t K, size_t N, uint32_t *words, float *scales) {
    const size_t kp = ceil_div(K, 4);
    for_each_channel(w_kn, K, N, [&](size_t n, const float *row) {
        {
            float max_abs = 0.0f;
            for (size_t k = 0; k < K; ++k) max_abs = std::fmax(max_abs, std::fabs(row[k]));
            float scale = max_abs == 0.0f ? 1.0f : max_abs / 240.0f;
            scales[n] = scale;
            const float inv = scale != 1.0f ? 1.0f / scale : 1.0f;
            pack_row<EncE4M3>(row, K, words + n * kp, [=](float x) { return x * inv; });
        }
    });
}

inline unsigned nearest16(float v, const float *c) {  // packed_tensor.rs:77-88
    float best_d = std::fabs(v - c[0]);
    unsigned best = 0;
    for (unsigned i = 1; i < 16; ++i) {
        float d = std::fabs(v - c[i]);
        if (d < best_d) {
            best_d = d;
            best = i;
        }
    }
    return best;
}

// src/packed_tensor.rs:18-75.  Assignment is data-parallel; the per-centroid sums keep the
// reference's element order (each centroid's members are added in stream order).
void kmeans16(const std::vector<float> &values, int iters, float *c) {
    const size_t n = values.size();
    std::fill(c, c + 16, 0.0f);
    if (n == 0) return;
    if (n == 1) {
        std::fill(c, c + 16, values[0]);
        return;
    }
    {
        std::vector<float> sorted(values);
        std::stable_sort(sorted.begin(), sorted.end());
        for (int i = 0; i < 16; ++i) {
            float pct = ((float)i + 0.5f) / 16.0f;
            size_t idx = (size_t)(pct * (float)n);
            c[i] = sorted[std::min(idx, n - 1)];
        }
    }
    std::vector<uint8_t> assign(n);
    for (int it = 0; it < iters; ++it) {
#pragma omp parallel for schedule(static)
        for (long i = 0; i < (long)n; ++i) assign[i] = (uint8_t)nearest16(values[i], c);
        float sums[16];
        size_t counts[16];
#pragma omp parallel for schedule(static, 1)
        for (int ci = 0; ci < 16; ++ci) {
            float s = 0.0f;
            size_t cnt = 0;
            for (size_t i = 0; i < n; ++i)
                if (assign[i] == ci) {
                    s += values[i];
                    ++cnt;
                }
            sums[ci] = s;
            counts[ci] = cnt;
        }
        for (int ci = 0; ci < 16; ++ci)
            if (counts[ci] > 0) c[ci] = sums[ci] / (float)counts[ci];
    }
    std::sort(c, c + 16);
}

// src/packed_tensor.rs:1209-1313 with qblock = 32.
void quantize_codebook(const float *w_kn, size_t K, size_t N, uint32_t *words, float *bscales,
                       float *codebook) {
    const size_t bpr = ceil_div(K, kBlock), kp = ceil_div(K, 8);
    std::vector<float> nk(N * K), normalized(N * K);
    for_each_channel(w_kn, K, N, [&](size_t n, const float *row) {
        std::memcpy(&nk[n * K], row, K * sizeof(float));
    });
#pragma omp parallel for schedule(static)
    for (long n = 0; n < (long)N; ++n) {
        for (size_t b = 0; b < bpr; ++b) {
            size_t lo = b * kBlock, hi = std::min(K, lo + kBlock);
            const float *src = &nk[(size_t)n * K];
            float mx = 0.0f;
            for (size_t k = lo; k < hi; ++k) mx = std::fmax(mx, std::fabs(src[k]));
            bscales[(size_t)n * bpr + b] = mx;
            float inv = mx > 0.0f ? 1.0f / mx : 0.0f;
            for (size_t k = lo; k < hi; ++k)
                normalized[(size_t)n * K + k] = mx > 0.0f ? src[k] * inv : 0.0f;
        }
    }
    kmeans16(normalized, 30, codebook);
#pragma omp parallel for schedule(static)
    for (long n = 0; n < (long)N; ++n) {
        const float *src = &nk[(size_t)n * K];
        for (size_t w = 0; w < kp; ++w) {
            uint32_t word = 0;
            for (size_t i = 0; i < 8; ++i) {
                size_t k = w * 8 + i;
                if (k >= K) break;
                float bs = bscales[(size_t)n * bpr + k / kBlock];
                float inv = bs > 0.0f ? 1.0f / bs : 0.0f;
                word |= nearest16(src[k] * inv, codebook) << (4 * i);
            }
            words[(size_t)n * kp + w] = word;
        }
    }
}

inline size_t items_of(int fmt) { return (fmt == FNN_FMT_I8 || fmt == FNN_FMT_F8) ? 4 : 8; }

}  // namespace

extern "C" {

size_t fnn_quant_packed_bytes(int fmt, size_t N, size_t K) {
    if (fmt < FNN_FMT_I8 || fmt > FNN_FMT_I4CB) return 0;
    return (N * ceil_div(K, items_of(fmt)) + kMargin) * 4;
}

size_t fnn_quant_num_scales(int fmt, size_t N, size_t K) {
    if (fmt < FNN_FMT_I8 || fmt > FNN_FMT_I4CB) return 0;
    return fmt == FNN_FMT_I4CB ? N * ceil_div(K, kBlock) : N;
}

int fnn_quantize_weights(int fmt, const float *w_kn, size_t K, size_t N, void *packed_out,
                         float *scales_out, float *zeros_out, float *codebook_out) {
    if (fmt < FNN_FMT_I8 || fmt > FNN_FMT_I4CB) return FNN_ERR_UNSUPPORTED;
    if (!w_kn || !packed_out || !scales_out || K == 0 || N == 0) return FNN_ERR_COMPILATION;
    uint32_t *words = (uint32_t *)packed_out;
    std::memset(words, 0, fnn_quant_packed_bytes(fmt, N, K));
    std::vector<float> ztmp;
    if (!zeros_out && (fmt == FNN_FMT_I8 || fmt == FNN_FMT_I4 || fmt == FNN_FMT_F4))
        return FNN_ERR_COMPILATION;
    switch (fmt) {
    case FNN_FMT_I8:
        quantize_asym<EncI8, false>(w_kn, K, N, words, scales_out, zeros_out);
        break;
    case FNN_FMT_I4:
        quantize_asym<EncI4, false>(w_kn, K, N, words, scales_out, zeros_out);
        break;
    case FNN_FMT_F4:
        quantize_asym<EncE2M1, true>(w_kn, K, N, words, scales_out, zeros_out);
        break;
    case FNN_FMT_F8:
        quantize_sym_e4m3(w_kn, K, N, words, scales_out);
        if (zeros_out) std::fill(zeros_out, zeros_out + N, 0.0f);
        break;
    case FNN_FMT_I4CB:
        if (!codebook_out) return FNN_ERR_COMPILATION;
        quantize_codebook(w_kn, K, N, words, scales_out, codebook_out);
        break;
    }
    return FNN_OK;
}

}  // extern "C"
