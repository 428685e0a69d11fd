/*
 * CPU oracle for fastnn's quantized-weight MatMul path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA path and the timed CPU baseline, never the product.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off, no -ffast-math: the
 * quantizers are required to reproduce the reference's f32 roundings exactly).
 *
 * Parity pinning: the reference (Rust) cannot be built here; this file is checked
 * against the reference's known-answer tests and a NumPy twin (see the header).
 */
#define _GNU_SOURCE
#include "fastnn_oracle.h"

#include <float.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ helpers */

static inline size_t div_ceil(size_t a, size_t b) { return (a + b - 1) / b; }

/* Rust `f32::round`: half away from zero == C roundf. */
/* Rust `x as i8` / `as u8`: saturating, NaN -> 0. */
static inline int sat_i8(float x) {
    if (isnan(x)) return 0;
    if (x <= -128.0f) return -128;
    if (x >= 127.0f) return 127;
    return (int)x;
}
static inline unsigned sat_u8(float x) {
    if (isnan(x)) return 0;
    if (x <= 0.0f) return 0;
    if (x >= 255.0f) return 255;
    return (unsigned)x;
}
/* Rust `f32::clamp(lo, hi)`: NaN stays NaN. */
static inline float clampf(float x, float lo, float hi) {
    if (x < lo) return lo;
    if (x > hi) return hi;
    return x;
}

int orc_items_per_word(int fmt) {
    switch (fmt) {
    case ORC_FMT_I8:
    case ORC_FMT_F8:
        return 4; /* src/dtypes/i8x4.rs:16, src/dtypes/f8x4.rs:111 */
    case ORC_FMT_I4:
    case ORC_FMT_F4:
    case ORC_FMT_I4CB:
        return 8; /* src/dtypes/i4x8.rs:16, src/dtypes/f4x8.rs:117 */
    default:
        return 0;
    }
}

size_t orc_words_per_row(int fmt, size_t inner) {
    int items = orc_items_per_word(fmt);
    return items ? div_ceil(inner, (size_t)items) : 0;
}

/* src/packed_tensor.rs:978-982 (and :700-704, :1263-1266): rows*k_packed + SIMD_MARGIN. */
size_t orc_packed_words(int fmt, size_t rows, size_t inner) {
    return rows * orc_words_per_row(fmt, inner) + ORC_SIMD_MARGIN_WORDS;
}

/* ------------------------------------------------------------ scalar codecs */

/* src/dtypes/f8x4.rs:23-38 */
float orc_e4m3_to_f32(uint8_t byte) {
    float sign = (byte & 0x80) ? -1.0f : 1.0f;
    int biased = (byte >> 3) & 0x0F;
    float mant = (float)(byte & 0x07);
    if (biased == 0) {
        if (mant == 0.0f) return 0.0f * sign;
        return sign * ldexpf(1.0f, 1 - 7) * (mant / 8.0f);
    }
    if (biased == 0x0F) return NAN;
    return sign * ldexpf(1.0f, biased - 7) * (1.0f + mant / 8.0f);
}

/* src/dtypes/f8x4.rs:41-77 */
uint8_t orc_f32_to_e4m3(float v) {
    if (isnan(v)) return 0x7F;
    uint8_t sign_bit = (v < 0.0f) ? 0x80 : 0x00;
    float abs_v = fabsf(v);
    if (abs_v == 0.0f) return signbit(v) ? 0x80 : 0x00;
    abs_v = fminf(abs_v, 240.0f);
    if (abs_v < 0.015625f) {
        unsigned m = sat_u8(roundf(abs_v * 512.0f));
        if (m >= 8) return sign_bit | 0x08;
        if (m == 0) return sign_bit;
        return (uint8_t)(sign_bit | m);
    }
    int e = (int)floorf(log2f(abs_v));
    unsigned biased = (unsigned)(e + 7) & 0xFF;
    float normalized = abs_v / ldexpf(1.0f, e);
    unsigned mant = sat_u8(roundf((normalized - 1.0f) * 8.0f));
    if (mant >= 8) {
        unsigned nb = biased + 1;
        if (nb >= 15) return sign_bit | 0x7B;
        return (uint8_t)(sign_bit | (nb << 3));
    }
    if (biased >= 15) return sign_bit | 0x7B;
    return (uint8_t)(sign_bit | (biased << 3) | mant);
}

static const float FP4_MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* src/dtypes/f4x8.rs:25-45: code 0x8 decodes to +0. */
float orc_fp4_to_f32(uint8_t code) {
    float mag = FP4_MAG[code & 7];
    return ((code & 8) && (code & 7)) ? -mag : mag;
}

/* src/dtypes/f4x8.rs:49-70: nearest magnitude, strict '<' so ties keep the lower index. */
uint8_t orc_f32_to_fp4(float v) {
    if (isnan(v)) return 0;
    int neg = signbit(v) ? 1 : 0;
    float a = fabsf(v);
    unsigned best_i = 0;
    float best_d = a;
    for (unsigned i = 0; i < 8; ++i) {
        float d = fabsf(a - FP4_MAG[i]);
        if (d < best_d) {
            best_d = d;
            best_i = i;
        }
    }
    return (uint8_t)((neg && best_i != 0) ? (best_i | 8) : best_i);
}

uint32_t orc_pack_word(int fmt, const float *vals) {
    uint32_t w = 0;
    switch (fmt) {
    case ORC_FMT_I4: /* src/dtypes/i4x8.rs:33-40 */
        for (int i = 0; i < 8; ++i) {
            int q = sat_i8(roundf(clampf(vals[i], -8.0f, 7.0f)));
            w |= ((uint32_t)(uint8_t)(int8_t)q & 0xFu) << (i * 4);
        }
        return w;
    case ORC_FMT_I8: /* src/dtypes/i8x4.rs:33-41 */
        for (int i = 0; i < 4; ++i) {
            int q = sat_i8(roundf(clampf(vals[i], -128.0f, 127.0f)));
            w |= ((uint32_t)(uint8_t)(int8_t)q) << (i * 8);
        }
        return w;
    case ORC_FMT_F8: /* src/dtypes/f8x4.rs:128-134 */
        for (int i = 0; i < 4; ++i) w |= (uint32_t)orc_f32_to_e4m3(vals[i]) << (i * 8);
        return w;
    case ORC_FMT_F4: /* src/dtypes/f4x8.rs:133-145 */
        for (int i = 0; i < 8; ++i) w |= (uint32_t)orc_f32_to_fp4(vals[i]) << (i * 4);
        return w;
    default:
        return 0;
    }
}

void orc_unpack_word(int fmt, uint32_t word, float *out) {
    switch (fmt) {
    case ORC_FMT_I4: /* src/dtypes/i4x8.rs:22-30: sign-extended nibbles */
        for (int i = 0; i < 8; ++i) {
            int32_t nib = (int32_t)((word >> (i * 4)) & 0xF);
            out[i] = (float)((int32_t)((uint32_t)nib << 28) >> 28);
        }
        break;
    case ORC_FMT_I4CB: /* raw unsigned nibble index (src/packed_tensor.rs:90-93) */
        for (int i = 0; i < 8; ++i) out[i] = (float)((word >> (i * 4)) & 0xF);
        break;
    case ORC_FMT_I8: /* src/dtypes/i8x4.rs:22-30 */
        for (int i = 0; i < 4; ++i) out[i] = (float)(int8_t)((word >> (i * 8)) & 0xFF);
        break;
    case ORC_FMT_F8: /* src/dtypes/f8x4.rs:115-124 (LUT == orc_e4m3_to_f32) */
        for (int i = 0; i < 4; ++i) out[i] = orc_e4m3_to_f32((uint8_t)((word >> (i * 8)) & 0xFF));
        break;
    case ORC_FMT_F4: /* src/dtypes/f4x8.rs:120-131 */
        for (int i = 0; i < 8; ++i) out[i] = orc_fp4_to_f32((uint8_t)((word >> (i * 4)) & 0xF));
        break;
    default:
        break;
    }
}

/* src/compiler/passes/quantization.rs:144-156, :361-373 */
void orc_transpose_kn_to_nk(const float *kn, size_t K, size_t N, float *nk) {
    for (size_t r = 0; r < K; ++r)
        for (size_t c = 0; c < N; ++c) nk[c * K + r] = kn[r * N + c];
}

/* ------------------------------------------------------------- quantizers */

/* Pack one row: lane i of word w holds f(data[w*items+i]); lanes past `inner`
 * keep the array default 0.0 and are packed as such
 * (src/packed_tensor.rs:993-1004, :717-728). */
static void pack_row_affine(int fmt, const float *row, size_t inner, float sub, float mul,
                            uint32_t *words_row) {
    int items = orc_items_per_word(fmt);
    size_t kp = div_ceil(inner, (size_t)items);
    for (size_t w = 0; w < kp; ++w) {
        float arr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < items; ++i) {
            size_t c = w * (size_t)items + (size_t)i;
            if (c < inner) arr[i] = (row[c] - sub) * mul;
        }
        words_row[w] = orc_pack_word(fmt, arr);
    }
}

/* src/packed_tensor.rs:205-273 */
void orc_from_f32_slice(int fmt, const float *data, size_t rows, size_t inner, float scale,
                        float zero, uint32_t *words) {
    int items = orc_items_per_word(fmt);
    size_t kp = div_ceil(inner, (size_t)items);
    memset(words, 0, (rows * kp + ORC_SIMD_MARGIN_WORDS) * sizeof(uint32_t));
    for (size_t r = 0; r < rows; ++r) {
        if (scale != 1.0f || zero != 0.0f) {
            float inv = 1.0f / scale;
            pack_row_affine(fmt, data + r * inner, inner, zero, inv, words + r * kp);
        } else {
            /* raw values: (x - 0) * 1 is exact, so the affine helper is equivalent */
            for (size_t w = 0; w < kp; ++w) {
                float arr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int i = 0; i < items; ++i) {
                    size_t c = w * (size_t)items + (size_t)i;
                    if (c < inner) arr[i] = data[r * inner + c];
                }
                words[r * kp + w] = orc_pack_word(fmt, arr);
            }
        }
    }
}

/* src/packed_tensor.rs:852-1049 with group_size == 0 (per output channel).
 * Integer branch :966-974, fp4 branch :950-965, packing :984-1005. */
static void quantize_per_channel_asym(int fmt, const float *data, size_t N, size_t K,
                                      uint32_t *words, float *scales, float *zeros) {
    const int bits = (fmt == ORC_FMT_I8) ? 8 : 4;
    const float unsigned_max = (float)((1u << bits) - 1u);
    const float signed_bias = (float)(1u << (bits - 1));
    const int is_fp4 = (fmt == ORC_FMT_F4); /* IS_FLOAT && MAX_REPRESENTABLE(6) < bias(8) */
    size_t kp = orc_words_per_row(fmt, K);

    for (size_t r = 0; r < N; ++r) {
        const float *row = data + r * K;
        float mn = FLT_MAX, mx = -FLT_MAX; /* f32::MAX / f32::MIN, :867-868 */
        for (size_t i = 0; i < K; ++i) {
            mn = fminf(mn, row[i]);
            mx = fmaxf(mx, row[i]);
        }
        float range = mx - mn;
        float scale, zp;
        if (range == 0.0f || unsigned_max == 0.0f) {
            scale = 1.0f;
            zp = 0.0f;
        } else if (is_fp4) {
            float sum = 0.0f; /* sequential f32 sum, :954 */
            for (size_t i = 0; i < K; ++i) sum += row[i];
            float mean = sum / (float)K;
            float dev = fmaxf(fabsf(mean - mn), fabsf(mx - mean));
            float max_dev = (dev == 0.0f) ? 1e-10f : dev;
            scale = max_dev / 4.0f;
            zp = mean;
        } else {
            float init_scale = range / unsigned_max;
            float lo = mn - init_scale;
            float hi = mx + init_scale;
            scale = (hi - lo) / unsigned_max;
            zp = lo + signed_bias * scale;
        }
        scales[r] = scale;
        zeros[r] = zp;
        float inv = (scale != 0.0f) ? 1.0f / scale : 0.0f;
        pack_row_affine(fmt, row, K, zp, inv, words + r * kp);
    }
}

/* src/packed_tensor.rs:661-742: scale = maxabs/240 (1 if 0), lane = x * (1/scale). */
static void quantize_per_channel_sym_f8(const float *data, size_t N, size_t K, uint32_t *words,
                                        float *scales, float *zeros) {
    size_t kp = orc_words_per_row(ORC_FMT_F8, K);
    for (size_t r = 0; r < N; ++r) {
        const float *row = data + r * K;
        float max_abs = 0.0f;
        for (size_t i = 0; i < K; ++i) max_abs = fmaxf(max_abs, fabsf(row[i]));
        float scale = (max_abs == 0.0f) ? 1.0f : max_abs / 240.0f;
        scales[r] = scale;
        if (zeros) zeros[r] = 0.0f;
        float inv = (scale != 1.0f) ? 1.0f / scale : 1.0f;
        for (size_t w = 0; w < kp; ++w) {
            float arr[4] = {0, 0, 0, 0};
            for (int i = 0; i < 4; ++i) {
                size_t c = w * 4 + (size_t)i;
                if (c < K) arr[i] = row[c] * inv;
            }
            words[r * kp + w] = orc_pack_word(ORC_FMT_F8, arr);
        }
    }
}

/* Stable ascending merge sort (Rust `sort_by(partial_cmp)` is a stable merge sort). */
static void stable_sort_f32(float *a, size_t n) {
    if (n < 2) return;
    float *tmp = (float *)malloc(n * sizeof(float));
    float *src = a, *dst = tmp;
    for (size_t width = 1; width < n; width *= 2) {
        for (size_t lo = 0; lo < n; lo += 2 * width) {
            size_t mid = lo + width < n ? lo + width : n;
            size_t hi = lo + 2 * width < n ? lo + 2 * width : n;
            size_t i = lo, j = mid, k = lo;
            while (i < mid && j < hi) dst[k++] = (src[j] < src[i]) ? src[j++] : src[i++];
            while (i < mid) dst[k++] = src[i++];
            while (j < hi) dst[k++] = src[j++];
        }
        float *t = src;
        src = dst;
        dst = t;
    }
    if (src != a) memcpy(a, src, n * sizeof(float));
    free(tmp);
}

static inline unsigned nearest16(float v, const float *c) {
    /* src/packed_tensor.rs:77-88 and :50-58: first minimum wins (strict '<'). */
    float best_d = fabsf(v - c[0]);
    unsigned best = 0;
    for (unsigned ci = 1; ci < 16; ++ci) {
        float d = fabsf(v - c[ci]);
        if (d < best_d) {
            best_d = d;
            best = ci;
        }
    }
    return best;
}

/* src/packed_tensor.rs:18-75 */
void orc_kmeans16(const float *values, size_t n, int max_iter, float *centroids) {
    for (int i = 0; i < 16; ++i) centroids[i] = 0.0f;
    if (n == 0) return;
    if (n == 1) {
        for (int i = 0; i < 16; ++i) centroids[i] = values[0];
        return;
    }
    float *sorted = (float *)malloc(n * sizeof(float));
    memcpy(sorted, values, n * sizeof(float));
    stable_sort_f32(sorted, n);
    for (int i = 0; i < 16; ++i) {
        float percentile = ((float)i + 0.5f) / 16.0f;
        float pos = percentile * (float)n;
        size_t idx = (size_t)pos; /* `as usize` truncation of a non-negative f32 */
        if (idx > n - 1) idx = n - 1;
        centroids[i] = sorted[idx];
    }
    free(sorted);

    uint8_t *assign = (uint8_t *)malloc(n);
    for (int it = 0; it < max_iter; ++it) {
        for (size_t vi = 0; vi < n; ++vi) assign[vi] = (uint8_t)nearest16(values[vi], centroids);
        size_t counts[16];
        float sums[16];
        for (int c = 0; c < 16; ++c) {
            counts[c] = 0;
            sums[c] = 0.0f;
        }
        for (size_t vi = 0; vi < n; ++vi) { /* sequential f32 sums, :63-66 */
            counts[assign[vi]] += 1;
            sums[assign[vi]] += values[vi];
        }
        for (int c = 0; c < 16; ++c)
            if (counts[c] > 0) centroids[c] = sums[c] / (float)counts[c];
    }
    free(assign);
    /* final ascending sort, :73 */
    for (int i = 1; i < 16; ++i) {
        float x = centroids[i];
        int j = i - 1;
        while (j >= 0 && centroids[j] > x) {
            centroids[j + 1] = centroids[j];
            --j;
        }
        centroids[j + 1] = x;
    }
}

/* src/packed_tensor.rs:1209-1313 with qblock = 32 (quantization.rs:375,436-440). */
static void quantize_codebook(const float *data, size_t N, size_t K, uint32_t *words,
                              float *block_scales, float *codebook) {
    const size_t qb = ORC_CODEBOOK_BLOCK;
    size_t bpr = div_ceil(K, qb);
    size_t kp = div_ceil(K, 8);
    float *normalized = (float *)malloc((N * K + 1) * sizeof(float));
    size_t pos = 0;
    for (size_t blk = 0; blk < N * bpr; ++blk) {
        size_t row = blk / bpr, bi = blk % bpr;
        size_t base = row * K + bi * qb;
        size_t end = base + qb < (row + 1) * K ? base + qb : (row + 1) * K;
        float max_abs = 0.0f;
        for (size_t i = base; i < end; ++i) max_abs = fmaxf(max_abs, fabsf(data[i]));
        block_scales[blk] = max_abs;
        if (max_abs > 0.0f) {
            float inv = 1.0f / max_abs;
            for (size_t i = base; i < end; ++i) normalized[pos++] = data[i] * inv;
        } else {
            for (size_t i = base; i < end; ++i) normalized[pos++] = 0.0f;
        }
    }
    orc_kmeans16(normalized, pos, 30, codebook);
    free(normalized);

    for (size_t row = 0; row < N; ++row) {
        for (size_t b = 0; b < bpr; ++b) {
            float bs = block_scales[row * bpr + b];
            float inv = (bs > 0.0f) ? 1.0f / bs : 0.0f;
            size_t base = row * K + b * qb;
            size_t end = base + qb < (row + 1) * K ? base + qb : (row + 1) * K;
            size_t len = end - base;
            for (size_t e = 0; e < len; e += 8) {
                size_t word_in_row = (b * qb + e) / 8;
                uint32_t w = 0;
                for (int i = 0; i < 8; ++i) {
                    size_t idx = base + e + (size_t)i;
                    if (idx < end) w |= (uint32_t)nearest16(data[idx] * inv, codebook) << (i * 4);
                }
                words[row * kp + word_in_row] = w;
            }
        }
    }
}

int orc_quantize(int fmt, const float *w_nk, size_t N, size_t K, uint32_t *words, float *scales,
                 float *zeros, float *codebook16) {
    if (orc_items_per_word(fmt) == 0) return -1;
    memset(words, 0, orc_packed_words(fmt, N, K) * sizeof(uint32_t));
    switch (fmt) {
    case ORC_FMT_I8:
    case ORC_FMT_I4:
    case ORC_FMT_F4:
        quantize_per_channel_asym(fmt, w_nk, N, K, words, scales, zeros);
        return 0;
    case ORC_FMT_F8:
        quantize_per_channel_sym_f8(w_nk, N, K, words, scales, zeros);
        return 0;
    case ORC_FMT_I4CB:
        quantize_codebook(w_nk, N, K, words, scales, codebook16);
        return 0;
    }
    return -1;
}

/* src/packed_tensor.rs:469-521 (and :275-403): unpack(q) * scale + zero, unfused. */
int orc_dequant(int fmt, const uint32_t *words, size_t N, size_t K, const float *scales,
                const float *zeros, const float *codebook16, float *out) {
    int items = orc_items_per_word(fmt);
    if (!items) return -1;
    size_t kp = div_ceil(K, (size_t)items);
    size_t bpr = div_ceil(K, (size_t)ORC_CODEBOOK_BLOCK);
    for (size_t r = 0; r < N; ++r) {
        for (size_t w = 0; w < kp; ++w) {
            float u[8];
            orc_unpack_word(fmt, words[r * kp + w], u);
            for (int i = 0; i < items; ++i) {
                size_t c = w * (size_t)items + (size_t)i;
                if (c >= K) break;
                if (fmt == ORC_FMT_I4CB) {
                    size_t blk = r * bpr + c / ORC_CODEBOOK_BLOCK;
                    out[r * K + c] = scales[blk] * codebook16[(unsigned)u[i]];
                } else {
                    float z = zeros ? zeros[r] : 0.0f;
                    volatile float prod = u[i] * scales[r];
                    out[r * K + c] = prod + z;
                }
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ GEMM */

static float dot_scalar(const float *a, const float *b, size_t len) {
    /* src/backend/cpu/microkernels/mod.rs:274-281 */
    float acc = 0.0f;
    for (size_t i = 0; i < len; ++i) acc += a[i] * b[i];
    return acc;
}

#if defined(__x86_64__)
/* src/backend/cpu/microkernels/mod.rs:391-431: four 16-lane FMA accumulators. */
__attribute__((target("avx512f"))) static float dot_avx512(const float *a, const float *b,
                                                           size_t len) {
    __m512 acc0 = _mm512_setzero_ps(), acc1 = acc0, acc2 = acc0, acc3 = acc0;
    size_t i = 0;
    for (; i + 64 <= len; i += 64) {
        acc0 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), acc0);
        acc1 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 16), _mm512_loadu_ps(b + i + 16), acc1);
        acc2 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 32), _mm512_loadu_ps(b + i + 32), acc2);
        acc3 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 48), _mm512_loadu_ps(b + i + 48), acc3);
    }
    for (; i + 16 <= len; i += 16)
        acc0 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), acc0);
    __m512 c = _mm512_add_ps(_mm512_add_ps(acc0, acc1), _mm512_add_ps(acc2, acc3));
    float total = _mm512_reduce_add_ps(c);
    for (; i < len; ++i) total += a[i] * b[i];
    return total;
}

__attribute__((target("avx2,fma"))) static float dot_avx2(const float *a, const float *b,
                                                          size_t len) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = acc0, acc2 = acc0, acc3 = acc0;
    size_t i = 0;
    for (; i + 32 <= len; i += 32) {
        acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
        acc1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), acc1);
        acc2 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 16), _mm256_loadu_ps(b + i + 16), acc2);
        acc3 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 24), _mm256_loadu_ps(b + i + 24), acc3);
    }
    for (; i + 8 <= len; i += 8)
        acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
    __m256 c = _mm256_add_ps(_mm256_add_ps(acc0, acc1), _mm256_add_ps(acc2, acc3));
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(c), _mm256_extractf128_ps(c, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
    float total = _mm_cvtss_f32(s);
    for (; i < len; ++i) total += a[i] * b[i];
    return total;
}
#endif

int orc_simd_level(void) {
#if defined(__x86_64__)
    if (__builtin_cpu_supports("avx512f")) return 5;
    if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 2;
#endif
    return 0;
}

/* src/backend/cpu/microkernels/mod.rs:254-272: AVX-512, else AVX2, else scalar. */
static float fma_f32_slice(const float *a, const float *b, size_t len) {
#if defined(__x86_64__)
    static int level = -1;
    if (level < 0) level = orc_simd_level();
    if (level == 5) return dot_avx512(a, b, len);
    if (level == 2) return dot_avx2(a, b, len);
#endif
    return dot_scalar(a, b, len);
}

/* src/backend/cpu/topology.rs:32-60: logical CPUs / SMT width. */
int orc_physical_cores(void) {
    long logical = sysconf(_SC_NPROCESSORS_ONLN);
    if (logical < 1) logical = 4;
    int smt = 1;
    FILE *f = fopen("/sys/devices/system/cpu/cpu0/topology/thread_siblings_list", "r");
    if (f) {
        char buf[256];
        if (fgets(buf, sizeof buf, f)) {
            int n = 1;
            for (char *p = buf; *p; ++p) {
                if (*p == ',') ++n;
                if (*p == '-') {
                    int lo = 0, hi = 0;
                    char *q = p;
                    while (q > buf && q[-1] >= '0' && q[-1] <= '9') --q;
                    lo = atoi(q);
                    hi = atoi(p + 1);
                    n += hi - lo;
                }
            }
            smt = n > 0 ? n : 1;
        }
        fclose(f);
    }
    int phys = (int)((logical + smt - 1) / smt);
    return phys > 0 ? phys : 1;
}

/* src/backend/cpu/microkernels/gemm.rs:23-32 with topology.rs:2-22. */
size_t orc_k_block_size(void) {
    long l2 = sysconf(_SC_LEVEL2_CACHE_SIZE);
    if (l2 <= 0) l2 = 256 * 1024;
    if (l2 < 128 * 1024) l2 = 128 * 1024;
    if (l2 > 8 * 1024 * 1024) l2 = 8 * 1024 * 1024;
    size_t tile = (((size_t)l2 / 2 / 4) / 4096) * 4096;
    if (tile < 4096) tile = 4096;
    if (tile > 65536) tile = 65536;
    return tile;
}

static inline float act_apply(float x, int epilogue) {
    switch (epilogue) {
    case ORC_EPI_RELU: /* src/backend/cpu/mod.rs:3140 */
        return fmaxf(x, 0.0f);
    case ORC_EPI_GELU: { /* src/backend/cpu/mod.rs:3153-3158 */
        float x3 = x * x * x;
        float tanh_arg = 0.7978846f * (x + 0.044715f * x3);
        float t = tanhf(tanh_arg);
        return 0.5f * x * (1.0f + t);
    }
    case ORC_EPI_SILU: /* src/backend/cpu/mod.rs:3171 */
        return x / (1.0f + expf(-x));
    default:
        return x;
    }
}

/* src/backend/cpu/matmul.rs:61-71 */
void orc_epilogue(float *out, size_t len, size_t n, const float *bias, int epilogue) {
    if (bias) {
        for (size_t i = 0; i < len; ++i) out[i] = act_apply(out[i] + bias[i % n], epilogue);
    } else {
        for (size_t i = 0; i < len; ++i) out[i] = act_apply(out[i], epilogue);
    }
}

/* src/backend/cpu/elementwise.rs:105-130 */
void orc_add_broadcast(const float *a, size_t a_len, const float *b, size_t b_len, float *out,
                       size_t out_len) {
    for (size_t i = 0; i < out_len; ++i) out[i] = a[i % a_len] + b[i % b_len];
}

/* src/backend/cpu/microkernels/ops.rs:979-1008 (rms_norm_f32_scalar). */
void orc_rms_norm(const float *in, size_t n, const float *w, size_t w_len, size_t row_size, float eps,
                  float *out) {
    if (row_size == 0) return;
    size_t rows = n / row_size;
    for (size_t r = 0; r < rows; ++r) {
        const float *x = in + r * row_size;
        float sq = 0.0f;
        for (size_t i = 0; i < row_size; ++i) sq += x[i] * x[i];
        float rms = sqrtf(sq / (float)row_size + eps);
        for (size_t i = 0; i < row_size; ++i) {
            float wi = i < w_len ? w[i] : 1.0f;
            out[r * row_size + i] = x[i] / rms * wi;
        }
    }
}

/* src/backend/cpu/microkernels/ops.rs:788-825 (fused_residual_add_layer_norm_f32_scalar). */
void orc_layer_norm(const float *in, const float *residual, size_t n, const float *w, size_t w_len,
                    const float *b, size_t b_len, size_t row_size, float eps, float *out) {
    if (row_size == 0) return;
    size_t rows = n / row_size;
    for (size_t r = 0; r < rows; ++r) {
        size_t s0 = r * row_size;
        float mean = 0.0f, m2 = 0.0f;
        unsigned count = 0;
        for (size_t i = 0; i < row_size; ++i) {
            count += 1;
            float x = residual ? in[s0 + i] + residual[s0 + i] : in[s0 + i];
            float delta = x - mean;
            mean += delta / (float)count;
            float delta2 = x - mean;
            m2 += delta * delta2;
        }
        float var = count > 1 ? m2 / (float)count : 0.0f;
        float inv_std = 1.0f / sqrtf(var + eps);
        for (size_t i = 0; i < row_size; ++i) {
            float x = residual ? in[s0 + i] + residual[s0 + i] : in[s0 + i];
            float wi = i < w_len ? w[i] : 1.0f;
            float bi = i < b_len ? b[i] : 0.0f;
            out[s0 + i] = (x - mean) * inv_std * wi + bi;
        }
    }
}

/* src/backend/cpu/microkernels/ops.rs:1363-1397 (softmax_f32_scalar_strided). */
void orc_softmax(const float *in, size_t n, size_t axis_dim, size_t stride, float *out) {
    if (axis_dim == 0) axis_dim = 1;
    if (stride == 0) stride = 1;
    size_t rows = n / axis_dim;
    for (size_t r = 0; r < rows; ++r) {
        size_t base = (r / stride) * axis_dim * stride + (r % stride);
        float mx = -INFINITY;
        for (size_t i = 0; i < axis_dim; ++i)
            if (in[base + i * stride] > mx) mx = in[base + i * stride];
        float sum = 0.0f;
        for (size_t i = 0; i < axis_dim; ++i) {
            float e = expf(in[base + i * stride] - mx);
            out[base + i * stride] = e;
            sum += e;
        }
        if (sum > 0.0f)
            for (size_t i = 0; i < axis_dim; ++i) out[base + i * stride] /= sum;
    }
}

/* src/backend/cpu/microkernels/gemm.rs:1982-2088 (gemm_batch_packed_simd), reached via
 * gemm_cpu_flat (:1610-1619) from quantized_matmul_dispatch (src/backend/cpu/matmul.rs:214-221).
 * Threads over batch rows only when M >= physical cores (:2019-2035). */
static void gemm_batch_packed(int fmt, const uint32_t *words, size_t N, size_t K,
                              const float *scales, const float *zeros, const float *act,
                              size_t M, float *out) {
    int items = orc_items_per_word(fmt);
    size_t kp = div_ceil(K, (size_t)items);
    size_t kblock = orc_k_block_size();
    int par = (int)M >= orc_physical_cores();
    (void)par;
    for (size_t i = 0; i < M * N; ++i) out[i] = 0.0f;

    float *scratch = (float *)malloc((kblock < K ? kblock : K) * sizeof(float) + 64);
    for (size_t k_start = 0; k_start < K; k_start += kblock) {
        size_t k_end = k_start + kblock < K ? k_start + kblock : K;
        size_t k_len = k_end - k_start;
        size_t p0 = k_start / (size_t)items, p1 = div_ceil(k_end, (size_t)items);
        for (size_t row = 0; row < N; ++row) {
            for (size_t p = p0; p < p1; ++p) {
                float u[8];
                orc_unpack_word(fmt, words[row * kp + p], u);
                size_t base = p * (size_t)items;
                for (int j = 0; j < items; ++j) {
                    size_t idx = base + (size_t)j;
                    if (idx >= k_start && idx < k_end) scratch[idx - k_start] = u[j];
                }
            }
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (par)
#endif
            for (long bi = 0; bi < (long)M; ++bi) {
                float acc = fma_f32_slice(scratch, act + (size_t)bi * K + k_start, k_len);
                out[(size_t)bi * N + row] += acc;
            }
        }
    }
    free(scratch);

    /* affine post-pass, :2048-2087 with mod.rs:284-295: dot*scale + zero*sum(a). */
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (par)
#endif
    for (long bi = 0; bi < (long)M; ++bi) {
        const float *in = act + (size_t)bi * K;
        float input_sum = 0.0f; /* sequential sum (affine_sum_term is called with zero = 1.0) */
        for (size_t i = 0; i < K; ++i) input_sum += in[i];
        for (size_t row = 0; row < N; ++row) {
            float scale = scales[row];
            float zero = zeros ? zeros[row] : 0.0f;
            volatile float a = out[(size_t)bi * N + row] * scale;
            volatile float b = zero * input_sum;
            out[(size_t)bi * N + row] = a + b;
        }
    }
}

/* f32 GEMM C[M,N] = A[M,K] * B where B[k][n] = b[k*ldk + n*ldn]: stands in for crate
 * gemm 0.19 / cblas_sgemm (src/backend/cpu/blas.rs:29-110). */
static void sgemm_strided(const float *a, const float *b, size_t ldk, size_t ldn, float *c,
                          size_t M, size_t K, size_t N) {
    if (ldn == K && ldk == 1) { /* B given as [N,K] rows: dot of contiguous rows */
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
        for (long n = 0; n < (long)N; ++n)
            for (size_t m = 0; m < M; ++m)
                c[m * N + (size_t)n] = fma_f32_slice(a + m * K, b + (size_t)n * K, K);
        return;
    }
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long m = 0; m < (long)M; ++m) {
        float *crow = c + (size_t)m * N;
        for (size_t n = 0; n < N; ++n) crow[n] = 0.0f;
        for (size_t k = 0; k < K; ++k) {
            float av = a[(size_t)m * K + k];
            const float *brow = b + k * ldk;
            for (size_t n = 0; n < N; ++n) crow[n] += av * brow[n * ldn];
        }
    }
}

int orc_qmatmul(int fmt, const uint32_t *words, size_t N, size_t K, const float *scales,
                const float *zeros, const float *codebook16, const float *act, size_t M,
                const float *bias, int epilogue, int mode, float *out) {
    if (!orc_items_per_word(fmt) || !words || !scales || !act || !out) return -1;

    if (mode == ORC_MODE_AS_WRITTEN && bias && epilogue != ORC_EPI_NONE) {
        /* MatMulAdd{Relu,Gelu,Silu} leaves a 3-input MatMul; the quantized dispatch only
         * matches exactly two input slices and returns Ok(()) without writing
         * (src/backend/cpu/matmul.rs:177). */
        return 1;
    }

    if (fmt == ORC_FMT_I4CB) {
        /* src/backend/cpu/matmul.rs:206-212: dequantize, then f32 GEMM. */
        float *wdeq = (float *)malloc((N * K + 1) * sizeof(float));
        orc_dequant(fmt, words, N, K, scales, NULL, codebook16, wdeq);
        if (mode == ORC_MODE_AS_WRITTEN)
            sgemm_strided(act, wdeq, N, 1, out, M, K, N); /* [N,K] buffer read as [K,N] */
        else
            sgemm_strided(act, wdeq, 1, K, out, M, K, N); /* A . Wdeq^T */
        free(wdeq);
    } else {
        gemm_batch_packed(fmt, words, N, K, scales, zeros, act, M, out);
    }

    if (mode == ORC_MODE_AS_WRITTEN) {
        /* bias without activation stays a separate add_f32 (correct); a fused
         * activation is silently dropped (src/backend/cpu/mod.rs:406-425,452-495). */
        if (bias) orc_epilogue(out, M * N, N, bias, ORC_EPI_NONE);
        return 0;
    }
    if (bias || epilogue != ORC_EPI_NONE) orc_epilogue(out, M * N, N, bias, epilogue);
    return 0;
}
