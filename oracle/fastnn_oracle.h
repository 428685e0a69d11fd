/*
 * CPU oracle for fastnn's quantized-weight MatMul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's Rust algorithm, used by the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark as the
 * checker.  Nothing in the shipped CUDA path links, loads or calls it.
 *
 * The reference is Rust and cannot be compiled where this oracle is built, so the
 * oracle is pinned against the reference's own known-answer tests (ported in
 * tests/test_oracle_kat.py) and against an independent NumPy twin (oracle/np_twin.py)
 * that must agree with it bit for bit.
 *
 * Every function cites the reference file:line (paths relative to the fastnn
 * repository root) whose behaviour it follows.
 */
#ifndef FASTNN_ORACLE_H
#define FASTNN_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Packed weight formats of the path. */
enum {
    ORC_FMT_I8 = 0,   /* I8x4, per-channel asymmetric   (src/dtypes/i8x4.rs)  */
    ORC_FMT_I4 = 1,   /* I4x8, per-channel asymmetric   (src/dtypes/i4x8.rs)  */
    ORC_FMT_F8 = 2,   /* F8x4 e4m3, per-channel symmetric (src/dtypes/f8x4.rs) */
    ORC_FMT_F4 = 3,   /* F4x8 e2m1, per-channel asymmetric (src/dtypes/f4x8.rs) */
    ORC_FMT_I4CB = 4  /* I4x8 words holding codebook indices, per-32 block scales */
};

enum { ORC_EPI_NONE = 0, ORC_EPI_RELU = 1, ORC_EPI_GELU = 2, ORC_EPI_SILU = 3 };

/* ORC_MODE_INTENDED: act((A . Wdeq^T) + bias).
 * ORC_MODE_AS_WRITTEN: what the reference CPU backend does today: the fused
 * bias/activation is dropped on quantized MatMuls (a 3-input MatMul writes
 * nothing at all) and the codebook GEMM reads the [N,K] dequantized buffer as
 * if it were [K,N]. */
enum { ORC_MODE_INTENDED = 0, ORC_MODE_AS_WRITTEN = 1 };

#define ORC_SIMD_MARGIN_WORDS 16
#define ORC_CODEBOOK_BLOCK 32

int orc_items_per_word(int fmt);
size_t orc_words_per_row(int fmt, size_t inner);
/* rows*ceil(inner/ITEMS) + 16 margin words (what as_bytes()/WriteConst carry). */
size_t orc_packed_words(int fmt, size_t rows, size_t inner);

/* scalar codecs */
uint8_t orc_f32_to_e4m3(float v);
float orc_e4m3_to_f32(uint8_t b);
uint8_t orc_f32_to_fp4(float v);
float orc_fp4_to_f32(uint8_t code);
uint32_t orc_pack_word(int fmt, const float *vals);
void orc_unpack_word(int fmt, uint32_t word, float *out);

/* [K,N] row-major -> [N,K] row-major, as the quantization pass does. */
void orc_transpose_kn_to_nk(const float *kn, size_t K, size_t N, float *nk);

/* PackedTensor::from_f32_slice: one (scale, zero) for the whole tensor. */
void orc_from_f32_slice(int fmt, const float *data, size_t rows, size_t inner,
                        float scale, float zero, uint32_t *words);

/* Quantize an [N,K] row-major f32 weight the way the compiler pass does for `fmt`.
 * words: orc_packed_words() u32 (margin zeroed).  scales: N floats (I4CB:
 * N*ceil(K/32)).  zeros: N floats (I8/I4/F4; F8 writes N zeros; I4CB unused).
 * codebook16: 16 floats (I4CB only).  Returns 0, or -1 on a bad format. */
int orc_quantize(int fmt, const float *w_nk, size_t N, size_t K, uint32_t *words,
                 float *scales, float *zeros, float *codebook16);

void orc_kmeans16(const float *values, size_t n, int max_iter, float *centroids16);

/* Dequantize to [N,K] f32: unpack(q)*scale + zero (two roundings). */
int orc_dequant(int fmt, const uint32_t *words, size_t N, size_t K, const float *scales,
                const float *zeros, const float *codebook16, float *out_nk);

/* Quantized MatMul, reference graph path.  act [M,K], out [M,N], both row-major f32.
 * bias may be NULL.  Returns 0 on success; 1 if (mode == AS_WRITTEN) left `out`
 * untouched because the reference would; -1 on bad arguments. */
int orc_qmatmul(int fmt, const uint32_t *words, size_t N, size_t K, const float *scales,
                const float *zeros, const float *codebook16, const float *act, size_t M,
                const float *bias, int epilogue, int mode, float *out);

/* act(x + bias[i % n]) in place over out[0..len). bias may be NULL. */
void orc_epilogue(float *out, size_t len, size_t n, const float *bias, int epilogue);

/* out[i] = a[i % a_len] + b[i % b_len]  (standalone add_f32 broadcast). */
void orc_add_broadcast(const float *a, size_t a_len, const float *b, size_t b_len,
                       float *out, size_t out_len);

/* rms_norm over rows of row_size elements: out = in / sqrt(mean(in^2) + eps) * w[i] (w = 1 beyond
 * w_len).  src/backend/cpu/microkernels/ops.rs:979-1008.  The fused residual variant takes the
 * hidden size (= weight length) as row size (tests/residual_add_norm.rs:327-355); the unfused
 * dispatch arm derives input_len / weight_len instead (src/backend/cpu/mod.rs:5053-5075), which
 * equals the hidden size only for square inputs -- callers choose by passing row_size. */
void orc_rms_norm(const float *in, size_t n, const float *w, size_t w_len, size_t row_size, float eps,
                  float *out);

/* fused_residual_add_layer_norm: x = main + residual per element, Welford mean / population variance
 * per row, out = (x - mean) * (1 / sqrt(var + eps)) * w[i] + b[i]; residual, w, b may be NULL
 * (w = 1, b = 0).  src/backend/cpu/microkernels/ops.rs:788-825. */
void orc_layer_norm(const float *in, const float *residual, size_t n, const float *w, size_t w_len,
                    const float *b, size_t b_len, size_t row_size, float eps, float *out);

/* softmax plan instruction over the axis of size axis_dim whose elements are `stride` apart;
 * n / axis_dim rows.  src/backend/cpu/microkernels/ops.rs:1363-1397. */
void orc_softmax(const float *in, size_t n, size_t axis_dim, size_t stride, float *out);

/* Introspection used by the CPU-baseline report. */
int orc_simd_level(void);      /* 0 scalar, 2 avx2+fma, 5 avx512f */
int orc_physical_cores(void);
size_t orc_k_block_size(void);

#ifdef __cplusplus
}
#endif
#endif
