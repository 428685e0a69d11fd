// Device layouts of a quantized weight: upload (with the reference's metadata checks),
// bit-preserving unrepack, and on-device dequantization.
#include "common.cuh"

#include <vector>
#include <string.h>

namespace fnn {

void free_qweight_aux(fnn_cuda_qweight *w) {
    if (w->frag) cudaFree(w->frag);
    if (w->frag_bs) cudaFree(w->frag_bs);
    w->frag = nullptr;
    w->frag_bs = nullptr;
}

// One thread per element of the [N,K] result: unpack(q)*scale + zero, two roundings.
__global__ void dequant_kernel(int fmt, const uint32_t *rows, size_t ld_words, size_t N, size_t K,
                               const float *scales, const float *zeros, const float *codebook,
                               size_t blocks_per_row, float *out) {
    size_t total = N * K;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    const int items = items_per_word(fmt);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        size_t n = idx / K, k = idx % K;
        uint32_t word = rows[n * ld_words + k / items];
        int lane = (int)(k % items);
        float r;
        if (fmt == FNN_FMT_I4CB) {
            uint32_t nib = (word >> (4 * lane)) & 0xFu;
            r = __fmul_rn(scales[n * blocks_per_row + k / kCodebookBlock], codebook[nib]);
        } else {
            float v;
            if (fmt == FNN_FMT_I8)
                v = i8_to_f32(word, lane);
            else if (fmt == FNN_FMT_I4)
                v = i4_to_f32(word, lane);
            else if (fmt == FNN_FMT_F8)
                v = e4m3_to_f32_exact((word >> (8 * lane)) & 0xFFu);
            else
                v = fp4_to_f32_exact((word >> (4 * lane)) & 0xFu);
            float z = zeros ? zeros[n] : 0.0f;
            r = __fadd_rn(__fmul_rn(v, scales[n]), z);
        }
        out[idx] = r;
    }
}

}  // namespace fnn

using namespace fnn;

extern "C" {

// `packed_on_device`: the payload already sits in device memory (a WriteConst slot of the arena).  Its
// rows are then used in place when their stride needs no padding, and copied device-to-device
// otherwise; nothing travels through the host.
static int qweight_build(fnn_cuda_ctx *ctx, int fmt, const void *packed, size_t packed_bytes, bool packed_on_device,
                         size_t N, size_t K, const float *scales, size_t n_scales, const float *zeros,
                         size_t n_zeros, size_t qblock, const float *codebook16, fnn_cuda_qweight **out) {
    clear_error();
    FNN_REQUIRE(ctx && out, FNN_ERR_DISPATCH, "qweight_upload: null argument");
    *out = nullptr;
    FNN_REQUIRE(valid_fmt(fmt), FNN_ERR_UNSUPPORTED, "qweight_upload: unknown format %d", fmt);
    FNN_REQUIRE(N > 0 && K > 0, FNN_ERR_DISPATCH, "qweight_upload: empty weight [%zu,%zu]", N, K);
    const char *kname = (fmt == FNN_FMT_I8)   ? "matmul_i8"
                        : (fmt == FNN_FMT_F8) ? "matmul_f8"
                        : (fmt == FNN_FMT_F4) ? "matmul_f4"
                                              : "matmul_i4";
    // Same checks, in the same order, as packed_tensor_from_meta
    // (src/backend/cpu/matmul.rs:81-152).
    FNN_REQUIRE(scales && n_scales > 0, FNN_ERR_DISPATCH,
                "%s: quantized weight metadata missing scales", kname);
    size_t nz = (n_zeros == 0 || !zeros) ? n_scales : n_zeros;
    FNN_REQUIRE(nz == n_scales, FNN_ERR_DISPATCH,
                "%s: quantized weight metadata length mismatch: %zu scales vs %zu zero_points",
                kname, n_scales, nz);
    bool per_block = qblock > 0 && n_scales > N && n_scales % N == 0;
    bool valid_len = n_scales == 1 || n_scales == N || (N > n_scales && N % n_scales == 0) ||
                     per_block;
    FNN_REQUIRE(valid_len, FNN_ERR_DISPATCH,
                "%s: quantized weight metadata length %zu incompatible with shape [%zu, %zu] "
                "(expected 1, %zu, or a divisor of %zu)",
                kname, n_scales, N, K, N, N);
    const size_t items = (size_t)items_per_word(fmt);
    const size_t wpr = div_ceil(K, items);
    const size_t expected_words = N * wpr;
    FNN_REQUIRE(packed && packed_bytes / 4 >= expected_words, FNN_ERR_DISPATCH,
                "%s: quantized weight payload too short: got %zu packed words for shape "
                "[%zu, %zu], expected at least %zu",
                kname, packed_bytes / 4, N, K, expected_words);
    if (fmt == FNN_FMT_I4CB) {
        FNN_REQUIRE(codebook16 != nullptr, FNN_ERR_DISPATCH, "%s: codebook weight without codebook",
                    kname);
        FNN_REQUIRE(qblock == (size_t)kCodebookBlock, FNN_ERR_UNSUPPORTED,
                    "%s: codebook block size %zu (only %d is produced by the compiler pass)", kname,
                    qblock, kCodebookBlock);
        FNN_REQUIRE(n_scales == N * div_ceil(K, qblock), FNN_ERR_DISPATCH,
                    "%s: expected %zu block scales, got %zu", kname, N * div_ceil(K, qblock),
                    n_scales);
    } else {
        FNN_REQUIRE(!per_block, FNN_ERR_UNSUPPORTED,
                    "%s: per-block scales without a codebook are not produced by the compiler pass",
                    kname);
    }

    FNN_CUDA_CHECK(cudaSetDevice(ctx->device), FNN_ERR_MEMORY);
    fnn_cuda_qweight *w = new fnn_cuda_qweight();
    w->ctx = ctx;
    w->fmt = fmt;
    w->N = N;
    w->K = K;
    w->qblock = (fmt == FNN_FMT_I4CB) ? qblock : 0;
    w->words_per_row = wpr;
    // rows are padded to 16 bytes; FP4 rows to 64 bytes (128 codes), which is what the 4-bit tensor-map
    // type of the tcgen05 kernel addresses
    w->ld_u4 = div_ceil(wpr, 4);
    if (fmt == FNN_FMT_F4) w->ld_u4 = div_ceil(w->ld_u4, 4) * 4;
    w->blocks_per_row = (fmt == FNN_FMT_I4CB) ? div_ceil(K, qblock) : 0;

    auto fail = [&](cudaError_t e, const char *what) {
        int rc = set_error(FNN_ERR_MEMORY, "qweight_upload: %s failed: %s", what,
                           cudaGetErrorString(e));
        fnn_cuda_qweight_free(w);
        return rc;
    };
    cudaError_t e;
    size_t row_bytes = w->ld_u4 * 16;
    if (packed_on_device && row_bytes == wpr * 4 && ((uintptr_t)packed & 31u) == 0) {
        // the arena slot is already [N][row_bytes]: read it where it is (the slot outlives the weight
        // handle: constants persist for the life of the plan's arena)
        w->rows = (uint4 *)packed;
        w->rows_owned = false;
    } else {
        if ((e = cudaMalloc((void **)&w->rows, N * row_bytes)) != cudaSuccess) return fail(e, "cudaMalloc(rows)");
        if (row_bytes != wpr * 4) {
            if ((e = cudaMemset(w->rows, 0, N * row_bytes)) != cudaSuccess) return fail(e, "cudaMemset");
        }
        if ((e = cudaMemcpy2D(w->rows, row_bytes, packed, wpr * 4, wpr * 4, N,
                              packed_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice)) != cudaSuccess)
            return fail(e, "cudaMemcpy2D(rows)");
    }

    // Expand per-tensor / per-group metadata to one entry per row (scale_for_row,
    // src/packed_tensor.rs:439-462), so kernels index by row only.
    std::vector<float> s_host, z_host;
    bool any_zero = false;
    if (fmt == FNN_FMT_I4CB) {
        s_host.assign(scales, scales + n_scales);
        // the tcgen05 kernel dequantizes to fp16 (block scale times centroid): keep it to weights
        // whose block scales and centroids are comfortably inside that range
        for (size_t i = 0; i < n_scales; ++i) {
            float v = scales[i];
            if (!(v == 0.0f || (v >= 1e-4f && v <= 3e4f))) w->fp16_ok = false;
        }
        for (int i = 0; i < 16; ++i)
            if (!(codebook16[i] >= -4.0f && codebook16[i] <= 4.0f)) w->fp16_ok = false;
    } else {
        s_host.resize(N);
        z_host.resize(N);
        size_t group = (n_scales == 1) ? N : N / n_scales;
        for (size_t r = 0; r < N; ++r) {
            size_t gi = (n_scales == 1) ? 0 : r / group;
            s_host[r] = scales[gi];
            z_host[r] = (zeros && n_zeros) ? zeros[gi] : 0.0f;
            any_zero = any_zero || (z_host[r] != 0.0f);
        }
    }
    if ((e = cudaMalloc((void **)&w->scales, s_host.size() * 4)) != cudaSuccess) return fail(e, "cudaMalloc(scales)");
    if ((e = cudaMemcpy(w->scales, s_host.data(), s_host.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
        return fail(e, "cudaMemcpy(scales)");
    w->has_zero = any_zero;
    if (any_zero) {
        if ((e = cudaMalloc((void **)&w->zeros, N * 4)) != cudaSuccess) return fail(e, "cudaMalloc(zeros)");
        if ((e = cudaMemcpy(w->zeros, z_host.data(), N * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
            return fail(e, "cudaMemcpy(zeros)");
    }
    if (fmt == FNN_FMT_I4CB) {
        if ((e = cudaMalloc((void **)&w->codebook, 16 * 4)) != cudaSuccess) return fail(e, "cudaMalloc(codebook)");
        if ((e = cudaMemcpy(w->codebook, codebook16, 16 * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
            return fail(e, "cudaMemcpy(codebook)");
    }
    *out = w;
    return FNN_OK;
}

int fnn_cuda_qweight_upload(fnn_cuda_ctx *ctx, int fmt, const void *packed, size_t packed_bytes,
                            size_t N, size_t K, const float *scales, size_t n_scales,
                            const float *zeros, size_t n_zeros, size_t qblock,
                            const float *codebook16, fnn_cuda_qweight **out) {
    return qweight_build(ctx, fmt, packed, packed_bytes, false, N, K, scales, n_scales, zeros, n_zeros, qblock,
                         codebook16, out);
}

int fnn_cuda_qweight_from_arena(fnn_cuda_ctx *ctx, int fmt, fnn_cuda_arena *arena, size_t offset,
                                size_t packed_bytes, size_t N, size_t K, const float *scales, size_t n_scales,
                                const float *zeros, size_t n_zeros, size_t qblock, const float *codebook16,
                                fnn_cuda_qweight **out) {
    clear_error();
    FNN_REQUIRE(ctx && arena && out, FNN_ERR_DISPATCH, "qweight_from_arena: null argument");
    FNN_REQUIRE((offset & 15u) == 0 && offset <= arena->bytes && packed_bytes <= arena->bytes - offset,
                FNN_ERR_DISPATCH, "qweight_from_arena: weight slice [%zu, +%zu) outside arena of %zu bytes or "
                "not 16-byte aligned", offset, packed_bytes, arena->bytes);
    // the WriteConst that filled the slot was enqueued on this stream: it must have landed before a
    // copy on another stream (cudaMemcpy2D) or the first kernel reads it
    FNN_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), FNN_ERR_MEMORY);
    return qweight_build(ctx, fmt, arena->base + offset, packed_bytes, true, N, K, scales, n_scales, zeros,
                         n_zeros, qblock, codebook16, out);
}

int fnn_cuda_qweight_free(fnn_cuda_qweight *w) {
    if (!w) return FNN_OK;
    cudaSetDevice(w->ctx->device);
    cudaStreamSynchronize(w->ctx->stream);
    free_qweight_aux(w);
    if (w->rows && w->rows_owned) cudaFree(w->rows);
    if (w->scales) cudaFree(w->scales);
    if (w->zeros) cudaFree(w->zeros);
    if (w->codebook) cudaFree(w->codebook);
    delete w;
    return FNN_OK;
}

size_t fnn_cuda_qweight_packed_bytes(fnn_cuda_qweight *w) {
    return w ? (w->N * w->words_per_row + kMarginWords) * 4 : 0;
}

int fnn_cuda_qweight_unrepack(fnn_cuda_qweight *w, void *host_out, size_t bytes) {
    clear_error();
    FNN_REQUIRE(w && host_out, FNN_ERR_DISPATCH, "qweight_unrepack: null argument");
    size_t need = fnn_cuda_qweight_packed_bytes(w);
    FNN_REQUIRE(bytes >= need, FNN_ERR_MEMORY, "qweight_unrepack: need %zu bytes, got %zu", need,
                bytes);
    FNN_CUDA_CHECK(cudaSetDevice(w->ctx->device), FNN_ERR_MEMORY);
    FNN_CUDA_CHECK(cudaStreamSynchronize(w->ctx->stream), FNN_ERR_MEMORY);
    FNN_CUDA_CHECK(cudaMemcpy2D(host_out, w->words_per_row * 4, w->rows, w->ld_u4 * 16,
                                w->words_per_row * 4, w->N, cudaMemcpyDeviceToHost),
                   FNN_ERR_MEMORY);
    memset((uint8_t *)host_out + w->N * w->words_per_row * 4, 0, kMarginWords * 4);
    return FNN_OK;
}

int fnn_cuda_qweight_dequant(fnn_cuda_qweight *w, fnn_cuda_arena *arena, size_t out_offset) {
    clear_error();
    FNN_REQUIRE(w && arena, FNN_ERR_DISPATCH, "qweight_dequant: null argument");
    size_t bytes = w->N * w->K * sizeof(float);
    FNN_REQUIRE((out_offset & 3u) == 0 && out_offset <= arena->bytes &&
                    bytes <= arena->bytes - out_offset,
                FNN_ERR_DISPATCH, "qweight_dequant: output slice outside arena");
    fnn_cuda_ctx *ctx = w->ctx;
    size_t total = w->N * w->K;
    size_t blocks = div_ceil(total, 256);
    size_t cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    dequant_kernel<<<(int)blocks, 256, 0, arena->ctx->stream>>>(
        w->fmt, (const uint32_t *)w->rows, w->ld_u4 * 4, w->N, w->K, w->scales, w->zeros,
        w->codebook, w->blocks_per_row, (float *)(arena->base + out_offset));
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    arena->ctx->launches++;
    return FNN_OK;
}

}  // extern "C"
