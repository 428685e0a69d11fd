// Row-wise plan instructions that sit between the quantized MatMuls of a transformer block:
// rms_norm, layer_norm (both with an optional residual input) and softmax, one block per row, f32 in
// and out inside the plan's arena.
//   rms_norm: out = x / sqrt(mean(x^2) + eps) * w[i]       (src/backend/cpu/microkernels/ops.rs:979-1008)
//   layer_norm: out = (x - mean) / sqrt(var + eps) * w[i] + b[i], x = main + residual
//                                                          (src/backend/cpu/microkernels/ops.rs:788-825, 1012-1044)
//   softmax : e = exp(in - max); out = e / sum(e) over an axis whose elements are `stride` apart
//                                                          (src/backend/cpu/microkernels/ops.rs:1363-1397)
#include "common.cuh"

namespace fnn {

namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float block_sum(float v, float *s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();   // s_red may still be read from an earlier reduction
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) t += s_red[w];   // same order in every thread
    return t;
}

__device__ __forceinline__ float block_max(float v, float *s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = -INFINITY;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) t = fmaxf(t, s_red[w]);
    return t;
}

// KIND 0: rms_norm, KIND 1: layer_norm (population variance); x = in (+ res when given).
template <int KIND>
__global__ void __launch_bounds__(kRowThreads)
row_norm_kernel(const float *in, const float *res, const float *__restrict__ w, size_t w_len,
                const float *__restrict__ b, size_t b_len, size_t row_size, float eps,
                float *out) {   // out may be in (in-place plan slot)
    __shared__ float s_red[kRowThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const float *x = in + (size_t)blockIdx.x * row_size;
    const float *r = res ? res + (size_t)blockIdx.x * row_size : nullptr;
    float *y = out + (size_t)blockIdx.x * row_size;
    float mean = 0.0f;
    if (KIND == 1) {
        float sm = 0.0f;
        for (size_t i = threadIdx.x; i < row_size; i += kRowThreads) sm += r ? __fadd_rn(x[i], r[i]) : x[i];
        mean = __fdiv_rn(block_sum(sm, s_red), (float)row_size);
    }
    float sq = 0.0f;
    for (size_t i = threadIdx.x; i < row_size; i += kRowThreads) {
        const float v = (r ? __fadd_rn(x[i], r[i]) : x[i]) - mean;
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, s_red);
    const float denom = sqrtf(__fadd_rn(__fdiv_rn(sq, (float)row_size), eps));
    const float inv_std = __fdiv_rn(1.0f, denom);
    for (size_t i = threadIdx.x; i < row_size; i += kRowThreads) {
        const float v = r ? __fadd_rn(x[i], r[i]) : x[i];
        const float wi = i < w_len ? w[i] : 1.0f;
        if (KIND == 0) {
            y[i] = __fmul_rn(__fdiv_rn(v, denom), wi);                      // x / rms * w
        } else {
            const float bi = i < b_len ? b[i] : 0.0f;
            y[i] = __fadd_rn(__fmul_rn(__fmul_rn(v - mean, inv_std), wi), bi);   // (x - mean) * inv_std * w + b
        }
    }
}

__global__ void __launch_bounds__(kRowThreads)
softmax_kernel(const float *in, size_t axis_dim, size_t stride, float *out) {   // out may be in
    __shared__ float s_red[kRowThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    const size_t base = (r / stride) * axis_dim * stride + (r % stride);
    float mx = -INFINITY;
    for (size_t i = threadIdx.x; i < axis_dim; i += kRowThreads) mx = fmaxf(mx, in[base + i * stride]);
    mx = block_max(mx, s_red);
    float sum = 0.0f;
    for (size_t i = threadIdx.x; i < axis_dim; i += kRowThreads) {
        const float e = expf(in[base + i * stride] - mx);
        out[base + i * stride] = e;
        sum += e;
    }
    sum = block_sum(sum, s_red);
    if (sum > 0.0f)
        for (size_t i = threadIdx.x; i < axis_dim; i += kRowThreads)
            out[base + i * stride] = __fdiv_rn(out[base + i * stride], sum);
}

bool span_in(const fnn_cuda_arena *a, size_t off, size_t bytes) {
    return off <= a->bytes && bytes <= a->bytes - off;
}

}  // namespace

}  // namespace fnn

using namespace fnn;

extern "C" {

int fnn_cuda_row_norm(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, int kind, size_t in_offset, size_t len,
                      long long res_offset, long long w_offset, size_t w_len, long long b_offset,
                      size_t b_len, size_t row_size, float eps, size_t out_offset) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "row_norm: null handle");
    FNN_REQUIRE(kind == 0 || kind == 1, FNN_ERR_UNSUPPORTED, "row_norm: unknown kind %d", kind);
    if (len == 0) return FNN_OK;
    FNN_REQUIRE(row_size > 0 && len % row_size == 0, FNN_ERR_DISPATCH,
                "row_norm: %zu elements are not whole rows of %zu", len, row_size);
    FNN_REQUIRE(((in_offset | out_offset) & 3u) == 0 && span_in(arena, in_offset, len * 4) &&
                    span_in(arena, out_offset, len * 4),
                FNN_ERR_DISPATCH, "row_norm: slice outside arena or misaligned");
    auto opt = [&](long long off, size_t n, const float **ptr, size_t *cnt, const char *what) -> int {
        *ptr = nullptr;
        *cnt = 0;
        if (off < 0 || n == 0) return FNN_OK;
        FNN_REQUIRE((off & 3) == 0 && span_in(arena, (size_t)off, n * 4), FNN_ERR_DISPATCH,
                    "row_norm: %s slice outside arena or misaligned", what);
        *ptr = (const float *)(arena->base + off);
        *cnt = n;
        return FNN_OK;
    };
    const float *w, *b, *res;
    size_t wn, bn, rn;
    int rc = opt(w_offset, w_len, &w, &wn, "weight");
    if (rc == FNN_OK) rc = opt(b_offset, b_len, &b, &bn, "bias");
    if (rc == FNN_OK) rc = opt(res_offset, len, &res, &rn, "residual");
    if (rc != FNN_OK) return rc;
    const size_t rows = len / row_size;
    FNN_REQUIRE(rows <= 0x7FFFFFFFu, FNN_ERR_DISPATCH, "row_norm: too many rows (%zu)", rows);
    const float *in = (const float *)(arena->base + in_offset);
    float *out = (float *)(arena->base + out_offset);
    cudaError_t e = kind == 0 ? launch_pdl(row_norm_kernel<0>, (int)rows, kRowThreads, 0, ctx, in, res, w,
                                           wn, b, bn, row_size, eps, out)
                              : launch_pdl(row_norm_kernel<1>, (int)rows, kRowThreads, 0, ctx, in, res, w,
                                           wn, b, bn, row_size, eps, out);
    FNN_CUDA_CHECK(e, FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

int fnn_cuda_rms_norm(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t in_offset, size_t len,
                      long long w_offset, size_t w_len, size_t row_size, float eps, size_t out_offset) {
    return fnn_cuda_row_norm(ctx, arena, 0, in_offset, len, -1, w_offset, w_len, -1, 0, row_size, eps,
                             out_offset);
}

int fnn_cuda_softmax(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t in_offset, size_t len,
                     size_t axis_dim, size_t stride, size_t out_offset) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "softmax: null handle");
    if (len == 0) return FNN_OK;
    if (axis_dim == 0) axis_dim = 1;   // the reference clamps both to at least one
    if (stride == 0) stride = 1;
    FNN_REQUIRE(len % (axis_dim * stride) == 0, FNN_ERR_DISPATCH,
                "softmax: %zu elements are not whole [axis %zu x stride %zu] groups", len, axis_dim, stride);
    FNN_REQUIRE(((in_offset | out_offset) & 3u) == 0 && span_in(arena, in_offset, len * 4) &&
                    span_in(arena, out_offset, len * 4),
                FNN_ERR_DISPATCH, "softmax: slice outside arena or misaligned");
    const size_t rows = len / axis_dim;
    FNN_REQUIRE(rows <= 0x7FFFFFFFu, FNN_ERR_DISPATCH, "softmax: too many rows (%zu)", rows);
    FNN_CUDA_CHECK(launch_pdl(softmax_kernel, (int)rows, kRowThreads, 0, ctx,
                              (const float *)(arena->base + in_offset), axis_dim, stride,
                              (float *)(arena->base + out_offset)),
                   FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

}  // extern "C"
