// Row-wise plan instructions that sit between the quantized MatMuls of a transformer block:
// rms_norm and softmax, one block per row, f32 in and out inside the plan's arena.
//   rms_norm: out = in / sqrt(mean(in^2) + eps) * w[i]     (src/backend/cpu/microkernels/ops.rs:979-1008)
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

__global__ void __launch_bounds__(kRowThreads)
rms_norm_kernel(const float *in, const float *__restrict__ w, size_t w_len, size_t row_size, float eps,
                float *out) {   // out may be in (in-place plan slot)
    __shared__ float s_red[kRowThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const float *x = in + (size_t)blockIdx.x * row_size;
    float *y = out + (size_t)blockIdx.x * row_size;
    float sq = 0.0f;
    for (size_t i = threadIdx.x; i < row_size; i += kRowThreads) sq = fmaf(x[i], x[i], sq);
    sq = block_sum(sq, s_red);
    const float rms = sqrtf(__fadd_rn(__fdiv_rn(sq, (float)row_size), eps));
    for (size_t i = threadIdx.x; i < row_size; i += kRowThreads) {
        const float wi = i < w_len ? w[i] : 1.0f;
        y[i] = __fmul_rn(__fdiv_rn(x[i], rms), wi);
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

int fnn_cuda_rms_norm(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t in_offset, size_t len,
                      long long w_offset, size_t w_len, size_t row_size, float eps, size_t out_offset) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "rms_norm: null handle");
    if (len == 0) return FNN_OK;
    FNN_REQUIRE(row_size > 0 && len % row_size == 0, FNN_ERR_DISPATCH,
                "rms_norm: %zu elements are not whole rows of %zu", len, row_size);
    FNN_REQUIRE(((in_offset | out_offset) & 3u) == 0 && span_in(arena, in_offset, len * 4) &&
                    span_in(arena, out_offset, len * 4),
                FNN_ERR_DISPATCH, "rms_norm: slice outside arena or misaligned");
    const float *w = nullptr;
    if (w_offset >= 0 && w_len > 0) {
        FNN_REQUIRE((w_offset & 3) == 0 && span_in(arena, (size_t)w_offset, w_len * 4), FNN_ERR_DISPATCH,
                    "rms_norm: weight slice outside arena or misaligned");
        w = (const float *)(arena->base + w_offset);
    } else {
        w_len = 0;
    }
    const size_t rows = len / row_size;
    FNN_REQUIRE(rows <= 0x7FFFFFFFu, FNN_ERR_DISPATCH, "rms_norm: too many rows (%zu)", rows);
    FNN_CUDA_CHECK(launch_pdl(rms_norm_kernel, (int)rows, kRowThreads, 0, ctx->stream,
                              (const float *)(arena->base + in_offset), w, w_len, row_size, eps,
                              (float *)(arena->base + out_offset)),
                   FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
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
    FNN_CUDA_CHECK(launch_pdl(softmax_kernel, (int)rows, kRowThreads, 0, ctx->stream,
                              (const float *)(arena->base + in_offset), axis_dim, stride,
                              (float *)(arena->base + out_offset)),
                   FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

}  // extern "C"
