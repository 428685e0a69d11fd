// Context, arena, plan-instruction kernels, replay and timing entry points of the C ABI.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

namespace fnn {

static thread_local char g_err[1024] = "";

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { g_err[0] = 0; }

int ensure_scratch(fnn_cuda_ctx *ctx, size_t bytes) {
    if (ctx->scratch_bytes >= bytes) return FNN_OK;
    FNN_REQUIRE(!ctx->capturing, FNN_ERR_MEMORY,
                "scratch buffer must grow (%zu -> %zu bytes) during graph capture; run the "
                "plan once before capturing it",
                ctx->scratch_bytes, bytes);
    // A captured graph may hold the old buffer's address (kernel arguments, memset nodes, tensor
    // maps), so an outgrown buffer is never freed while the context lives: it is retired and
    // released by fnn_cuda_ctx_destroy.
    size_t want = bytes + (bytes >> 2);
    void *grown = nullptr;
    FNN_CUDA_CHECK(cudaMalloc(&grown, want), FNN_ERR_MEMORY);
    if (ctx->scratch) ctx->retired_scratch.push_back(ctx->scratch);
    ctx->scratch = grown;
    ctx->scratch_bytes = want;
    return FNN_OK;
}

// Rows of `width` bytes from src (pitch spitch) to dst (pitch dpitch).  VEC bytes per thread and
// access: 16 when every pointer, pitch and the width are multiples of 16, else 4, else 1.  A kernel
// rather than a copy-engine node: inside a captured plan a memcpy node cannot overlap its
// neighbours the way programmatic dependent launches do, and costs several microseconds.
template <typename V>
__global__ void copy2d_kernel(unsigned char *dst, size_t dpitch, const unsigned char *src, size_t spitch,
                              size_t width_v, size_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = width_v * rows, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / width_v, c = i - r * width_v;
        reinterpret_cast<V *>(dst + r * dpitch)[c] = reinterpret_cast<const V *>(src + r * spitch)[c];
    }
}

// The common case of the element-wise instruction: operands as long as the output (no broadcast),
// 16-byte aligned, four elements per thread and access.
__global__ void elementwise_vec_kernel(int op, const float4 *a, const float4 *b, float4 *out, size_t n4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int base = op & 0xFF, act = op >> 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 x = a[i];
        float4 y = x;
        if (base == FNN_EW_ADD || base == FNN_EW_MUL || base == FNN_EW_SUB) y = b[i];
        float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w}, r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            switch (base) {
            case FNN_EW_ADD:
                r[j] = __fadd_rn(xs[j], ys[j]);
                break;
            case FNN_EW_MUL:
                r[j] = __fmul_rn(xs[j], ys[j]);
                break;
            case FNN_EW_SUB:
                r[j] = __fsub_rn(xs[j], ys[j]);
                break;
            case FNN_EW_RELU:
                r[j] = apply_act(xs[j], FNN_EPI_RELU);
                break;
            case FNN_EW_GELU:
                r[j] = apply_act(xs[j], FNN_EPI_GELU);
                break;
            default:
                r[j] = apply_act(xs[j], FNN_EPI_SILU);
                break;
            }
            if (act) r[j] = apply_act(r[j], act);
        }
        out[i] = make_float4(r[0], r[1], r[2], r[3]);
    }
}

// out[i] = op(a[i % a_len], b[i % b_len]); unary ops read a only.
__global__ void elementwise_kernel(int op, const float *a, size_t a_len, const float *b,
                                   size_t b_len, float *out, size_t out_len) {
    // launched as a programmatic dependent: nothing here is independent of the kernel before it
    pdl_launch_dependents();
    pdl_wait();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < out_len; i += stride) {
        float x = a[i % a_len];
        float r;
        switch (op & 0xFF) {
        case FNN_EW_ADD:
            r = __fadd_rn(x, b[i % b_len]);
            break;
        case FNN_EW_MUL:
            r = __fmul_rn(x, b[i % b_len]);
            break;
        case FNN_EW_SUB:
            r = __fsub_rn(x, b[i % b_len]);
            break;
        case FNN_EW_RELU:
            r = apply_act(x, FNN_EPI_RELU);
            break;
        case FNN_EW_GELU:
            r = apply_act(x, FNN_EPI_GELU);
            break;
        case FNN_EW_SILU:
            r = apply_act(x, FNN_EPI_SILU);
            break;
        default:
            r = x;
        }
        out[i] = apply_act(r, op >> 8);
    }
}

__global__ void fill_kernel(float *dst, size_t n, float value) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = value;
}

__global__ void flush_kernel(uint4 *buf, size_t n, uint32_t v) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        buf[i] = make_uint4(v, v, v, v);
}

static int grid_for(const fnn_cuda_ctx *ctx, size_t work_items, int block) {
    size_t blocks = div_ceil(work_items, (size_t)block);
    size_t cap = (size_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

static bool span_ok(const fnn_cuda_arena *a, size_t off, size_t bytes) {
    return off <= a->bytes && bytes <= a->bytes - off;
}

}  // namespace fnn

using namespace fnn;

extern "C" {

const char *fnn_cuda_last_error(void) { return g_err; }

static int ctx_create(int device, bool use_given_stream, void *stream, fnn_cuda_ctx **out) {
    clear_error();
    FNN_REQUIRE(out != nullptr, FNN_ERR_DISPATCH, "ctx_create: out is null");
    *out = nullptr;
    int count = 0;
    FNN_CUDA_CHECK(cudaGetDeviceCount(&count), FNN_ERR_UNSUPPORTED);
    FNN_REQUIRE(device >= 0 && device < count, FNN_ERR_UNSUPPORTED,
                "ctx_create: device %d not present (%d CUDA devices)", device, count);
    FNN_CUDA_CHECK(cudaSetDevice(device), FNN_ERR_UNSUPPORTED);
    cudaDeviceProp prop;
    FNN_CUDA_CHECK(cudaGetDeviceProperties(&prop, device), FNN_ERR_UNSUPPORTED);
    FNN_REQUIRE(prop.major == 10, FNN_ERR_UNSUPPORTED,
                "ctx_create: this library is built for sm_100a only; device %d is sm_%d%d",
                device, prop.major, prop.minor);
    fnn_cuda_ctx *ctx = new fnn_cuda_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->total_mem = prop.totalGlobalMem;
    if (use_given_stream) {
        ctx->stream = (cudaStream_t)stream;   // a null handle is the legacy default stream
        ctx->owns_stream = false;
    } else {
        cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            delete ctx;
            return set_error(FNN_ERR_MEMORY, "cudaStreamCreate failed: %s", cudaGetErrorString(e));
        }
        ctx->owns_stream = true;
    }
    cudaError_t e = cudaMalloc((void **)&ctx->err_flag, 2 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->err_flag, 0, 2 * sizeof(int));
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&ctx->err_host, sizeof(int), cudaHostAllocDefault);
    if (e == cudaSuccess) *ctx->err_host = 0;
    if (e == cudaSuccess) e = cudaMalloc((void **)&ctx->sk_flags, 2048 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctx->sk_flags, 0, 2048 * sizeof(unsigned));
    if (e != cudaSuccess) {
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return set_error(FNN_ERR_MEMORY, "ctx_create: %s", cudaGetErrorString(e));
    }
    *out = ctx;
    return FNN_OK;
}

int fnn_cuda_ctx_create(int device, fnn_cuda_ctx **out) { return ctx_create(device, false, nullptr, out); }

int fnn_cuda_ctx_create_on_stream(int device, void *stream, fnn_cuda_ctx **out) {
    return ctx_create(device, true, stream, out);
}

void *fnn_cuda_ctx_stream(fnn_cuda_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int fnn_cuda_ctx_set_overlap(fnn_cuda_ctx *ctx, int enabled) {
    FNN_REQUIRE(ctx, FNN_ERR_DISPATCH, "ctx_set_overlap: null context");
    ctx->overlap_launches = enabled != 0;
    return FNN_OK;
}

int fnn_cuda_ctx_destroy(fnn_cuda_ctx *ctx) {
    if (!ctx) return FNN_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 64; ++i) {
        if (ctx->ev_start[i]) cudaEventDestroy(ctx->ev_start[i]);
        if (ctx->ev_stop[i]) cudaEventDestroy(ctx->ev_stop[i]);
    }
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (void *p : ctx->retired_scratch) cudaFree(p);
    if (ctx->err_flag) cudaFree(ctx->err_flag);
    if (ctx->err_host) cudaFreeHost(ctx->err_host);
    if (ctx->sk_flags) cudaFree(ctx->sk_flags);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return FNN_OK;
}

int fnn_cuda_sync(fnn_cuda_ctx *ctx) {
    FNN_REQUIRE(ctx, FNN_ERR_DISPATCH, "sync: null context");
    // the device error flag travels to pinned host memory at the tail of the stream: one wait, not a
    // stream synchronize followed by a blocking 4-byte copy (which cost about 8 us per step of the
    // host-to-host path)
    FNN_CUDA_CHECK(cudaMemcpyAsync(ctx->err_host, ctx->err_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), FNN_ERR_DISPATCH);
    const int flag = *ctx->err_host;
    if (flag != 0) {
        cudaMemset(ctx->err_flag, 0, sizeof(int));
        *ctx->err_host = 0;
        return set_error(FNN_ERR_DISPATCH,
                         "a kernel gave up on a bounded wait (device error flag 0x%x)", flag);
    }
    return FNN_OK;
}

int fnn_cuda_launch_count(fnn_cuda_ctx *ctx, uint64_t *out) {
    FNN_REQUIRE(ctx && out, FNN_ERR_DISPATCH, "launch_count: null argument");
    *out = ctx->launches;
    return FNN_OK;
}

int fnn_cuda_device_info(fnn_cuda_ctx *ctx, int *sm_count, int *cc_major, int *cc_minor,
                         size_t *total_mem) {
    FNN_REQUIRE(ctx, FNN_ERR_DISPATCH, "device_info: null context");
    if (sm_count) *sm_count = ctx->sm_count;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    if (total_mem) *total_mem = ctx->total_mem;
    return FNN_OK;
}

// ---- arena ---------------------------------------------------------------------------

int fnn_cuda_arena_alloc(fnn_cuda_ctx *ctx, size_t bytes, fnn_cuda_arena **out) {
    clear_error();
    FNN_REQUIRE(ctx && out, FNN_ERR_MEMORY, "arena_alloc: null argument");
    *out = nullptr;
    FNN_CUDA_CHECK(cudaSetDevice(ctx->device), FNN_ERR_MEMORY);
    size_t padded = div_ceil(bytes > 0 ? bytes : 1, 256) * 256;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, padded);
    if (e != cudaSuccess)
        return set_error(FNN_ERR_MEMORY, "arena_alloc: cudaMalloc(%zu) failed: %s", padded,
                         cudaGetErrorString(e));
    e = cudaMemsetAsync(p, 0, padded, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return set_error(FNN_ERR_MEMORY, "arena_alloc: memset failed: %s", cudaGetErrorString(e));
    }
    fnn_cuda_arena *a = new fnn_cuda_arena();
    a->ctx = ctx;
    a->base = (uint8_t *)p;
    a->bytes = bytes;
    a->owned = true;
    *out = a;
    return FNN_OK;
}

int fnn_cuda_arena_wrap(fnn_cuda_ctx *ctx, void *device_ptr, size_t bytes, fnn_cuda_arena **out) {
    clear_error();
    FNN_REQUIRE(ctx && out && device_ptr, FNN_ERR_MEMORY, "arena_wrap: null argument");
    FNN_REQUIRE(((uintptr_t)device_ptr & 255u) == 0, FNN_ERR_MEMORY,
                "arena_wrap: device pointer must be 256-byte aligned");
    fnn_cuda_arena *a = new fnn_cuda_arena();
    a->ctx = ctx;
    a->base = (uint8_t *)device_ptr;
    a->bytes = bytes;
    a->owned = false;
    *out = a;
    return FNN_OK;
}

int fnn_cuda_arena_free(fnn_cuda_arena *a) {
    if (!a) return FNN_OK;
    if (a->owned && a->base) {
        cudaSetDevice(a->ctx->device);
        cudaStreamSynchronize(a->ctx->stream);
        cudaFree(a->base);
    }
    delete a;
    return FNN_OK;
}

static int arena_copy(fnn_cuda_arena *a, size_t offset, void *host, size_t bytes, bool to_device,
                      bool async) {
    clear_error();
    FNN_REQUIRE(a && (host || bytes == 0), FNN_ERR_MEMORY, "arena copy: null argument");
    int rc = FNN_OK;
    if (!span_ok(a, offset, bytes)) {
        // Clamp like CpuBuffer does (src/backend/cpu/mod.rs:7228-7238) but report it.
        size_t avail = offset < a->bytes ? a->bytes - offset : 0;
        rc = set_error(FNN_ERR_MEMORY, "arena %s out of range: offset %zu + %zu > %zu",
                       to_device ? "write" : "read", offset, bytes, a->bytes);
        bytes = bytes < avail ? bytes : avail;
    }
    if (bytes == 0) return rc;
    cudaStream_t s = a->ctx->stream;
    cudaError_t e;
    if (to_device)
        e = cudaMemcpyAsync(a->base + offset, host, bytes, cudaMemcpyHostToDevice, s);
    else
        e = cudaMemcpyAsync(host, a->base + offset, bytes, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess)
        return set_error(FNN_ERR_MEMORY, "arena copy failed: %s", cudaGetErrorString(e));
    if (!async && !a->ctx->capturing) {
        e = cudaStreamSynchronize(s);
        if (e != cudaSuccess)
            return set_error(FNN_ERR_MEMORY, "arena copy sync failed: %s", cudaGetErrorString(e));
    }
    return rc;
}

int fnn_cuda_arena_write(fnn_cuda_arena *a, size_t offset, const void *host, size_t bytes) {
    return arena_copy(a, offset, (void *)host, bytes, true, false);
}
int fnn_cuda_arena_read(fnn_cuda_arena *a, size_t offset, void *host, size_t bytes) {
    return arena_copy(a, offset, host, bytes, false, false);
}
int fnn_cuda_arena_write_async(fnn_cuda_arena *a, size_t offset, const void *pinned, size_t bytes) {
    return arena_copy(a, offset, (void *)pinned, bytes, true, true);
}
int fnn_cuda_arena_read_async(fnn_cuda_arena *a, size_t offset, void *pinned, size_t bytes) {
    return arena_copy(a, offset, pinned, bytes, false, true);
}
void *fnn_cuda_arena_device_ptr(fnn_cuda_arena *a) { return a ? a->base : nullptr; }
size_t fnn_cuda_arena_size(fnn_cuda_arena *a) { return a ? a->bytes : 0; }

int fnn_cuda_host_alloc(size_t bytes, void **out) {
    clear_error();
    FNN_REQUIRE(out, FNN_ERR_MEMORY, "host_alloc: out is null");
    FNN_CUDA_CHECK(cudaHostAlloc(out, bytes > 0 ? bytes : 1, cudaHostAllocDefault), FNN_ERR_MEMORY);
    return FNN_OK;
}
int fnn_cuda_host_free(void *ptr) {
    if (ptr) cudaFreeHost(ptr);
    return FNN_OK;
}

// ---- hot path dispatch --------------------------------------------------------------------

static int qmatmul_impl(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a, float *out,
                        const float *bias, size_t M, int epilogue, int path) {
    FNN_REQUIRE(ctx && w, FNN_ERR_DISPATCH, "qmatmul: null handle");
    FNN_REQUIRE(w->ctx->device == ctx->device, FNN_ERR_DISPATCH,
                "qmatmul: weight lives on device %d, context on %d", w->ctx->device, ctx->device);
    FNN_REQUIRE(epilogue >= FNN_EPI_NONE && epilogue <= FNN_EPI_SILU, FNN_ERR_DISPATCH,
                "qmatmul: unknown epilogue %d", epilogue);
    if (M == 0 || w->N == 0) return FNN_OK;
    QmmArgs args{w, a, out, bias, M, epilogue};
    switch (path) {
    case FNN_PATH_AUTO:
        // Measured crossover.  The 8-bit fragment kernel wins up to 8 batch rows (beyond that it runs
        // 16-row groups at twice the time and the tcgen05 sequence, about 14.5 us at K=4096 N=11008, is
        // ahead); FP8, which rides the fp16 fragment kernel, up to 4.  Layers with tiles for at most a
        // quarter of the SMs keep the fragment kernels longer (12 and 8 rows): there the tcgen05
        // kernel is bound by its fixed cost of about 18 us.
        {
            const bool frag_ok = qmm_mma_supported(w, M) && auto_uses_mma(w);
            const size_t tiles128 = div_ceil(w->N, (size_t)128);
            const bool narrow = tiles128 * 4 <= (size_t)ctx->sm_count;
            const size_t frag_max =
                !frag_ok ? 0 : (w->fmt == FNN_FMT_F8 ? (narrow ? 8 : 4) : (narrow ? 12 : 8));
            if (qmm_tc_supported(w, M) && M > frag_max && M > 4) return launch_qmm_tc(ctx, args);
        }
        // tiny layers stay on the row kernel: a 16-row x 128-k fragment tile would be mostly padding
        if (qmm_mma_supported(w, M) && auto_uses_mma(w)) return launch_qmm_mma(ctx, args);
        return launch_qmm_rows(ctx, args);
    case FNN_PATH_ROWS:
        return launch_qmm_rows(ctx, args);
    case FNN_PATH_MMA:
        FNN_REQUIRE(qmm_mma_supported(w, M), FNN_ERR_UNSUPPORTED,
                    "qmatmul: tensor-core skinny path does not cover fmt=%d N=%zu K=%zu M=%zu",
                    w->fmt, w->N, w->K, M);
        return launch_qmm_mma(ctx, args);
    case FNN_PATH_TC:
        FNN_REQUIRE(qmm_tc_supported(w, M), FNN_ERR_UNSUPPORTED,
                    "qmatmul: tcgen05 path does not cover fmt=%d N=%zu K=%zu M=%zu", w->fmt,
                    w->N, w->K, M);
        return launch_qmm_tc(ctx, args);
    default:
        return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: unknown path %d", path);
    }
}

int fnn_cuda_qmatmul(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, fnn_cuda_arena *arena,
                     size_t a_offset, size_t out_offset, int64_t bias_offset, size_t M,
                     int epilogue, int path) {
    clear_error();
    FNN_REQUIRE(ctx && w && arena, FNN_ERR_DISPATCH, "qmatmul: null handle");
    FNN_REQUIRE((a_offset & 15u) == 0 && (out_offset & 15u) == 0, FNN_ERR_DISPATCH,
                "qmatmul: slot offsets must be 16-byte aligned (planner aligns to 64)");
    FNN_REQUIRE(span_ok(arena, a_offset, M * w->K * sizeof(float)), FNN_ERR_DISPATCH,
                "qmatmul: activation slice [%zu, +%zu) outside arena of %zu bytes", a_offset,
                M * w->K * sizeof(float), arena->bytes);
    FNN_REQUIRE(span_ok(arena, out_offset, M * w->N * sizeof(float)), FNN_ERR_DISPATCH,
                "qmatmul: output slice [%zu, +%zu) outside arena of %zu bytes", out_offset,
                M * w->N * sizeof(float), arena->bytes);
    const float *bias = nullptr;
    if (bias_offset >= 0) {
        FNN_REQUIRE(((size_t)bias_offset & 3u) == 0 &&
                        span_ok(arena, (size_t)bias_offset, w->N * sizeof(float)),
                    FNN_ERR_DISPATCH, "qmatmul: bias slice outside arena");
        bias = (const float *)(arena->base + bias_offset);
    }
    return qmatmul_impl(ctx, w, (const float *)(arena->base + a_offset),
                        (float *)(arena->base + out_offset), bias, M, epilogue, path);
}

int fnn_cuda_qmatmul_ptr(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                         float *out_dev, const float *bias_dev, size_t M, int epilogue,
                         int path) {
    clear_error();
    FNN_REQUIRE(a_dev && out_dev, FNN_ERR_DISPATCH, "qmatmul_ptr: null device pointer");
    FNN_REQUIRE(((uintptr_t)a_dev & 15u) == 0 && ((uintptr_t)out_dev & 15u) == 0,
                FNN_ERR_DISPATCH, "qmatmul_ptr: pointers must be 16-byte aligned");
    return qmatmul_impl(ctx, w, a_dev, out_dev, bias_dev, M, epilogue, path);
}

const char *fnn_cuda_last_path(fnn_cuda_ctx *ctx) { return ctx ? ctx->last_path : ""; }

// ---- column-sharded layers: peer memory and the fused GEMV + all-gather ----------------------

int fnn_cuda_ipc_export(fnn_cuda_arena *arena, void *handle64) {
    clear_error();
    FNN_REQUIRE(arena && handle64 && arena->owned, FNN_ERR_MEMORY,
                "ipc_export: needs an arena allocated by fnn_cuda_arena_alloc");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    FNN_CUDA_CHECK(cudaSetDevice(arena->ctx->device), FNN_ERR_MEMORY);
    FNN_CUDA_CHECK(cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle64, arena->base), FNN_ERR_MEMORY);
    return FNN_OK;
}

int fnn_cuda_ipc_open(fnn_cuda_ctx *ctx, const void *handle64, void **device_ptr) {
    clear_error();
    FNN_REQUIRE(ctx && handle64 && device_ptr, FNN_ERR_MEMORY, "ipc_open: null argument");
    FNN_CUDA_CHECK(cudaSetDevice(ctx->device), FNN_ERR_MEMORY);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    FNN_CUDA_CHECK(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess), FNN_ERR_MEMORY);
    return FNN_OK;
}

int fnn_cuda_ipc_close(fnn_cuda_ctx *ctx, void *device_ptr) {
    if (!ctx || !device_ptr) return FNN_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    FNN_CUDA_CHECK(cudaIpcCloseMemHandle(device_ptr), FNN_ERR_MEMORY);
    return FNN_OK;
}

int fnn_cuda_qmatmul_gather(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                            const float *bias_dev, size_t M, int epilogue, int rank, int world,
                            void *const *peer_bases, size_t gather_offset, size_t counter_offset,
                            size_t n_stride) {
    clear_error();
    FNN_REQUIRE(ctx && w && a_dev && peer_bases, FNN_ERR_DISPATCH, "qmatmul_gather: null argument");
    FNN_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, FNN_ERR_DISPATCH,
                "qmatmul_gather: rank %d of %d (at most 8 ranks of one node)", rank, world);
    FNN_REQUIRE(n_stride >= w->N && (gather_offset & 15u) == 0 && (counter_offset & 15u) == 0,
                FNN_ERR_DISPATCH, "qmatmul_gather: n_stride %zu < shard width %zu, or misaligned offsets",
                n_stride, w->N);
    FNN_REQUIRE(epilogue >= FNN_EPI_NONE && epilogue <= FNN_EPI_SILU, FNN_ERR_DISPATCH,
                "qmatmul_gather: unknown epilogue %d", epilogue);
    FNN_REQUIRE(M >= 1 && M <= (size_t)kGatherRows && qmm_mma_supported(w, M), FNN_ERR_UNSUPPORTED,
                "qmatmul_gather: the fused gather serves 1..%d batch rows on the fragment kernels "
                "(fmt=%d, M=%zu, K=%zu); gather other cases with a collective", kGatherRows, w->fmt, M, w->K);
    GatherArgs g{};
    for (int r = 0; r < world; ++r) {
        FNN_REQUIRE(peer_bases[r] != nullptr, FNN_ERR_DISPATCH, "qmatmul_gather: peer %d has no buffer", r);
        g.peer_words[r] = (unsigned long long *)((uint8_t *)peer_bases[r] + gather_offset);
    }
    uint8_t *mine = (uint8_t *)peer_bases[rank] + counter_offset;
    g.step_ctr = (unsigned *)mine;   // u32 steps | i32 blocks done | i32 rows of the last step
    g.done_ctr = (int *)(mine + 4);
    g.last_m = (int *)(mine + 8);
    g.err_flag = ctx->err_flag;
    g.rank = rank;
    g.world = world;
    g.n_stride = (int)n_stride;
    int rc = prepare_qmm_mma(ctx, w);
    if (rc != FNN_OK) return rc;
    QmmArgs args{w, a_dev, nullptr, bias_dev, M, epilogue, &g};
    return launch_qmm_mma(ctx, args);   // 8-bit operand kernel for I8 / I4 / FP4, fp16 kernel for the rest
}

int fnn_cuda_qmatmul_allgather(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev, const float *bias_dev,
                               size_t M, int epilogue, int rank, int world, void *const *peer_bases,
                               size_t out_offset, size_t counter_offset, size_t n_total, size_t col0) {
    clear_error();
    FNN_REQUIRE(ctx && w && a_dev && peer_bases, FNN_ERR_DISPATCH, "qmatmul_allgather: null argument");
    FNN_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, FNN_ERR_DISPATCH,
                "qmatmul_allgather: rank %d of %d (at most 8 ranks of one node)", rank, world);
    FNN_REQUIRE(col0 + w->N <= n_total && n_total < (1u << 30) && (out_offset & 15u) == 0 &&
                    (counter_offset & 7u) == 0 && ((uintptr_t)a_dev & 15u) == 0,
                FNN_ERR_DISPATCH, "qmatmul_allgather: columns [%zu, +%zu) outside a row of %zu, or misaligned offsets",
                col0, w->N, n_total);
    FNN_REQUIRE(epilogue >= FNN_EPI_NONE && epilogue <= FNN_EPI_SILU, FNN_ERR_DISPATCH,
                "qmatmul_allgather: unknown epilogue %d", epilogue);
    FNN_REQUIRE(M >= 1 && qmm_tc_supported(w, M), FNN_ERR_UNSUPPORTED,
                "qmatmul_allgather: the tcgen05 kernel does not cover fmt=%d K=%zu", w->fmt, w->K);
    AllGatherArgs g{};
    for (int r = 0; r < world; ++r) {
        FNN_REQUIRE(peer_bases[r] != nullptr, FNN_ERR_DISPATCH, "qmatmul_allgather: peer %d has no buffer", r);
        g.peer_out[r] = (float *)((uint8_t *)peer_bases[r] + out_offset);
        g.peer_arrive[r] = (unsigned *)((uint8_t *)peer_bases[r] + counter_offset);
    }
    g.ticket = ctx->err_flag + 1;
    g.rank = rank;
    g.world = world;
    g.n_total = (int)n_total;
    g.col0 = (int)col0;
    QmmArgs args{w, a_dev, nullptr, bias_dev, M, epilogue, nullptr, &g};
    return launch_qmm_tc(ctx, args);
}

int fnn_cuda_gather_wait(fnn_cuda_ctx *ctx, void *my_base, size_t gather_offset, size_t counter_offset,
                         int world, size_t n_stride, void *out_dev) {
    clear_error();
    FNN_REQUIRE(ctx && my_base && world >= 1 && world <= 8 && n_stride > 0, FNN_ERR_DISPATCH,
                "gather_wait: bad argument");
    FNN_REQUIRE(gather_offset % 8 == 0 && counter_offset % 4 == 0, FNN_ERR_DISPATCH,
                "gather_wait: offsets must be aligned (gather 8, counters 4)");
    return launch_gather_wait(ctx, (const unsigned long long *)((uint8_t *)my_base + gather_offset),
                              (const unsigned *)((uint8_t *)my_base + counter_offset), world, (int)n_stride,
                              (float *)out_dev);
}

int fnn_cuda_qweight_prepare(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, int path) {
    clear_error();
    FNN_REQUIRE(ctx && w, FNN_ERR_DISPATCH, "qweight_prepare: null handle");
    FNN_CUDA_CHECK(cudaSetDevice(ctx->device), FNN_ERR_MEMORY);
    int rc = FNN_OK;
    if (path == FNN_PATH_MMA || (path == FNN_PATH_AUTO && auto_uses_mma(w) && qmm_mma_supported(w, 1)))
        rc = prepare_qmm_mma(ctx, w);
    if (rc == FNN_OK && (path == FNN_PATH_TC || (path == FNN_PATH_AUTO && qmm_tc_supported(w, 128))))
        rc = prepare_qmm_tc(ctx, w);
    return rc;
}

// ---- remaining plan instructions --------------------------------------------------------------

int fnn_cuda_elementwise(fnn_cuda_ctx *ctx, int op, fnn_cuda_arena *arena, size_t a_offset,
                         size_t a_len, size_t b_offset, size_t b_len, size_t out_offset,
                         size_t out_len) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "elementwise: null handle");
    const int base = op & 0xFF, act = op >> 8;
    bool binary = (base == FNN_EW_ADD || base == FNN_EW_MUL || base == FNN_EW_SUB);
    bool unary = (base == FNN_EW_RELU || base == FNN_EW_GELU || base == FNN_EW_SILU);
    FNN_REQUIRE((binary || unary) && act >= FNN_EPI_NONE && act <= FNN_EPI_SILU && (binary || act == 0),
                FNN_ERR_UNSUPPORTED, "elementwise: unknown op 0x%x", op);
    if (out_len == 0) return FNN_OK;
    FNN_REQUIRE(a_len > 0 && (!binary || b_len > 0), FNN_ERR_DISPATCH,
                "elementwise: empty operand");
    FNN_REQUIRE(((a_offset | b_offset | out_offset) & 3u) == 0, FNN_ERR_DISPATCH,
                "elementwise: offsets must be 4-byte aligned");
    FNN_REQUIRE(span_ok(arena, a_offset, a_len * 4) && span_ok(arena, out_offset, out_len * 4) &&
                    (!binary || span_ok(arena, b_offset, b_len * 4)),
                FNN_ERR_DISPATCH, "elementwise: slice outside arena");
    const float *a = (const float *)(arena->base + a_offset);
    const float *b = binary ? (const float *)(arena->base + b_offset) : a;
    float *o = (float *)(arena->base + out_offset);
    const bool same_len = a_len == out_len && (!binary || b_len == out_len);
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                           reinterpret_cast<uintptr_t>(o)) & 15u) == 0;
    if (same_len && aligned && out_len % 4 == 0) {
        FNN_CUDA_CHECK(launch_pdl(elementwise_vec_kernel, grid_for(ctx, out_len / 4, 256), 256, 0, ctx, op,
                                  reinterpret_cast<const float4 *>(a), reinterpret_cast<const float4 *>(b),
                                  reinterpret_cast<float4 *>(o), out_len / 4),
                       FNN_ERR_DISPATCH);
    } else {
        FNN_CUDA_CHECK(launch_pdl(elementwise_kernel, grid_for(ctx, out_len, 256), 256, 0, ctx, op, a,
                                  a_len, b, binary ? b_len : (size_t)1, o, out_len),
                       FNN_ERR_DISPATCH);
    }
    ctx->launches++;
    return FNN_OK;
}

// Device-to-device copy of `rows` rows of `width` bytes as a kernel on the context's stream.
static int launch_copy2d(fnn_cuda_ctx *ctx, unsigned char *dst, size_t dpitch, const unsigned char *src,
                         size_t spitch, size_t width, size_t rows) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | dpitch | spitch | width;
    if ((bits & 15u) == 0) {
        FNN_CUDA_CHECK(launch_pdl(copy2d_kernel<uint4>, grid_for(ctx, width / 16 * rows, 256), 256, 0, ctx, dst,
                                  dpitch, src, spitch, width / 16, rows),
                       FNN_ERR_DISPATCH);
    } else if ((bits & 3u) == 0) {
        FNN_CUDA_CHECK(launch_pdl(copy2d_kernel<uint32_t>, grid_for(ctx, width / 4 * rows, 256), 256, 0, ctx, dst,
                                  dpitch, src, spitch, width / 4, rows),
                       FNN_ERR_DISPATCH);
    } else {
        FNN_CUDA_CHECK(launch_pdl(copy2d_kernel<unsigned char>, grid_for(ctx, width * rows, 256), 256, 0, ctx, dst,
                                  dpitch, src, spitch, width, rows),
                       FNN_ERR_DISPATCH);
    }
    ctx->launches++;
    return FNN_OK;
}

int fnn_cuda_memcpy(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t dst_offset,
                    size_t src_offset, size_t bytes) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "memcpy: null handle");
    FNN_REQUIRE(span_ok(arena, dst_offset, bytes) && span_ok(arena, src_offset, bytes),
                FNN_ERR_DISPATCH, "memcpy: slice outside arena");
    if (bytes == 0) return FNN_OK;
    return launch_copy2d(ctx, arena->base + dst_offset, bytes, arena->base + src_offset, bytes, bytes, 1);
}

int fnn_cuda_memcpy2d(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t dst_offset, size_t dst_pitch,
                      size_t src_offset, size_t src_pitch, size_t width, size_t rows) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "memcpy2d: null handle");
    if (width == 0 || rows == 0) return FNN_OK;
    FNN_REQUIRE(width <= dst_pitch && width <= src_pitch &&
                    span_ok(arena, dst_offset, (rows - 1) * dst_pitch + width) &&
                    span_ok(arena, src_offset, (rows - 1) * src_pitch + width),
                FNN_ERR_DISPATCH, "memcpy2d: rows outside arena or wider than their pitch");
    return launch_copy2d(ctx, arena->base + dst_offset, dst_pitch, arena->base + src_offset, src_pitch, width,
                         rows);
}

int fnn_cuda_fill(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t offset, size_t bytes,
                  float value) {
    clear_error();
    FNN_REQUIRE(ctx && arena, FNN_ERR_DISPATCH, "fill: null handle");
    FNN_REQUIRE((offset & 3u) == 0 && span_ok(arena, offset, bytes), FNN_ERR_DISPATCH,
                "fill: slice outside arena or misaligned");
    size_t n = bytes / 4;
    if (n == 0) return FNN_OK;
    fill_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>((float *)(arena->base + offset), n,
                                                                value);
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

// ---- replay and timing -------------------------------------------------------------------------

int fnn_cuda_graph_begin(fnn_cuda_ctx *ctx) {
    clear_error();
    FNN_REQUIRE(ctx && !ctx->capturing, FNN_ERR_DISPATCH, "graph_begin: already capturing");
    FNN_CUDA_CHECK(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed),
                   FNN_ERR_DISPATCH);
    ctx->capturing = true;
    ctx->launches_at_capture = ctx->launches;
    return FNN_OK;
}

int fnn_cuda_graph_end(fnn_cuda_ctx *ctx, fnn_cuda_graph **out) {
    clear_error();
    FNN_REQUIRE(ctx && out && ctx->capturing, FNN_ERR_DISPATCH, "graph_end: not capturing");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    FNN_CUDA_CHECK(cudaStreamEndCapture(ctx->stream, &g), FNN_ERR_DISPATCH);
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return set_error(FNN_ERR_DISPATCH, "cudaGraphInstantiate failed: %s",
                         cudaGetErrorString(e));
    }
    fnn_cuda_graph *h = new fnn_cuda_graph();
    h->ctx = ctx;
    h->graph = g;
    h->exec = ex;
    // launches recorded during capture did not run; they are counted per replay instead
    h->launches_per_replay = ctx->launches - ctx->launches_at_capture;
    ctx->launches = ctx->launches_at_capture;
    *out = h;
    return FNN_OK;
}

int fnn_cuda_graph_launch(fnn_cuda_ctx *ctx, fnn_cuda_graph *g) {
    FNN_REQUIRE(ctx && g && g->exec, FNN_ERR_DISPATCH, "graph_launch: null handle");
    FNN_CUDA_CHECK(cudaGraphLaunch(g->exec, ctx->stream), FNN_ERR_DISPATCH);
    ctx->launches += g->launches_per_replay;
    return FNN_OK;
}

int fnn_cuda_graph_free(fnn_cuda_graph *g) {
    if (!g) return FNN_OK;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return FNN_OK;
}

int fnn_cuda_timer_start(fnn_cuda_ctx *ctx, int slot) {
    FNN_REQUIRE(ctx && slot >= 0 && slot < 64, FNN_ERR_DISPATCH, "timer: bad slot %d", slot);
    if (!ctx->ev_start[slot]) {
        FNN_CUDA_CHECK(cudaEventCreate(&ctx->ev_start[slot]), FNN_ERR_DISPATCH);
        FNN_CUDA_CHECK(cudaEventCreate(&ctx->ev_stop[slot]), FNN_ERR_DISPATCH);
    }
    FNN_CUDA_CHECK(cudaEventRecord(ctx->ev_start[slot], ctx->stream), FNN_ERR_DISPATCH);
    return FNN_OK;
}

int fnn_cuda_timer_stop(fnn_cuda_ctx *ctx, int slot) {
    FNN_REQUIRE(ctx && slot >= 0 && slot < 64 && ctx->ev_stop[slot], FNN_ERR_DISPATCH,
                "timer_stop: slot %d was never started", slot);
    FNN_CUDA_CHECK(cudaEventRecord(ctx->ev_stop[slot], ctx->stream), FNN_ERR_DISPATCH);
    return FNN_OK;
}

int fnn_cuda_timer_elapsed_ms(fnn_cuda_ctx *ctx, int slot, float *ms) {
    FNN_REQUIRE(ctx && ms && slot >= 0 && slot < 64 && ctx->ev_stop[slot], FNN_ERR_DISPATCH,
                "timer_elapsed: slot %d was never started", slot);
    FNN_CUDA_CHECK(cudaEventSynchronize(ctx->ev_stop[slot]), FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(cudaEventElapsedTime(ms, ctx->ev_start[slot], ctx->ev_stop[slot]),
                   FNN_ERR_DISPATCH);
    return FNN_OK;
}

int fnn_cuda_flush_l2(fnn_cuda_ctx *ctx) {
    FNN_REQUIRE(ctx, FNN_ERR_DISPATCH, "flush_l2: null context");
    if (!ctx->flush_buf) {
        FNN_REQUIRE(!ctx->capturing, FNN_ERR_MEMORY, "flush_l2: first call during capture");
        ctx->flush_bytes = (size_t)256 << 20;  // twice the 126 MB L2
        FNN_CUDA_CHECK(cudaMalloc(&ctx->flush_buf, ctx->flush_bytes), FNN_ERR_MEMORY);
    }
    static uint32_t tick = 0;
    size_t n = ctx->flush_bytes / sizeof(uint4);
    flush_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>((uint4 *)ctx->flush_buf, n, ++tick);
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    return FNN_OK;
}

}  // extern "C"
