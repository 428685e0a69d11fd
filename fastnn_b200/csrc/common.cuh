// Shared declarations of the sm_100a backend library: handle structs, error plumbing and
// the register-level decoders of fastnn's packed weight words.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <string>
#include <vector>

#include "../../include/fastnn_cuda.h"

namespace fnn {

// ---- error plumbing ---------------------------------------------------------------
int set_error(int code, const char *fmt, ...);
void clear_error();

#define FNN_CUDA_CHECK(expr, code)                                                         \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return fnn::set_error((code), "%s failed: %s (%s:%d)", #expr,                  \
                                  cudaGetErrorString(_e), __FILE__, __LINE__);             \
    } while (0)

#define FNN_REQUIRE(cond, code, ...)                                                       \
    do {                                                                                   \
        if (!(cond)) return fnn::set_error((code), __VA_ARGS__);                           \
    } while (0)

static inline size_t div_ceil(size_t a, size_t b) { return (a + b - 1) / b; }

// Items per u32 word (src/dtypes/*.rs `ITEMS`).
__host__ __device__ static inline int items_per_word(int fmt) {
    return (fmt == FNN_FMT_I8 || fmt == FNN_FMT_F8) ? 4 : 8;
}
static inline bool valid_fmt(int fmt) { return fmt >= FNN_FMT_I8 && fmt <= FNN_FMT_I4CB; }

constexpr int kMarginWords = 16;   // SIMD margin appended by the reference packers
constexpr int kCodebookBlock = 32; // quantization.rs:375

}  // namespace fnn

// ---- handles ------------------------------------------------------------------------

struct fnn_cuda_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t total_mem = 0;
    uint64_t launches = 0;
    const char *last_path = "";
    bool capturing = false;
    uint64_t launches_at_capture = 0;
    cudaEvent_t ev_start[64] = {};
    cudaEvent_t ev_stop[64] = {};
    void *flush_buf = nullptr;
    size_t flush_bytes = 0;
    // scratch for the tensor-core paths (activation conversion, split-K partials)
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    std::vector<void *> retired_scratch;   // outgrown scratch buffers (captured graphs may still name them)
    int *err_flag = nullptr;  // device flag written by bounded waits that gave up; err_flag[1]: CTA ticket of
                              // the fused GEMM + all-gather
    int *err_host = nullptr;  // pinned host copy of err_flag[0], refreshed by fnn_cuda_sync
    bool overlap_launches = true;   // programmatic dependent launch (fnn_cuda_ctx_set_overlap)
    unsigned *sk_flags = nullptr;   // 2 x 1024 zeroed counters of the tcgen05 kernel's split-K hand-over
};

struct fnn_cuda_arena {
    fnn_cuda_ctx *ctx = nullptr;
    uint8_t *base = nullptr;
    size_t bytes = 0;
    bool owned = false;
};

struct fnn_cuda_qweight {
    fnn_cuda_ctx *ctx = nullptr;
    int fmt = 0;
    size_t N = 0, K = 0;
    size_t qblock = 0;
    size_t words_per_row = 0;   // reference row length in u32
    size_t ld_u4 = 0;           // row stride of the row-padded layout, in 16-byte units
    uint4 *rows = nullptr;      // row-padded layout [N][ld_u4] (reference bit order)
    bool rows_owned = true;     // false: `rows` points into the arena slot the payload was written to
    float *scales = nullptr;    // [N] (I4CB: [N][blocks_per_row])
    float *zeros = nullptr;     // [N] or nullptr when every zero point is 0
    float *codebook = nullptr;  // [16] for I4CB
    size_t blocks_per_row = 0;
    bool has_zero = false;
    // fragment-major copy for the skinny tensor-core kernel (built on demand)
    uint4 *frag = nullptr;
    size_t frag_bytes = 0;
    float *frag_bs = nullptr;   // I4CB block scales in fragment order
    bool fp16_ok = true;         // codebook format: false when block scales or centroids would leave the fp16 range
                                // of the tcgen05 kernel's dequantized operand
};

struct fnn_cuda_graph {
    fnn_cuda_ctx *ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches_per_replay = 0;
};

// ---- device-side decoders -------------------------------------------------------------
// Each returns the exact f32 value the reference's `unpack_to_f32` produces for the lane.

namespace fnn {

// e4m3 -> f32 (src/dtypes/f8x4.rs:23-38).  Exponent 15 is NaN for every mantissa.
__device__ __forceinline__ float e4m3_to_f32_exact(uint32_t byte) {
    uint32_t mag = byte & 0x7Fu;
    // (mag << 20) places exponent and mantissa in f32 position with bias 0+..; scaling
    // by 2^120 rebiases (7 -> 127) and also turns the f32 subnormal into m * 2^-9.
    float v = __uint_as_float(mag << 20) * 0x1p120f;
    if ((mag & 0x78u) == 0x78u) v = __uint_as_float(0x7FC00000u);
    return __uint_as_float(__float_as_uint(v) | ((byte & 0x80u) << 24));
}

// Hot-loop variant: identical on every code the reference quantizer can emit
// (|v| <= 240, i.e. codes <= 0x77 / 0xF7); codes with exponent 15 decode as finite.
__device__ __forceinline__ float e4m3_to_f32_fast(uint32_t byte) {
    float v = __uint_as_float((byte & 0x7Fu) << 20) * 0x1p120f;
    return __uint_as_float(__float_as_uint(v) | ((byte & 0x80u) << 24));
}

// e2m1 -> f32 (src/dtypes/f4x8.rs:21-39).  Code 0x8 decodes to +0.
__device__ __forceinline__ float fp4_to_f32_exact(uint32_t code) {
    uint32_t mag = code & 7u;
    float v = __uint_as_float(mag << 22) * 0x1p126f;
    uint32_t sign = (mag != 0u) ? ((code & 8u) << 28) : 0u;
    return __uint_as_float(__float_as_uint(v) | sign);
}

// Sign-extended nibble (src/dtypes/i4x8.rs:22-30).
__device__ __forceinline__ float i4_to_f32(uint32_t word, int i) {
    return (float)(((int32_t)(word << (28 - 4 * i))) >> 28);
}

__device__ __forceinline__ float i8_to_f32(uint32_t word, int i) {
    return (float)(int8_t)((word >> (8 * i)) & 0xFFu);
}

// act(x) of the fused epilogue (src/backend/cpu/mod.rs:3140-3171).
__device__ __forceinline__ float apply_act(float x, int epi) {
    switch (epi) {
    case FNN_EPI_RELU:
        return fmaxf(x, 0.0f);
    case FNN_EPI_GELU: {
        float x3 = x * x * x;
        float t = tanhf(0.7978846f * (x + 0.044715f * x3));
        return 0.5f * x * (1.0f + t);
    }
    case FNN_EPI_SILU:
        return x / (1.0f + expf(-x));
    default:
        return x;
    }
}

// The same functions through the hardware exp2 / reciprocal units (relative error of a few 1e-7 on
// the exponential's result; the reference's own SIMD exp is good to 2e-5,
// src/backend/cpu/microkernels/activations.rs:336-373).  Used where the epilogue competes with the
// tensor pipe for issue slots.  tanh(u) = 1 - 2 / (1 + e^(2u)).
__device__ __forceinline__ float apply_act_fast(float x, int epi) {
    switch (epi) {
    case FNN_EPI_RELU:
        return fmaxf(x, 0.0f);
    case FNN_EPI_GELU: {
        const float u = 0.7978846f * (x + 0.044715f * x * x * x);
        const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
        return 0.5f * x * (1.0f + t);
    }
    case FNN_EPI_SILU:
        return __fdividef(x, 1.0f + __expf(-x));
    default:
        return x;
    }
}

// dot*scale + zero*sum(a) with the reference's separate roundings
// (src/backend/cpu/microkernels/mod.rs:293-295), then act(x + bias).
__device__ __forceinline__ float finish_output(float dot, float scale, float zero, float rowsum,
                                               bool has_bias, float bias, int epi) {
    float x = __fadd_rn(__fmul_rn(dot, scale), __fmul_rn(zero, rowsum));
    if (has_bias) x = __fadd_rn(x, bias);
    return apply_act(x, epi);
}
__device__ __forceinline__ float finish_output_fast(float dot, float scale, float zero, float rowsum,
                                                    bool has_bias, float bias, int epi) {
    float x = __fadd_rn(__fmul_rn(dot, scale), __fmul_rn(zero, rowsum));
    if (has_bias) x = __fadd_rn(x, bias);
    return apply_act_fast(x, epi);
}

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched through launch_pdl may start while the kernel before it on the stream is still
// running: everything that does not depend on that kernel (weight prefetch, scales, shared-memory
// set-up) runs under its tail, and pdl_wait() blocks until the earlier kernel has completed and its
// memory is visible.  Every block must reach pdl_wait() before it touches activations, outputs or
// counters.  Without the launch attribute both instructions do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), int grid, int block, size_t smem, const fnn_cuda_ctx *ctx,
                              Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->overlap_launches ? 1 : 0;   // without it every kernel waits for the one before it
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

// ---- launchers implemented in the kernel translation units ---------------------------------
// Fused all-gather of the outputs over peer memory (column-sharded layers, one rank per GPU).
// Fused GEMV + all-gather.  Every output travels as one 8-byte word {value bits, step number}: the
// store is a single access, so a reader that sees the step number of a word also has its value and
// no fence or flag handshake is needed on either side.
struct GatherArgs {
    unsigned long long *peer_words[8];   // every rank's [2 slots][world][kGatherRows][n_stride] words
    unsigned *step_ctr;   // local: number of completed steps
    int *done_ctr;        // local: blocks finished in the current launch
    int *last_m;          // local: batch rows of the last completed step
    int *err_flag;
    int rank, world, n_stride;
};
constexpr int kGatherRows = 4;   // batch rows a gathered slot holds (the fused path serves M <= 4)

#ifdef __CUDACC__
// One gathered output: {value bits, step number} in a single 8-byte access at system scope.
__device__ __forceinline__ void st_word_sys(unsigned long long *p, float v, unsigned step) {
    const unsigned long long w = ((unsigned long long)step << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word_sys(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
// Polls one word until it carries `step` (or a later one); false after about a second of cycles.
__device__ __forceinline__ bool wait_word(const unsigned long long *p, unsigned step, unsigned long long &w) {
    const long long t0 = clock64();
    for (;;) {
        w = ld_word_sys(p);
        if ((int)((unsigned)(w >> 32) - step) >= 0) return true;
        if (clock64() - t0 > 2000000000LL) return false;
    }
}

// Per-thread state of one fused-gather launch.
struct GatherCursor {
    unsigned step;                          // the step this launch produces (1, 2, ...)
    const unsigned long long *prev_words;   // this rank's slot of the previous step
    int prev_per_rank, prev_total, prev_i;  // words per rank / in all / this thread's first word
    unsigned long long prev_w0;             // first poll of this thread's first word
};

// Reads the counters (steps, blocks done, rows of the last step: one 16-byte load; every block does
// this before any block can advance them) and issues the first poll of the previous step's words.
__device__ __forceinline__ GatherCursor gather_begin(const GatherArgs &g, int global_tid) {
    GatherCursor c{};
    unsigned c0, c1, c2, c3;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3) : "l"(g.step_ctr) : "memory");
    c.step = c0 + 1u;
    c.prev_i = global_tid;
    if (c.step > 1u) {
        c.prev_words = g.peer_words[g.rank] + (size_t)((c.step - 1u) & 1u) * g.world * kGatherRows * g.n_stride;
        c.prev_per_rank = (int)c2 * g.n_stride;
        c.prev_total = g.world * c.prev_per_rank;
        if (c.prev_i < c.prev_total) {
            const int r = c.prev_i / c.prev_per_rank;
            c.prev_w0 = ld_word_sys(c.prev_words + (size_t)r * kGatherRows * g.n_stride +
                                    (c.prev_i - r * c.prev_per_rank));
        }
    }
    return c;
}

// The grid checks that every word of the previous step has arrived in this rank's buffer (a few
// words per thread, bounded polls).  A peer whose previous step is visible here has finished reading
// the slot this step overwrites.
__device__ __forceinline__ void gather_check_prev(const GatherArgs &g, const GatherCursor &c, int grid_threads) {
    bool first = true;
    for (int i = c.prev_i; i < c.prev_total; i += grid_threads) {
        const int r = i / c.prev_per_rank;
        unsigned long long w = c.prev_w0;
        if (!(first && (int)((unsigned)(w >> 32) - (c.step - 1u)) >= 0) &&
            !wait_word(c.prev_words + (size_t)r * kGatherRows * g.n_stride + (i - r * c.prev_per_rank),
                       c.step - 1u, w)) {
            atomicOr(g.err_flag, 0x100);
            break;
        }
        first = false;
    }
}

// This rank's output (m, n) goes straight into every rank's buffer (plain peer stores).
__device__ __forceinline__ void gather_store(const GatherArgs &g, unsigned step, int m, int n, float v) {
    const size_t at = (((size_t)(step & 1u) * g.world + g.rank) * kGatherRows + m) * g.n_stride + n;
    for (int r = 0; r < g.world; ++r) st_word_sys(g.peer_words[r] + at, v, step);
}

// End of a fused-gather launch (all threads of the block call it).  Columns between the shard's width
// and the common stride are never computed: block 0 marks them as arrived so that readers can poll
// whole rows.  The last block to finish advances the step counter.
__device__ __forceinline__ void gather_finish(const GatherArgs &g, unsigned step, int M, int N) {
    const int tid = threadIdx.x, NT = blockDim.x;
    if (blockIdx.x == 0) {
        const int pad = g.n_stride - N;
        for (int i = tid; i < pad * M; i += NT) gather_store(g, step, i / pad, N + i % pad, 0.0f);
    }
    __syncthreads();
    if (tid == 0) {
        const int ticket = atomicAdd(g.done_ctr, 1);
        if (ticket == (int)gridDim.x - 1) {
            *g.done_ctr = 0;
            // A launch whose check of the previous step gave up advances nothing: the host sees the
            // error at its next fnn_cuda_sync and has to zero the gather buffers on every rank before
            // it uses them again (words of this step may have been published in part).
            int failed;
            asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(failed) : "l"(g.err_flag) : "memory");
            if (!(failed & 0x100)) {
                *g.last_m = M;
                *g.step_ctr = step;
            }
        }
    }
}
#endif

// Fused GEMM + all-gather for any batch size (tcgen05 kernel): every rank stores its [M, n_local]
// block into columns [col0, col0 + n_local) of every rank's [M, n_total] f32 output and, when its last
// CTA is done, adds one to every rank's arrival counter (release at system scope).
struct AllGatherArgs {
    float *peer_out[8];          // every rank's [M, n_total] output
    unsigned *peer_arrive[8];    // every rank's {arrivals, consumed} pair (one arrival per rank and launch)
    int *ticket;                 // local: CTAs of this launch that have stored their outputs
    int rank;
    int world, n_total, col0;
};

struct QmmArgs {
    const fnn_cuda_qweight *w;
    const float *a;    // [M,K]
    float *out;        // [M,N]
    const float *bias; // [N] or nullptr
    size_t M;
    int epilogue;
    const GatherArgs *gather = nullptr;
    const AllGatherArgs *allgather = nullptr;
};

int launch_qmm_rows(fnn_cuda_ctx *ctx, const QmmArgs &args);
bool qmm_mma_supported(const fnn_cuda_qweight *w, size_t M);
int launch_qmm_mma(fnn_cuda_ctx *ctx, const QmmArgs &args);
int prepare_qmm_mma(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w);
bool qmm_mma8_supported(const fnn_cuda_qweight *w, size_t M);
int launch_qmm_mma8(fnn_cuda_ctx *ctx, const QmmArgs &args);
int launch_gather_wait(fnn_cuda_ctx *ctx, const unsigned long long *my_words, const unsigned *counters,
                       int world, int n_stride, float *out);
int prepare_qmm_tc(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w);
// shapes automatic dispatch sends to the skinny tensor-core kernel
static inline bool auto_uses_mma(const fnn_cuda_qweight *w) { return w->K >= 512 && w->N >= 64; }
bool qmm_tc_supported(const fnn_cuda_qweight *w, size_t M);
int launch_qmm_tc(fnn_cuda_ctx *ctx, const QmmArgs &args);
void free_qweight_aux(fnn_cuda_qweight *w);

int ensure_scratch(fnn_cuda_ctx *ctx, size_t bytes);

}  // namespace fnn
