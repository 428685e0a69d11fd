/*
 * fastnn_cuda.h -- C ABI of the B200 (sm_100a) backend for fastnn's quantized-weight
 * MatMul path.
 *
 * A Rust `CudaBackend` implementing fastnn's `Backend` trait (src/backend/mod.rs:152-254)
 * binds exactly these symbols through `extern "C"`; the Python mirror in this
 * repository binds them through ctypes.  Plain pointers and sizes only; every function
 * returns an `int` status (FNN_OK == 0) and never throws or aborts.  The message for
 * the last failure on the calling thread is available from fnn_cuda_last_error().
 *
 * There is no CPU fallback behind any entry point.
 *
 * File paths in the comments are relative to the fastnn repository root.
 */
#ifndef FASTNN_CUDA_H
#define FASTNN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  They map onto BackendError (src/backend/mod.rs:6-12). */
enum {
    FNN_OK = 0,
    FNN_ERR_COMPILATION = 1, /* BackendError::Compilation  */
    FNN_ERR_DISPATCH = 2,    /* BackendError::Dispatch     */
    FNN_ERR_MEMORY = 3,      /* BackendError::Memory       */
    FNN_ERR_UNSUPPORTED = 4  /* BackendError::UnsupportedOp */
};

/* Packed weight formats: the four packed-word dtypes on the path plus the codebook
 * variant of I4x8 (src/dtypes/{i8x4,i4x8,f8x4,f4x8}.rs, src/packed_tensor.rs:1209). */
enum {
    FNN_FMT_I8 = 0,   /* kernel "matmul_i8": per-channel scale + zero          */
    FNN_FMT_I4 = 1,   /* kernel "matmul_i4": per-channel scale + zero          */
    FNN_FMT_F8 = 2,   /* kernel "matmul_f8": e4m3, per-channel scale           */
    FNN_FMT_F4 = 3,   /* kernel "matmul_f4": e2m1, per-channel scale + zero    */
    FNN_FMT_I4CB = 4  /* kernel "matmul_i4" with codebooks: per-32 block scale */
};

/* Fused epilogue, from the MatMul node's `fused_op` attribute
 * (src/backend/cpu/mod.rs:406-413): act(x + bias[j]). */
enum { FNN_EPI_NONE = 0, FNN_EPI_RELU = 1, FNN_EPI_GELU = 2, FNN_EPI_SILU = 3 };

/* Which kernel family fnn_cuda_qmatmul may pick. */
enum {
    FNN_PATH_AUTO = 0,
    FNN_PATH_ROWS = 1, /* f32 CUDA-core row kernel (any shape)                */
    FNN_PATH_MMA = 2,  /* skinny-M tensor-core kernel, fragment-major weights  */
    FNN_PATH_TC = 3    /* tcgen05 / TMEM / TMA GEMM (5 batch rows and more)    */
};

/* Elementwise kernels of the plan ("add_f32", "mul_f32", "relu_f32", ...;
 * src/backend/cpu/mod.rs:627-640, src/backend/cpu/elementwise.rs:105-130).  The op+activation
 * kernels ("add_relu_f32", "mul_gelu_f32", ...; src/backend/cpu/mod.rs:642-672) are
 * `binary_op | (FNN_EPI_* << 8)`. */
enum {
    FNN_EW_ADD = 0,
    FNN_EW_MUL = 1,
    FNN_EW_SUB = 2,
    FNN_EW_RELU = 10,
    FNN_EW_GELU = 11,
    FNN_EW_SILU = 12
};

typedef struct fnn_cuda_ctx fnn_cuda_ctx;
typedef struct fnn_cuda_arena fnn_cuda_arena;
typedef struct fnn_cuda_qweight fnn_cuda_qweight;
typedef struct fnn_cuda_graph fnn_cuda_graph;

/* ---- context ------------------------------------------------------------------
 * One per executor.  All work of a context is asynchronous on one CUDA stream;
 * calls are serialized by the caller, as `CpuBackend::dispatch` is single-threaded
 * by contract (src/backend/cpu/mod.rs:176-187). */
int fnn_cuda_ctx_create(int device, fnn_cuda_ctx **out);   /* on a private non-blocking stream */
/* Same, but runs on the stream the caller gives (a `cudaStream_t` passed as void*) and never on
 * another one: a null handle is the legacy default stream (on which stream capture, and so
 * fnn_cuda_graph_begin, is not possible). */
int fnn_cuda_ctx_create_on_stream(int device, void *stream, fnn_cuda_ctx **out);
/* The `cudaStream_t` the context launches on (so that a caller can order its own work against it). */
void *fnn_cuda_ctx_stream(fnn_cuda_ctx *ctx);
/* Kernels are launched as programmatic dependents of the kernel before them on the stream: a
 * kernel's prologue (weight prefetch, scales, barrier set-up) runs under its predecessor's tail and
 * it waits only where it first touches what the predecessor wrote.  enabled == 0 turns that off
 * for the launches that follow (every kernel then starts after the previous one has finished),
 * which is how a launch is timed on its own. */
int fnn_cuda_ctx_set_overlap(fnn_cuda_ctx *ctx, int enabled);
int fnn_cuda_ctx_destroy(fnn_cuda_ctx *ctx);
int fnn_cuda_sync(fnn_cuda_ctx *ctx);
/* Message of the last failing call on this thread ("" if none). */
const char *fnn_cuda_last_error(void);
/* Number of kernels this library has launched on `ctx` since creation. */
int fnn_cuda_launch_count(fnn_cuda_ctx *ctx, uint64_t *out);
/* Device facts for sizing and reports. */
int fnn_cuda_device_info(fnn_cuda_ctx *ctx, int *sm_count, int *cc_major, int *cc_minor,
                         size_t *total_mem);

/* ---- arena ---------------------------------------------------------------------
 * Backend::allocate_arena / write_arena / read_arena (src/backend/mod.rs:157,243,
 * 250; CPU impl src/backend/cpu/mod.rs:188-279, 7228-7238).  The arena is one device
 * allocation holding every slot of the compiler's MemoryPlan at its planned offset
 * (src/compiler/passes/memory_planning.rs:17-29); it is zero-filled on allocation. */
int fnn_cuda_arena_alloc(fnn_cuda_ctx *ctx, size_t bytes, fnn_cuda_arena **out);
/* Wrap device memory the caller owns (kept alive by the caller). */
int fnn_cuda_arena_wrap(fnn_cuda_ctx *ctx, void *device_ptr, size_t bytes, fnn_cuda_arena **out);
int fnn_cuda_arena_free(fnn_cuda_arena *arena);
/* Host -> arena.  Out-of-range spans are clamped like the CPU backend does and
 * reported as FNN_ERR_MEMORY. */
int fnn_cuda_arena_write(fnn_cuda_arena *arena, size_t offset, const void *host, size_t bytes);
/* Arena -> host; synchronizes the context's stream first. */
int fnn_cuda_arena_read(fnn_cuda_arena *arena, size_t offset, void *host, size_t bytes);
/* Asynchronous variants for pinned host memory (no implicit synchronization). */
int fnn_cuda_arena_write_async(fnn_cuda_arena *arena, size_t offset, const void *pinned,
                               size_t bytes);
int fnn_cuda_arena_read_async(fnn_cuda_arena *arena, size_t offset, void *pinned, size_t bytes);
void *fnn_cuda_arena_device_ptr(fnn_cuda_arena *arena);
size_t fnn_cuda_arena_size(fnn_cuda_arena *arena);
/* Pinned host staging buffers for the executor's input/output copies. */
int fnn_cuda_host_alloc(size_t bytes, void **out);
int fnn_cuda_host_free(void *ptr);

/* ---- quantized weights -----------------------------------------------------------
 * Replaces get_or_cache_packed + packed_tensor_from_meta
 * (src/backend/cpu/mod.rs:62-89, src/backend/cpu/matmul.rs:81-152): takes the WriteConst
 * payload of a quantized weight Constant -- `[N][ceil(K/ITEMS)]` u32 rows followed by
 * 16 margin words (src/packed_tensor.rs:978-982) -- plus the fields of
 * QuantizedWeightMeta (src/backend/mod.rs:43-58), validates them with the same rules,
 * and builds the device layout the kernels read.  Every quantized bit and every scale
 * is preserved; fnn_cuda_qweight_unrepack() returns the original byte stream.
 *
 * scales: N floats (I4CB: N*ceil(K/qblock)); a single scale/zero is broadcast to all
 * rows.  zeros: N floats or n_zeros == 0 (then zero).  codebook16: 16 floats for
 * I4CB, else NULL.  qblock: 32 for I4CB, else 0. */
int fnn_cuda_qweight_upload(fnn_cuda_ctx *ctx, int fmt, const void *packed, size_t packed_bytes,
                            size_t N, size_t K, const float *scales, size_t n_scales,
                            const float *zeros, size_t n_zeros, size_t qblock,
                            const float *codebook16, fnn_cuda_qweight **out);
/* The same for a payload that Instruction::WriteConst has already written into the arena (what
 * Backend::dispatch sees on the first execution): the packed rows are read where they are -- no copy,
 * no trip through the host -- whenever their stride needs no padding (K a multiple of 32 codes; 128
 * for FP4), and copied device-to-device otherwise.  The slot must stay untouched for the life of the
 * handle, which the memory plan guarantees for constants
 * (src/compiler/passes/memory_planning.rs:376-397). */
int fnn_cuda_qweight_from_arena(fnn_cuda_ctx *ctx, int fmt, fnn_cuda_arena *arena, size_t offset,
                                size_t packed_bytes, size_t N, size_t K, const float *scales,
                                size_t n_scales, const float *zeros, size_t n_zeros, size_t qblock,
                                const float *codebook16, fnn_cuda_qweight **out);
/* Build the device layout a kernel family needs (fragment-major for FNN_PATH_MMA; the tcgen05
 * kernel reads the packed rows and needs none; FNN_PATH_AUTO builds what automatic dispatch can
 * pick for this shape) now instead of at its first use.  Call it from Backend::compile, outside any
 * graph capture. */
int fnn_cuda_qweight_prepare(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, int path);
int fnn_cuda_qweight_free(fnn_cuda_qweight *w);
/* Reference-layout byte count: (N*ceil(K/ITEMS) + 16) * 4. */
size_t fnn_cuda_qweight_packed_bytes(fnn_cuda_qweight *w);
/* Device layout -> reference byte stream (margin zero-filled), into host memory. */
int fnn_cuda_qweight_unrepack(fnn_cuda_qweight *w, void *host_out, size_t bytes);
/* Dequantize on the device to f32 [N,K] at arena+out_offset with the reference's two
 * roundings, unpack(q)*scale + zero (src/packed_tensor.rs:469-521). */
int fnn_cuda_qweight_dequant(fnn_cuda_qweight *w, fnn_cuda_arena *arena, size_t out_offset);

/* ---- the hot path -----------------------------------------------------------------
 * Replaces quantized_matmul_dispatch<T> -> gemm_cpu_flat -> gemm_batch_packed_simd
 * (src/backend/cpu/matmul.rs:165-225, src/backend/cpu/microkernels/gemm.rs:1982-2088):
 *   out[m,n] = act( (sum_k unpack(q[n,k]) * a[m,k]) * scale[n] + zero[n] * sum_k a[m,k]
 *                   + bias[n] )
 * a: f32 [M,K] row-major at arena+a_offset; out: f32 [M,N] row-major at
 * arena+out_offset; bias: f32 [N] at arena+bias_offset, or bias_offset < 0 for none.
 * The epilogue follows matmul_activation_dispatch (src/backend/cpu/matmul.rs:61-71). */
int fnn_cuda_qmatmul(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, fnn_cuda_arena *arena,
                     size_t a_offset, size_t out_offset, int64_t bias_offset, size_t M,
                     int epilogue, int path);
/* Same with explicit device pointers (activations/outputs outside any arena). */
int fnn_cuda_qmatmul_ptr(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                         float *out_dev, const float *bias_dev, size_t M, int epilogue,
                         int path);
/* The same quantized MatMul for callers that must not trigger a device allocation -- no
 * counterpart in the reference, which runs on host memory only.  Some hosts hand every byte
 * of device memory to an allocator of their own, or run a latency-critical loop in which
 * cudaMalloc/cudaFree (which can synchronize the whole device) are off limits; fnn_cuda_qmatmul
 * may grow the context's scratch buffer on a larger problem, this entry point never calls
 * cudaMalloc, cudaFree or any allocating routine; after the first call per device (which makes the
 * CUDA runtime load the module and materialise the array) free device memory does not change
 * across a call.  It runs the tcgen05 kernel with the rewritten
 * activations placed in an 8 MiB scratch array that is part of the library image (every GPU
 * that loads the library holds it until the process exits).  The rewritten activations must
 * fit in it: about T * M * K bytes with M and K rounded up to the kernel's tiles (T = 2 byte
 * planes; 3 for FP8/FP4 below 128 batch rows) -- for example M = 512 at K = 4096, or M = 256 at
 * K = 8192.  A larger problem is refused with FNN_ERR_MEMORY and both sizes in the message.
 * a_dev [M,K], out_dev [M,N], bias_dev [N] or NULL are device pointers owned by the caller.
 * All five formats are served where the tcgen05 kernel is (K >= 128; the codebook format: K a
 * multiple of 128).  The first call on a device looks up the scratch array's device
 * address; make that call before any stream capture.  All calls share the array and it keeps
 * the previous call's contents (stale batch rows beyond M only reach accumulator columns that are
 * never stored), so two
 * calls that overlap on the GPU -- different streams or contexts of one device -- race. */
int fnn_cuda_qmatmul_noalloc(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                             float *out_dev, const float *bias_dev, size_t M, int epilogue);
/* Name of the kernel family the last fnn_cuda_qmatmul on `ctx` launched. */
const char *fnn_cuda_last_path(fnn_cuda_ctx *ctx);

/* ---- column-sharded layers on the GPUs of one node --------------------------------------------
 * No counterpart in the reference (it has no collective of any kind).  A layer is sharded by
 * output columns = contiguous ranges of packed rows, one process per GPU.  Each rank allocates one
 * shared arena with fnn_cuda_arena_alloc, exports it, and opens its peers':
 *   [gather_offset]  u64 words[2 slots][world][4 rows][n_stride]   (n_stride >= widest shard)
 *   [counter_offset] u32 steps | i32 blocks | i32 rows of the last step   (16 bytes)
 * both zero at start (fnn_cuda_arena_alloc clears the arena).
 * fnn_cuda_qmatmul_gather is the GEMV fused with the all-gather.  Every output travels as one 8-byte
 * word {f32 value, step number} that the epilogue stores into every rank's
 * words[step & 1][rank][row][column] with one plain peer store over NVLink: a reader that sees the
 * step number of a word has its value too, so neither side needs a fence or a flag handshake and the
 * producer never waits.  The consumer polls: the next fnn_cuda_qmatmul_gather on the stream first
 * checks, one word per thread over its grid, that the previous step has arrived in full (which also
 * proves that every peer is done reading the slot it is about to overwrite), and
 * fnn_cuda_gather_wait does the same for the last step and, when out_dev is given, writes the values
 * there as plain f32 [world][M][n_stride] for any other consumer.  Polls are bounded (about one
 * second, so ranks whose launches drift further apart than that report it too): if a word never
 * arrives the context's error flag is raised, that launch does not advance the step counter, and
 * fnn_cuda_sync reports it; words of the failed step may have been published in part, so the gather
 * buffers and counters have to be zeroed on every rank before they are used again.  Every rank must
 * make the same sequence of calls with the same n_stride (the check of the previous step indexes
 * with it).  Serves all five formats with 1..4 batch rows (the HBM-bound case where a separate
 * collective costs more than the GEMV); larger batches use fnn_cuda_qmatmul_allgather below. */
int fnn_cuda_ipc_export(fnn_cuda_arena *arena, void *handle64);
int fnn_cuda_ipc_open(fnn_cuda_ctx *ctx, const void *handle64, void **device_ptr);
int fnn_cuda_ipc_close(fnn_cuda_ctx *ctx, void *device_ptr);
int fnn_cuda_qmatmul_gather(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                            const float *bias_dev, size_t M, int epilogue, int rank, int world,
                            void *const *peer_bases, size_t gather_offset, size_t counter_offset,
                            size_t n_stride);
int fnn_cuda_gather_wait(fnn_cuda_ctx *ctx, void *my_base, size_t gather_offset, size_t counter_offset,
                         int world, size_t n_stride, void *out_dev);
/* The same fusion for any batch size, on the tcgen05 kernel (no counterpart in the reference).  Every
 * rank's shared arena holds, at the same offsets on every rank,
 *   [out_offset]      f32 [M][n_total]   the gathered rows, ready to be the next layer's activations
 *   [counter_offset]  u32 arrivals | u32 consumed                       (8 bytes, zero at start)
 * The epilogue stores this rank's [M, n_local] block into columns [col0, col0 + n_local) of every
 * rank's rows with plain peer stores over NVLink.  The CTA that leaves last on a rank fences at
 * system scope, adds one to every rank's `arrivals` (release) and then waits (bounded, about a
 * second; on expiry the context's error flag is raised and nothing is consumed) until `world`
 * arrivals beyond `consumed` are in, and advances
 * `consumed`: when the call's kernel has finished, the rows are complete, and whatever follows it
 * on the stream may read them.  The counters only grow and live in device memory: a captured graph
 * of such steps can be replayed.  A buffer may be reused by a later step once every rank has read it,
 * which a chain of at least two gathered layers guarantees (a rank can only finish the step after
 * next when its peers have started theirs).  Every rank must make the same sequence of calls, each
 * rank on its own GPU.  Serves what the tcgen05 kernel serves (K >= 128). */
int fnn_cuda_qmatmul_allgather(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                               const float *bias_dev, size_t M, int epilogue, int rank, int world,
                               void *const *peer_bases, size_t out_offset, size_t counter_offset,
                               size_t n_total, size_t col0);

/* ---- remaining plan instructions ---------------------------------------------------
 * Binary ops broadcast by modulo, out[i] = op(a[i % a_len], b[i % b_len])
 * (src/backend/cpu/elementwise.rs:105-130); unary ops ignore b.  Lengths in floats.
 * `out` may alias `a` (the planner reuses slots in place,
 * src/compiler/passes/memory_planning.rs:491-618). */
int fnn_cuda_elementwise(fnn_cuda_ctx *ctx, int op, fnn_cuda_arena *arena, size_t a_offset,
                         size_t a_len, size_t b_offset, size_t b_len, size_t out_offset,
                         size_t out_len);
/* Instruction::MemCopy and Instruction::Fill (src/backend/mod.rs:82-89). */
/* rms_norm over rows of row_size floats: out = in / sqrt(mean(in^2) + eps) * w[i]
 * (src/backend/cpu/microkernels/ops.rs:979-1008).  w_offset < 0: no weight.  The caller passes the
 * row size: the hidden size (= weight length), as the reference's fused residual variant does
 * (tests/residual_add_norm.rs:327-355); its unfused dispatch arm derives len / w_len instead
 * (src/backend/cpu/mod.rs:5053-5075).  out may be in. */
int fnn_cuda_rms_norm(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t in_offset, size_t len,
                      long long w_offset, size_t w_len, size_t row_size, float eps, size_t out_offset);
/* The general row normalisation behind "rms_norm", "fused_residual_add_rms_norm" and
 * "fused_residual_add_layer_norm" (src/backend/cpu/mod.rs:2424-2500, 5053-5230): kind 0 = rms_norm,
 * 1 = layer_norm with population variance; x = in + residual when res_offset >= 0; weight and bias are
 * optional (offset < 0), default 1 and 0 (src/backend/cpu/microkernels/ops.rs:788-825, 1012-1044). */
int fnn_cuda_row_norm(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, int kind, size_t in_offset, size_t len,
                      long long res_offset, long long w_offset, size_t w_len, long long b_offset,
                      size_t b_len, size_t row_size, float eps, size_t out_offset);
/* softmax along an axis of axis_dim elements that are `stride` floats apart; len / axis_dim rows
 * (kernel "softmax", params [axis_dim, stride]: src/backend/cpu/mod.rs:1002-1050, 3488-3514;
 * src/backend/cpu/microkernels/ops.rs:1363-1397).  out may be in. */
int fnn_cuda_softmax(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t in_offset, size_t len,
                     size_t axis_dim, size_t stride, size_t out_offset);
int fnn_cuda_memcpy(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t dst_offset,
                    size_t src_offset, size_t bytes);
int fnn_cuda_fill(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t offset, size_t bytes,
                  float value);
/* Strided copy inside the arena: `rows` rows of `width` bytes, row r from src_offset + r*src_pitch
 * to dst_offset + r*dst_pitch -- a column range of a row-major matrix (kernel "slice_f32" of the reference's
 * plans with unit stride on the innermost dimension, src/backend/cpu/mod.rs:1250, 4721-4760). */
int fnn_cuda_memcpy2d(fnn_cuda_ctx *ctx, fnn_cuda_arena *arena, size_t dst_offset, size_t dst_pitch,
                      size_t src_offset, size_t src_pitch, size_t width, size_t rows);

/* ---- replay and timing --------------------------------------------------------------
 * A static-shape plan is replayed unchanged after its first execution
 * (src/backend/executor.rs:639-667); capture it once and relaunch it as a CUDA graph.
 * Between begin and end every call on `ctx` is recorded instead of executed.  A graph keeps the
 * addresses it was captured with: the context's scratch buffer is never freed while the context
 * lives (when a later, larger call outgrows it the old one is retired, not released), so a graph
 * stays valid whatever runs on the context afterwards. */
int fnn_cuda_graph_begin(fnn_cuda_ctx *ctx);
int fnn_cuda_graph_end(fnn_cuda_ctx *ctx, fnn_cuda_graph **out);
int fnn_cuda_graph_launch(fnn_cuda_ctx *ctx, fnn_cuda_graph *g);
int fnn_cuda_graph_free(fnn_cuda_graph *g);
/* CUDA-event stopwatch on the context's stream; replaces the wall clock of
 * Backend::dispatch_profile (src/backend/mod.rs:178-211).  `slot` in [0, 64). */
int fnn_cuda_timer_start(fnn_cuda_ctx *ctx, int slot);
int fnn_cuda_timer_stop(fnn_cuda_ctx *ctx, int slot);
/* Waits for the stop event; milliseconds between start and stop. */
int fnn_cuda_timer_elapsed_ms(fnn_cuda_ctx *ctx, int slot, float *ms);
/* Overwrite a scratch buffer larger than L2 so the next kernel starts cold. */
int fnn_cuda_flush_l2(fnn_cuda_ctx *ctx);

/* ---- host-side compile-time pass -------------------------------------------------------
 * The weight-quantization pass itself (src/compiler/passes/quantization.rs:36-273,
 * 281-495 calling src/packed_tensor.rs:661-742, 852-1049, 1209-1313).  Host code, as in
 * the reference: w_kn is the graph constant, f32 [K,N] row-major; it is transposed to
 * [N,K] and quantized per output channel (I4CB: per 32-element block with one 16-entry
 * codebook).  packed_out: fnn_quant_packed_bytes() bytes.  scales_out: N floats
 * (I4CB: N*ceil(K/32)); zeros_out: N floats (ignored for F8 and I4CB); codebook_out: 16
 * floats (I4CB only). */
size_t fnn_quant_packed_bytes(int fmt, size_t N, size_t K);
size_t fnn_quant_num_scales(int fmt, size_t N, size_t K);
int fnn_quantize_weights(int fmt, const float *w_kn, size_t K, size_t N, void *packed_out,
                         float *scales_out, float *zeros_out, float *codebook_out);

#ifdef __cplusplus
}
#endif
#endif /* FASTNN_CUDA_H */
