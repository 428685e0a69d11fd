// tcgen05 / TMEM / TMA kernel for the quantized MatMul.
//
// Weight operand (the MMA's M side, 128 output channels per CTA tile), always fetched from the
// packed rows as the reference stores them -- no expanded copy exists in device memory:
//   I8    kind::i8, FP8 kind::f8f6f4 (e4m3): TMA drops the K-contiguous rows into 128-byte-swizzled
//         shared memory and the tensor core reads them; no ALU touches a weight bit
//   FP4   kind::f8f6f4 with an e2m1 A operand: the 4-bit tensor-map type unpacks sixteen packed
//         codes (8 bytes) into each 16-byte slot of the swizzled tile; again no ALU
//   I4    TMA brings the packed nibbles (64 bytes per row and K block); transform warps widen them
//         in shared memory to int8 holding 16*q (two logic operations per eight weights) for
//         kind::i8
//   I4CB  TMA brings the nibbles and the block scales; transform warps write fp16 of
//         block scale x centroid (one rounding) for kind::f16
//
// Orientation: the weight tile is the MMA's M operand and the batch is its N operand, so the same
// kernel serves one batch row and thousands:
//     D[n, (t,m)] += W[n, k] * Aq_t[m, k]          (accumulators in TMEM, 128 lanes = n)
// f32 activations are first rewritten by `act_prep_kernel` as T narrow terms per element
//   int8:  a ~= dq[m] * (128*hi + lo)             (15-bit fixed point per row, T = 2)
//   e4m3:  a ~= dq[m] * (t1 + t2 + t3)            (three 4-bit-significand terms, T = 3)
//   fp16:  one term (codebook format)
// The epilogue reads the accumulators with tcgen05.ld, recombines the terms and applies
//     out[m,n] = act(dq[m]*scale[n]*acc + zero[n]*sum_k a[m,k] + bias[n])
// (src/backend/cpu/microkernels/gemm.rs:2048-2087, src/backend/cpu/matmul.rs:61-71).
//
// Warp roles: warp 0 = TMA producer and TMEM owner, warp 1 = MMA issuer, warps 2-9 = epilogue (a TMEM
// lane quadrant each, two warps per quadrant), warps 10-17 = transform (I4 / I4CB only).  Every
// mbarrier wait is bounded: a wait that runs out raises the context's error flag, every role leaves
// its loop, TMEM is freed and the kernel returns.
#include "common.cuh"

#include <algorithm>
#include <cuda.h>
#include <cuda_fp8.h>

namespace fnn {

namespace {

constexpr int kTileN = 128;        // weight rows (output channels) per CTA tile = MMA M
constexpr int kKBlockBytes = 128;  // bytes of K per pipeline stage = one 128B swizzle row
constexpr int kEpiWarps = 8;                      // two per TMEM lane quadrant
constexpr int kXfWarps = 8;                       // transform warps (formats widened in shared memory)
constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: far beyond any legitimate wait

enum { KIND_I8 = 0, KIND_F8 = 1, KIND_F16 = 2 };
// How the weight tile reaches the MMA: straight from TMA (I8, FP8, FP4), or through the transform
// warps (I4 -> int8, codebook -> fp16).
enum { WF_TMA = 0, WF_I4 = 1, WF_CB = 2 };
constexpr int kFmtE4M3 = 0, kFmtE2M1 = 5;        // operand format codes of kind::f8f6f4

// ---- PTX wrappers -------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after raising the error flags) if the phase never completes or
// another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *err_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) {
            *abort_flag = 1;
            atomicOr(err_flag, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0,
                                            int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
// Brings a tensor map (a kernel parameter) into the descriptor cache ahead of its first copy.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap *map, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1),
                 "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    if (KIND == KIND_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if (KIND == KIND_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// 32 lanes x 16 consecutive 32-bit columns of TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128B-swizzled
// (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);  // start address / 16
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                       // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                       // layout type: SWIZZLE_128B
    return d;
}

// Instruction descriptor: D format, A/B formats, K-major both, N (>>3) and M (>>4).  `a_fmt`: the
// A operand's format code for kind::f8f6f4 (e4m3 or e2m1); B is e4m3 there.  Format 0 is F16 for
// kind::f16.
__host__ __device__ constexpr uint32_t make_idesc(int kind, int n_cols, int a_fmt) {
    return (kind == KIND_I8 ? (2u << 4) | (1u << 7) | (1u << 10)   // S32 accum, signed 8-bit A and B
                            : (1u << 4) | ((uint32_t)a_fmt << 7) | (0u << 10))  // F32 accum
           | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
}
// generic-proxy writes to shared memory -> visible to the async proxy (the tensor core's reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One activation, already divided by the row's step, as T narrow terms: an int8 pair hi * 128 + lo
// (15 bits), or an e4m3 code followed by the codes of what the earlier terms left over.
template <int KIND, int T>
__device__ __forceinline__ void split_terms(float x, uint8_t t[3]) {
    if (KIND == KIND_I8) {
        int q = __float2int_rn(x);
        q = max(-16256, min(16256, q));
        const int hi = (q + 64) >> 7;
        const int lo = q - hi * 128;
        t[0] = (uint8_t)(int8_t)hi;
        t[1] = (uint8_t)(int8_t)lo;
    } else {
        float r = x;
#pragma unroll
        for (int i = 0; i < T; ++i) {
            __nv_fp8_storage_t c = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
            t[i] = (uint8_t)c;
            r -= __half2float(__half(__nv_cvt_fp8_to_halfraw(c, __NV_E4M3)));
        }
    }
}

// The activations are written by the kernel before this one on the stream, so they may only be
// read after griddepcontrol.wait.  A load through a `const __restrict__` pointer counts as invariant
// for the compiler, which may then move it above the wait (it did: a chain of layers read the
// previous run's activations).  The activation pointers of these kernels therefore carry no
// __restrict__, and the unrolled loads of the register form are volatile asm, which keeps its place
// after the (volatile asm) wait.
__device__ __forceinline__ float4 ld_after_wait(const float4 *p) {
    float4 v;
    asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// ---- activation rewrite ---------------------------------------------------------------------
// One block per batch row.  Writes T byte planes Bq[t][m][Kp] (rows zero-padded to Kp), the
// per-row factor dq[m] and the row sum.  PERM8: inside every group of eight k the bytes are stored
// in the order 0,2,4,6,1,3,5,7 -- the order in which the I4 transform emits its weights.
template <int KIND, int T, bool PERM8>
__global__ void __launch_bounds__(256)
act_prep_kernel(const float *act, int M, int K, int Kp, int Mpad, uint8_t *bq, float *dq, float *rowsum) {
    __shared__ float s_max[8], s_sum[8];
    // reads the activations and overwrites planes the previous tensor-core kernel may still read
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    const float *row = act + (size_t)m * K;
    float mx = 0.0f, sum = 0.0f;
    for (int k = tid; k < K; k += 256) {
        float a = row[k];
        mx = fmaxf(mx, fabsf(a));
        sum += a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    }
    if ((tid & 31) == 0) {
        s_max[tid >> 5] = mx;
        s_sum[tid >> 5] = sum;
    }
    __syncthreads();
    mx = 0.0f;
    sum = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        mx = fmaxf(mx, s_max[w]);
        sum += s_sum[w];
    }
    if (KIND == KIND_F16) {
        // one fp16 term; the row is scaled by a power of two so that its largest element sits just
        // below 2^15 (exact, any f32 magnitude fits): bq is [Mpad][Kp bytes] of halves
        int ex = 15;
        if (mx > 0.0f && isfinite(mx)) (void)frexpf(mx, &ex);
        const int e = max(-120, min(120, 15 - ex));
        const float up = ldexpf(1.0f, e);
        if (tid == 0) {
            dq[m] = ldexpf(1.0f, -e);
            rowsum[m] = sum;
        }
        __half *dst = reinterpret_cast<__half *>(bq + (size_t)m * Kp);
        for (int k = tid; k < Kp / 2; k += 256) dst[k] = __float2half_rn(k < K ? row[k] * up : 0.0f);
        return;
    }
    const float full = (KIND == KIND_I8) ? 16256.0f : 448.0f;
    const float step = (mx > 0.0f && isfinite(mx)) ? mx / full : 1.0f;
    const float inv = 1.0f / step;
    if (tid == 0) {
        dq[m] = step;
        rowsum[m] = sum;
    }
    for (int k = tid; k < Kp; k += 256) {
        uint8_t t[3];
        split_terms<KIND, T>((k < K) ? row[k] * inv : 0.0f, t);
        const int i8 = k & 7;
        const int kk = PERM8 ? ((k & ~7) | ((i8 >> 1) + (i8 & 1) * 4)) : k;
#pragma unroll
        for (int i = 0; i < T; ++i) bq[((size_t)i * Mpad + m) * Kp + kk] = t[i];
    }
}

// The same rewrite for rows of a multiple of 8 and at most 16384 elements that start on 16 bytes
// (every layer of a real model): the row is read once, eight consecutive elements per thread and
// step with all loads in flight together, stays in registers between the scan and the rewrite, and
// every plane is written eight bytes at a time.
constexpr int kPrepHold = 8;   // units of eight elements a thread can hold
template <int KIND, int T, bool PERM8>
__global__ void __launch_bounds__(256)
act_prep_regs_kernel(const float *act, int M, int K, int Kp, int Mpad, uint8_t *bq, float *dq, float *rowsum) {
    __shared__ float s_max[8], s_sum[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    const float4 *row4 = reinterpret_cast<const float4 *>(act + (size_t)m * K);
    const int units = K >> 3;
    float v[kPrepHold][8];
#pragma unroll
    for (int i = 0; i < kPrepHold; ++i) {
        const int u = tid + i * 256;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (u < units) {
            a = ld_after_wait(row4 + 2 * u);
            b = ld_after_wait(row4 + 2 * u + 1);
        }
        v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
        v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
    }
    float mx = 0.0f, sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kPrepHold; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            mx = fmaxf(mx, fabsf(v[i][j]));
            sum += v[i][j];
        }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    }
    if ((tid & 31) == 0) {
        s_max[tid >> 5] = mx;
        s_sum[tid >> 5] = sum;
    }
    __syncthreads();
    mx = 0.0f;
    sum = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        mx = fmaxf(mx, s_max[w]);
        sum += s_sum[w];
    }
    if (KIND == KIND_F16) {
        int ex = 15;
        if (mx > 0.0f && isfinite(mx)) (void)frexpf(mx, &ex);
        const int e = max(-120, min(120, 15 - ex));
        const float up = ldexpf(1.0f, e);
        if (tid == 0) {
            dq[m] = ldexpf(1.0f, -e);
            rowsum[m] = sum;
        }
        uint4 *dst = reinterpret_cast<uint4 *>(bq + (size_t)m * Kp);   // Kp = 2 K bytes here
#pragma unroll
        for (int i = 0; i < kPrepHold; ++i) {
            const int u = tid + i * 256;
            if (u >= units) continue;
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 x = __floats2half2_rn(v[i][2 * j] * up, v[i][2 * j + 1] * up);
                h[j] = *reinterpret_cast<const uint32_t *>(&x);
            }
            dst[u] = make_uint4(h[0], h[1], h[2], h[3]);
        }
        return;
    }
    const float full = (KIND == KIND_I8) ? 16256.0f : 448.0f;
    const float step = (mx > 0.0f && isfinite(mx)) ? mx / full : 1.0f;
    const float inv = 1.0f / step;
    if (tid == 0) {
        dq[m] = step;
        rowsum[m] = sum;
        if (Kp > K) {   // K is 8 mod 16: one more unit of zeros pads the row to 16 bytes
#pragma unroll
            for (int i = 0; i < T; ++i)
                *reinterpret_cast<uint2 *>(bq + ((size_t)i * Mpad + m) * Kp + K) = make_uint2(0u, 0u);
        }
    }
#pragma unroll
    for (int i = 0; i < kPrepHold; ++i) {
        const int u = tid + i * 256;
        if (u >= units) continue;
        uint32_t w[T][2];
#pragma unroll
        for (int t = 0; t < T; ++t) w[t][0] = w[t][1] = 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint8_t t[3];
            split_terms<KIND, T>(v[i][j] * inv, t);
            const int pos = PERM8 ? ((j >> 1) + (j & 1) * 4) : j;
#pragma unroll
            for (int q = 0; q < T; ++q) w[q][pos >> 2] |= (uint32_t)t[q] << (8 * (pos & 3));
        }
#pragma unroll
        for (int q = 0; q < T; ++q)
            *reinterpret_cast<uint2 *>(bq + ((size_t)q * Mpad + m) * Kp + (size_t)u * 8) = make_uint2(w[q][0], w[q][1]);
    }
}

// The epilogue arithmetic of one chunk: 16 batch rows of one output channel.  `fac` carries the
// rows' dq (lanes 0-15) and row sums (lanes 16-31).  No branches: EPI is a compile-time constant.
template <int KIND, int T, int EPI>
__device__ __forceinline__ void finish_chunk(const uint32_t (&r)[T][16], float fac, float scale, float zero,
                                             float bias, bool has_bias, float acc_scale, float (&v)[16]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float dq_m = __shfl_sync(0xFFFFFFFFu, fac, j);
        const float rs_m = __shfl_sync(0xFFFFFFFFu, fac, 16 + j);
        float acc;
        if (T == 1)
            acc = __uint_as_float(r[0][j]);
        else if (KIND == KIND_I8)
            acc = ((float)(int)r[0][j] * 128.0f + (float)(int)r[T > 1 ? 1 : 0][j]) * acc_scale;
        else if (T == 3)
            acc = (__uint_as_float(r[0][j]) + __uint_as_float(r[T > 1 ? 1 : 0][j])) + __uint_as_float(r[T - 1][j]);
        else
            acc = __uint_as_float(r[0][j]) + __uint_as_float(r[T > 1 ? 1 : 0][j]);
        // dot*scale + zero*sum(a) with the reference's separate roundings, then act(x + bias)
        const float x = __fadd_rn(__fmul_rn(acc * dq_m, scale), __fmul_rn(zero, rs_m));
        v[j] = apply_act_fast(has_bias ? __fadd_rn(x, bias) : x, EPI);
    }
}

// ---- main kernel ------------------------------------------------------------------------------

struct TcParams {
    const float *scales;
    const float *zeros;
    const float *bias;
    const float *dq;
    const float *rowsum;
    const float *codebook;   // WF_CB: 16 centroids
    float *out;
    int *err_flag;
    int M, N, K;
    int Mb;        // batch rows per tile
    int n_tiles, m_tiles;
    int kblocks;   // pipeline stages' worth of K: ceil(operand bytes per row / (128 * atoms))
    AllGatherArgs ag;   // ag.world > 0: outputs go to every rank's gathered buffer
    // Work split along K as well as over tiles (layers with too few tiles to give every SM one): every CTA
    // takes an equal, contiguous share of all (tile, K block) steps; where a share ends inside a tile
    // the CTAs that hold the tile's later K blocks leave their raw accumulators in `sk_ws` and raise
    // their flag, and the CTA that holds its first K block adds them up in CTA order and finishes it.
    int sk_steps;        // steps per CTA; 0: every CTA takes whole tiles
    float *sk_ws;        // [grid][T * Mb columns][128 rows] raw accumulators (int32 bits for kind::i8)
    unsigned *sk_flags;  // [grid] epilogue warps of a CTA that have stored their part of its partial (0 .. 8);
                         // [1024 + grid] epilogue warps of the finishing CTA that have consumed it
    int a_fmt;     // A operand format of kind::f8f6f4
    float acc_scale;   // 1/16 when the int8 operand carries 16*q (I4)
    int stages;
    int epilogue;
};

// The sequence of (tile, K block range) segments one CTA works through; every role of the CTA walks it
// with its own copy.  Whole tiles, blockIdx.x + i * gridDim.x, when sk_steps == 0; otherwise the
// CTA's contiguous share [blockIdx.x * sk_steps, +sk_steps) of the linear (tile, K block) space, cut
// at tile boundaries.
struct Segments {
    int kblocks, total_tiles, sk_steps;
    long long cur, end;   // linear step range (split mode)
    int tile;             // next tile (whole-tile mode)
    __device__ Segments(const TcParams &p, int total) : kblocks(p.kblocks), total_tiles(total), sk_steps(p.sk_steps) {
        cur = (long long)blockIdx.x * sk_steps;
        end = min(cur + sk_steps, (long long)total * kblocks);
        tile = blockIdx.x;
    }
    __device__ bool next(int &t, int &kb0, int &kb1) {
        if (sk_steps == 0) {
            if (tile >= total_tiles) return false;
            t = tile;
            kb0 = 0;
            kb1 = kblocks;
            tile += gridDim.x;
            return true;
        }
        if (cur >= end) return false;
        t = (int)(cur / kblocks);
        kb0 = (int)(cur - (long long)t * kblocks);
        kb1 = (int)min((long long)kblocks, kb0 + (end - cur));
        cur += kb1 - kb0;
        return true;
    }
};

// ATOMS: 128-byte swizzle atoms of K per pipeline stage (2 for fp16 operands: a stage is 128 k for
// every format).  Shared memory per stage: operand tile, raw tile (transformed formats), activations.
template <int KIND, int T, int WF>
__global__ void __launch_bounds__((2 + kEpiWarps + (WF == WF_TMA ? 0 : kXfWarps)) * 32, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
              const __grid_constant__ CUtensorMap map_s, TcParams p) {
    constexpr int ATOMS = (KIND == KIND_F16) ? 2 : 1;
    constexpr int kRawBytes = (WF == WF_TMA) ? 0 : kTileN * 64;        // packed nibbles: 64 bytes per row
    constexpr int kScBytes = (WF == WF_CB) ? kTileN * 16 : 0;          // four block scales per row
    constexpr int kXf0 = 2 + kEpiWarps;                                // first transform warp
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment is what the 128B swizzle atoms need
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int BNt = T * p.Mb;                               // MMA N: (term, batch row) columns
    const int a_atom = kTileN * kKBlockBytes;               // 16 KB operand atom
    const int a_bytes = ATOMS * a_atom;
    const int b_bytes = BNt * kKBlockBytes;                 // activation atom
    const int b_atom = (b_bytes + 1023) & ~1023;
    const int b_stride = ATOMS * b_atom;
    unsigned char *s_a = smem;
    unsigned char *s_b = s_a + (size_t)p.stages * a_bytes;
    unsigned char *s_raw = s_b + (size_t)p.stages * b_stride;             // [stages][raw | scales]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_raw + (size_t)p.stages * (kRawBytes + kScBytes));
    uint64_t *full = bars, *empty = bars + p.stages, *rawfull = bars + 2 * p.stages;
    uint64_t *tfull = bars + 3 * p.stages, *tempty = tfull + 2;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);
    float *s_cb = reinterpret_cast<float *>(s_tmem + 2);                  // [16]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();   // barrier set-up and the TMEM allocation below run under the previous kernel's tail
    // TMEM columns: two accumulator buffers of BNt columns, power of two >= 32
    uint32_t ncols = 32;
    while ((int)ncols < 2 * BNt) ncols <<= 1;

    const int total_tiles = p.n_tiles * p.m_tiles;
    // weights of stage `st`: the operand tile itself, or the packed nibbles (+ block scales) for the
    // transform warps
    auto load_w = [&](int st, int nt, int kb) {
        if (WF == WF_TMA) {
#pragma unroll
            for (int at = 0; at < ATOMS; ++at)
                tma_load_2d(s_a + (size_t)st * a_bytes + at * a_atom, &map_w, &full[st],
                            (kb * ATOMS + at) * kKBlockBytes, nt * kTileN);
        } else {
            unsigned char *raw = s_raw + (size_t)st * (kRawBytes + kScBytes);
            mbar_expect_tx(&rawfull[st], (uint32_t)(kRawBytes + kScBytes));
            tma_load_2d(raw, &map_w, &rawfull[st], kb * 64, nt * kTileN);
            if (WF == WF_CB) tma_load_2d(raw + kRawBytes, &map_s, &rawfull[st], kb * 16, nt * kTileN);
        }
    };
    // bytes the copies of a stage report to its barrier; the unpacking 4-bit tensor-map type counts
    // the packed source bytes (half of the 16 KB tile it writes)
    const uint32_t full_tx =
        (uint32_t)((WF == WF_TMA ? (p.a_fmt == kFmtE2M1 ? a_bytes / 2 : a_bytes) : 0) + ATOMS * b_bytes);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
        if (WF == WF_CB) prefetch_tensormap(&map_s);
        for (int s = 0; s < p.stages; ++s) {
            // the MMA issuer waits for the activation tile (one arrival with a byte count) and, for the
            // formats widened in shared memory, for every transform warp
            mbar_init(&full[s], 1 + (WF == WF_TMA ? 0 : kXfWarps));
            mbar_init(&empty[s], 1);
            mbar_init(&rawfull[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], kEpiWarps);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // This thread is the TMA producer.  The weights do not depend on the kernel before this one on
        // the stream: the first ring of weight tiles is requested here, before the rest of the CTA
        // has finished setting up and before griddepcontrol.wait; the matching activation tiles
        // follow in the producer's loop.
        Segments segs(p, total_tiles);
        int tile, kb0, kb1;
        if (segs.next(tile, kb0, kb1)) {
            const int head = min(p.stages, kb1 - kb0), nt = tile / p.m_tiles;
            for (int i = 0; i < head; ++i) {
                mbar_expect_tx(&full[i], full_tx);   // stage i: all stages start empty
                load_w(i, nt, kb0 + i);
            }
            // The activation planes may still be being written: an L2 prefetch of the first tile reads
            // nothing into this SM, but it has the address translated before the copies that follow
            // griddepcontrol.wait ask for it (L2 is the point of coherence, so nothing stale can result).
            tma_prefetch_3d(&map_a, kb0 * ATOMS * kKBlockBytes, (tile % p.m_tiles) * p.Mb, 0);
        }
    }
    if (WF == WF_CB && threadIdx.x >= 64 && threadIdx.x < 80) s_cb[threadIdx.x - 64] = p.codebook[threadIdx.x - 64];
    if (warp == 1) {   // the MMA warp owns the tensor memory: it allocates and frees it
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(s_tmem)),
                     "r"(ncols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto load_b = [&](int st, int mt, int kb) {
#pragma unroll
                for (int at = 0; at < ATOMS; ++at)
                    tma_load_3d(s_b + (size_t)st * b_stride + at * b_atom, &map_a, &full[st],
                                (kb * ATOMS + at) * kKBlockBytes, mt * p.Mb, 0);
            };
            // The first ring of weight tiles is already on its way (requested during set-up); the
            // activation planes depend on the kernel before this one: their tiles follow
            // griddepcontrol.wait.
            Segments segs(p, total_tiles);
            int tile, kb0, kb1;
            bool have = segs.next(tile, kb0, kb1);
            const int head = have ? min(p.stages, kb1 - kb0) : 0;
            if (head > 0) {
                const int mt = tile % p.m_tiles;
                pdl_wait();
                for (int i = 0; i < head; ++i) load_b(i, mt, kb0 + i);
                s = head;
                if (s == p.stages) {
                    s = 0;
                    phase ^= 1;
                }
            } else {
                pdl_wait();
            }
            bool first = true;
            for (; have && ok; have = segs.next(tile, kb0, kb1)) {
                const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
                for (int kb = kb0 + (first ? head : 0); kb < kb1; ++kb) {
                    if (!mbar_wait(&empty[s], phase ^ 1, s_abort, p.err_flag, 0x10)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], full_tx);
                    load_w(s, nt, kb);
                    load_b(s, mt, kb);
                    if (++s == p.stages) {
                        s = 0;
                        phase ^= 1;
                    }
                }
                first = false;
            }
            if (!ok) {  // let copies already in flight land before the CTA can exit
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(KIND, BNt, p.a_fmt);
            int s = 0;
            uint32_t phase = 0;
            int as = 0;
            uint32_t aphase = 0;
            bool ok = true;
            Segments segs(p, total_tiles);
            int tile, kb0, kb1;
            while (ok && segs.next(tile, kb0, kb1)) {
                if (!mbar_wait(&tempty[as], aphase ^ 1, s_abort, p.err_flag, 0x20)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BNt);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full[s], phase, s_abort, p.err_flag, 0x40)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int at = 0; at < ATOMS; ++at) {
                        const uint64_t da = make_desc_sw128(smem_u32(s_a + (size_t)s * a_bytes + at * a_atom));
                        const uint64_t db = make_desc_sw128(smem_u32(s_b + (size_t)s * b_stride + at * b_atom));
#pragma unroll
                        for (int k = 0; k < kKBlockBytes / 32; ++k) {
                            // advance both operands by 32 bytes of K inside the swizzled row
                            tc_mma<KIND>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                                         (kb > kb0 || at > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    tc_commit(&empty[s]);  // frees the stage once these MMAs have read it
                    if (++s == p.stages) {
                        s = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                tc_commit(&tfull[as]);  // accumulator complete
                if (++as == 2) {
                    as = 0;
                    aphase ^= 1;
                }
            }
        }
    } else if (WF != WF_TMA && warp >= kXf0) {
        // ---------------- transform warps: packed nibbles -> operand tile ----------------
        // All transform warps work on every pipeline step together (every warp meets every phase of
        // every barrier in order, which is what a parity wait needs; letting warps run steps apart
        // would let one of them see a barrier two phases behind and take it for ready).  A work item is
        // one 16-byte unit of a row (32 codes = one scale block of the codebook format); consecutive
        // threads take consecutive units, so the reads of the raw tile are contiguous, and the writes
        // follow the 128-byte swizzle (16-byte chunk index XOR row mod 8).
        const int xt = threadIdx.x - kXf0 * 32;
        int s = 0;
        uint32_t phase = 0;
        bool ok = true;
        Segments segs(p, total_tiles);
        int tile, kb0, kb1;
        while (ok && segs.next(tile, kb0, kb1)) {
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!mbar_wait(&rawfull[s], phase, s_abort, p.err_flag, 0x200)) {
                    ok = false;
                    break;
                }
                const unsigned char *raw = s_raw + (size_t)s * (kRawBytes + kScBytes);
                unsigned char *dst = s_a + (size_t)s * a_bytes;
#pragma unroll
                for (int it = 0; it < (kTileN * 4) / (kXfWarps * 32); ++it) {
                    const int item = xt + it * kXfWarps * 32;
                    const int row = item >> 2, c = item & 3;
                    const uint4 w = *reinterpret_cast<const uint4 *>(raw + item * 16);
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                    if (WF == WF_I4) {
                        // 16*q as int8: even codes of a word, then odd codes (the activation planes
                        // carry the same order inside every group of eight k)
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            o[2 * j] = (ww[j] << 4) & 0xF0F0F0F0u;
                            o[2 * j + 1] = ww[j] & 0xF0F0F0F0u;
                        }
                        unsigned char *r = dst + row * 128;
                        *reinterpret_cast<uint4 *>(r + (((2 * c) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4 *>(r + (((2 * c + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    } else {
                        // fp16 of block scale x centroid, one rounding; the unit is one scale block
                        const float bs = *reinterpret_cast<const float *>(raw + kRawBytes + row * 16 + c * 4);
                        unsigned char *r = dst + (c >> 1) * a_atom + row * 128;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t h[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float lo = __fmul_rn(bs, s_cb[(ww[j] >> (8 * q)) & 0xFu]);
                                const float hi = __fmul_rn(bs, s_cb[(ww[j] >> (8 * q + 4)) & 0xFu]);
                                const __half2 v = __floats2half2_rn(lo, hi);
                                h[q] = *reinterpret_cast<const uint32_t *>(&v);
                            }
                            *reinterpret_cast<uint4 *>(r + ((((c & 1) * 4 + j) ^ (row & 7)) << 4)) =
                                make_uint4(h[0], h[1], h[2], h[3]);
                        }
                    }
                }
                fence_proxy_async();   // these stores are read by the tensor core (async proxy)
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
                if (++s == p.stages) {
                    s = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp < kXf0) {
        // ---------------- epilogue (8 warps: a TMEM lane quadrant each, two warps per quadrant
        // taking alternate 16-column chunks) ----------------
        pdl_wait();   // dq, rowsum and the output buffer belong to kernels before this one
        const int quad = warp & 3;
        const int chunk0 = ((warp - 2) >> 2) * 16;
        int as = 0;
        uint32_t aphase = 0;
        const bool has_zero = p.zeros != nullptr;
        Segments segs(p, total_tiles);
        int tile, kb0, kb1;
        const int row = quad * 32 + lane;            // this thread's row of the tile = its TMEM lane
        // dq and rowsum of a chunk's 16 batch rows, spread over the lanes (lane j: dq, lane 16 + j: rowsum)
        auto load_rowfac = [&](int mt, int c0) -> float {
            const int j = lane & 15, m = mt * p.Mb + c0 + j;
            const bool want = c0 + j < p.Mb && m < p.M && (lane < 16 || has_zero);
            return want ? (lane < 16 ? p.dq : p.rowsum)[m] : 0.0f;
        };
        while (segs.next(tile, kb0, kb1)) {
            const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
            // Everything the epilogue needs besides the accumulator is requested before the wait for
            // it, so these loads (a trip to L2 or HBM each) run under the tile's main loop.
            const int n = nt * kTileN + row;
            const bool n_ok = n < p.N;
            float scale = 0.0f, zero = 0.0f, bias = 0.0f, fac = 0.0f;
            if (kb0 == 0) {
                scale = n_ok ? (p.scales ? __ldg(p.scales + n) : 1.0f) : 0.0f;
                zero = (n_ok && has_zero) ? __ldg(p.zeros + n) : 0.0f;
                bias = (n_ok && p.bias) ? p.bias[n] : 0.0f;
                fac = load_rowfac(mt, chunk0);
            }
            if (!mbar_wait(&tfull[as], aphase, s_abort, p.err_flag, 0x80)) break;
            tc_fence_after();
            const uint32_t t_base = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(as * BNt);
            if (kb0 > 0) {
                // A later part of a tile's K range: leave the raw accumulators for the CTA that holds
                // the tile's first K blocks ([column][row]: a warp stores 32 consecutive rows).
                float *ws = p.sk_ws + (size_t)blockIdx.x * BNt * kTileN;
                for (int c0 = chunk0; c0 < p.Mb; c0 += 16 * (kEpiWarps / 4)) {
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        uint32_t x[16];
                        tmem_ld16(t_base + (uint32_t)(t * p.Mb + c0), x);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < p.Mb) ws[(size_t)(t * p.Mb + c0 + j) * kTileN + row] = __uint_as_float(x[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&tempty[as]);
                    // this warp's part of the partial is stored: count it in (release); the finishing
                    // CTA reads once all eight warps have
                    __threadfence();
                    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sk_flags + blockIdx.x) : "memory");
                }
            } else {
                // This CTA finishes the tile.  If its share ended before the tile's last K block, the next
                // CTA(s) hold the rest: wait (bounded) for their partials and add them in CTA order.
                const int others = (kb1 < p.kblocks) ? (p.kblocks - kb1 + p.sk_steps - 1) / p.sk_steps : 0;
                bool partials_ok = true;
                for (int o = 1; o <= others; ++o) {
                    const unsigned *flag = p.sk_flags + blockIdx.x + o;
                    const long long t0 = clock64();
                    for (;;) {
                        unsigned f;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(flag) : "memory");
                        if (f >= (unsigned)kEpiWarps) break;
                        if (*s_abort || clock64() - t0 > kWaitCycles) {
                            *s_abort = 1;
                            atomicOr(p.err_flag, 0x800);
                            partials_ok = false;
                            break;
                        }
                    }
                    if (!partials_ok) break;
                }
                for (int c0 = chunk0; c0 < p.Mb && partials_ok; c0 += 16 * (kEpiWarps / 4)) {
                    uint32_t r[T][16];
#pragma unroll
                    for (int t = 0; t < T; ++t) tmem_ld16(t_base + (uint32_t)(t * p.Mb + c0), r[t]);
                    const float fac_next = load_rowfac(mt, c0 + 16 * (kEpiWarps / 4));   // next chunk's
                    tmem_ld_wait();
                    for (int o = 1; o <= others; ++o) {
                        const float *ws = p.sk_ws + (size_t)(blockIdx.x + o) * BNt * kTileN;
#pragma unroll
                        for (int t = 0; t < T; ++t) {
                            // all 16 loads of a term in flight together (a warp reads 32 consecutive rows)
                            uint32_t x[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                x[j] = (c0 + j < p.Mb)
                                           ? __float_as_uint(__ldcg(ws + (size_t)(t * p.Mb + c0 + j) * kTileN + row))
                                           : 0u;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                r[t][j] = (KIND == KIND_I8)
                                              ? (uint32_t)((int)r[t][j] + (int)x[j])
                                              : __float_as_uint(__uint_as_float(r[t][j]) + __uint_as_float(x[j]));
                        }
                    }
                    // The 16 outputs are computed in straight-line code (one specialisation per
                    // activation, no branch per output: with a branch per output the two warps a
                    // scheduler has here ran them one after another at full instruction latency), then
                    // stored under a predicate.
                    float v[16];
                    switch (p.epilogue) {
                    case FNN_EPI_RELU:
                        finish_chunk<KIND, T, FNN_EPI_RELU>(r, fac, scale, zero, bias, p.bias != nullptr, p.acc_scale, v);
                        break;
                    case FNN_EPI_GELU:
                        finish_chunk<KIND, T, FNN_EPI_GELU>(r, fac, scale, zero, bias, p.bias != nullptr, p.acc_scale, v);
                        break;
                    case FNN_EPI_SILU:
                        finish_chunk<KIND, T, FNN_EPI_SILU>(r, fac, scale, zero, bias, p.bias != nullptr, p.acc_scale, v);
                        break;
                    default:
                        finish_chunk<KIND, T, FNN_EPI_NONE>(r, fac, scale, zero, bias, p.bias != nullptr, p.acc_scale, v);
                        break;
                    }
                    const int m0 = mt * p.Mb + c0;
                    const int jmax = n_ok ? min(16, min(p.Mb - c0, p.M - m0)) : 0;   // rows of this chunk that exist
                    if (p.ag.world == 0) {   // a warp writes 32 consecutive n
                        float *dst = p.out + (size_t)m0 * p.N + n;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < jmax) dst[(size_t)j * p.N] = v[j];
                    } else {   // plain peer stores over NVLink (and one local store)
                        const size_t at = (size_t)m0 * p.ag.n_total + p.ag.col0 + n;
                        for (int rk = 0; rk < p.ag.world; ++rk) {
                            float *dst = p.ag.peer_out[rk] + at;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (j < jmax) dst[(size_t)j * p.ag.n_total] = v[j];
                        }
                    }
                    fac = fac_next;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty[as]);
                if (lane == 0) {
                    // the last of the eight warps to have read a partial hands its counters back for the
                    // next launch (nobody else touches them until then)
                    for (int o = 1; o <= others; ++o) {
                        unsigned *done = p.sk_flags + 1024 + blockIdx.x + o;
                        if (atomicAdd(done, 1u) == (unsigned)kEpiWarps - 1u) {
                            *done = 0u;
                            p.sk_flags[blockIdx.x + o] = 0u;
                        }
                    }
                }
            }
            if (++as == 2) {
                as = 0;
                aphase ^= 1;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols)
                     : "memory");
    }
    if (p.ag.world > 0 && threadIdx.x == 32) {
        // Every store of this CTA happened before the barrier above.  A device-scope fence and a ticket
        // hand them to the CTA that leaves last on this rank; that one CTA makes everything visible
        // system-wide (one system-scope fence per launch: 148 of them at once cost about 10 us) and
        // adds one arrival to every rank's counter (release).  It then waits (bounded) until every
        // rank's arrival for this step is in before the kernel ends, so whatever follows on the
        // stream reads complete rows without a separate consumer kernel.  counters = {arrivals,
        // consumed} live in device memory and only grow: a captured graph can be replayed.
        __threadfence();
        const int ticket = atomicAdd(p.ag.ticket, 1);
        if (ticket == (int)gridDim.x - 1) {
            *p.ag.ticket = 0;
            __threadfence_system();
            for (int r = 0; r < p.ag.world; ++r)
                asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.ag.peer_arrive[r]) : "memory");
            unsigned *counters = p.ag.peer_arrive[p.ag.rank];
            const unsigned want = counters[1] + (unsigned)p.ag.world;
            const long long t0 = clock64();
            for (;;) {
                unsigned got;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(counters) : "memory");
                if ((int)(got - want) >= 0) {
                    counters[1] = want;
                    break;
                }
                if (clock64() - t0 > kWaitCycles) {   // gives up without consuming
                    atomicOr(p.err_flag, 0x400);
                    break;
                }
            }
        }
    }
}

// ---- host side -----------------------------------------------------------------------------------

// cuTensorMapEncodeTiled is looked up through the runtime, so the library itself carries no
// link-time dependency on libcuda (it must load, and fail cleanly, on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int encode_map(CUtensorMap *map, void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
               const cuuint32_t *box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B,
               CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        FNN_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres),
                       FNN_ERR_UNSUPPORTED);
        FNN_REQUIRE(fn != nullptr && qres == cudaDriverEntryPointSuccess, FNN_ERR_UNSUPPORTED,
                    "the CUDA driver does not provide cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(map, dtype, (cuuint32_t)rank, base, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(FNN_ERR_DISPATCH, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FNN_OK;
}

// Tensor map of the weight operand over the packed rows (row stride ld_u4 * 16 bytes).
//   I8 / FP8: 128 bytes x 128 rows per box, 128-byte swizzle: the operand tile itself.
//   FP4:      the 4-bit type that unpacks sixteen codes (8 bytes) into every 16-byte slot: 128 codes
//             x 128 rows per box, 128-byte swizzle.  Needs 32-byte aligned rows.
//   I4 / I4CB: the packed nibbles as bytes, 64 bytes x 128 rows, unswizzled (the transform warps
//             read them linearly).
int encode_weight_map(CUtensorMap *map, const fnn_cuda_qweight *w) {
    const cuuint64_t row_bytes = (cuuint64_t)w->ld_u4 * 16;
    cuuint64_t strides[1] = {row_bytes};
    if (w->fmt == FNN_FMT_I8 || w->fmt == FNN_FMT_F8) {
        cuuint64_t dims[2] = {(cuuint64_t)w->K, (cuuint64_t)w->N};
        cuuint32_t box[2] = {(cuuint32_t)kKBlockBytes, (cuuint32_t)kTileN};
        return encode_map(map, (void *)w->rows, 2, dims, strides, box);
    }
    if (w->fmt == FNN_FMT_F4) {
        cuuint64_t dims[2] = {row_bytes * 2, (cuuint64_t)w->N};   // in codes; a multiple of 128
        cuuint32_t box[2] = {128, (cuuint32_t)kTileN};
        return encode_map(map, (void *)w->rows, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B);
    }
    cuuint64_t dims[2] = {row_bytes, (cuuint64_t)w->N};
    cuuint32_t box[2] = {64, (cuuint32_t)kTileN};
    return encode_map(map, (void *)w->rows, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Scratch of one call: the rewritten activations Bq[T][Mpad][Kp], then dq[Mpad] and rowsum[Mpad].
// `fixed_scratch` null: the context's growable buffer; otherwise a caller-supplied region of
// `fixed_bytes` that must already be large enough (the entry point that may not allocate).
template <int KIND, int T, int WF>
int launch_tc(fnn_cuda_ctx *ctx, const QmmArgs &a, uint8_t *fixed_scratch = nullptr, size_t fixed_bytes = 0) {
    const fnn_cuda_qweight *w = a.w;
    constexpr int ES = (KIND == KIND_F16) ? 2 : 1;  // bytes per operand element
    constexpr int ATOMS = (KIND == KIND_F16) ? 2 : 1;
    const int M = (int)a.M, N = (int)w->N, K = (int)w->K;
    const int Kbytes = K * ES;
    const int Kp = (Kbytes + 15) & ~15;  // row bytes; TMA strides are multiples of 16 bytes
    // batch rows per tile: T*Mb is the MMA N (multiple of 16, at most 256)
    const int mb_max = (T == 1) ? 256 : (T == 2) ? 128 : 80;
    int Mb = std::min(mb_max, (M + 15) & ~15);
    const int m_tiles = (M + Mb - 1) / Mb;
    const int Mpad = m_tiles * Mb;

    const size_t bq_bytes = (size_t)T * Mpad * Kp;
    const size_t bq_al = (bq_bytes + 255) & ~(size_t)255;
    const size_t need = bq_al + (size_t)Mpad * 8 + 256;
    // A layer with few tiles and long K loops is bound by the per-CTA rate of those loops: a 128-byte
    // K block costs four MMA instructions of about 60 cycles each however few batch columns they
    // carry.  Such layers split every tile's K loop into `parts` shares on different SMs; the partial
    // accumulators of a tile meet in a workspace behind the activation planes and the CTA with the
    // first share adds them up.  `parts` comes from measured costs: a pipeline step of one CTA (0.35
    // us; 0.8 with two atoms per step), an extra partial for the finishing CTA to read (1 us per 128
    // accumulator columns) and about 3 us for the hand-over; shares shorter than that buy nothing.
    const int n_tiles = (N + kTileN - 1) / kTileN;
    const int kblocks = (Kbytes + kKBlockBytes * ATOMS - 1) / (kKBlockBytes * ATOMS);
    const int sms = std::min(ctx->sm_count, 1024);
    const int tiles = n_tiles * m_tiles;
    int parts = 1;
    if (!fixed_scratch && ctx->sk_flags != nullptr) {
        const double t_step = ATOMS == 2 ? 0.8 : 0.35, c_part = 0.5 + (double)(T * Mb) / 128.0;
        double best = 3.0;   // microseconds a split has to save before it is worth the hand-over
        for (int q = 2; q <= std::min(sms / std::max(tiles, 1), 12); ++q) {
            const double gain = kblocks * t_step * (1.0 - 1.0 / q) - c_part * (q - 1) - 3.0;
            if (gain > best) {
                best = gain;
                parts = q;
            }
        }
    }
    // More tiles than SMs, and a last wave that leaves many of them idle (224 tiles on 148 SMs): at
    // medium batch every CTA takes an equal share of all steps instead of whole tiles; a share then
    // starts and ends inside a tile, so a CTA hands over or adds at most one partial at either end.
    int even_steps = 0;
    if (parts == 1 && !fixed_scratch && ctx->sk_flags != nullptr && tiles > sms && T * Mb <= 128) {
        const double t_step = ATOMS == 2 ? 0.8 : 0.35, c_part = 0.5 + (double)(T * Mb) / 128.0;
        const long long steps = (long long)tiles * kblocks;
        const long long share = (steps + sms - 1) / sms;
        const double whole = (double)((tiles + sms - 1) / sms) * kblocks * t_step;
        const double even = (double)share * t_step + 2.0 * c_part + 3.0;
        if (whole - even > 3.0 && share >= 16) even_steps = (int)share;
    }
    const bool split_k = parts > 1 || even_steps > 0;
    const size_t ws_off = (need + 255) & ~(size_t)255;
    const size_t ws_bytes = split_k ? (size_t)sms * T * Mb * kTileN * 4 : 0;
    int rc = FNN_OK;
    uint8_t *bq;
    if (fixed_scratch) {
        FNN_REQUIRE(need <= fixed_bytes, FNN_ERR_MEMORY,
                    "qmatmul_noalloc: M=%d, K=%d needs %zu bytes of activation scratch; the built-in "
                    "scratch holds %zu (use fnn_cuda_qmatmul for larger problems)",
                    M, K, need, fixed_bytes);
        bq = fixed_scratch;
    } else {
        rc = ensure_scratch(ctx, ws_off + ws_bytes);
        if (rc != FNN_OK) return rc;
        bq = (uint8_t *)ctx->scratch;
    }
    float *dq = (float *)(bq + bq_al);
    float *rowsum = dq + Mpad;
    // Batch rows M .. Mpad of the planes are never written: a batch row is one column of the MMA, so
    // whatever those rows hold only reaches accumulator columns that the epilogue does not store.
    // same shared-memory carve-out as the main kernel: alternating carve-outs between consecutive
    // kernels makes every SM reconfigure (and drain) twice per call
    const bool regs_ok = K % 8 == 0 && K <= kPrepHold * 256 * 8 && (reinterpret_cast<uintptr_t>(a.a) & 15) == 0;
    auto prep = regs_ok ? act_prep_regs_kernel<KIND, T, WF == WF_I4> : act_prep_kernel<KIND, T, WF == WF_I4>;
    FNN_CUDA_CHECK(cudaFuncSetAttribute(prep, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(launch_pdl(prep, M, 256, 0, ctx, a.a, M, K, Kp, Mpad, bq, dq, rowsum),
                   FNN_ERR_DISPATCH);
    ctx->launches++;

    CUtensorMap map_w, map_a, map_s;
    rc = encode_weight_map(&map_w, w);
    if (rc != FNN_OK) return rc;
    {
        cuuint64_t dims[3] = {(cuuint64_t)Kp, (cuuint64_t)Mpad, (cuuint64_t)T};
        cuuint64_t strides[2] = {(cuuint64_t)Kp, (cuuint64_t)Kp * Mpad};
        cuuint32_t box[3] = {(cuuint32_t)kKBlockBytes, (cuuint32_t)Mb, (cuuint32_t)T};
        rc = encode_map(&map_a, bq, 3, dims, strides, box);
        if (rc != FNN_OK) return rc;
    }
    if (WF == WF_CB) {
        // block scales f32 [N][K/32] as bytes: four scales (16 bytes) per row and stage
        cuuint64_t dims[2] = {(cuuint64_t)w->blocks_per_row * 4, (cuuint64_t)w->N};
        cuuint64_t strides[1] = {(cuuint64_t)w->blocks_per_row * 4};
        cuuint32_t box[2] = {16, (cuuint32_t)kTileN};
        rc = encode_map(&map_s, (void *)w->scales, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != FNN_OK) return rc;
    } else {
        map_s = map_a;   // unused
    }
    TcParams p{};
    p.scales = (w->fmt == FNN_FMT_I4CB) ? nullptr : w->scales;  // block scales are folded into the operand
    p.zeros = w->zeros;
    p.bias = a.bias;
    p.dq = dq;
    p.rowsum = rowsum;
    p.codebook = w->codebook;
    p.out = a.out;
    p.err_flag = ctx->err_flag;
    p.M = M;
    p.N = N;
    p.K = K;
    p.Mb = Mb;
    p.n_tiles = n_tiles;
    p.m_tiles = m_tiles;
    p.kblocks = kblocks;
    p.a_fmt = (w->fmt == FNN_FMT_F4) ? kFmtE2M1 : kFmtE4M3;
    p.acc_scale = (WF == WF_I4) ? 0.0625f : 1.0f;
    p.epilogue = a.epilogue;
    if (a.allgather) p.ag = *a.allgather;
    const int a_bytes = ATOMS * kTileN * kKBlockBytes;
    const int b_stride = ATOMS * ((T * Mb * kKBlockBytes + 1023) & ~1023);
    const int raw_bytes = (WF == WF_TMA) ? 0 : kTileN * 64 + (WF == WF_CB ? kTileN * 16 : 0);
    int stages = (int)((200 * 1024) / (size_t)(a_bytes + b_stride + raw_bytes));
    stages = std::max(2, std::min(stages, 8));
    p.stages = stages;
    const size_t smem = 1024 + (size_t)stages * (a_bytes + b_stride + raw_bytes) + (3 * stages + 4) * 8 + 64 + 64;
    int grid = std::min(tiles, ctx->sm_count);
    if (split_k) {
        const long long steps = (long long)tiles * kblocks;
        p.sk_steps = even_steps > 0 ? even_steps : (kblocks + parts - 1) / parts;
        grid = (int)std::min<long long>(sms, (steps + p.sk_steps - 1) / p.sk_steps);
        p.sk_ws = (float *)(bq + ws_off);
        p.sk_flags = ctx->sk_flags;
    }
    const int threads = (2 + kEpiWarps + (WF == WF_TMA ? 0 : kXfWarps)) * 32;
    auto kern = qmm_tc_kernel<KIND, T, WF>;
    FNN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(launch_pdl(kern, grid, threads, smem, ctx, map_w, map_a, map_s, p), FNN_ERR_DISPATCH);
    ctx->launches++;
    ctx->last_path = fixed_scratch ? "tc-noalloc" : "tc";
    return FNN_OK;
}

}  // namespace

int dispatch_tc(fnn_cuda_ctx *ctx, const QmmArgs &a, uint8_t *fixed, size_t fixed_bytes);

bool qmm_tc_supported(const fnn_cuda_qweight *w, size_t M) {
    (void)M;
    // I8 / FP8 / FP4 codes are operands as stored; I4 and the codebook format are widened in shared
    // memory.  The codebook format becomes fp16 of block scale x centroid (only when those stay inside
    // the fp16 range) and its block scales travel by TMA, four per row and stage (K a multiple of 128).
    if (w->fmt == FNN_FMT_I4CB && (!w->fp16_ok || w->K % 128 != 0)) return false;
    return w->K >= 128 && w->N >= 1 && w->N < (1u << 30) && w->K < (1u << 29);
}

// Nothing to build: every format is read from the packed rows.
int prepare_qmm_tc(fnn_cuda_ctx *, fnn_cuda_qweight *) { return FNN_OK; }

// Format -> (MMA kind, activation terms, weight path).  `fixed`: caller-supplied scratch or null.
int dispatch_tc(fnn_cuda_ctx *ctx, const QmmArgs &a, uint8_t *fixed, size_t fixed_bytes) {
    switch (a.w->fmt) {
    case FNN_FMT_I8:
        return launch_tc<KIND_I8, 2, WF_TMA>(ctx, a, fixed, fixed_bytes);
    case FNN_FMT_I4:
        return launch_tc<KIND_I8, 2, WF_I4>(ctx, a, fixed, fixed_bytes);
    case FNN_FMT_F8:
    case FNN_FMT_F4:
        // three e4m3 terms keep f32-grade accuracy while the scan of the weights is the bound;
        // two terms (~1e-3 of the output norm) once the tensor core is
        return a.M >= 128 ? launch_tc<KIND_F8, 2, WF_TMA>(ctx, a, fixed, fixed_bytes)
                          : launch_tc<KIND_F8, 3, WF_TMA>(ctx, a, fixed, fixed_bytes);
    case FNN_FMT_I4CB:
        return launch_tc<KIND_F16, 1, WF_CB>(ctx, a, fixed, fixed_bytes);
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: tcgen05 path does not cover format %d", a.w->fmt);
}

int launch_qmm_tc(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    FNN_REQUIRE(a.M < (1u << 24), FNN_ERR_DISPATCH, "qmatmul: M=%zu too large for the tcgen05 path", a.M);
    return dispatch_tc(ctx, a, nullptr, 0);
}

}  // namespace fnn

// ---- entry point that allocates nothing ---------------------------------------------------------

namespace {
// Activation scratch of fnn_cuda_qmatmul_noalloc.  Lives in the module image: every GPU that
// loads the library holds these 8 MiB until the process exits.
constexpr size_t kNoAllocScratchBytes = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
// In host code the symbol above is only a stand-in; the device address is looked up once per
// device (with that device current) and kept here.
static void *g_noalloc_scratch_addr[64] = {};
}  // namespace

extern "C" int fnn_cuda_qmatmul_noalloc(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w, const float *a_dev,
                                        float *out_dev, const float *bias_dev, size_t M, int epilogue) {
    using namespace fnn;
    clear_error();
    FNN_REQUIRE(ctx && w && a_dev && out_dev, FNN_ERR_DISPATCH, "qmatmul_noalloc: null argument");
    FNN_REQUIRE(w->ctx->device == ctx->device, FNN_ERR_DISPATCH,
                "qmatmul_noalloc: weight lives on device %d, context on %d", w->ctx->device, ctx->device);
    FNN_REQUIRE(ctx->device >= 0 && ctx->device < 64, FNN_ERR_UNSUPPORTED,
                "qmatmul_noalloc: device index %d out of range", ctx->device);
    FNN_REQUIRE(epilogue >= FNN_EPI_NONE && epilogue <= FNN_EPI_SILU, FNN_ERR_DISPATCH,
                "qmatmul_noalloc: unknown epilogue %d", epilogue);
    FNN_REQUIRE(((uintptr_t)a_dev & 15u) == 0 && ((uintptr_t)out_dev & 15u) == 0, FNN_ERR_DISPATCH,
                "qmatmul_noalloc: pointers must be 16-byte aligned");
    FNN_REQUIRE(qmm_tc_supported(w, M), FNN_ERR_UNSUPPORTED,
                "qmatmul_noalloc: format %d / K=%zu is not served by this entry point", w->fmt, w->K);
    FNN_REQUIRE(M < (1u << 24), FNN_ERR_DISPATCH, "qmatmul_noalloc: M=%zu too large", M);
    if (M == 0) return FNN_OK;
    FNN_CUDA_CHECK(cudaSetDevice(ctx->device), FNN_ERR_DISPATCH);
    if (!g_noalloc_scratch_addr[ctx->device]) {
        void *ptr = nullptr;
        FNN_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch), FNN_ERR_MEMORY);
        FNN_REQUIRE(ptr != nullptr, FNN_ERR_MEMORY, "qmatmul_noalloc: scratch symbol has no address");
        g_noalloc_scratch_addr[ctx->device] = ptr;
    }
    uint8_t *scratch = (uint8_t *)g_noalloc_scratch_addr[ctx->device];
    QmmArgs args{w, a_dev, out_dev, bias_dev, M, epilogue};
    return dispatch_tc(ctx, args, scratch, kNoAllocScratchBytes);
}
