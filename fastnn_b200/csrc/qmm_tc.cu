// tcgen05 / TMEM / TMA kernel for the quantized MatMul.  I8 runs through kind::i8 and FP8-e4m3 through
// kind::f8f6f4 with no weight bit touched by an ALU: TMA drops the reference's own K-contiguous rows
// into 128-byte-swizzled shared memory and the tensor core reads them from there.  I4 (as int8), FP4
// (as the e4m3 code of the same value) and the codebook format (fp16 of block scale x centroid,
// kind::f16) read a tile-major, pre-swizzled expansion of their codes.
//
// Orientation: the weight tile is the MMA's M operand (128 output channels per CTA) and the
// batch is its N operand, so the same kernel serves one batch row and thousands:
//     D[n, (t,m)] += W[n, k] * Aq_t[m, k]          (accumulators in TMEM, 128 lanes = n)
// f32 activations are first rewritten by `act_prep_kernel` as T narrow terms per element
//   int8:  a ~= dq[m] * (128*hi + lo)             (15-bit fixed point per row, T = 2)
//   e4m3:  a ~= dq[m] * (t1 + t2 + t3)            (three 4-bit-significand terms, T = 3)
// which keeps the result within ~3e-4 of the f32-accumulated reference.  The epilogue reads the
// accumulators with tcgen05.ld, recombines the terms and applies
//     out[m,n] = act(dq[m]*scale[n]*acc + zero[n]*sum_k a[m,k] + bias[n])
// (src/backend/cpu/microkernels/gemm.rs:2048-2087, src/backend/cpu/matmul.rs:61-71).
//
// Warp roles (320 threads): warp 0 = TMA producer and TMEM owner, warp 1 = MMA issuer,
// warps 2-9 = epilogue (a TMEM lane quadrant each, two warps per quadrant).  Every mbarrier wait is bounded: a wait
// that runs out raises the context's error flag, every role leaves its loop, TMEM is freed and
// the kernel returns.
#include "common.cuh"

#include <algorithm>
#include <cuda.h>
#include <cuda_fp8.h>

namespace fnn {

namespace {

constexpr int kTileN = 128;        // weight rows (output channels) per CTA tile = MMA M
constexpr int kKBlockBytes = 128;  // bytes of K per pipeline stage = one 128B swizzle row
constexpr int kEpiWarps = 8;                      // two per TMEM lane quadrant
constexpr int kThreadsTc = (2 + kEpiWarps) * 32;
constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: far beyond any legitimate wait

enum { KIND_I8 = 0, KIND_F8 = 1, KIND_F16 = 2 };

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
// Untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
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

// Instruction descriptor: D format, A/B formats, K-major both, N (>>3) and M (>>4).
__host__ __device__ constexpr uint32_t make_idesc(int kind, int n_cols) {
    return (kind == KIND_I8 ? (2u << 4) | (1u << 7) | (1u << 10)   // S32 accum, signed 8-bit A and B
                            : (1u << 4) | (0u << 7) | (0u << 10))  // F32 accum; format 0 = E4M3 (f8f6f4) or F16 (f16)
           | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
}

// ---- activation rewrite ---------------------------------------------------------------------
// One block per batch row.  Writes T byte planes Bq[t][m][Kp] (rows zero-padded to Kp), the
// per-row factor dq[m] and the row sum.
template <int KIND, int T>
__global__ void __launch_bounds__(256)
act_prep_kernel(const float *__restrict__ act, int M, int K, int Kp, int Mpad, uint8_t *__restrict__ bq,
                float *__restrict__ dq, float *__restrict__ rowsum) {
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
    const float full = (KIND == KIND_I8) ? 16256.0f : 448.0f;
    if (KIND == KIND_F16) {
        // one fp16 term, no rescaling: bq is [Mpad][Kp bytes] of halves
        if (tid == 0) {
            dq[m] = 1.0f;
            rowsum[m] = sum;
        }
        __half *dst = reinterpret_cast<__half *>(bq + (size_t)m * Kp);
        for (int k = tid; k < Kp / 2; k += 256) dst[k] = __float2half_rn(k < K ? row[k] : 0.0f);
        return;
    }
    const float step = (mx > 0.0f && isfinite(mx)) ? mx / full : 1.0f;
    const float inv = 1.0f / step;
    if (tid == 0) {
        dq[m] = step;
        rowsum[m] = sum;
    }
    for (int k = tid; k < Kp; k += 256) {
        const float x = (k < K) ? row[k] * inv : 0.0f;
        uint8_t t[3];
        if (KIND == KIND_I8) {
            int q = __float2int_rn(x);
            q = max(-16256, min(16256, q));
            int hi = (q + 64) >> 7;
            int lo = q - hi * 128;
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
#pragma unroll
        for (int i = 0; i < T; ++i) bq[((size_t)i * Mpad + m) * Kp + k] = t[i];
    }
}

// ---- main kernel ------------------------------------------------------------------------------

struct TcParams {
    const float *scales;
    const float *zeros;
    const float *bias;
    const float *dq;
    const float *rowsum;
    float *out;
    int *err_flag;
    int M, N, K;
    int Mb;        // batch rows per tile
    int n_tiles, m_tiles;
    int kblocks;   // ceil(K / 128)
    int tiled;     // weights come from the tile-major copy (one contiguous, pre-swizzled 16 KB per stage)
    const unsigned char *w_tiles;
    int stages;
    int epilogue;
};

template <int KIND, int T>
__global__ void __launch_bounds__(kThreadsTc, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
              TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment is what the 128B swizzle atoms need
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int BNt = T * p.Mb;                       // MMA N: (term, batch row) columns
    const int a_bytes = kTileN * kKBlockBytes;      // 16 KB weight tile per stage
    const int b_bytes = BNt * kKBlockBytes;         // activation tile per stage
    const int b_stride = (b_bytes + 1023) & ~1023;
    unsigned char *s_a = smem;
    unsigned char *s_b = smem + (size_t)p.stages * a_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_b + (size_t)p.stages * b_stride);
    uint64_t *full = bars, *empty = bars + p.stages;
    uint64_t *tfull = bars + 2 * p.stages, *tempty = tfull + 2;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();   // barrier set-up and the TMEM allocation below run under the previous kernel's tail
    // TMEM columns: two accumulator buffers of BNt columns, power of two >= 32
    uint32_t ncols = 32;
    while ((int)ncols < 2 * BNt) ncols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], kEpiWarps);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(s_tmem)),
                     "r"(ncols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    const int total_tiles = p.n_tiles * p.m_tiles;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto load_a = [&](int st, int nt, int kb) {
                if (p.tiled)
                    bulk_load(s_a + (size_t)st * a_bytes, p.w_tiles + (size_t)(nt * p.kblocks + kb) * a_bytes,
                              a_bytes, &full[st]);
                else
                    tma_load_2d(s_a + (size_t)st * a_bytes, &map_w, &full[st], kb * kKBlockBytes, nt * kTileN);
            };
            // The weights do not depend on the kernel before this one on the stream, the activation
            // planes do: the first ring of weight tiles is requested before griddepcontrol.wait, the
            // matching activation tiles after it.
            const int head = (blockIdx.x < total_tiles) ? min(p.stages, p.kblocks) : 0;
            if (head > 0) {
                const int nt = blockIdx.x / p.m_tiles, mt = blockIdx.x - nt * p.m_tiles;
                for (int kb = 0; kb < head; ++kb) {
                    mbar_expect_tx(&full[kb], (uint32_t)(a_bytes + b_bytes));   // stage kb: all stages start empty
                    load_a(kb, nt, kb);
                }
                pdl_wait();
                for (int kb = 0; kb < head; ++kb)
                    tma_load_3d(s_b + (size_t)kb * b_stride, &map_a, &full[kb], kb * kKBlockBytes, mt * p.Mb, 0);
                s = head;
                if (s == p.stages) {
                    s = 0;
                    phase ^= 1;
                }
            } else {
                pdl_wait();
            }
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
                for (int kb = (tile == (int)blockIdx.x ? head : 0); kb < p.kblocks; ++kb) {
                    if (!mbar_wait(&empty[s], phase ^ 1, s_abort, p.err_flag, 0x10)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], (uint32_t)(a_bytes + b_bytes));
                    load_a(s, nt, kb);
                    tma_load_3d(s_b + (size_t)s * b_stride, &map_a, &full[s], kb * kKBlockBytes, mt * p.Mb, 0);
                    if (++s == p.stages) {
                        s = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {  // let copies already in flight land before the CTA can exit
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(KIND, BNt);
            int s = 0;
            uint32_t phase = 0;
            int as = 0;
            uint32_t aphase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(&tempty[as], aphase ^ 1, s_abort, p.err_flag, 0x20)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BNt);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(&full[s], phase, s_abort, p.err_flag, 0x40)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = make_desc_sw128(smem_u32(s_a + (size_t)s * a_bytes));
                    const uint64_t db = make_desc_sw128(smem_u32(s_b + (size_t)s * b_stride));
#pragma unroll
                    for (int k = 0; k < kKBlockBytes / 32; ++k) {
                        // advance both operands by 32 bytes of K inside the swizzled row
                        tc_mma<KIND>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
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
    } else {
        // ---------------- epilogue (8 warps: a TMEM lane quadrant each, two warps per quadrant
        // taking alternate 16-column chunks) ----------------
        pdl_wait();   // dq, rowsum and the output buffer belong to kernels before this one
        const int quad = warp & 3;
        const int chunk0 = ((warp - 2) >> 2) * 16;
        int as = 0;
        uint32_t aphase = 0;
        const bool has_zero = p.zeros != nullptr;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
            if (!mbar_wait(&tfull[as], aphase, s_abort, p.err_flag, 0x80)) break;
            tc_fence_after();
            const int n = nt * kTileN + quad * 32 + lane;
            const bool n_ok = n < p.N;
            const float scale = n_ok ? (p.scales ? p.scales[n] : 1.0f) : 0.0f;
            const float zero = (n_ok && has_zero) ? p.zeros[n] : 0.0f;
            const float bias = (n_ok && p.bias) ? p.bias[n] : 0.0f;
            const uint32_t t_base = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(as * BNt);
            for (int c0 = chunk0; c0 < p.Mb; c0 += 16 * (kEpiWarps / 4)) {
                uint32_t r[T][16];
#pragma unroll
                for (int t = 0; t < T; ++t) tmem_ld16(t_base + (uint32_t)(t * p.Mb + c0), r[t]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = mt * p.Mb + c0 + j;
                    if (m >= p.M || c0 + j >= p.Mb) continue;
                    float acc;
                    if (T == 1)
                        acc = __uint_as_float(r[0][j]);
                    else if (KIND == KIND_I8)
                        acc = (float)(int)r[0][j] * 128.0f + (float)(int)r[1][j];
                    else if (T == 3)
                        acc = (__uint_as_float(r[0][j]) + __uint_as_float(r[1][j])) +
                              __uint_as_float(r[T - 1][j]);
                    else
                        acc = __uint_as_float(r[0][j]) + __uint_as_float(r[T > 1 ? 1 : 0][j]);
                    const float dot = acc * p.dq[m];
                    const float v = finish_output_fast(dot, scale, zero, has_zero ? p.rowsum[m] : 0.0f,
                                                       p.bias != nullptr, bias, p.epilogue);
                    if (n_ok) p.out[(size_t)m * p.N + n] = v;  // a warp writes 32 consecutive n
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[as]);
            if (++as == 2) {
                as = 0;
                aphase ^= 1;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols)
                     : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------

struct TcWeightMaps {
    CUtensorMap w;
};

// cuTensorMapEncodeTiled is looked up through the runtime, so the library itself carries no
// link-time dependency on libcuda (it must load, and fail cleanly, on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int encode_map(CUtensorMap *map, void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
               const cuuint32_t *box) {
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
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, base, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(FNN_ERR_DISPATCH, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FNN_OK;
}

// Tensor map of the weight operand.  With the tile-major copy the tensor is [tiles * K blocks * 128
// rows][128 bytes] and the box of (row tile nt, K block kb) starts at row (nt * kblocks + kb) * 128:
// 16 KB of contiguous memory.  Without it (8-bit codes that were never prepared) the rows are read in
// place, 128 bytes from each of 128 rows.
int encode_weight_map(CUtensorMap *map, const fnn_cuda_qweight *w, int Kbytes) {
    cuuint32_t box[2] = {(cuuint32_t)kKBlockBytes, (cuuint32_t)kTileN};
    if (w->tc) {
        const size_t n_tiles = div_ceil(w->N, (size_t)kTileN);
        cuuint64_t dims[2] = {(cuuint64_t)kKBlockBytes, (cuuint64_t)(n_tiles * w->tc_kblocks * kTileN)};
        cuuint64_t strides[1] = {(cuuint64_t)kKBlockBytes};
        return encode_map(map, w->tc, 2, dims, strides, box);
    }
    cuuint64_t dims[2] = {(cuuint64_t)Kbytes, (cuuint64_t)w->N};
    cuuint64_t strides[1] = {(cuuint64_t)w->ld_u4 * 16};
    return encode_map(map, (void *)w->rows, 2, dims, strides, box);
}

// Scratch of one call: the rewritten activations Bq[T][Mpad][Kp], then dq[Mpad] and rowsum[Mpad].
// `fixed_scratch` null: the context's growable buffer; otherwise a caller-supplied region of
// `fixed_bytes` that must already be large enough (the entry point that may not allocate).
template <int KIND, int T>
int launch_tc(fnn_cuda_ctx *ctx, const QmmArgs &a, uint8_t *fixed_scratch = nullptr, size_t fixed_bytes = 0) {
    const fnn_cuda_qweight *w = a.w;
    constexpr int ES = (KIND == KIND_F16) ? 2 : 1;  // bytes per operand element
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
    int rc = FNN_OK;
    uint8_t *bq;
    if (fixed_scratch) {
        FNN_REQUIRE(need <= fixed_bytes, FNN_ERR_MEMORY,
                    "qmatmul_noalloc: M=%d, K=%d needs %zu bytes of activation scratch; the built-in "
                    "scratch holds %zu (use fnn_cuda_qmatmul for larger problems)",
                    M, K, need, fixed_bytes);
        bq = fixed_scratch;
    } else {
        rc = ensure_scratch(ctx, need);
        if (rc != FNN_OK) return rc;
        bq = (uint8_t *)ctx->scratch;
    }
    float *dq = (float *)(bq + bq_al);
    float *rowsum = dq + Mpad;
    if (Mpad > M)  // padded batch rows of every term plane must read as zero
        FNN_CUDA_CHECK(cudaMemset2DAsync(bq + (size_t)M * Kp, (size_t)Mpad * Kp, 0,
                                         (size_t)(Mpad - M) * Kp, T, ctx->stream),
                       FNN_ERR_DISPATCH);
    // same shared-memory carve-out as the main kernel: alternating carve-outs between consecutive
    // kernels makes every SM reconfigure (and drain) twice per call
    FNN_CUDA_CHECK(cudaFuncSetAttribute(act_prep_kernel<KIND, T>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(launch_pdl(act_prep_kernel<KIND, T>, M, 256, 0, ctx->stream, a.a, M, K, Kp, Mpad, bq, dq, rowsum),
                   FNN_ERR_DISPATCH);
    ctx->launches++;

    CUtensorMap map_w, map_a;
    {
        rc = encode_weight_map(&map_w, w, Kbytes);
        if (rc != FNN_OK) return rc;
    }
    {
        cuuint64_t dims[3] = {(cuuint64_t)Kp, (cuuint64_t)Mpad, (cuuint64_t)T};
        cuuint64_t strides[2] = {(cuuint64_t)Kp, (cuuint64_t)Kp * Mpad};
        cuuint32_t box[3] = {(cuuint32_t)kKBlockBytes, (cuuint32_t)Mb, (cuuint32_t)T};
        rc = encode_map(&map_a, bq, 3, dims, strides, box);
        if (rc != FNN_OK) return rc;
    }

    TcParams p{};
    p.scales = (w->fmt == FNN_FMT_I4CB) ? nullptr : w->scales;  // block scales are folded into the copy
    p.zeros = w->zeros;
    p.bias = a.bias;
    p.dq = dq;
    p.rowsum = rowsum;
    p.out = a.out;
    p.err_flag = ctx->err_flag;
    p.M = M;
    p.N = N;
    p.K = K;
    p.Mb = Mb;
    p.n_tiles = (N + kTileN - 1) / kTileN;
    p.m_tiles = m_tiles;
    p.kblocks = (Kbytes + kKBlockBytes - 1) / kKBlockBytes;
    p.tiled = w->tc != nullptr;
    p.w_tiles = (const unsigned char *)w->tc;
    p.epilogue = a.epilogue;
    const int a_bytes = kTileN * kKBlockBytes;
    const int b_stride = (T * Mb * kKBlockBytes + 1023) & ~1023;
    int stages = (int)((200 * 1024) / (size_t)(a_bytes + b_stride));
    stages = std::max(2, std::min(stages, 8));
    p.stages = stages;
    const size_t smem = 1024 + (size_t)stages * (a_bytes + b_stride) + (2 * stages + 4) * 8 + 64;
    const int grid = std::min(p.n_tiles * p.m_tiles, ctx->sm_count);
    auto kern = qmm_tc_kernel<KIND, T>;
    FNN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(launch_pdl(kern, grid, kThreadsTc, smem, ctx->stream, map_w, map_a, p), FNN_ERR_DISPATCH);
    ctx->launches++;
    ctx->last_path = fixed_scratch ? "tc-noalloc" : "tc";
    return FNN_OK;
}

// Position i of the tile-major copy -> (weight row n, byte offset inside the row's operand bytes).
// Each 16 KB tile is stored the way the 128-byte swizzle lays it out in shared memory (16-byte chunk
// index XOR row mod 8), so that one untiled bulk copy of 16 KB brings it in ready for the MMA.
__device__ __forceinline__ void tile_pos(size_t i, size_t kblocks, size_t &n, size_t &byte) {
    const size_t r = (i / kKBlockBytes) % kTileN;
    const size_t bs = i % kKBlockBytes;
    const size_t b = (((bs >> 4) ^ (r & 7)) << 4) | (bs & 15);
    const size_t blk = i / ((size_t)kKBlockBytes * kTileN);   // nt * kblocks + kb
    n = (blk / kblocks) * kTileN + r;
    byte = (blk % kblocks) * kKBlockBytes + b;
}

// Codebook weights -> fp16 of blockscale * centroid (one rounding), tile-major, for kind::f16.
__global__ void expand_codebook_kernel(const uint32_t *rows, size_t ld_words, size_t N, size_t K,
                                       const float *bscales, size_t bpr, const float *codebook,
                                       size_t kblocks, size_t total_halves, __half *out) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_halves; i += stride) {
        size_t n, byte;
        tile_pos(i * 2, kblocks, n, byte);
        const size_t k = byte / 2;
        float v = 0.0f;
        if (n < N && k < K) {
            const uint32_t nib = (rows[n * ld_words + k / 8] >> (4 * (k % 8))) & 0xFu;
            v = __fmul_rn(bscales[n * bpr + k / kCodebookBlock], codebook[nib]);
        }
        out[i] = __float2half_rn(v);
    }
}

// 4-bit codes -> one byte per weight, exactly: e2m1 -> the e4m3 code of the same value,
// two's-complement nibble -> int8; tile-major.
__global__ void expand_nibbles_kernel(int fmt, const uint32_t *rows, size_t ld_words, size_t N, size_t K,
                                      size_t kblocks, size_t total, uint8_t *out) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t n, k;
        tile_pos(i, kblocks, n, k);
        uint8_t v = 0;
        if (n < N && k < K) {
            const uint32_t nib = (rows[n * ld_words + k / 8] >> (4 * (k % 8))) & 0xFu;
            if (fmt == FNN_FMT_I4) {
                v = (uint8_t)(int8_t)(((int32_t)(nib << 28)) >> 28);
            } else {
                // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 as e4m3 (bias 7, 3 mantissa bits)
                const uint8_t lut[8] = {0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C};
                v = (uint8_t)(lut[nib & 7u] | ((nib & 8u) << 4));
            }
        }
        out[i] = v;
    }
}

}  // namespace

bool qmm_tc_supported(const fnn_cuda_qweight *w, size_t M) {
    (void)M;
    // codes the tensor core takes natively (I8, FP8), after an exact one-byte expansion (I4, FP4),
    // or -- the codebook format, whose block scales vary inside K -- as an fp16 copy of
    // blockscale * centroid (only when those stay inside the fp16 range)
    if (w->fmt == FNN_FMT_I4CB && !w->fp16_ok) return false;
    return w->K >= 128 && w->N >= 1 && w->N < (1u << 30) && w->K < (1u << 29);
}

int prepare_qmm_tc(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w) {
    // 8-bit codes are read in place from the rows (a tile-major copy measured within 4 % of that at
    // every batch size and would double their footprint); the formats that need a byte or fp16
    // expansion anyway get it tile-major
    if (w->tc || w->fmt == FNN_FMT_I8 || w->fmt == FNN_FMT_F8) return FNN_OK;
    FNN_REQUIRE(!ctx->capturing, FNN_ERR_MEMORY,
                "first tcgen05 use of a weight happened during graph capture; run the plan once before "
                "capturing it");
    const size_t kbytes = (w->fmt == FNN_FMT_I4CB) ? w->K * 2 : w->K;   // operand bytes per row
    const size_t kblocks = div_ceil(kbytes, (size_t)kKBlockBytes);
    const size_t total = div_ceil(w->N, (size_t)kTileN) * kblocks * kTileN * kKBlockBytes;
    void *buf = nullptr;
    FNN_CUDA_CHECK(cudaMalloc(&buf, total), FNN_ERR_MEMORY);
    const auto blocks_for = [&](size_t items) {
        return (int)std::min<size_t>(div_ceil(items, 256), (size_t)ctx->sm_count * 16);
    };
    if (w->fmt == FNN_FMT_I4CB) {
        expand_codebook_kernel<<<blocks_for(total / 2), 256, 0, ctx->stream>>>(
            (const uint32_t *)w->rows, w->ld_u4 * 4, w->N, w->K, w->scales, w->blocks_per_row, w->codebook,
            kblocks, total / 2, (__half *)buf);
    } else {
        expand_nibbles_kernel<<<blocks_for(total), 256, 0, ctx->stream>>>(
            w->fmt, (const uint32_t *)w->rows, w->ld_u4 * 4, w->N, w->K, kblocks, total, (uint8_t *)buf);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        cudaFree(buf);
        return set_error(FNN_ERR_DISPATCH, "tile-major copy: %s", cudaGetErrorString(e));
    }
    ctx->launches++;
    w->tc = buf;
    w->tc_bytes = total;
    w->tc_kblocks = kblocks;
    return FNN_OK;
}

int launch_qmm_tc(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    FNN_REQUIRE(a.M < (1u << 24), FNN_ERR_DISPATCH, "qmatmul: M=%zu too large for the tcgen05 path", a.M);
    int rc = prepare_qmm_tc(ctx, const_cast<fnn_cuda_qweight *>(a.w));
    if (rc != FNN_OK) return rc;
    switch (a.w->fmt) {
    case FNN_FMT_I8:
    case FNN_FMT_I4:
        return launch_tc<KIND_I8, 2>(ctx, a);
    case FNN_FMT_F8:
    case FNN_FMT_F4:
        // three e4m3 terms keep f32-grade accuracy while the scan of the weights is the bound;
        // two terms (~1e-3 of the output norm) once the tensor core is
        return a.M >= 128 ? launch_tc<KIND_F8, 2>(ctx, a) : launch_tc<KIND_F8, 3>(ctx, a);
    case FNN_FMT_I4CB:
        return launch_tc<KIND_F16, 1>(ctx, a);
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: tcgen05 path does not cover format %d", a.w->fmt);
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
    FNN_REQUIRE(qmm_tc_supported(w, M) && w->fmt != FNN_FMT_I4CB, FNN_ERR_UNSUPPORTED,
                "qmatmul_noalloc: format %d / K=%zu is not served by this entry point", w->fmt, w->K);
    // 4-bit formats read a byte-expanded copy that fnn_cuda_qweight_prepare(.., FNN_PATH_TC)
    // builds; building it here would allocate
    FNN_REQUIRE(w->tc != nullptr || w->fmt == FNN_FMT_I8 || w->fmt == FNN_FMT_F8, FNN_ERR_MEMORY,
                "qmatmul_noalloc: call fnn_cuda_qweight_prepare(ctx, w, FNN_PATH_TC) once for 4-bit "
                "weights before using the entry point that may not allocate");
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
    switch (w->fmt) {
    case FNN_FMT_I8:
    case FNN_FMT_I4:
        return launch_tc<KIND_I8, 2>(ctx, args, scratch, kNoAllocScratchBytes);
    case FNN_FMT_F8:
    case FNN_FMT_F4:
        return M >= 128 ? launch_tc<KIND_F8, 2>(ctx, args, scratch, kNoAllocScratchBytes)
                        : launch_tc<KIND_F8, 3>(ctx, args, scratch, kNoAllocScratchBytes);
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul_noalloc: format %d", w->fmt);
}
