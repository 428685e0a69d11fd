// f32 CUDA-core row kernel for the quantized MatMul: every format, every shape.
//
// One warp owns R output rows (weight rows n) for a tile of MT batch rows.  Lanes read the
// packed row with 128-bit loads (consecutive lanes -> consecutive 16 bytes), decode the
// codes to exact f32 in registers, multiply with activations staged in shared memory and
// reduce with warp shuffles.  Accumulation is f32 throughout, the affine post-step and the
// epilogue use the reference's separate roundings
// (src/backend/cpu/microkernels/gemm.rs:1982-2088, microkernels/mod.rs:284-295).
//
// HBM-bound at M = 1; for larger M the tensor-core kernels take over and this kernel remains
// the path for ragged shapes (K not a multiple of the packing unit, tiny N).
#include "common.cuh"

#include <cuda_fp8.h>
#include <cuda_fp4.h>

namespace fnn {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

// ---- per-format decode of one u32 into PER exact floats -----------------------------------

template <int FMT>
struct Dec;

template <>
struct Dec<FNN_FMT_I8> {
    static constexpr int PER = 4;
    __device__ __forceinline__ static void run(uint32_t w, float *v, const float *) {
        // q + 128 in each byte, placed in the mantissa of 2^23: exact int -> float.
        uint32_t x = w ^ 0x80808080u;
        v[0] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7440)) - 8388736.0f;
        v[1] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7441)) - 8388736.0f;
        v[2] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7442)) - 8388736.0f;
        v[3] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7443)) - 8388736.0f;
    }
};

template <>
struct Dec<FNN_FMT_I4> {
    static constexpr int PER = 8;
    __device__ __forceinline__ static void run(uint32_t w, float *v, const float *) {
        uint32_t x = w ^ 0x88888888u;  // q + 8 per nibble
        uint32_t lo = x & 0x0F0F0F0Fu;  // elements 0,2,4,6
        uint32_t hi = (x >> 4) & 0x0F0F0F0Fu;  // elements 1,3,5,7
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            v[2 * b] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7440 | b)) - 8388616.0f;
            v[2 * b + 1] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7440 | b)) - 8388616.0f;
        }
    }
};

template <>
struct Dec<FNN_FMT_F8> {
    static constexpr int PER = 4;
    __device__ __forceinline__ static void run(uint32_t w, float *v, const float *) {
        // Hardware e4m3 -> f16 (exact), then f16 -> f32 (exact).  Equal to the reference
        // LUT (src/dtypes/f8x4.rs:83-92) on every code its encoder emits (<= 0x77).
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xFFFFu), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
        float2 a = __half22float2(*reinterpret_cast<__half2 *>(&lo));
        float2 b = __half22float2(*reinterpret_cast<__half2 *>(&hi));
        v[0] = a.x;
        v[1] = a.y;
        v[2] = b.x;
        v[3] = b.y;
    }
};

template <>
struct Dec<FNN_FMT_F4> {
    static constexpr int PER = 8;
    __device__ __forceinline__ static void run(uint32_t w, float *v, const float *) {
        // Hardware e2m1 -> f16.  Code 0x8 gives -0.0 where the reference LUT gives +0.0
        // (src/dtypes/f4x8.rs:31-36); the two are equal in every product and sum.
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(
                (__nv_fp4x2_storage_t)((w >> (8 * b)) & 0xFFu), __NV_E2M1);
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&h));
            v[2 * b] = f.x;
            v[2 * b + 1] = f.y;
        }
    }
};

template <>
struct Dec<FNN_FMT_I4CB> {
    static constexpr int PER = 8;
    // cb: 16-entry codebook in shared memory (16 consecutive banks: conflict-free).
    __device__ __forceinline__ static void run(uint32_t w, float *v, const float *cb) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = cb[(w >> (4 * i)) & 0xFu];
    }
};

// Shared-memory position of tile element k.  The tile is stored as PER planes so that lane l
// reading 16 bytes for chunk c = l (+32 per iteration) hits consecutive banks, and each plane
// is padded by 4 floats so that the staging stores are conflict-free too.
template <int PER>
__device__ __forceinline__ int act_pos(int k, int plane_stride) {
    int c = k / (4 * PER);
    int r = k % (4 * PER);
    int plane = r / 4;  // == j * (PER/4) + q
    return plane * plane_stride + c * 4 + (r & 3);
}

template <int FMT, int MT, int R>
__global__ void __launch_bounds__(kThreads)
qmm_rows_kernel(const uint4 *__restrict__ rows, size_t ld_u4, const float *__restrict__ scales,
                const float *__restrict__ zeros, const float *__restrict__ codebook,
                size_t blocks_per_row, const float *__restrict__ act, float *__restrict__ out,
                const float *__restrict__ bias, int M, int N, int K, int KT, int epilogue) {
    constexpr int PER = Dec<FMT>::PER;
    constexpr int EPC = 4 * PER;  // elements per 16-byte chunk
    extern __shared__ float s_act[];  // [MT][PER planes][plane_stride]
    __shared__ float s_cb[16];
    __shared__ float s_rowsum[kWarps][MT];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = (blockIdx.x * kWarps + warp) * R;
    const int m0 = blockIdx.y * MT;
    const int NC = KT / EPC;
    const int plane_stride = NC * 4 + 4;
    const int m_stride = PER * plane_stride;
    const int Kpad = (int)ld_u4 * EPC;
    const bool has_zero = zeros != nullptr;

    if (FMT == FNN_FMT_I4CB && tid < 16) s_cb[tid] = codebook[tid];

    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;
    float rs[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) rs[m] = 0.0f;

    for (int k0 = 0; k0 < Kpad; k0 += KT) {
        const int tile_len = min(KT, Kpad - k0);
        __syncthreads();  // previous tile fully consumed
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const bool m_ok = (m0 + m) < M;
            const float *src = act + (size_t)(m0 + m) * K + k0;
            for (int k = tid; k < tile_len; k += kThreads) {
                float a = (m_ok && (k0 + k) < K) ? src[k] : 0.0f;
                s_act[m * m_stride + act_pos<PER>(k, plane_stride)] = a;
                rs[m] += a;
            }
        }
        __syncthreads();

        const int nchunk = tile_len / EPC;
        const size_t u4_base = (size_t)(k0 / EPC);
#pragma unroll 2
        for (int c = lane; c < nchunk; c += 32) {
            uint4 wv[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                wv[r] = make_uint4(0, 0, 0, 0);
                if (row0 + r < N) wv[r] = __ldg(rows + (size_t)(row0 + r) * ld_u4 + u4_base + c);
            }
            float part[R][MT];
            float bs[R];
            if (FMT == FNN_FMT_I4CB) {
                // one 16-byte chunk is exactly one 32-element scale block
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    bs[r] = 0.0f;
                    size_t blk = (size_t)(k0 / kCodebookBlock) + c;
                    if (row0 + r < N && blk < blocks_per_row)
                        bs[r] = __ldg(scales + (size_t)(row0 + r) * blocks_per_row + blk);
#pragma unroll
                    for (int m = 0; m < MT; ++m) part[r][m] = 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float wf[R][PER];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    uint32_t word = (j == 0) ? wv[r].x : (j == 1) ? wv[r].y : (j == 2) ? wv[r].z : wv[r].w;
                    Dec<FMT>::run(word, wf[r], s_cb);
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float av[PER];
#pragma unroll
                    for (int q = 0; q < PER / 4; ++q) {
                        const float4 t = *reinterpret_cast<const float4 *>(
                            s_act + m * m_stride + (j * (PER / 4) + q) * plane_stride + c * 4);
                        av[4 * q] = t.x;
                        av[4 * q + 1] = t.y;
                        av[4 * q + 2] = t.z;
                        av[4 * q + 3] = t.w;
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        float s = (FMT == FNN_FMT_I4CB) ? part[r][m] : acc[r][m];
#pragma unroll
                        for (int i = 0; i < PER; ++i) s = fmaf(wf[r][i], av[i], s);
                        if (FMT == FNN_FMT_I4CB)
                            part[r][m] = s;
                        else
                            acc[r][m] = s;
                    }
                }
            }
            if (FMT == FNN_FMT_I4CB) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int m = 0; m < MT; ++m) acc[r][m] = fmaf(bs[r], part[r][m], acc[r][m]);
            }
        }
    }

    // sum(a) per batch row, reduced in a fixed order (needed only with zero points)
    if (has_zero) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = rs[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0) s_rowsum[warp][m] = v;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            acc[r][m] = v;
        }
    __syncthreads();

    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m0 + m >= M) continue;
            float rowsum = 0.0f;
            if (has_zero) {
#pragma unroll
                for (int wi = 0; wi < kWarps; ++wi) rowsum += s_rowsum[wi][m];
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                int n = row0 + r;
                if (n >= N) continue;
                float scale = (FMT == FNN_FMT_I4CB) ? 1.0f : scales[n];
                float zero = has_zero ? zeros[n] : 0.0f;
                float b = bias ? bias[n] : 0.0f;
                out[(size_t)(m0 + m) * N + n] =
                    (FMT == FNN_FMT_I4CB)
                        ? apply_act(bias ? __fadd_rn(acc[r][m], b) : acc[r][m], epilogue)
                        : finish_output(acc[r][m], scale, zero, rowsum, bias != nullptr, b, epilogue);
            }
        }
    }
}

template <int FMT, int MT, int R>
int launch_one(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    constexpr int PER = Dec<FMT>::PER;
    const fnn_cuda_qweight *w = a.w;
    int KT = 8192 / MT;
    if (KT > 4096) KT = 4096;
    int Kpad = (int)w->ld_u4 * 4 * PER;
    if (KT > Kpad) KT = ((Kpad + 4 * PER - 1) / (4 * PER)) * (4 * PER);
    int NC = KT / (4 * PER);
    size_t smem = (size_t)MT * PER * (NC * 4 + 4) * sizeof(float);
    dim3 grid((unsigned)div_ceil(w->N, (size_t)kWarps * R), (unsigned)div_ceil(a.M, (size_t)MT));
    auto kern = qmm_rows_kernel<FMT, MT, R>;
    if (smem > 48 * 1024)
        FNN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)smem),
                       FNN_ERR_DISPATCH);
    kern<<<grid, kThreads, smem, ctx->stream>>>(w->rows, w->ld_u4, w->scales, w->zeros, w->codebook,
                                                w->blocks_per_row, a.a, a.out, a.bias, (int)a.M,
                                                (int)w->N, (int)w->K, KT, a.epilogue);
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    ctx->launches++;
    ctx->last_path = "rows";
    return FNN_OK;
}

template <int FMT>
int launch_fmt(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    constexpr bool four_bit = Dec<FMT>::PER == 8;
    if (a.M == 1) return four_bit ? launch_one<FMT, 1, 4>(ctx, a) : launch_one<FMT, 1, 2>(ctx, a);
    if (a.M == 2) return launch_one<FMT, 2, 2>(ctx, a);
    if (a.M <= 4) return launch_one<FMT, 4, 2>(ctx, a);
    return launch_one<FMT, 8, 2>(ctx, a);
}

}  // namespace

int launch_qmm_rows(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    FNN_REQUIRE(a.M <= 65535u * 8u, FNN_ERR_DISPATCH, "qmatmul: M=%zu too large for the row kernel",
                a.M);
    FNN_REQUIRE(a.w->N < (1u << 30) && a.w->K < (1u << 30), FNN_ERR_DISPATCH,
                "qmatmul: dimension exceeds 2^30");
    switch (a.w->fmt) {
    case FNN_FMT_I8:
        return launch_fmt<FNN_FMT_I8>(ctx, a);
    case FNN_FMT_I4:
        return launch_fmt<FNN_FMT_I4>(ctx, a);
    case FNN_FMT_F8:
        return launch_fmt<FNN_FMT_F8>(ctx, a);
    case FNN_FMT_F4:
        return launch_fmt<FNN_FMT_F4>(ctx, a);
    case FNN_FMT_I4CB:
        return launch_fmt<FNN_FMT_I4CB>(ctx, a);
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: unknown format %d", a.w->fmt);
}

}  // namespace fnn
