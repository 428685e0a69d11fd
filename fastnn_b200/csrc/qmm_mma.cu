// Skinny-M tensor-core kernel for the quantized MatMul (1 <= M <= 64 per launch).
//
// The op is bound by the HBM scan of the packed weights, so the kernel is built around that
// scan: weights live in a fragment-major layout where every warp-wide 128-bit load reads 512
// contiguous bytes and each lane receives exactly the codes of its own `mma.sync` A fragment
// (16 weight rows x 16 k).  Codes are expanded to exact fp16 in registers (byte/nibble
// permutes and half2 arithmetic, ~1 ALU op per weight), activations are staged once per block
// in shared memory as fp16 (two-term hi/lo split for M <= 16, which keeps f32-grade accuracy),
// products accumulate in f32 in the tensor cores, K is split across the warps of a block and
// reduced through shared memory in a fixed order, and the affine step, bias and activation
// are applied in the epilogue:
//   out[m,n] = act(acc[m,n] * scale[n] + zero[n] * sum_k a[m,k] + bias[n])
// (src/backend/cpu/microkernels/gemm.rs:2048-2087, src/backend/cpu/matmul.rs:61-71).
//
// Fragment-major layout ("frag"): for row tile rt (16 rows), k-block kb (64 k for 8-bit codes,
// 128 k for 4-bit), half h (rows g / g+8) and lane l = g*4 + c, the 16-byte unit
//   frag[((rt*KB + kb)*2 + h)*32 + l]  ==  bytes [ (kb*4 + c)*16, +16 ) of reference row rt*16 + h*8 + g.
// It is a permutation of the reference's 16-byte units: no bit inside a unit changes.
#include "common.cuh"

#include <algorithm>

#include <cuda_fp8.h>
#include <cuda_fp4.h>

namespace fnn {

namespace {

constexpr int kW = 8;             // warps per block
constexpr int kThreadsMma = kW * 32;
constexpr int kU = 2;             // k-blocks per prefetch chunk

template <int FMT>
struct FragTraits {
    static constexpr bool four_bit = (FMT == FNN_FMT_I4 || FMT == FNN_FMT_F4 || FMT == FNN_FMT_I4CB);
    static constexpr int KBLK = four_bit ? 128 : 64;  // k per k-block (4 lanes x 16 bytes per row)
    static constexpr int VEC = four_bit ? 4 : 2;      // B vectors (2 MMAs each) per k-block
    static constexpr int PAD_BYTES = four_bit ? 64 : 16;  // row padding of the activation tile
};

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b),
                        *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

// Position of element i (0..7) of an 8-group inside the staged activation tile.  I4 pairs
// nibbles (0,4),(1,5),(2,6),(3,7) when it masks two codes at once, so the activations are
// stored in that order; every other format decodes adjacent pairs.
template <int FMT>
__device__ __forceinline__ int pos8(int i) {
    return (FMT == FNN_FMT_I4) ? ((i & 3) * 2 + (i >> 2)) : i;
}

// Staged position (in halves) of activation k within its row.
template <int FMT>
__device__ __forceinline__ int act_pos(int k) {
    if (FragTraits<FMT>::four_bit) {
        int kb = k >> 7, r = k & 127;
        int c = r >> 5, j = (r >> 3) & 3, i = r & 7;
        return (kb << 7) + j * 32 + c * 8 + pos8<FMT>(i);
    }
    return k;
}

// One 32-bit word of codes -> half2 registers in A-fragment order.
//   8-bit: h[0] = (e0,e1) [slot k 2c..], h[1] = (e2,e3) [slot k 2c+8..]            -> 1 MMA
//   4-bit: h[0],h[1] -> MMA 2j ; h[2],h[3] -> MMA 2j+1
template <int FMT>
struct MmaDec;

template <>
struct MmaDec<FNN_FMT_I8> {
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h, const uint32_t *, uint32_t) {
        uint32_t x = w ^ 0x80808080u;  // q + 128
        h[0] = h2_sub(__byte_perm(x, 0x64646464u, 0x4140), 0x64806480u);  // (1024+u) - 1152
        h[1] = h2_sub(__byte_perm(x, 0x64646464u, 0x4342), 0x64806480u);
    }
};

template <>
struct MmaDec<FNN_FMT_I4> {
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h, const uint32_t *, uint32_t) {
        uint32_t x = w ^ 0x88888888u;  // q + 8 per nibble
        uint32_t y = x >> 8;
        h[0] = h2_sub((x & 0x000F000Fu) | 0x64006400u, 0x64086408u);               // (e0,e4)
        h[1] = h2_fma((x & 0x00F000F0u) | 0x64006400u, 0x2C002C00u, 0xD480D480u);  // (e1,e5)
        h[2] = h2_sub((y & 0x000F000Fu) | 0x64006400u, 0x64086408u);               // (e2,e6)
        h[3] = h2_fma((y & 0x00F000F0u) | 0x64006400u, 0x2C002C00u, 0xD480D480u);  // (e3,e7)
    }
};

template <>
struct MmaDec<FNN_FMT_F8> {
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h, const uint32_t *, uint32_t) {
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xFFFFu), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
        h[0] = *reinterpret_cast<uint32_t *>(&lo);
        h[1] = *reinterpret_cast<uint32_t *>(&hi);
    }
};

template <>
struct MmaDec<FNN_FMT_F4> {
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h, const uint32_t *, uint32_t) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            __half2_raw r = __nv_cvt_fp4x2_to_halfraw2(
                (__nv_fp4x2_storage_t)((w >> (8 * b)) & 0xFFu), __NV_E2M1);
            h[b] = *reinterpret_cast<uint32_t *>(&r);
        }
    }
};

template <>
struct MmaDec<FNN_FMT_I4CB> {
    // lut: per-lane copy of the 256-entry table byte -> half2(cb[lo nibble], cb[hi nibble]);
    // bs2: half2 of the lane's block scale (a 16-byte unit is exactly one 32-element block).
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h, const uint32_t *lut,
                                               uint32_t bs2) {
#pragma unroll
        for (int b = 0; b < 4; ++b) h[b] = h2_mul(lut[((w >> (8 * b)) & 0xFFu) * 32], bs2);
    }
};

__device__ __forceinline__ void mma_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct MmaParams {
    const uint4 *frag;
    const float *frag_bs;  // I4CB block scales in fragment order
    const float *scales;
    const float *zeros;
    const float *codebook;
    const float *act;
    float *out;
    const float *bias;
    int *err_flag;
    int M, N, K;
    int KB;          // k-blocks per row (padded)
    int ntiles;      // row tiles of 16
    int tiles_per_block;
    int Kc;          // activations staged per pass (multiple of KBLK)
    int split;       // 1: hi/lo activation split (cols m and Mh+m), Mh = 4*CG; 0: Mh = 8*CG
    int epilogue;
};

template <int FMT, int CG>
__global__ void __launch_bounds__(kThreadsMma, (CG <= 2) ? 3 : (CG == 4 ? 2 : 1))
qmm_mma_kernel(MmaParams p) {
    using T = FragTraits<FMT>;
    constexpr int KBLK = T::KBLK, VEC = T::VEC;
    constexpr int COLS = 8 * CG;
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = 2 * p.Kc + T::PAD_BYTES;  // bytes per staged activation row
    unsigned char *s_act = smem;                                         // [COLS][RS]
    float *s_red = reinterpret_cast<float *>(s_act + (size_t)COLS * RS);  // [2][kW][CG*128]
    float *s_out = s_red + 2 * kW * CG * 128;                            // [tiles_per_block][CG*128]
    float *s_rs_part = s_out + (size_t)p.tiles_per_block * CG * 128;     // [kW][64]
    float *s_rs = s_rs_part + kW * 64;                                   // [64]
    uint32_t *s_lut = reinterpret_cast<uint32_t *>(s_rs + 64);           // I4CB: [256][32]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int Mh = p.split ? 4 * CG : 8 * CG;
    const int tile0 = blockIdx.x * p.tiles_per_block;
    const int tiles_here = min(p.tiles_per_block, p.ntiles - tile0);
    const bool has_zero = p.zeros != nullptr;

    for (int i = tid; i < p.tiles_per_block * CG * 128; i += kThreadsMma) s_out[i] = 0.0f;
    if (tid < 64) s_rs[tid] = 0.0f;
    if (FMT == FNN_FMT_I4CB) {
        for (int i = tid; i < 256 * 32; i += kThreadsMma) {
            int b = i >> 5;
            __half2 v = __floats2half2_rn(p.codebook[b & 15], p.codebook[b >> 4]);
            s_lut[i] = *reinterpret_cast<uint32_t *>(&v);
        }
    }
    // columns that carry no batch row stay zero for the whole kernel
    for (int col = 0; col < COLS; ++col) {
        const bool used = p.split ? (col < p.M || (col >= Mh && col < Mh + p.M)) : (col < p.M);
        if (used) continue;
        uint32_t *row = reinterpret_cast<uint32_t *>(s_act + (size_t)col * RS);
        for (int i = tid; i < RS / 4; i += kThreadsMma) row[i] = 0u;
    }

    float acc[CG][4];
#pragma unroll
    for (int cg = 0; cg < CG; ++cg)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[cg][r] = 0.0f;
    int red_buf = 0;

    const int Kpad = p.KB * KBLK;
    for (int k0 = 0; k0 < Kpad; k0 += p.Kc) {
        const int kc_len = min(p.Kc, Kpad - k0);
        __syncthreads();  // previous pass fully consumed (and the zero fills above are done)
        // ---- stage activations [M][k0, k0+kc_len) as fp16 (hi | lo) ------------------------
        for (int m = 0; m < p.M; ++m) {
            const float *src = p.act + (size_t)m * p.K;
            __half *row_hi = reinterpret_cast<__half *>(s_act + (size_t)m * RS);
            __half *row_lo = reinterpret_cast<__half *>(s_act + (size_t)(Mh + m) * RS);
            float part = 0.0f;
            for (int k = tid; k < kc_len; k += kThreadsMma) {
                float a = (k0 + k < p.K) ? __ldg(src + k0 + k) : 0.0f;
                part += a;
                if (fabsf(a) > 65000.0f) atomicOr(p.err_flag, 2);  // outside fp16 range
                __half hi = __float2half_rn(a);
                int pos = act_pos<FMT>(k);
                row_hi[pos] = hi;
                if (p.split) row_lo[pos] = __float2half_rn(a - __half2float(hi));
            }
            if (has_zero) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
                if (lane == 0) s_rs_part[warp * 64 + m] = part;
            }
        }
        __syncthreads();
        if (has_zero && tid < p.M) {
            float s = s_rs[tid];
#pragma unroll
            for (int w = 0; w < kW; ++w) s += s_rs_part[w * 64 + tid];
            s_rs[tid] = s;
        }

        // ---- stream this K range of every tile of the block -------------------------------
        const int KBc = kc_len / KBLK;
        const int kb0 = k0 / KBLK;
        const int nch = (KBc + kU - 1) / kU;
        const int cpw = (nch + kW - 1) / kW;   // chunks per warp per tile
        const int nitems = tiles_here * cpw;

        uint4 cur[kU][2], nxt[kU][2];
        float cur_bs[kU][2], nxt_bs[kU][2];
        auto load = [&](int it, uint4 (&buf)[kU][2], float (&bs)[kU][2]) {
            const int tl = it / cpw;
            const int ch = warp + (it - tl * cpw) * kW;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int kb = ch * kU + u;
                const bool ok = (it < nitems) && (ch < nch) && (kb < KBc);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    buf[u][h] = make_uint4(0, 0, 0, 0);
                    bs[u][h] = 0.0f;
                    if (ok) {
                        size_t idx = (((size_t)(tile0 + tl) * p.KB + kb0 + kb) * 2 + h) * 32 + lane;
                        buf[u][h] = __ldg(p.frag + idx);
                        if (FMT == FNN_FMT_I4CB) bs[u][h] = __ldg(p.frag_bs + idx);
                    }
                }
            }
        };

        if (nitems > 0) load(0, cur, cur_bs);
        for (int it = 0; it < nitems; ++it) {
            load(it + 1, nxt, nxt_bs);
            const int tl = it / cpw;
            const int ch = warp + (it - tl * cpw) * kW;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int kb = ch * kU + u;  // may be past the range: weights are zero then
                const int kb_s = min(kb, KBc - 1);
                // byte offset of this lane's first B vector of the k-block in a staged row
                const int voff = T::four_bit ? (kb_s * KBLK + c * 8) * 2 : (kb_s * KBLK + c * 16) * 2;
                uint32_t bs2[2] = {0u, 0u};
                if (FMT == FNN_FMT_I4CB) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        __half2 t = __float2half2_rn(cur_bs[u][h]);
                        bs2[h] = *reinterpret_cast<uint32_t *>(&t);
                    }
                }
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    // A registers for the two MMAs this B vector feeds
                    uint32_t alo[4], ahi[4];
                    if (T::four_bit) {
                        uint32_t wl = (v == 0) ? cur[u][0].x : (v == 1) ? cur[u][0].y : (v == 2) ? cur[u][0].z : cur[u][0].w;
                        uint32_t wh = (v == 0) ? cur[u][1].x : (v == 1) ? cur[u][1].y : (v == 2) ? cur[u][1].z : cur[u][1].w;
                        MmaDec<FMT>::run(wl, alo, s_lut + lane, bs2[0]);
                        MmaDec<FMT>::run(wh, ahi, s_lut + lane, bs2[1]);
                    } else {
                        uint32_t wl0 = (v == 0) ? cur[u][0].x : cur[u][0].z;
                        uint32_t wl1 = (v == 0) ? cur[u][0].y : cur[u][0].w;
                        uint32_t wh0 = (v == 0) ? cur[u][1].x : cur[u][1].z;
                        uint32_t wh1 = (v == 0) ? cur[u][1].y : cur[u][1].w;
                        MmaDec<FMT>::run(wl0, alo, nullptr, 0u);
                        MmaDec<FMT>::run(wl1, alo + 2, nullptr, 0u);
                        MmaDec<FMT>::run(wh0, ahi, nullptr, 0u);
                        MmaDec<FMT>::run(wh1, ahi + 2, nullptr, 0u);
                    }
                    const int boff = voff + (T::four_bit ? v * 64 : v * 16);
#pragma unroll
                    for (int cg = 0; cg < CG; ++cg) {
                        const uint4 b = *reinterpret_cast<const uint4 *>(
                            s_act + (size_t)(cg * 8 + g) * RS + boff);
                        mma_16816(acc[cg], alo[0], ahi[0], alo[1], ahi[1], b.x, b.y);
                        mma_16816(acc[cg], alo[2], ahi[2], alo[3], ahi[3], b.z, b.w);
                    }
                }
            }
            // last chunk of a tile: reduce the warps' partial tiles in a fixed order
            if (it - tl * cpw == cpw - 1) {
                float *red = s_red + (size_t)red_buf * kW * CG * 128;
#pragma unroll
                for (int cg = 0; cg < CG; ++cg)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        red[(warp * CG + cg) * 128 + r * 32 + lane] = acc[cg][r];
                        acc[cg][r] = 0.0f;
                    }
                __syncthreads();
                for (int e = tid; e < CG * 128; e += kThreadsMma) {
                    float s = 0.0f;
#pragma unroll
                    for (int w = 0; w < kW; ++w) s += red[w * CG * 128 + e];
                    s_out[tl * CG * 128 + e] += s;
                }
                red_buf ^= 1;
            }
#pragma unroll
            for (int u = 0; u < kU; ++u)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    cur[u][h] = nxt[u][h];
                    cur_bs[u][h] = nxt_bs[u][h];
                }
        }
    }
    __syncthreads();

    // ---- epilogue: out[m][n] for the block's tiles ---------------------------------------
    const int total = tiles_here * 16 * p.M;
    for (int i = tid; i < total; i += kThreadsMma) {
        const int tl = i / (16 * p.M);
        const int rem = i - tl * 16 * p.M;
        const int m = rem >> 4, r16 = rem & 15;  // consecutive threads -> consecutive n
        const int n = (tile0 + tl) * 16 + r16;
        if (n >= p.N) continue;
        auto frag_at = [&](int col) {
            const int cg = col >> 3, cc = col & 7;
            const int reg = (r16 >> 3) * 2 + (cc & 1);
            const int ln = (r16 & 7) * 4 + (cc >> 1);
            return s_out[tl * CG * 128 + cg * 128 + reg * 32 + ln];
        };
        float dot = frag_at(m);
        if (p.split) dot += frag_at(Mh + m);
        const float bias = p.bias ? p.bias[n] : 0.0f;
        float r;
        if (FMT == FNN_FMT_I4CB) {
            r = apply_act(p.bias ? __fadd_rn(dot, bias) : dot, p.epilogue);
        } else {
            r = finish_output(dot, p.scales[n], has_zero ? p.zeros[n] : 0.0f,
                              has_zero ? s_rs[m] : 0.0f, p.bias != nullptr, bias, p.epilogue);
        }
        p.out[(size_t)m * p.N + n] = r;
    }
}

// rows layout -> fragment-major layout (zero padded to whole tiles / k-blocks)
__global__ void to_frag_kernel(const uint4 *rows, size_t ld_u4, size_t N, size_t KB, size_t ntiles,
                               uint4 *frag) {
    size_t total = ntiles * KB * 2 * 32;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t lane = i & 31, h = (i >> 5) & 1, t = i >> 6;
        size_t kb = t % KB, rt = t / KB;
        size_t row = rt * 16 + h * 8 + (lane >> 2);
        size_t unit = kb * 4 + (lane & 3);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < N && unit < ld_u4) v = rows[row * ld_u4 + unit];
        frag[i] = v;
    }
}

// I4CB block scales [N][bpr] -> fragment order (one scale per 16-byte unit)
__global__ void to_frag_scales_kernel(const float *scales, size_t bpr, size_t N, size_t KB,
                                      size_t ntiles, float *out) {
    size_t total = ntiles * KB * 2 * 32;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t lane = i & 31, h = (i >> 5) & 1, t = i >> 6;
        size_t kb = t % KB, rt = t / KB;
        size_t row = rt * 16 + h * 8 + (lane >> 2);
        size_t blk = kb * 4 + (lane & 3);
        out[i] = (row < N && blk < bpr) ? scales[row * bpr + blk] : 0.0f;
    }
}

template <int FMT>
int kblk_of() {
    return FragTraits<FMT>::KBLK;
}

int kblk_for(int fmt) {
    return (fmt == FNN_FMT_I8 || fmt == FNN_FMT_F8) ? 64 : 128;
}

int ensure_frag(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w) {
    if (w->frag) return FNN_OK;
    FNN_REQUIRE(!ctx->capturing, FNN_ERR_MEMORY,
                "first tensor-core use of a weight happened during graph capture; run the plan once "
                "before capturing it");
    const size_t KB = div_ceil(w->K, (size_t)kblk_for(w->fmt));
    const size_t ntiles = div_ceil(w->N, 16);
    const size_t units = ntiles * KB * 64;
    FNN_CUDA_CHECK(cudaMalloc((void **)&w->frag, units * sizeof(uint4)), FNN_ERR_MEMORY);
    w->frag_bytes = units * sizeof(uint4);
    int blocks = (int)std::min<size_t>(div_ceil(units, 256), (size_t)ctx->sm_count * 16);
    to_frag_kernel<<<blocks, 256, 0, ctx->stream>>>(w->rows, w->ld_u4, w->N, KB, ntiles, w->frag);
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    ctx->launches++;
    if (w->fmt == FNN_FMT_I4CB) {
        FNN_CUDA_CHECK(cudaMalloc((void **)&w->frag_bs, units * sizeof(float)), FNN_ERR_MEMORY);
        to_frag_scales_kernel<<<blocks, 256, 0, ctx->stream>>>(w->scales, w->blocks_per_row, w->N, KB,
                                                             ntiles, w->frag_bs);
        FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
        ctx->launches++;
    }
    return FNN_OK;
}

template <int FMT, int CG>
int launch_mma(fnn_cuda_ctx *ctx, const QmmArgs &a, const float *act, float *out, int M, int split) {
    using T = FragTraits<FMT>;
    const fnn_cuda_qweight *w = a.w;
    MmaParams p{};
    p.frag = w->frag;
    p.frag_bs = w->frag_bs;
    p.scales = w->scales;
    p.zeros = w->zeros;
    p.codebook = w->codebook;
    p.act = act;
    p.out = out;
    p.bias = a.bias;
    p.err_flag = ctx->err_flag;
    p.M = M;
    p.N = (int)w->N;
    p.K = (int)w->K;
    p.KB = (int)div_ceil(w->K, (size_t)T::KBLK);
    p.ntiles = (int)div_ceil(w->N, 16);
    p.split = split;
    p.epilogue = a.epilogue;

    // Stage as much of K as keeps two to three blocks per SM resident.
    const int Kpad = p.KB * T::KBLK;
    const size_t lut = (FMT == FNN_FMT_I4CB) ? 256 * 32 * 4 : 0;
    const size_t act_budget = (CG <= 2 ? 72 : 110) * 1024 - (CG <= 2 ? lut : 0);
    int Kc = Kpad;
    while ((size_t)(8 * CG) * (2 * Kc + T::PAD_BYTES) > act_budget && Kc > T::KBLK * kU) {
        Kc = (Kc / 2 + T::KBLK - 1) / T::KBLK * T::KBLK;
    }
    p.Kc = Kc;
    const size_t act_bytes = (size_t)(8 * CG) * (2 * Kc + T::PAD_BYTES);
    auto smem_for = [&](int tpb) {
        return act_bytes + (size_t)(2 * kW * CG * 128 + tpb * CG * 128 + kW * 64 + 64) * 4 + lut;
    };
    int blocks_per_sm = (int)std::max<size_t>(1, std::min<size_t>(3, (200 * 1024) / smem_for(2)));
    int tpb = (int)div_ceil((size_t)p.ntiles, (size_t)ctx->sm_count * blocks_per_sm);
    if (tpb < 1) tpb = 1;
    if (tpb > 32 / CG) tpb = 32 / CG;  // keeps the per-block output accumulator at 16 KB
    p.tiles_per_block = tpb;
    const size_t smem = smem_for(tpb);
    const int grid = (int)div_ceil((size_t)p.ntiles, (size_t)tpb);
    auto kern = qmm_mma_kernel<FMT, CG>;
    FNN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   FNN_ERR_DISPATCH);
    kern<<<grid, kThreadsMma, smem, ctx->stream>>>(p);
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

template <int FMT>
int launch_mma_fmt(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    const size_t N = a.w->N, K = a.w->K;
    for (size_t m0 = 0; m0 < a.M; m0 += 64) {
        const int M = (int)std::min<size_t>(64, a.M - m0);
        const float *act = a.a + m0 * K;
        float *out = a.out + m0 * N;
        int rc;
        if (M <= 4)
            rc = launch_mma<FMT, 1>(ctx, a, act, out, M, 1);
        else if (M <= 8)
            rc = launch_mma<FMT, 2>(ctx, a, act, out, M, 1);
        else if (M <= 16)
            rc = launch_mma<FMT, 4>(ctx, a, act, out, M, 1);
        else if (M <= 32)
            rc = launch_mma<FMT, 4>(ctx, a, act, out, M, 0);
        else
            rc = launch_mma<FMT, 8>(ctx, a, act, out, M, 0);
        if (rc != FNN_OK) return rc;
    }
    ctx->last_path = "mma";
    return FNN_OK;
}

}  // namespace

bool qmm_mma_supported(const fnn_cuda_qweight *w, size_t M) {
    (void)M;
    return w->N < (1u << 27) && w->K < (1u << 27) && w->mma_ok;
}

int launch_qmm_mma(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    int rc = ensure_frag(ctx, const_cast<fnn_cuda_qweight *>(a.w));
    if (rc != FNN_OK) return rc;
    switch (a.w->fmt) {
    case FNN_FMT_I8:
        return launch_mma_fmt<FNN_FMT_I8>(ctx, a);
    case FNN_FMT_I4:
        return launch_mma_fmt<FNN_FMT_I4>(ctx, a);
    case FNN_FMT_F8:
        return launch_mma_fmt<FNN_FMT_F8>(ctx, a);
    case FNN_FMT_F4:
        return launch_mma_fmt<FNN_FMT_F4>(ctx, a);
    case FNN_FMT_I4CB:
        return launch_mma_fmt<FNN_FMT_I4CB>(ctx, a);
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: unknown format %d", a.w->fmt);
}

}  // namespace fnn
