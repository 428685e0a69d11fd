// Skinny-M tensor-core kernel for the quantized MatMul on fp16 operands (1 <= M <= 64 per launch).
//
// The op is bound by the HBM scan of the packed weights, so the kernel is built around that
// scan: weights live in a fragment-major layout where every warp-wide 128-bit load reads 512
// contiguous bytes and each lane receives exactly the codes of its own `mma.sync` A fragment
// (16 weight rows x 16 k).  Codes are expanded to exact fp16 in registers (byte/nibble
// permutes and half2 arithmetic, ~1 ALU op per weight), activations are staged once per block
// in shared memory as fp16 -- each row scaled by a power of two so that its largest element sits
// just below 2^15 (any f32 magnitude is representable, small rows keep their low bits), and split
// into two terms hi + lo up to 32 batch rows, which keeps f32-grade accuracy -- products
// accumulate in f32 in the tensor cores, K is split across the warps of a block and
// reduced through shared memory in a fixed order, and the affine step, bias and activation
// are applied in the epilogue:
//   out[m,n] = act(acc[m,n] * scale[n] + zero[n] * sum_k a[m,k] + bias[n])
// (src/backend/cpu/microkernels/gemm.rs:2048-2087, src/backend/cpu/matmul.rs:61-71).
//
// Fragment-major layout ("frag"): for row tile rt (16 rows), k-block kb (64 k for 8-bit codes,
// 128 k for 4-bit), half h (rows g / g+8) and lane l = g*4 + c, the 16-byte unit
//   frag[((rt*KB + kb)*2 + h)*32 + l]  ==  bytes [ (kb*4 + c)*16, +16 ) of reference row rt*16 + h*8 + g.
// It is a permutation of the reference's 16-byte units: no bit inside a unit changes.
#include "frag_common.cuh"

#include <cuda_fp8.h>
#include <cuda_fp4.h>

namespace fnn {

namespace {

using frag::cp_async16;
using frag::cp_async4;
using frag::cp_async_commit;
using frag::cp_async_wait;
using frag::group_barrier;

constexpr int kW = frag::kWarpsPerGroup;   // warps per group
constexpr int kU = frag::kChunkBlocks;     // k-blocks per prefetch chunk
constexpr int kMaxRows = 64;               // batch rows per launch

template <int FMT>
struct FragTraits {
    static constexpr bool four_bit = (FMT == FNN_FMT_I4 || FMT == FNN_FMT_F4);
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

// Position of element i (0..7) of an 8-group inside the staged activation tile.  I4 and F4
// pair nibbles (0,4),(1,5),(2,6),(3,7) when they mask two codes at once, so the activations
// are stored in that order; the other formats decode adjacent pairs.
template <int FMT>
__device__ __forceinline__ int pos8(int i) {
    return (FMT == FNN_FMT_I4 || FMT == FNN_FMT_F4) ? ((i & 3) * 2 + (i >> 2)) : i;
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
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h) {
        uint32_t x = w ^ 0x80808080u;  // q + 128
        h[0] = h2_sub(__byte_perm(x, 0x64646464u, 0x4140), 0x64806480u);  // (1024+u) - 1152
        h[1] = h2_sub(__byte_perm(x, 0x64646464u, 0x4342), 0x64806480u);
    }
};

template <>
struct MmaDec<FNN_FMT_I4> {
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h) {
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
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h) {
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xFFFFu), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
        h[0] = *reinterpret_cast<uint32_t *>(&lo);
        h[1] = *reinterpret_cast<uint32_t *>(&hi);
    }
};

template <>
struct MmaDec<FNN_FMT_F4> {
    __device__ __forceinline__ static void run(uint32_t w, uint32_t *h) {
        // e2m1 is a tiny float: its (e1 e0 m) bits dropped into fp16 bits [11:9] read as
        // 2^(e-15)*(1+m/2) (or the subnormal m*2^-15), so one multiply by 2^14 rebiases it exactly.
        // Nibbles i and i+4 sit at the same offset of the two halves and move with one shift.
        const uint32_t kMag = 0x0E000E00u, kSign = 0x80008000u, kTwo14 = 0x74007400u;
        h[0] = h2_mul(((w << 9) & kMag) | ((w << 12) & kSign), kTwo14);  // (e0,e4)
        h[1] = h2_mul(((w << 5) & kMag) | ((w << 8) & kSign), kTwo14);   // (e1,e5)
        h[2] = h2_mul(((w << 1) & kMag) | ((w << 4) & kSign), kTwo14);   // (e2,e6)
        h[3] = h2_mul(((w >> 3) & kMag) | (w & kSign), kTwo14);          // (e3,e7)
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
    const float *scales;
    const float *zeros;
    const float *act;
    float *out;
    const float *bias;
    int M, N, K;
    int KB;          // k-blocks per row (padded)
    int ntiles;      // row tiles of 16
    int tiles_per_group;
    int Kc;          // activations staged per pass (multiple of KBLK)
    int split;       // 1: hi/lo activation split (cols m and Mh+m), Mh = 4*CG; 0: Mh = 8*CG
    int epilogue;
    int gather_on;   // fused all-gather epilogue (one 8-column group only, M <= kGatherRows)
    GatherArgs g;
};

// Warp groups per block for a given number of 8-column groups (register budget).
__host__ __device__ constexpr int groups_for(int cg) { return cg == 1 ? 3 : (cg <= 4 ? 2 : 1); }

// Stages of each lane's private cp.async ring (weights in flight = STAGES - 1 chunks per lane).
__host__ __device__ constexpr int stages_for(int cg) { return cg == 4 ? 2 : 3; }

// One block per SM.  Its G groups of 8 warps share the staged activations; each group streams
// its own row tiles, splitting K across its warps.
template <int FMT, int CG, int G>
__global__ void __launch_bounds__(G * kW * 32, 1)
qmm_mma_kernel(MmaParams p) {
    using T = FragTraits<FMT>;
    constexpr int KBLK = T::KBLK, VEC = T::VEC;
    constexpr int COLS = 8 * CG;
    constexpr int NT = G * kW * 32;   // threads per block
    constexpr int NW = G * kW;        // warps per block
    constexpr int S = stages_for(CG);
    constexpr int UNITS = kU * 2;     // 16-byte units per lane per chunk
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = 2 * p.Kc + T::PAD_BYTES;  // bytes per staged activation row
    const int act_rows = p.split ? 2 * p.M : p.M;  // only real batch rows are staged
    unsigned char *s_ring = smem;                                         // [NW][S][UNITS][32] uint4
    unsigned char *s_act = s_ring + (size_t)NW * S * UNITS * 512;
    float *s_red = reinterpret_cast<float *>(s_act + (size_t)act_rows * RS);  // [G][2][kW][CG*128]
    float *s_out = s_red + G * 2 * kW * CG * 128;                         // [G][tiles_per_group][CG*128]
    const int Mr = (p.M + 3) & ~3;
    float *s_part = s_out + (size_t)G * p.tiles_per_group * CG * 128;     // [NW][Mr][2]
    float *s_rs = s_part + NW * Mr * 2;                                   // [Mr] row sums
    float *s_mx = s_rs + Mr;                                              // [Mr] row maxima
    float *s_up = s_mx + Mr;                                              // [Mr] power-of-two row factor
    float *s_dq = s_up + Mr;                                              // [Mr] its inverse
    float *s_meta = s_dq + Mr;                                            // [G][tiles_per_group][16][3]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = warp / kW, gw = warp % kW, gtid = tid - group * kW * 32;
    const int g = lane >> 2, c = lane & 3;
    const int Mh = p.split ? 4 * CG : 8 * CG;
    // group ids interleave across SMs so consecutive tiles land on different SMs
    const int gg = group * gridDim.x + blockIdx.x, GG = gridDim.x * G;
    const int tiles_here = gg < p.ntiles ? (p.ntiles - gg + GG - 1) / GG : 0;  // tiles gg, gg+GG, ...
    // the next kernel on the stream may be set up as soon as an SM has room: its own prologue (scales,
    // lookup table, first weight copies) then runs under this kernel's tail
    pdl_launch_dependents();
    GatherCursor gc{};
    const bool has_zero = p.zeros != nullptr;
    float *my_out = s_out + (size_t)group * p.tiles_per_group * CG * 128;
    float *my_red = s_red + (size_t)group * 2 * kW * CG * 128;

    unsigned char *my_ring = s_ring + (size_t)warp * S * UNITS * 512 + lane * 16;

    // scale / zero / bias of the group's rows: fetched now, used by the epilogue
    float *my_meta = s_meta + (size_t)group * p.tiles_per_group * 48;
    for (int i = gtid; i < tiles_here * 16; i += kW * 32) {
        const int n = (gg + (i >> 4) * GG) * 16 + (i & 15);
        const bool in = n < p.N;
        my_meta[i * 3 + 0] = in ? __ldg(p.scales + n) : 1.0f;
        my_meta[i * 3 + 1] = (in && has_zero) ? __ldg(p.zeros + n) : 0.0f;
        my_meta[i * 3 + 2] = (in && p.bias) ? __ldg(p.bias + n) : 0.0f;
    }
    for (int i = tid; i < G * p.tiles_per_group * CG * 128; i += NT) s_out[i] = 0.0f;
    // staged row holding batch column (cg*8 + g), or -1 when that column carries no batch row
    int brow[CG];
#pragma unroll
    for (int cg = 0; cg < CG; ++cg) {
        const int col = cg * 8 + g;
        if (p.split)
            brow[cg] = (col < Mh) ? (col < p.M ? col : -1) : (col - Mh < p.M ? p.M + col - Mh : -1);
        else
            brow[cg] = col < p.M ? col : -1;
    }

    float acc[CG][4];
#pragma unroll
    for (int cg = 0; cg < CG; ++cg)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[cg][r] = 0.0f;
    int red_buf = 0;
    const bool vec_ok = (p.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.act) & 15u) == 0);

    const int Kpad = p.KB * KBLK;
    for (int k0 = 0; k0 < Kpad; k0 += p.Kc) {
        const int kc_len = min(p.Kc, Kpad - k0);
        const int KBc = kc_len / KBLK;
        const int kb0 = k0 / KBLK;
        const int nch = (KBc + kU - 1) / kU;
        const int cpw = (nch + kW - 1) / kW;   // chunks per warp per tile

        // issue-side cursor: the next item (tile, chunk-of-this-warp) whose copies go into the ring
        // (an empty group once the warp's items are exhausted)
        int i_tl = 0, i_j = 0, i_st = 0;
        auto issue_next = [&]() {
            const bool valid = i_tl < tiles_here;
            const int ch = gw + i_j * kW;
            const size_t tile_unit = ((size_t)(gg + i_tl * GG) * p.KB + kb0) * 64 + lane;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int kb = ch * kU + u;
                const bool ok = valid && (kb < KBc);
                const size_t idx = ok ? tile_unit + (size_t)kb * 64 : 0;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    cp_async16(my_ring + (size_t)(i_st * UNITS + u * 2 + h) * 512, p.frag + idx + h * 32,
                               ok ? 16 : 0);
            }
            cp_async_commit();
            if (++i_j == cpw) {
                i_j = 0;
                ++i_tl;
            }
            if (++i_st == S) i_st = 0;
        };
        // the first weights are in flight while the activations are being staged
#pragma unroll
        for (int i = 0; i < S - 1; ++i) issue_next();

        if (k0 == 0) {
            // everything above (scales, lookup table, the first weight copies) is independent of the
            // kernel before this one on the stream; the activations and the gather counters are not
            pdl_wait();
            if (CG == 1 && p.gather_on) gc = gather_begin(p.g, blockIdx.x * NT + tid);
            // per-row maximum and sum; the row is staged as a * 2^e with the largest element in
            // [2^14, 2^15): exact, inside the fp16 range whatever the magnitude of the activations
            frag::scan_rows<NT, 4>(p.act, p.M, p.K, vec_ok, s_part, s_mx, s_rs);
            if (tid < p.M) {
                const float bm = s_mx[tid];
                int ex = 15;
                if (bm > 0.0f && isfinite(bm)) (void)frexpf(bm, &ex);   // bm = f * 2^ex, f in [0.5, 1)
                const int e = max(-120, min(120, 15 - ex));
                s_up[tid] = ldexpf(1.0f, e);
                s_dq[tid] = ldexpf(1.0f, -e);
            }
        }
        __syncthreads();  // previous pass fully consumed (and the fills above are done)
        // ---- stage activations [M][k0, k0+kc_len) as fp16 (hi | lo) ----------------------------
        // Work item of a warp = 32 groups of eight consecutive k of one batch row: two 16-byte loads
        // per lane, one 16-byte store per plane (an 8-group is contiguous in the staged order of every
        // format).  Two items are in flight per warp.
        if (vec_ok) {
            const int chunks = kc_len / 8, cg32 = (chunks + 31) / 32, witems = p.M * cg32;
            for (int w0 = warp; w0 < witems; w0 += 2 * NW) {
                float4 v[2][2];
                int mm[2], cc[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int wi = w0 + q * NW;
                    mm[q] = wi / cg32;
                    cc[q] = (wi - mm[q] * cg32) * 32 + lane;
                    v[q][0] = v[q][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (wi < witems && cc[q] < chunks) {
                        const int k = k0 + cc[q] * 8;
                        const float *src = p.act + (size_t)mm[q] * p.K + k;
                        if (k < p.K) v[q][0] = __ldg(reinterpret_cast<const float4 *>(src));
                        if (k + 4 < p.K) v[q][1] = __ldg(reinterpret_cast<const float4 *>(src) + 1);
                    }
                }
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int wi = w0 + q * NW;
                    if (wi >= witems) break;   // warp-uniform
                    const float e[8] = {v[q][0].x, v[q][0].y, v[q][0].z, v[q][0].w,
                                        v[q][1].x, v[q][1].y, v[q][1].z, v[q][1].w};
                    const float up = s_up[mm[q]];
                    __align__(16) __half hi[8];
                    __align__(16) __half lo[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a = e[i] * up;
                        const int pos = FragTraits<FMT>::four_bit ? pos8<FMT>(i) : i;
                        hi[pos] = __float2half_rn(a);
                        lo[pos] = __float2half_rn(a - __half2float(hi[pos]));
                    }
                    if (cc[q] < chunks) {
                        const int base = act_pos<FMT>(cc[q] * 8) * 2;   // bytes; 8-groups stay together
                        *reinterpret_cast<uint4 *>(s_act + (size_t)mm[q] * RS + base) =
                            *reinterpret_cast<const uint4 *>(hi);
                        if (p.split)
                            *reinterpret_cast<uint4 *>(s_act + (size_t)(p.M + mm[q]) * RS + base) =
                                *reinterpret_cast<const uint4 *>(lo);
                    }
                }
            }
        } else {
            for (int m = 0; m < p.M; ++m) {
                const float *src = p.act + (size_t)m * p.K;
                const float up = s_up[m];
                for (int k = tid; k < kc_len; k += NT) {
                    const float a = (k0 + k < p.K) ? __ldg(src + k0 + k) * up : 0.0f;
                    const __half h = __float2half_rn(a);
                    const int pos = act_pos<FMT>(k);
                    reinterpret_cast<__half *>(s_act + (size_t)m * RS)[pos] = h;
                    if (p.split)
                        reinterpret_cast<__half *>(s_act + (size_t)(p.M + m) * RS)[pos] =
                            __float2half_rn(a - __half2float(h));
                }
            }
        }
        __syncthreads();
        // fused gather: the first poll of the previous step's words was issued before the staging
        if (CG == 1 && p.gather_on && k0 == 0 && gc.step > 1u) gather_check_prev(p.g, gc, gridDim.x * NT);

        // ---- stream this K range of every tile of the group -------------------------------
        int c_st = 0;
        for (int tl = 0; tl < tiles_here; ++tl)
        for (int j = 0; j < cpw; ++j) {
            issue_next();
            cp_async_wait<S - 1>();  // the current item has landed in this lane's ring
            const int ch = gw + j * kW;
            uint4 cur[kU][2];
#pragma unroll
            for (int u = 0; u < kU; ++u)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int slot = c_st * UNITS + u * 2 + h;
                    cur[u][h] = *reinterpret_cast<const uint4 *>(my_ring + (size_t)slot * 512);
                }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int kb = ch * kU + u;  // may be past the range: the weights are zero then
                const int kb_s = min(kb, KBc - 1);
                // byte offset of this lane's first B vector of the k-block in a staged row
                const int voff = T::four_bit ? (kb_s * KBLK + c * 8) * 2 : (kb_s * KBLK + c * 16) * 2;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    // A registers for the two MMAs this B vector feeds
                    uint32_t alo[4], ahi[4];
                    if (T::four_bit) {
                        uint32_t wl = (v == 0) ? cur[u][0].x : (v == 1) ? cur[u][0].y : (v == 2) ? cur[u][0].z : cur[u][0].w;
                        uint32_t wh = (v == 0) ? cur[u][1].x : (v == 1) ? cur[u][1].y : (v == 2) ? cur[u][1].z : cur[u][1].w;
                        MmaDec<FMT>::run(wl, alo);
                        MmaDec<FMT>::run(wh, ahi);
                    } else {
                        uint32_t wl0 = (v == 0) ? cur[u][0].x : cur[u][0].z;
                        uint32_t wl1 = (v == 0) ? cur[u][0].y : cur[u][0].w;
                        uint32_t wh0 = (v == 0) ? cur[u][1].x : cur[u][1].z;
                        uint32_t wh1 = (v == 0) ? cur[u][1].y : cur[u][1].w;
                        MmaDec<FMT>::run(wl0, alo);
                        MmaDec<FMT>::run(wl1, alo + 2);
                        MmaDec<FMT>::run(wh0, ahi);
                        MmaDec<FMT>::run(wh1, ahi + 2);
                    }
                    const int boff = voff + (T::four_bit ? v * 64 : v * 16);
#pragma unroll
                    for (int cg = 0; cg < CG; ++cg) {
                        uint4 b = make_uint4(0, 0, 0, 0);
                        if (brow[cg] >= 0)
                            b = *reinterpret_cast<const uint4 *>(s_act + (size_t)brow[cg] * RS + boff);
                        mma_16816(acc[cg], alo[0], ahi[0], alo[1], ahi[1], b.x, b.y);
                        mma_16816(acc[cg], alo[2], ahi[2], alo[3], ahi[3], b.z, b.w);
                    }
                }
            }
            // last chunk of a tile: reduce the group's partial tiles in a fixed order
            if (++c_st == S) c_st = 0;
            if (j == cpw - 1) {
                float *red = my_red + (size_t)red_buf * kW * CG * 128;
#pragma unroll
                for (int cg = 0; cg < CG; ++cg)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        red[(gw * CG + cg) * 128 + r * 32 + lane] = acc[cg][r];
                        acc[cg][r] = 0.0f;
                    }
                group_barrier(group);
                for (int e = gtid; e < CG * 128; e += kW * 32) {
                    float s = 0.0f;
#pragma unroll
                    for (int w = 0; w < kW; ++w) s += red[w * CG * 128 + e];
                    my_out[tl * CG * 128 + e] += s;
                }
                red_buf ^= 1;
            }
        }
        cp_async_wait<0>();
    }
    __syncthreads();

    // ---- epilogue: out[m][n] for the group's tiles ---------------------------------------
    const int total = tiles_here * 16 * p.M;
    for (int i = gtid; i < total; i += kW * 32) {
        const int tl = i / (16 * p.M);
        const int rem = i - tl * 16 * p.M;
        const int m = rem >> 4, r16 = rem & 15;  // consecutive threads -> consecutive n
        const int n = (gg + tl * GG) * 16 + r16;
        if (n >= p.N) continue;
        auto frag_at = [&](int col) {
            const int cg = col >> 3, cc = col & 7;
            const int reg = (r16 >> 3) * 2 + (cc & 1);
            const int ln = (r16 & 7) * 4 + (cc >> 1);
            return my_out[tl * CG * 128 + cg * 128 + reg * 32 + ln];
        };
        float dot = frag_at(m);
        if (p.split) dot += frag_at(Mh + m);
        dot *= s_dq[m];   // power of two: exact
        const float *meta = my_meta + (tl * 16 + r16) * 3;
        const float bias = meta[2];
        const float r = finish_output(dot, meta[0], meta[1], has_zero ? s_rs[m] : 0.0f, p.bias != nullptr,
                                      bias, p.epilogue);
        if (CG == 1 && p.gather_on)
            gather_store(p.g, gc.step, m, n, r);
        else
            p.out[(size_t)m * p.N + n] = r;
    }
    if (CG == 1 && p.gather_on) gather_finish(p.g, gc.step, p.M, p.N);
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

// Codebook format: the unit of lane (g, c) carries word c of each of the four 32-element scale blocks
// of the k-block (a 4 x 4 transpose of 32-bit words inside every 64 bytes of a row), so that one
// m16n8k32 MMA covers exactly one scale block.  No bit inside a word moves.
__global__ void to_frag_cb_kernel(const uint32_t *rows, size_t ld_words, size_t N, size_t KB, size_t ntiles,
                                  uint4 *frag) {
    size_t total = ntiles * KB * 2 * 32;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t lane = i & 31, h = (i >> 5) & 1, t = i >> 6;
        size_t kb = t % KB, rt = t / KB;
        size_t row = rt * 16 + h * 8 + (lane >> 2), c = lane & 3;
        uint32_t v[4] = {0, 0, 0, 0};
        if (row < N) {
            for (size_t b = 0; b < 4; ++b) {
                size_t word = (kb * 4 + b) * 4 + c;
                if (word < ld_words) v[b] = rows[row * ld_words + word];
            }
        }
        frag[i] = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// I4CB block scales [N][bpr] -> fragment order (the slot of lane (g, c) holds block kb*4 + c)
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
    if (w->fmt == FNN_FMT_I4CB)
        to_frag_cb_kernel<<<blocks, 256, 0, ctx->stream>>>((const uint32_t *)w->rows, w->ld_u4 * 4, w->N, KB,
                                                         ntiles, w->frag);
    else
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

template <int FMT, int CG, int G>
int launch_mma_g(fnn_cuda_ctx *ctx, const QmmArgs &a, const float *act, float *out, int M, int split) {
    using T = FragTraits<FMT>;
    const fnn_cuda_qweight *w = a.w;
    MmaParams p{};
    p.frag = w->frag;
    p.scales = w->scales;
    p.zeros = w->zeros;
    p.act = act;
    p.out = out;
    p.bias = a.bias;
    p.M = M;
    p.N = (int)w->N;
    p.K = (int)w->K;
    p.KB = (int)div_ceil(w->K, (size_t)T::KBLK);
    p.ntiles = (int)div_ceil(w->N, 16);
    p.split = split;
    p.epilogue = a.epilogue;
    p.gather_on = (a.gather != nullptr && CG == 1);
    if (p.gather_on) p.g = *a.gather;

    // One block per SM: weight ring + as much of K as fits beside the reduction buffers.
    const int act_rows = split ? 2 * M : M;
    const int Mr = (M + 3) & ~3;
    const size_t ring = (size_t)G * kW * stages_for(CG) * kU * 2 * 512;
    const size_t fixed = ring + (size_t)(G * 2 * kW * CG * 128 + G * kW * Mr * 2 + 4 * Mr) * 4;
    const size_t per_tile = (size_t)G * (CG * 512 + 192);  // output accumulator + row metadata
    frag::FragSizing sz;
    const bool fits = frag::size_frag_launch(
        ctx->sm_count, p.ntiles, G, p.KB * T::KBLK, T::KBLK, fixed, per_tile,
        [&](int kc) { return (size_t)act_rows * (2 * kc + T::PAD_BYTES); }, &sz);
    FNN_REQUIRE(fits, FNN_ERR_UNSUPPORTED,
                "qmatmul: shared memory budget exceeded for M=%d on the skinny tensor-core path", M);
    p.tiles_per_group = sz.tiles_per_group;
    p.Kc = sz.Kc;
    const size_t smem = sz.smem;
    const int grid = sz.grid;
    auto kern = qmm_mma_kernel<FMT, CG, G>;
    FNN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(launch_pdl(kern, grid, G * kW * 32, smem, ctx, p), FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

// Groups per block: the most the register and shared-memory budget allows (groups_for) while that
// still gives (nearly) every SM a block; for the single-column-group kernels, layers with fewer row
// tiles run fewer groups per block so that the tiles spread over more SMs.
template <int FMT, int CG>
int launch_mma(fnn_cuda_ctx *ctx, const QmmArgs &a, const float *act, float *out, int M, int split) {
    constexpr int GMAX = groups_for(CG);
    if (CG == 1) {
        const int ntiles = (int)div_ceil(a.w->N, 16), want = ctx->sm_count * 4 / 5;
        if (GMAX >= 3 && (ntiles + 2) / 3 >= want) return launch_mma_g<FMT, CG, GMAX>(ctx, a, act, out, M, split);
        if ((ntiles + 1) / 2 >= want) return launch_mma_g<FMT, CG, (GMAX < 2 ? GMAX : 2)>(ctx, a, act, out, M, split);
        return launch_mma_g<FMT, CG, 1>(ctx, a, act, out, M, split);
    }
    return launch_mma_g<FMT, CG, GMAX>(ctx, a, act, out, M, split);
}

template <int FMT>
int launch_mma_fmt(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    const size_t N = a.w->N, K = a.w->K;
    for (size_t m0 = 0; m0 < a.M; m0 += kMaxRows) {
        const int M = (int)std::min<size_t>(kMaxRows, a.M - m0);
        const float *act = a.a + m0 * K;
        float *out = a.out + m0 * N;
        int rc;
        // two-term fp16 activations (f32-grade results) up to 32 batch rows: the hi and lo terms of a
        // row are two of the 8 * CG MMA columns; one term beyond, where the tcgen05 kernel is the
        // intended path and this one only runs on request
        if (M <= 4)
            rc = launch_mma<FMT, 1>(ctx, a, act, out, M, 1);
        else if (M <= 8)
            rc = launch_mma<FMT, 2>(ctx, a, act, out, M, 1);
        else if (M <= 16)
            rc = launch_mma<FMT, 4>(ctx, a, act, out, M, 1);
        else if (M <= 32)
            rc = launch_mma<FMT, 8>(ctx, a, act, out, M, 1);
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
    return w->N < (1u << 27) && w->K < (1u << 27);
}

int prepare_qmm_mma(fnn_cuda_ctx *ctx, fnn_cuda_qweight *w) { return ensure_frag(ctx, w); }

int launch_qmm_mma(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    int rc = ensure_frag(ctx, const_cast<fnn_cuda_qweight *>(a.w));
    if (rc != FNN_OK) return rc;
    // up to sixteen batch rows the 8-bit operand kernel serves I8 / I4 / FP4 / the codebook format from
    // the same fragment layout with exact integer products; the fp16 kernel below serves FP8 and larger
    // batches
    if (qmm_mma8_supported(a.w, a.M)) return launch_qmm_mma8(ctx, a);
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
        // block scales inside K: only the 8-bit operand kernel carries them; larger batches run
        // through it sixteen rows at a time
        for (size_t m0 = 0; m0 < a.M; m0 += 16) {
            QmmArgs part = a;
            part.a = a.a + m0 * a.w->K;
            part.out = a.out + m0 * a.w->N;
            part.M = std::min<size_t>(16, a.M - m0);
            rc = launch_qmm_mma8(ctx, part);
            if (rc != FNN_OK) return rc;
        }
        return FNN_OK;
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: unknown format %d", a.w->fmt);
}

}  // namespace fnn
