// Skinny-M kernel (1 <= M <= 16) on 8-bit tensor-core operands: the HBM scan of the weights with
// almost no instruction per weight.
//
// Same skeleton as the fp16 fragment kernel (fragment-major weights, one block per SM, groups of
// eight warps that split K, a private cp.async ring per lane), but the codes are fed to
// `mma.sync.m16n8k32` as 8-bit operands:
//   I8   -> s8 operands as stored (no decode at all)
//   I4   -> s8 operands holding 16*q: two masks per word of eight codes
//   FP4  -> s8 operands holding 2*|v| through a byte-permute table, positive and negative codes
//           in separate operands (two accumulators, subtracted at the end): no sign arithmetic
//   I4CB -> the 16 centroids as 14-bit fixed point, 128*hi + lo with hi, lo in [0, 127], looked up from
//           two byte-permute tables with the raw index as selector (two operands, two MMAs per
//           32-element scale block); the block scale multiplies the block's exact integer sum in f32
// (FP8 is not served here: `mma.sync` with e4m3 operands measured slower than the fp16 kernel on this
// part) and the f32 activations are rewritten while they are staged, per batch row, as
//   a ~= dq * (128*hi + lo)        (15-bit fixed point, exact int32 accumulation)
// Partial sums are integers, so the split-K reduction is exact in any order.
// Epilogue as everywhere:  out = act(dq*acc*scale[n] + zero[n]*sum_k a[m,k] + bias[n])
// (src/backend/cpu/microkernels/gemm.rs:2048-2087, src/backend/cpu/matmul.rs:61-71).
#include "frag_common.cuh"

namespace fnn {

namespace {

using frag::cp_async_commit;
using frag::cp_async_wait;
using frag::group_barrier;

constexpr int kW8 = frag::kWarpsPerGroup;   // warps per group
constexpr int kU8 = frag::kChunkBlocks;     // k-blocks per ring chunk
constexpr int kS8 = 3;   // ring stages per lane (two chunks, 96 KB per SM, in flight)
constexpr int kMma8MaxRows = 16;   // four 8-column groups of (term, batch row) columns

template <int FMT>
struct T8 {
    static constexpr bool four_bit = (FMT == FNN_FMT_I4 || FMT == FNN_FMT_F4 || FMT == FNN_FMT_I4CB);
    static constexpr bool codebook = (FMT == FNN_FMT_I4CB);
    static constexpr int KBLK = four_bit ? 128 : 64;       // k per k-block (4 lanes x 16 bytes per row)
    static constexpr int MMAS = four_bit ? 4 : 2;          // m16n8k32 MMAs per k-block
    static constexpr int PAD = four_bit ? 16 : 64;         // activation row padding (bank spread)
};


__device__ __forceinline__ void mma_s8(int *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// prmt.b32 in its default mode: selector nibble n picks byte n&7 of {a, b}; bit 3 of the nibble
// replaces the byte by its sign bit replicated eight times.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Eight 4-bit codes of one word -> the two A registers of one m16n8k32 MMA.
//   I4: lo = 16*q of codes 0,2,4,6 ; hi = 16*q of codes 1,3,5,7 (the activations are staged in the
//       matching order 0,2,4,6,1,3,5,7 of each 8-group)
__device__ __forceinline__ void decode_i4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    lo = (w << 4) & 0xF0F0F0F0u;
    hi = w & 0xF0F0F0F0u;
}
//   F4 (sign | 3-bit magnitude code): the magnitudes 0,.5,1,1.5,2,3,4,6 doubled are the bytes of a
//   table that prmt indexes with the raw code.  A code with its sign bit set makes prmt return the
//   replicated top bit of the table byte, i.e. 0 -- so the raw word yields the positive weights
//   (negative ones as 0) and the word with all sign bits flipped yields the negative weights'
//   magnitudes: pos/neg operands in natural element order, seven ALU operations per eight weights.
__device__ __forceinline__ void decode_f4(uint32_t w, uint32_t &plo, uint32_t &phi, uint32_t &nlo,
                                          uint32_t &nhi) {
    const uint32_t t0 = 0x03020100u, t1 = 0x0C080604u;
    const uint32_t f = w ^ 0x88888888u;
    plo = prmt(t0, t1, w);
    phi = prmt(t0, t1, w >> 16);
    nlo = prmt(t0, t1, f);
    nhi = prmt(t0, t1, f >> 16);
}

//   I4CB (index into 16 centroids): every centroid is carried as v = 128*hi + lo, hi and lo in
//   [0, 127], so a table byte never has its top bit set.  Indices 0..7 come out of one prmt on the
//   raw word (indices 8..15 select "replicated top bit" = 0 there), indices 8..15 out of a second
//   prmt on the word with every index's bit 3 flipped (indices 0..7 give 0 there).  The two halves
//   are not merged: each is an operand of its own MMA into the same accumulator, which costs tensor
//   issue slots (idle here) instead of logic instructions (the limiter).
struct CbTables {
    uint32_t hi[4], lo[4];   // bytes of entries 0-3, 4-7, 8-11, 12-15
};
struct CbOperands {
    uint32_t hi_a[2], hi_b[2], lo_a[2], lo_b[2];   // [codes 0..3 | codes 4..7]; _a: indices 0..7, _b: 8..15
};
__device__ __forceinline__ void decode_cb(const CbTables &t, uint32_t w, CbOperands &o) {
    const uint32_t f = w ^ 0x88888888u, w16 = w >> 16, f16 = f >> 16;
    o.hi_a[0] = prmt(t.hi[0], t.hi[1], w);
    o.hi_a[1] = prmt(t.hi[0], t.hi[1], w16);
    o.hi_b[0] = prmt(t.hi[2], t.hi[3], f);
    o.hi_b[1] = prmt(t.hi[2], t.hi[3], f16);
    o.lo_a[0] = prmt(t.lo[0], t.lo[1], w);
    o.lo_a[1] = prmt(t.lo[0], t.lo[1], w16);
    o.lo_b[0] = prmt(t.lo[2], t.lo[3], f);
    o.lo_b[1] = prmt(t.lo[2], t.lo[3], f16);
}
constexpr int kCbHalf = 8192;   // centroid c is carried as v = round(c / cmax * 8191) + 8192

// Staged byte position of activation k inside its row: where its group of eight goes, plus its place
// inside the group.  I4 reorders inside the group (0,2,4,6,1,3,5,7: even codes of a word, then odd);
// the codebook format keeps the group but orders the sixteen groups of a 128-k block by (word c of a
// scale block, scale block b) instead of (b, c), so that the 32 bytes one lane needs for the four MMAs
// of a k-block are contiguous.
template <int FMT>
__device__ __forceinline__ int group_pos8(int k8) {   // k8: a multiple of 8
    if (FMT == FNN_FMT_I4CB) {
        const int r = k8 & 127, b = r >> 5, c = (r >> 3) & 3;
        return (k8 & ~127) + c * 32 + b * 8;
    }
    return k8;
}
template <int FMT>
__device__ __forceinline__ int inner_pos8(int i) {    // i in [0, 8)
    return FMT == FNN_FMT_I4 ? ((i >> 1) + (i & 1) * 4) : i;
}
template <int FMT>
__device__ __forceinline__ int act_pos8(int k) {
    return group_pos8<FMT>(k & ~7) + inner_pos8<FMT>(k & 7);
}

struct P8 {
    const uint4 *frag;
    const float *frag_bs;   // I4CB: block scales in fragment order
    const float *codebook;  // I4CB: 16 centroids
    const float *scales;
    const float *zeros;
    const float *act;
    float *out;
    const float *bias;
    int M, N, K;
    int KB, ntiles, tiles_per_group;
    int Kc;      // activations staged per pass (multiple of KBLK)
    int epilogue;
    int gather_on;
    GatherArgs g;
};

// MULTI: more than one batch row (all rows scanned and staged together); the single-row instantiation
// keeps the shortest prologue.  CG 8-column groups hold the (term, batch row) columns: up to 4 * CG rows.
template <int FMT, int CG, int kG8, bool MULTI>
__global__ void __launch_bounds__(kG8 * kW8 * 32, (kG8 == 1 && CG == 1 && !MULTI && !T8<FMT>::codebook) ? 3 : 1)
qmm_mma8_kernel(P8 p) {
    using TT = T8<FMT>;
    constexpr int KBLK = TT::KBLK, MMAS = TT::MMAS;
    constexpr int NT = kG8 * kW8 * 32, NW = kG8 * kW8;
    constexpr int UNITS = kU8 * 2;
    constexpr int MR = 4 * CG;                 // batch rows this instantiation can hold
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = p.Kc + TT::PAD;             // bytes per staged activation row
    const int cols = 2 * p.M;                  // (term, batch row) columns in use
    constexpr bool CB = TT::codebook;
    unsigned char *s_ring = smem;                                         // [NW][S][UNITS][32] uint4
    float *s_ring_bs = reinterpret_cast<float *>(s_ring + (size_t)NW * kS8 * UNITS * 512);   // I4CB: [NW][S][UNITS][32]
    unsigned char *s_act = reinterpret_cast<unsigned char *>(s_ring_bs + (CB ? (size_t)NW * kS8 * UNITS * 32 : 0));  // [cols][RS]
    float *s_red = reinterpret_cast<float *>(s_act + (((size_t)cols * RS + 15) & ~(size_t)15));
    float *s_out = s_red + kG8 * 2 * kW8 * CG * 128;                      // [G][tiles_per_group][CG*128]
    float *s_meta = s_out + (size_t)kG8 * p.tiles_per_group * CG * 128;   // [G][tiles_per_group][16][3]
    float *s_part = s_meta + (size_t)kG8 * p.tiles_per_group * 48;        // [NW][MR][2]
    float *s_dq = s_part + NW * MR * 2;                                   // [MR]
    float *s_rs = s_dq + MR;                                              // [MR]
    float *s_mx = s_rs + MR;                                              // [MR]
    // I4CB: -8192 * (sum of the staged bytes of a 32-element block), per block and column
    int *s_boff = reinterpret_cast<int *>(s_mx + MR);                     // [Kc / 32][8 * CG]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = warp / kW8, gw = warp % kW8, gtid = tid - group * kW8 * 32;
    const int g = lane >> 2, c = lane & 3;
    const int gg = group * gridDim.x + blockIdx.x, GG = gridDim.x * kG8;
    // the next kernel on the stream may be set up as soon as an SM has room: its own prologue (scales,
    // first weight copies) then runs under this kernel's tail
    pdl_launch_dependents();
    GatherCursor gc{};
    const int tiles_here = gg < p.ntiles ? (p.ntiles - gg + GG - 1) / GG : 0;
    const bool has_zero = p.zeros != nullptr;
    float *my_out = s_out + (size_t)group * p.tiles_per_group * CG * 128;
    float *my_red = s_red + (size_t)group * 2 * kW8 * CG * 128;
    float *my_meta = s_meta + (size_t)group * p.tiles_per_group * 48;
    unsigned char *my_ring = s_ring + (size_t)warp * kS8 * UNITS * 512 + lane * 16;
    float *my_ring_bs = s_ring_bs + (size_t)warp * kS8 * UNITS * 32;

    // I4CB: the centroids as 14-bit fixed point (every thread builds its own copy of the two tables)
    CbTables cbt{};
    float cb_unit = 0.0f;   // value of one fixed-point step
    if (CB) {
        float cv[16], cmax = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            cv[j] = __ldg(p.codebook + j);
            cmax = fmaxf(cmax, fabsf(cv[j]));
        }
        const float to_fix = cmax > 0.0f ? (float)(kCbHalf - 1) / cmax : 0.0f;
        cb_unit = cmax / (float)(kCbHalf - 1);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int v = __float2int_rn(cv[j] * to_fix) + kCbHalf;   // 1 .. 16383
            cbt.hi[j >> 2] |= (uint32_t)(v >> 7) << ((j & 3) * 8);
            cbt.lo[j >> 2] |= (uint32_t)(v & 127) << ((j & 3) * 8);
        }
    }

    for (int i = gtid; i < tiles_here * 16; i += kW8 * 32) {
        const int n = (gg + (i >> 4) * GG) * 16 + (i & 15);
        const bool in = n < p.N;
        my_meta[i * 3 + 0] = (in && !CB) ? __ldg(p.scales + n) : 1.0f;
        my_meta[i * 3 + 1] = (in && has_zero) ? __ldg(p.zeros + n) : 0.0f;
        my_meta[i * 3 + 2] = (in && p.bias) ? __ldg(p.bias + n) : 0.0f;
    }
    for (int i = tid; i < kG8 * p.tiles_per_group * CG * 128; i += NT) s_out[i] = 0.0f;

    // staged row holding batch column (cg*8 + g), or -1
    int brow[CG];
#pragma unroll
    for (int cg = 0; cg < CG; ++cg) brow[cg] = (cg * 8 + g < cols) ? cg * 8 + g : -1;

    int acci[CG][4], accn[FMT == FNN_FMT_F4 ? CG : 1][4];   // accn: FP4's negative-weight sums
    float accf[CB ? CG : 1][4];                              // I4CB: block sums times block scales
#pragma unroll
    for (int cg = 0; cg < CG; ++cg)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            acci[cg][r] = 0;
            if (FMT == FNN_FMT_F4) accn[cg][r] = 0;
            if constexpr (CB) accf[cg][r] = 0.0f;
        }
    int red_buf = 0;

    const bool vec_ok = (p.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.act) & 15u) == 0);
    const int Kpad = p.KB * KBLK;
    // groups of eight activations a thread keeps (single row, K <= 4096 per group of warps in the
    // block); three-group blocks have no registers to spare for it
    constexpr bool kCanHold = !MULTI && kG8 <= 2;
    constexpr int kHeld = 2;
    float hv[kCanHold ? kHeld : 1][8];
    bool held = false;
    for (int k0 = 0; k0 < Kpad; k0 += p.Kc) {
        const int kc_len = min(p.Kc, Kpad - k0);
        const int KBc = kc_len / KBLK;
        const int kb0 = k0 / KBLK;
        const int nch = (KBc + kU8 - 1) / kU8;
        const int cpw = (nch + kW8 - 1) / kW8;
        // issue-side cursor: the next item (tile, chunk-of-this-warp) whose copies go into the ring
        int i_tl = 0, i_j = 0, i_st = 0;
        auto issue_next = [&]() {
            const bool valid = i_tl < tiles_here;
            const int ch = gw + i_j * kW8;
            const uint4 *tile_src = p.frag + ((size_t)(gg + i_tl * GG) * p.KB + kb0) * 64 + lane;
#pragma unroll
            for (int u = 0; u < kU8; ++u) {
                const int kb = ch * kU8 + u;
                const bool ok = valid && (kb < KBc);
                const uint4 *src = ok ? tile_src + (size_t)kb * 64 : p.frag;
                frag::cp_async16(my_ring + (size_t)(i_st * UNITS + u * 2) * 512, src, ok ? 16 : 0);
                frag::cp_async16(my_ring + (size_t)(i_st * UNITS + u * 2 + 1) * 512, src + 32, ok ? 16 : 0);
                if (CB) {   // one block scale per 16-byte unit
                    const float *bsrc = p.frag_bs + (ok ? (src - p.frag) : 0);
                    frag::cp_async4(my_ring_bs + (i_st * UNITS + u * 2) * 32 + lane, bsrc, ok ? 4 : 0);
                    frag::cp_async4(my_ring_bs + (i_st * UNITS + u * 2 + 1) * 32 + lane, bsrc + 32, ok ? 4 : 0);
                }
            }
            cp_async_commit();
            if (++i_j == cpw) {
                i_j = 0;
                ++i_tl;
            }
            if (++i_st == kS8) i_st = 0;
        };
#pragma unroll
        for (int i = 0; i < kS8 - 1; ++i) issue_next();

        if (k0 == 0) {   // under the first weight loads: the per-row scan of the activations
            // everything above (scales, the first weight copies) is independent of the kernel before
            // this one on the stream; the activations and the gather counters are not
            pdl_wait();
            if (p.gather_on) gc = gather_begin(p.g, blockIdx.x * NT + tid);
            // ---- per-row step and sum: max |a| over the whole row first ---------------------
            if (kCanHold && vec_ok && p.K % 8 == 0 && p.K <= NT * 8 * kHeld && kc_len >= Kpad) {
                // A single batch row that is staged in one pass: every thread keeps its groups of eight
                // consecutive activations in registers between the scan and the rewrite, so the row is
                // read once.
                held = true;
                float mx = 0.0f, sum = 0.0f;
#pragma unroll
                for (int j = 0; j < kHeld; ++j) {
                    const int g8 = tid + j * NT;
                    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
                    if (g8 * 8 < p.K) {
                        a = __ldg(reinterpret_cast<const float4 *>(p.act) + 2 * g8);
                        b = __ldg(reinterpret_cast<const float4 *>(p.act) + 2 * g8 + 1);
                    }
                    hv[j][0] = a.x; hv[j][1] = a.y; hv[j][2] = a.z; hv[j][3] = a.w;
                    hv[j][4] = b.x; hv[j][5] = b.y; hv[j][6] = b.z; hv[j][7] = b.w;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        mx = fmaxf(mx, fabsf(hv[j][q]));
                        sum += hv[j][q];
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
                    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
                }
                if (lane == 0) {
                    s_part[warp * 2] = mx;
                    s_part[warp * 2 + 1] = sum;
                }
                __syncthreads();
                if (tid == 0) {   // fixed order: the sums do not depend on scheduling
                    float bm = 0.0f, bs = 0.0f;
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        bm = fmaxf(bm, s_part[w * 2]);
                        bs += s_part[w * 2 + 1];
                    }
                    s_mx[0] = bm;
                    s_rs[0] = bs;
                }
                __syncthreads();
            } else {
                frag::scan_rows<NT, MULTI ? 4 : 1>(p.act, p.M, p.K, vec_ok, s_part, s_mx, s_rs);
            }
            if (tid < p.M) {
                const float bm = s_mx[tid];
                s_dq[tid] = (bm > 0.0f && isfinite(bm)) ? bm / 16256.0f : 1.0f;
            }   // (published by the barrier below)

            // the first poll of the previous step's words was issued at the top; its latency is hidden by now
            if (p.gather_on && gc.step > 1u) gather_check_prev(p.g, gc, gridDim.x * NT);
        }

        __syncthreads();  // previous pass fully consumed
        // ---- stage the activation bytes of [k0, k0 + kc_len) --------------------------------
        if (MULTI && vec_ok && (p.K % 8 == 0)) {
            // eight activations of four rows per thread and step: two 16-byte loads per row in flight,
            // one 8-byte store per (row, plane)
            const int n8 = kc_len / 8;
            for (int i8 = tid; i8 < n8; i8 += NT) {
                const bool in = k0 + i8 * 8 < p.K;
                for (int mb = 0; mb < p.M; mb += 4) {
                    float4 v[4][2];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        v[m][0] = v[m][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (mb + m < p.M && in) {
                            const float4 *src =
                                reinterpret_cast<const float4 *>(p.act + (size_t)(mb + m) * p.K + k0 + i8 * 8);
                            v[m][0] = __ldg(src);
                            v[m][1] = __ldg(src + 1);
                        }
                    }
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        if (mb + m < p.M) {
                            const float inv = 1.0f / s_dq[mb + m];
                            const float e[8] = {v[m][0].x, v[m][0].y, v[m][0].z, v[m][0].w,
                                                v[m][1].x, v[m][1].y, v[m][1].z, v[m][1].w};
                            uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                int q = __float2int_rn(e[j] * inv);
                                q = max(-16256, min(16256, q));
                                const int h = (q + 64) >> 7;
                                const int pos = inner_pos8<FMT>(j);   // position inside the 8-group
                                hi[pos >> 2] |= (uint32_t)(h & 0xFF) << ((pos & 3) * 8);
                                lo[pos >> 2] |= (uint32_t)((q - h * 128) & 0xFF) << ((pos & 3) * 8);
                            }
                            const int gp = group_pos8<FMT>(i8 * 8);
                            *reinterpret_cast<uint2 *>(s_act + (size_t)(mb + m) * RS + gp) = make_uint2(hi[0], hi[1]);
                            *reinterpret_cast<uint2 *>(s_act + (size_t)(p.M + mb + m) * RS + gp) =
                                make_uint2(lo[0], lo[1]);
                        }
                    }
                }
            }
        } else if (kCanHold && held) {
            const float inv = 1.0f / s_dq[0];
#pragma unroll
            for (int j = 0; j < kHeld; ++j) {
                const int g8 = tid + j * NT;
                if (g8 * 8 >= kc_len) continue;   // (beyond K the held values are zero: the padding of the last block)
                uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) {
                    int q = __float2int_rn(hv[j][q8] * inv);
                    q = max(-16256, min(16256, q));
                    const int h = (q + 64) >> 7;
                    const int pos = inner_pos8<FMT>(q8);
                    hi[pos >> 2] |= (uint32_t)(h & 0xFF) << ((pos & 3) * 8);
                    lo[pos >> 2] |= (uint32_t)((q - h * 128) & 0xFF) << ((pos & 3) * 8);
                }
                const int gp = group_pos8<FMT>(g8 * 8);
                *reinterpret_cast<uint2 *>(s_act + gp) = make_uint2(hi[0], hi[1]);
                *reinterpret_cast<uint2 *>(s_act + (size_t)RS + gp) = make_uint2(lo[0], lo[1]);
            }
        } else
        for (int m = 0; m < p.M; ++m) {
            const float *row = p.act + (size_t)m * p.K;
            const float inv = 1.0f / s_dq[m];
            auto put = [&](int k, float a) {
                const float x = a * inv;
                const int pos = act_pos8<FMT>(k);
                int q = __float2int_rn(x);
                q = max(-16256, min(16256, q));
                const int hi = (q + 64) >> 7;
                s_act[(size_t)m * RS + pos] = (unsigned char)(signed char)hi;
                s_act[(size_t)(p.M + m) * RS + pos] = (unsigned char)(signed char)(q - hi * 128);
            };
            if (vec_ok) {
                const int n4 = kc_len / 4;
                for (int b4 = 0; b4 < n4; b4 += 2 * NT) {
                    float4 v[2];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int i4 = b4 + q * NT + tid;
                        v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (i4 < n4 && k0 + i4 * 4 < p.K)
                            v[q] = __ldg(reinterpret_cast<const float4 *>(row + k0 + i4 * 4));
                    }
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int i4 = b4 + q * NT + tid;
                        if (i4 < n4) {
                            put(i4 * 4 + 0, v[q].x);
                            put(i4 * 4 + 1, v[q].y);
                            put(i4 * 4 + 2, v[q].z);
                            put(i4 * 4 + 3, v[q].w);
                        }
                    }
                }
            } else {
                for (int k = tid; k < kc_len; k += NT) put(k, (k0 + k < p.K) ? __ldg(row + k0 + k) : 0.0f);
            }
        }
        __syncthreads();
        if (CB) {
            // -8192 * sum of each 32-element block of every staged column: the centroids are carried
            // with an offset of 8192, which the second MMA of a block takes back through its C operand
            const int nblk = kc_len / 32;
            for (int i = tid; i < nblk * 8 * CG; i += NT) {
                const int blk = i / (8 * CG), col = i - blk * (8 * CG), kb = blk >> 2, b = blk & 3;
                int sum = 0;
                if (col < cols) {
                    const unsigned char *src = s_act + (size_t)col * RS + kb * 128 + b * 8;
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {   // the block's eight bytes of each of its four words
                        const uint2 x = *reinterpret_cast<const uint2 *>(src + c4 * 32);
                        sum = __dp4a((int)x.x, 0x01010101, sum);
                        sum = __dp4a((int)x.y, 0x01010101, sum);
                    }
                }
                s_boff[i] = -kCbHalf * sum;
            }
            __syncthreads();
        }

        // ---- stream this K range of every tile of the group ----------------------------------
        int c_st = 0;
        for (int tl = 0; tl < tiles_here; ++tl)
        for (int j = 0; j < cpw; ++j) {
            issue_next();
            cp_async_wait<kS8 - 1>();
            const int ch = gw + j * kW8;
#pragma unroll(CB ? 1 : kU8)
            for (int u = 0; u < kU8; ++u) {
                const int slot = c_st * UNITS + u * 2;
                const uint4 wl = *reinterpret_cast<const uint4 *>(my_ring + (size_t)slot * 512);
                const uint4 wh = *reinterpret_cast<const uint4 *>(my_ring + (size_t)(slot + 1) * 512);
                const int kb_s = min(ch * kU8 + u, KBc - 1);
                if constexpr (CB) {
                    // The unit of lane (g, c) holds word c of the four 32-element blocks of this
                    // k-block: block b is two MMAs for the hi bytes of the centroids plus two for the lo
                    // bytes, eight codes of rows g and g + 8 per lane, and its integer sum is scaled by the
                    // block scale of each row, which sits in the ring slot of lane (g, b).
                    const uint32_t wl4[4] = {wl.x, wl.y, wl.z, wl.w}, wh4[4] = {wh.x, wh.y, wh.z, wh.w};
                    const float4 bl4 = *reinterpret_cast<const float4 *>(my_ring_bs + slot * 32 + (lane & ~3));
                    const float4 bh4 = *reinterpret_cast<const float4 *>(my_ring_bs + (slot + 1) * 32 + (lane & ~3));
                    const float bs_lo[4] = {bl4.x, bl4.y, bl4.z, bl4.w}, bs_hi[4] = {bh4.x, bh4.y, bh4.z, bh4.w};
                    const unsigned char *ap[CG];   // this lane's activation bytes: 8 per scale block
                    const int *op[CG];             // -8192 * block sums of its two columns
#pragma unroll
                    for (int cg = 0; cg < CG; ++cg) {
                        ap[cg] = s_act + (size_t)max(brow[cg], 0) * RS + kb_s * 128 + c * 32;
                        op[cg] = s_boff + (size_t)kb_s * 4 * 8 * CG + cg * 8 + 2 * c;
                    }
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        CbOperands rg, rh;   // row g, row g + 8
                        decode_cb(cbt, wl4[b], rg);
                        decode_cb(cbt, wh4[b], rh);
#pragma unroll
                        for (int cg = 0; cg < CG; ++cg) {
                            uint2 bb = *reinterpret_cast<const uint2 *>(ap[cg] + b * 8);
                            if (brow[cg] < 0) bb = make_uint2(0u, 0u);
                            const uint32_t b0 = bb.x, b1 = bb.y;
                            const int2 off = *reinterpret_cast<const int2 *>(op[cg] + b * 8 * CG);
                            int dh[4] = {0, 0, 0, 0};
                            int dl[4] = {off.x, off.y, off.x, off.y};
                            mma_s8(dh, rg.hi_a[0], rh.hi_a[0], rg.hi_a[1], rh.hi_a[1], b0, b1);
                            mma_s8(dh, rg.hi_b[0], rh.hi_b[0], rg.hi_b[1], rh.hi_b[1], b0, b1);
                            mma_s8(dl, rg.lo_a[0], rh.lo_a[0], rg.lo_a[1], rh.lo_a[1], b0, b1);
                            mma_s8(dl, rg.lo_b[0], rh.lo_b[0], rg.lo_b[1], rh.lo_b[1], b0, b1);
                            accf[cg][0] = fmaf(bs_lo[b], (float)(dh[0] * 128 + dl[0]), accf[cg][0]);
                            accf[cg][1] = fmaf(bs_lo[b], (float)(dh[1] * 128 + dl[1]), accf[cg][1]);
                            accf[cg][2] = fmaf(bs_hi[b], (float)(dh[2] * 128 + dl[2]), accf[cg][2]);
                            accf[cg][3] = fmaf(bs_hi[b], (float)(dh[3] * 128 + dl[3]), accf[cg][3]);
                        }
                    }
                    continue;
                }
                // this lane's activation bytes of the k-block: 16 (8-bit codes) or 32 (4-bit)
                const int boff = kb_s * KBLK + c * (KBLK / 4);
#pragma unroll
                for (int v = 0; v < MMAS / 2; ++v) {  // one 16-byte activation vector feeds two MMAs
                    uint32_t a[2][4];                // [mma][a0 a1 a2 a3]
                    uint32_t an[2][4];               // FP4 only: magnitudes of the negative weights
                    if (TT::four_bit) {
                        const uint32_t wl0 = v ? wl.z : wl.x, wl1 = v ? wl.w : wl.y;
                        const uint32_t wh0 = v ? wh.z : wh.x, wh1 = v ? wh.w : wh.y;
                        if (FMT == FNN_FMT_I4) {
                            decode_i4(wl0, a[0][0], a[0][2]);
                            decode_i4(wh0, a[0][1], a[0][3]);
                            decode_i4(wl1, a[1][0], a[1][2]);
                            decode_i4(wh1, a[1][1], a[1][3]);
                        } else {
                            decode_f4(wl0, a[0][0], a[0][2], an[0][0], an[0][2]);
                            decode_f4(wh0, a[0][1], a[0][3], an[0][1], an[0][3]);
                            decode_f4(wl1, a[1][0], a[1][2], an[1][0], an[1][2]);
                            decode_f4(wh1, a[1][1], a[1][3], an[1][1], an[1][3]);
                        }
                    } else {
                        a[0][0] = wl.x; a[0][2] = wl.y; a[0][1] = wh.x; a[0][3] = wh.y;
                        a[1][0] = wl.z; a[1][2] = wl.w; a[1][1] = wh.z; a[1][3] = wh.w;
                    }
#pragma unroll
                    for (int cg = 0; cg < CG; ++cg) {
                        uint4 b = make_uint4(0, 0, 0, 0);
                        if (brow[cg] >= 0)
                            b = *reinterpret_cast<const uint4 *>(s_act + (size_t)brow[cg] * RS + boff + v * 16);
                        mma_s8(acci[cg], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma_s8(acci[cg], a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
                        if (FMT == FNN_FMT_F4) {
                            mma_s8(accn[FMT == FNN_FMT_F4 ? cg : 0], an[0][0], an[0][1], an[0][2], an[0][3], b.x, b.y);
                            mma_s8(accn[FMT == FNN_FMT_F4 ? cg : 0], an[1][0], an[1][1], an[1][2], an[1][3], b.z, b.w);
                        }
                    }
                }
            }
            if (++c_st == kS8) c_st = 0;
            if (j == cpw - 1) {
                // last chunk of a tile: fixed-order reduction over the group's warps
                float *red = my_red + (size_t)red_buf * kW8 * CG * 128;
#pragma unroll
                for (int cg = 0; cg < CG; ++cg)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        red[(gw * CG + cg) * 128 + r * 32 + lane] =
                            CB ? accf[CB ? cg : 0][r]
                               : (float)(FMT == FNN_FMT_F4 ? acci[cg][r] - accn[FMT == FNN_FMT_F4 ? cg : 0][r]
                                                           : acci[cg][r]);
                        acci[cg][r] = 0;
                        if (FMT == FNN_FMT_F4) accn[cg][r] = 0;
                        if constexpr (CB) accf[cg][r] = 0.0f;
                    }
                group_barrier(group);
                for (int e = gtid; e < CG * 128; e += kW8 * 32) {
                    float s = 0.0f;
#pragma unroll
                    for (int w = 0; w < kW8; ++w) s += red[w * CG * 128 + e];
                    my_out[tl * CG * 128 + e] += s;
                }
                red_buf ^= 1;
            }
        }
        cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned step = gc.step;

    // ---- epilogue ----------------------------------------------------------------------------
    const int total = tiles_here * 16 * p.M;
    for (int i = gtid; i < total; i += kW8 * 32) {
        const int tl = i / (16 * p.M);
        const int rem = i - tl * 16 * p.M;
        const int m = rem >> 4, r16 = rem & 15;
        const int n = (gg + tl * GG) * 16 + r16;
        if (n >= p.N) continue;
        auto at = [&](int col) {
            const int cg = col >> 3, cc = col & 7;
            return my_out[tl * CG * 128 + cg * 128 + ((r16 >> 3) * 2 + (cc & 1)) * 32 + (r16 & 7) * 4 + (cc >> 1)];
        };
        float acc = at(m) * 128.0f + at(p.M + m);
        if (FMT == FNN_FMT_I4) acc *= 0.0625f;  // operands carried 16*q
        if (FMT == FNN_FMT_F4) acc *= 0.5f;     // operands carried 2*|v|
        const float *meta = my_meta + (tl * 16 + r16) * 3;
        float v;
        if (CB) {   // no per-row scale or zero point: the block scales are inside acc
            const float dot = acc * s_dq[m] * cb_unit;
            v = apply_act(p.bias ? __fadd_rn(dot, meta[2]) : dot, p.epilogue);
        } else {
            v = finish_output(acc * s_dq[m], meta[0], meta[1], has_zero ? s_rs[m] : 0.0f, p.bias != nullptr,
                              meta[2], p.epilogue);
        }
        if (!p.gather_on) {
            p.out[(size_t)m * p.N + n] = v;
        } else {
            gather_store(p.g, step, m, n, v);
        }
    }
    if (p.gather_on) gather_finish(p.g, step, p.M, p.N);
}

template <int FMT, int CG, int kG8, bool MULTI>
int launch8(fnn_cuda_ctx *ctx, const QmmArgs &a, int blocks_per_sm = 1) {
    using TT = T8<FMT>;
    const fnn_cuda_qweight *w = a.w;
    P8 p{};
    p.frag = w->frag;
    p.frag_bs = w->frag_bs;
    p.codebook = w->codebook;
    p.scales = w->scales;
    p.zeros = w->zeros;
    p.act = a.a;
    p.out = a.out;
    p.bias = a.bias;
    p.M = (int)a.M;
    p.N = (int)w->N;
    p.K = (int)w->K;
    p.KB = (int)div_ceil(w->K, (size_t)TT::KBLK);
    p.ntiles = (int)div_ceil(w->N, 16);
    p.epilogue = a.epilogue;
    p.gather_on = a.gather != nullptr;
    if (a.gather) p.g = *a.gather;
    const int cols = 2 * p.M;   // int8 pairs
    constexpr int MR = 4 * CG;
    const size_t ring = (size_t)kG8 * kW8 * kS8 * kU8 * 2 * (512 + (TT::codebook ? 128 : 0));
    const size_t fixed = ring + (size_t)(kG8 * 2 * kW8 * CG * 128 + kG8 * kW8 * MR * 2 + 3 * MR) * 4 + 64;
    const size_t per_tile = (size_t)kG8 * (CG * 512 + 192);
    frag::FragSizing sz;
    const bool fits = frag::size_frag_launch(
        ctx->sm_count, p.ntiles, kG8, p.KB * TT::KBLK, TT::KBLK, fixed, per_tile,
        [&](int kc) {
            return ((((size_t)cols * (kc + TT::PAD)) + 15) & ~(size_t)15) +
                   (TT::codebook ? (size_t)(kc / 32) * 8 * CG * 4 : 0);
        },
        &sz, blocks_per_sm);
    if (!fits && blocks_per_sm > 1) return launch8<FMT, CG, kG8, MULTI>(ctx, a, 1);
    FNN_REQUIRE(fits, FNN_ERR_UNSUPPORTED,
                "qmatmul: shared memory budget exceeded for M=%d on the 8-bit fragment kernel", p.M);
    p.tiles_per_group = sz.tiles_per_group;
    p.Kc = sz.Kc;
    auto kern = qmm_mma8_kernel<FMT, CG, kG8, MULTI>;
    FNN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sz.smem),
                   FNN_ERR_DISPATCH);
    FNN_CUDA_CHECK(launch_pdl(kern, sz.grid, kG8 * kW8 * 32, sz.smem, ctx, p), FNN_ERR_DISPATCH);
    ctx->launches++;
    ctx->last_path = "mma8";
    return FNN_OK;
}

// Groups per block: three while that still gives (nearly) every SM a block; layers with fewer row
// tiles run two or one group per block so that the tiles spread over more SMs.  Two and four column
// groups (5..8 and 9..16 batch rows) keep more accumulators per thread and run at most two groups.
template <int FMT, int CG>
int launch8_cg(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    const int ntiles = (int)div_ceil(a.w->N, 16), want = ctx->sm_count * 4 / 5;
    if (CG == 1) {
        const bool multi = a.M > 1;
        // (the codebook format keeps its two lookup tables in registers: two groups at most)
        if constexpr (!T8<FMT>::codebook) {
            // A single batch row on a layer with one to three tiles per group runs as three independent
            // one-group blocks per SM instead of one three-group block: blocks of the next kernel on the
            // stream then take the place of single finished blocks and prefetch their weights under
            // this kernel's tail (config 2: 9.8 -> 9.0 us per step).  Smaller layers lose more to the
            // smaller blocks' repeated prologue than they gain, larger ones have no tail to speak of.
            if (!multi && ntiles >= 3 * ctx->sm_count && ntiles < 9 * ctx->sm_count)
                return launch8<FMT, 1, 1, false>(ctx, a, 3);
            if ((ntiles + 2) / 3 >= want)
                return multi ? launch8<FMT, 1, 3, true>(ctx, a) : launch8<FMT, 1, 3, false>(ctx, a);
        }
        if ((ntiles + 1) / 2 >= want)
            return multi ? launch8<FMT, 1, 2, true>(ctx, a) : launch8<FMT, 1, 2, false>(ctx, a);
        return multi ? launch8<FMT, 1, 1, true>(ctx, a) : launch8<FMT, 1, 1, false>(ctx, a);
    }
    if ((ntiles + 1) / 2 >= want) return launch8<FMT, CG, 2, true>(ctx, a);
    return launch8<FMT, CG, 1, true>(ctx, a);
}

template <int FMT>
int launch8_fmt(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    const int M = (int)a.M;
    FNN_REQUIRE(M >= 1 && M <= kMma8MaxRows, FNN_ERR_UNSUPPORTED,
                "qmatmul: the 8-bit fragment kernel holds up to %d batch rows as int8 pairs (M=%d)",
                kMma8MaxRows, M);
    if (M <= 4) return launch8_cg<FMT, 1>(ctx, a);
    if (M <= 8) return launch8_cg<FMT, 2>(ctx, a);
    return launch8_cg<FMT, 4>(ctx, a);
}

}  // namespace

bool qmm_mma8_supported(const fnn_cuda_qweight *w, size_t M) {
    // Every format whose values are small integers (I8, I4, and FP4 doubled) runs on s8 operands with
    // the activations as exact int8 pairs; `mma.sync` with e4m3 operands runs at a fraction of the
    // fp16 rate on this part, so FP8 stays on the fp16 kernel.
    return (w->fmt == FNN_FMT_I8 || w->fmt == FNN_FMT_I4 || w->fmt == FNN_FMT_F4 || w->fmt == FNN_FMT_I4CB) &&
           M >= 1 &&
           M <= (size_t)kMma8MaxRows &&
           w->N < (1u << 27) &&
           w->K < (1u << 27);
}

// Consumer side of the fused gather: polls (bounded) every word of the last completed step in this
// rank's buffer and, if `out` is given, writes the values as plain f32 [world][rows][n_stride].
__global__ void gather_wait_kernel(const unsigned long long *words, const unsigned *counters, int world,
                                   int n_stride, float *out, int *err_flag) {
    const unsigned step = counters[0];
    const int rows = (int)counters[2];
    if (step == 0u) return;
    const unsigned long long *slot = words + (size_t)(step & 1u) * world * kGatherRows * n_stride;
    const int per_rank = rows * n_stride;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < world * per_rank; i += gridDim.x * blockDim.x) {
        const int r = i / per_rank;
        unsigned long long w;
        if (!wait_word(slot + (size_t)r * kGatherRows * n_stride + (i - r * per_rank), step, w)) {
            atomicOr(err_flag, 0x100);
            return;
        }
        if (out) out[i] = __uint_as_float((unsigned)w);
    }
}

int launch_gather_wait(fnn_cuda_ctx *ctx, const unsigned long long *my_words, const unsigned *counters,
                       int world, int n_stride, float *out) {
    const int blocks = (int)div_ceil((size_t)world * kGatherRows * n_stride, 256 * 4);
    gather_wait_kernel<<<blocks < 1 ? 1 : blocks, 256, 0, ctx->stream>>>(my_words, counters, world, n_stride,
                                                                        out, ctx->err_flag);
    FNN_CUDA_CHECK(cudaGetLastError(), FNN_ERR_DISPATCH);
    ctx->launches++;
    return FNN_OK;
}

int launch_qmm_mma8(fnn_cuda_ctx *ctx, const QmmArgs &a) {
    switch (a.w->fmt) {
    case FNN_FMT_I8:
        return launch8_fmt<FNN_FMT_I8>(ctx, a);
    case FNN_FMT_I4:
        return launch8_fmt<FNN_FMT_I4>(ctx, a);
    case FNN_FMT_F4:
        return launch8_fmt<FNN_FMT_F4>(ctx, a);
    case FNN_FMT_I4CB:
        return launch8_fmt<FNN_FMT_I4CB>(ctx, a);
    }
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: the 8-bit fragment kernel does not cover format %d",
                     a.w->fmt);
}

}  // namespace fnn
