// Pieces the two fragment kernels (fp16 operands, 8-bit operands) share: the cp.async ring
// primitives, the named barrier of a warp group, the scan of the activation rows that every block
// runs under its first weight copies, and the launch sizing.
#pragma once

#include "common.cuh"

#include <algorithm>

namespace fnn {
namespace frag {

constexpr int kWarpsPerGroup = 8;   // warps that split K of one 16-row tile
constexpr int kChunkBlocks = 2;     // k-blocks per ring chunk

// 16-byte global -> shared copy that bypasses registers; src_bytes == 0 writes zeros.
__device__ __forceinline__ void cp_async16(void *dst, const void *src, int src_bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src, int src_bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Barrier over the eight warps of one group (named barrier 1 + group).
__device__ __forceinline__ void group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kWarpsPerGroup * 32) : "memory");
}

// Block-wide scan of the activation rows: s_mx[m] = max_k |a[m,k]|, s_sum[m] = sum_k a[m,k].
// All threads walk the rows R at a time (R independent loads in flight per thread); the
// warps' partials are folded by one thread per row in a fixed order, so the sums do not depend on
// scheduling.  s_part holds [NW][rows rounded up to R][2] floats.  Ends with a block barrier.
template <int NT, int R>
__device__ __forceinline__ void scan_rows(const float *__restrict__ act, int M, int K, bool vec_ok,
                                          float *s_part, float *s_mx, float *s_sum) {
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Mr = (M + R - 1) / R * R;
    for (int mb = 0; mb < M; mb += R) {
        float mx[R], sum[R];
#pragma unroll
        for (int m = 0; m < R; ++m) mx[m] = sum[m] = 0.0f;
        if (vec_ok) {
            for (int i = tid; i < K / 4; i += NT) {
#pragma unroll
                for (int m = 0; m < R; ++m) {
                    if (mb + m < M) {
                        const float4 v = __ldg(reinterpret_cast<const float4 *>(act + (size_t)(mb + m) * K) + i);
                        mx[m] = fmaxf(fmaxf(mx[m], fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
                        sum[m] += (v.x + v.y) + (v.z + v.w);
                    }
                }
            }
        } else {
            for (int k = tid; k < K; k += NT) {
#pragma unroll
                for (int m = 0; m < R; ++m) {
                    if (mb + m < M) {
                        const float a = __ldg(act + (size_t)(mb + m) * K + k);
                        mx[m] = fmaxf(mx[m], fabsf(a));
                        sum[m] += a;
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < R; ++m) {
            if (mb + m < M) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xFFFFFFFFu, mx[m], o));
                    sum[m] += __shfl_xor_sync(0xFFFFFFFFu, sum[m], o);
                }
                if (lane == 0) {
                    s_part[(warp * Mr + mb + m) * 2] = mx[m];
                    s_part[(warp * Mr + mb + m) * 2 + 1] = sum[m];
                }
            }
        }
    }
    __syncthreads();
    if (tid < M) {
        float bm = 0.0f, bs = 0.0f;
        for (int w = 0; w < NW; ++w) {
            bm = fmaxf(bm, s_part[(w * Mr + tid) * 2]);
            bs += s_part[(w * Mr + tid) * 2 + 1];
        }
        s_mx[tid] = bm;
        s_sum[tid] = bs;
    }
    __syncthreads();
}

// Launch sizing shared by both kernels.  One block per SM whenever the per-group accumulators of
// ceil(tiles / groups) tiles fit next to at least one ring chunk of activations; otherwise more
// blocks, run in waves.  `fixed`: bytes that do not depend on the tile count or on Kc; `per_tile`:
// bytes per tile slot of the block; `row_bytes(Kc)`: staged activation bytes for a K range of Kc.
struct FragSizing {
    int grid, tiles_per_group, Kc;
    size_t smem;
};
// `blocks_per_sm` > 1: several smaller blocks share an SM (each gets that fraction of the shared
// memory), so that blocks of the next kernel on the stream become resident, and prefetch, as soon as
// single blocks of this one retire.
template <typename RowBytes>
inline bool size_frag_launch(int sm_count, int ntiles, int groups, int Kpad, int kblk, size_t fixed,
                             size_t per_tile, RowBytes act_bytes, FragSizing *out, int blocks_per_sm = 1) {
    const size_t cap = (size_t)226 * 1024 / blocks_per_sm - (blocks_per_sm > 1 ? 1024 : 0);
    sm_count *= blocks_per_sm;
    const size_t min_act = act_bytes(kblk * kChunkBlocks);
    if (fixed + per_tile + min_act > cap) return false;
    int grid = sm_count;
    int tpg = (int)div_ceil((size_t)ntiles, (size_t)grid * groups);
    const int tpg_max = (int)((cap - fixed - min_act) / per_tile);
    if (tpg > tpg_max) {
        tpg = tpg_max;
        grid = (int)div_ceil((size_t)ntiles, (size_t)groups * tpg);
    }
    if (tpg < 1) tpg = 1;
    grid = (int)std::min<size_t>((size_t)grid, div_ceil((size_t)ntiles, (size_t)groups));
    const size_t act_budget = cap - fixed - (size_t)tpg * per_tile;
    int Kc = Kpad;
    while (act_bytes(Kc) > act_budget && Kc > kblk * kChunkBlocks) Kc = (Kc / 2 + kblk - 1) / kblk * kblk;
    out->grid = grid;
    out->tiles_per_group = tpg;
    out->Kc = Kc;
    out->smem = act_bytes(Kc) + fixed + (size_t)tpg * per_tile;
    return true;
}

}  // namespace frag
}  // namespace fnn
