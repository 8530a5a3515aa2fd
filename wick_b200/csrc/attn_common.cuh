// Shared pieces of the exact single-query attention kernels (kernels_attn.cu, kernels_batch.cu).
#pragma once
#include "common.cuh"

namespace wick {

constexpr int ATTN_V_TILE = 32;  // cached rows staged per step of the weighted-V pass

// attn_values (cpu.rs:1463-1509): out[d] = sum over t, in ascending t, of fma(sc[t], V[t][d], acc): one serial fused chain
// per output dim, which is the reference's order and cannot be split.  What can be done in parallel is fetching the rows:
// ALL threads of the CTA copy ATTN_V_TILE rows of the head's V slice at a time into shared memory (16-byte asynchronous
// copies, two tiles in flight), and the first `hd` threads run the chains out of shared memory.
// vt: 2 * ATTN_V_TILE * hd floats of shared memory (16-byte aligned); v_head = v_cache + head offset; must be called by
// every thread of the CTA (it synchronises the CTA).
__device__ __forceinline__ void attn_values_staged(const float* __restrict__ sc, const float* __restrict__ v_head, int kv_dim, int hd, int seq,
                                                   float* __restrict__ vt, float* __restrict__ out_head) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int pieces = hd / 4;  // 16-byte pieces per row
    auto stage = [&](int tile) {
        const int t0 = tile * ATTN_V_TILE;
        const int rows = min(ATTN_V_TILE, seq - t0);
        float* dst = vt + (tile & 1) * ATTN_V_TILE * hd;
        for (int i = tid; i < rows * pieces; i += nthr) {
            const int r = i / pieces, c = i - r * pieces;
            const float* src = v_head + (size_t)(t0 + r) * kv_dim + c * 4;
            const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst + r * hd + c * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (seq + ATTN_V_TILE - 1) / ATTN_V_TILE;
    float acc = 0.0f;
    stage(0);
    for (int tile = 0; tile < n_tiles; tile++) {
        if (tile + 1 < n_tiles) {
            stage(tile + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // every thread's copies of this tile have landed
        if (tid < hd) {
            const int t0 = tile * ATTN_V_TILE;
            const int rows = min(ATTN_V_TILE, seq - t0);
            const float* v = vt + (tile & 1) * ATTN_V_TILE * hd + tid;
#pragma unroll 8
            for (int r = 0; r < rows; r++) acc = __fmaf_rn(sc[t0 + r], v[r * hd], acc);
        }
        __syncthreads();  // the buffer may be refilled by the copy of tile + 2
    }
    if (tid < hd) out_head[tid] = acc;
}

}  // namespace wick
