// Tensor-core (tcgen05 + TMEM + TMA) prefill GEMM: host-side handles and launch wrappers (gemm_tc.cu).
#pragma once
#include <cuda.h>

#include "kernels.cuh"

namespace wick {

// A second, GEMM-friendly copy of a quantised matrix: plain int8 values row-major (Q4_0 nibbles are
// widened to nib - 8) so that TMA can place 128-byte row segments straight into the swizzled operand
// layout, plus its scales as f32, block-major so that one k-block's 128 row scales are contiguous.
struct TcWeight {
    int8_t* q = nullptr;      // [m_pad][k]
    float* scales_t = nullptr;  // [k/32][m_pad]
    int m = 0, k = 0, m_pad = 0;
    CUtensorMap map;          // rows of this matrix, box 128 bytes x 128 rows, 128B swizzle
    size_t q_bytes() const { return (size_t)m_pad * k; }
    size_t s_bytes() const { return (size_t)(k / QK) * m_pad * sizeof(float); }
};

// Up to three matrices with the same k that share one set of quantised activations (gate + up, or
// Q + K + V): their tiles are scheduled as one grid so that narrow matrices do not leave SMs idle.
struct TcJob {
    CUtensorMap map_w[3];
    const float* scales_t[3];
    float* out[3];        // [n][m[i]] each
    int m[3], m_pad[3];
    int tile_start[4];    // first linear tile of each matrix; [count..3] = total
    int count;
};

// True when the shapes meet the kernel's requirements (k a multiple of 128).
bool tc_gemm_supported(int m, int k);
// Tokens per tile (64 or 128) the launcher chooses for n tokens and `row_tiles` 128-row tiles.
int tc_gemm_bn(int n, int row_tiles);

// Fills `out` (q / scales_t must already point at q_bytes() / s_bytes() of device memory, zeroed by
// this call) from the grouped layout of `w`, and encodes its tensor map.  Returns cudaSuccess or the
// failing CUDA error; a tensor-map failure is reported as cudaErrorInvalidValue.
cudaError_t tc_weight_fill(cudaStream_t st, const DevWeight& w, TcWeight* out);

// Tensor map over quantised activations xq [rows_cap][k] int8 with a box of bn rows.
cudaError_t tc_make_activation_map(const int8_t* xq, int rows_cap, int k, int bn, CUtensorMap* out);

// out[i][j][r] for matrix i < count (<= 3, equal k), token j < n, row r < m_i (token-major, like
// launch_gemm).  map_x[0] / map_x[1]: activation maps with 64 / 128 rows per box.  sums: optional
// [n][m][k/32] int32 block sums (count == 1 only).  err: device word that receives a non-zero code
// if a bounded wait expired.
cudaError_t launch_gemm_tc(cudaStream_t st, const TcWeight* const* w, float* const* out, int count, const CUtensorMap* map_x,
                           const float* x_scales, int n, int32_t* sums, uint32_t* err);

// The bit-exact variant (the arithmetic of gemm_q*_q8_0_neon, simd.rs:696-1019, in its order): the
// activation operand is the masked expansion xm [4 * n][k] of xq (row 4*j + l = token j with every
// byte outside NEON lane group l zeroed), so that one MMA yields the four lane partials of a block
// as four columns; the epilogue keeps the reference's eight unfused chains per output.
constexpr int TC_EXACT_TOKENS = 16;  // tokens per tile (64 MMA columns)
void launch_tc_mask_expand(cudaStream_t st, const int8_t* xq, int n, int k, int8_t* xm);
// map_xm: tc_make_activation_map(xm, 4 * rows_cap, k, 64, ..); map_xm_narrow (optional): the same with 32 rows per box,
// for the 8-token tiles small batches run with.
cudaError_t launch_gemm_tc_exact(cudaStream_t st, const TcWeight* const* w, float* const* out, int count, const CUtensorMap& map_xm,
                                 const float* x_scales, int n, uint32_t* err, const CUtensorMap* map_xm_narrow = nullptr);

}  // namespace wick
