// Q6_K vocabulary matrix (token_embd of llama.cpp-made Q4_0 files): load-time re-layout, embedding rows
// (dequantize_q6_k_block, wick/src/quant.rs:380-413) and the logits mat-vec (gemv_q6k_q8_0_neon,
// wick/src/backend/simd.rs:552-672).
#include "kernels.cuh"

namespace wick {

namespace {

// One thread per super-block: raw 210-byte block (2-byte aligned) -> the four planes of DevQ6K.
__global__ void k_repack_q6k(const uint16_t* __restrict__ raw, uint16_t* ql, uint16_t* qh, uint16_t* sc, uint16_t* d, size_t n_blocks) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks) return;
    const uint16_t* b = raw + i * 105;
    for (int j = 0; j < 64; j++) ql[i * 64 + j] = b[j];
    for (int j = 0; j < 32; j++) qh[i * 32 + j] = b[64 + j];
    for (int j = 0; j < 8; j++) sc[i * 8 + j] = b[96 + j];
    d[i] = b[104];
}

__global__ void k_embed_q6k(DevQ6K w, const uint32_t* __restrict__ tokens, const DecodeCtl* __restrict__ ctl, float* __restrict__ out) {
    const int j = blockIdx.x;
    uint32_t tok = tokens ? tokens[j] : ctl->token;
    if (tok >= (uint32_t)w.m) tok = 0;  // host validates ids; never index outside the table
    for (int e = threadIdx.x; e < w.k; e += blockDim.x) out[(size_t)j * w.k + e] = q6k_elem(w, tok, e);
}

// Logits mat-vec.  The reference keeps ONE serial f32 sum per row, over 16-element sub-blocks in the order
// (super-block, pass, half, j = 0..3 at element offsets +0, +32, +64, +96); term = ((d * scale) * d_x) *
// float(int dot), every product and the add unfused.  A warp takes ROWS rows: lane u of a row pass owns unit
// u = (super-block, pass, half) and computes its four terms (three 16-byte loads of weights, four of the
// input); the terms go to shared memory and one lane per row adds them in order.
constexpr int Q6K_ROWS = 8;      // rows per warp
constexpr int Q6K_WARPS = 4;     // warps per CTA

__global__ void __launch_bounds__(32 * Q6K_WARPS)
k_gemv_q6k(DevQ6K w, const float* __restrict__ xs, const int8_t* __restrict__ xq, float* __restrict__ y) {
    extern __shared__ float q6k_terms[];  // [warp][ROWS][k/16]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = w.k, units = k / 64, nsub = k / 16;
    float* terms = q6k_terms + (size_t)warp * Q6K_ROWS * nsub;
    const int row0 = (blockIdx.x * Q6K_WARPS + warp) * Q6K_ROWS;
    for (int r = 0; r < Q6K_ROWS; r++) {
        const int row = row0 + r;
        if (row >= w.m) break;
        for (int u = lane; u < units; u += 32) {
            const int bi = u >> 2, pass = (u >> 1) & 1, half = u & 1;
            const uint8_t* qlp = w.ql + (size_t)row * (k / 2) + (size_t)bi * 128 + 64 * pass + 16 * half;
            const uint4 lo = *reinterpret_cast<const uint4*>(qlp);
            const uint4 hi = *reinterpret_cast<const uint4*>(qlp + 32);
            const uint4 hh = *reinterpret_cast<const uint4*>(w.qh + (size_t)row * (k / 4) + (size_t)bi * 64 + 32 * pass + 16 * half);
            const float d = __half2float(w.d[(size_t)row * (k / QK_K) + bi]);
            const int8_t* scp = w.sc + (size_t)row * (k / 16) + (size_t)bi * 16 + 8 * pass + half;
            const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w}, qw[4] = {hh.x, hh.y, hh.z, hh.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int e0 = bi * 256 + pass * 128 + half * 16 + 32 * j;  // first element of the sub-block
                const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xq + e0));
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                int dot = 0;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint32_t src = (j & 1) ? hw[c] : lw[c];
                    const uint32_t nib = j < 2 ? (src & 0x0F0F0F0Fu) : ((src >> 4) & 0x0F0F0F0Fu);
                    const uint32_t q = nib | (((qw[c] >> (2 * j)) & 0x03030303u) << 4);   // four values 0..63
                    dot = __dp4a((int)__vsub4(q, 0x20202020u), (int)xw[c], dot);           // (q - 32) as int8
                }
                const float dj = __fmul_rn(__fmul_rn(d, (float)scp[2 * j]), __ldg(xs + (e0 >> 5)));
                terms[(size_t)r * nsub + u * 4 + j] = __fmul_rn(dj, (float)dot);
            }
        }
    }
    __syncwarp();
    if (lane < Q6K_ROWS && row0 + lane < w.m) {
        const float4* t4 = reinterpret_cast<const float4*>(terms + (size_t)lane * nsub);
        float sum = 0.0f;
        for (int i = 0; i < nsub / 4; i++) {
            const float4 t = t4[i];
            sum = __fadd_rn(sum, t.x);
            sum = __fadd_rn(sum, t.y);
            sum = __fadd_rn(sum, t.z);
            sum = __fadd_rn(sum, t.w);
        }
        y[row0 + lane] = sum;
    }
}

}  // namespace

void launch_repack_q6k(cudaStream_t st, const uint8_t* raw, const DevQ6K& w) {
    const size_t n_blocks = (size_t)w.m * (w.k / QK_K);
    if (!n_blocks) return;
    g_kernel_launches++;
    k_repack_q6k<<<(unsigned)((n_blocks + 127) / 128), 128, 0, st>>>(
        reinterpret_cast<const uint16_t*>(raw), (uint16_t*)w.ql, (uint16_t*)w.qh, (uint16_t*)w.sc, (uint16_t*)w.d, n_blocks);
}

void launch_embed_q6k(cudaStream_t st, const DevQ6K& w, const uint32_t* tokens, const DecodeCtl* ctl, float* out, int n) {
    g_kernel_launches++;
    k_embed_q6k<<<n, 256, 0, st>>>(w, tokens, ctl, out);
}

size_t gemv_q6k_smem(int k) { return (size_t)Q6K_WARPS * Q6K_ROWS * (k / 16) * sizeof(float); }

void launch_gemv_q6k(cudaStream_t st, const DevQ6K& w, const float* xs, const int8_t* xq, float* y) {
    const int rows_per_cta = Q6K_WARPS * Q6K_ROWS;
    g_kernel_launches++;
    k_gemv_q6k<<<(w.m + rows_per_cta - 1) / rows_per_cta, 32 * Q6K_WARPS, gemv_q6k_smem(w.k), st>>>(w, xs, xq, y);
}

}  // namespace wick
