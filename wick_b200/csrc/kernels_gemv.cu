// Integer GEMV / GEMM with the reference's exact f32 accumulation tree.
//
// wick's NEON kernels (wick/src/backend/simd.rs:328-415, :440-524, :59-86) keep, per
// output element, two 4-lane f32 accumulators: even blocks feed sumv0, odd blocks sumv1;
// lane l of a block's vdotq_s32 result covers elements {4l..4l+3} and {16+4l..16+4l+3};
// each update is acc[l] = acc[l] + float(p[l]) * (f16(d_w) * d_x) with separately rounded
// multiply and add; the result is ((a0+a1)+(a2+a3)) of sumv0 plus the same of sumv1.
// That is eight independent serial chains per output, so ONE THREAD OWNS ONE CHAIN
// (row, parity, lane): it walks the blocks of its parity in order, and three shuffle-adds
// in the order lane^1, lane^2, parity^1 reproduce vaddvq + the final add.  Integer sums are
// exact; every f32 operation is an explicit *_rn intrinsic.
#include "kernels.cuh"

namespace wick {

// 16*p for lane-word `w` of a Q4_0 block: moving a nibble to the top of its byte and
// flipping bit 7 gives the signed byte 16*(nib-8); dp4a then yields 16*sum, shifted back.
__device__ __forceinline__ int lane_sum_q4(uint32_t w, int x_lo, int x_hi) {
    int hi = (int)((w & 0xF0F0F0F0u) ^ 0x80808080u);
    int lo = (int)(((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u);
    return __dp4a(hi, x_hi, __dp4a(lo, x_lo, 0)) >> 4;
}
__device__ __forceinline__ int lane_sum_q8(int w_lo, int w_hi, int x_lo, int x_hi) {
    return __dp4a(w_hi, x_hi, __dp4a(w_lo, x_lo, 0));
}

// Lane layout of a warp that owns one 4-row group: lane = p*16 + r*4 + l (parity, row in
// group, word) -- the word order of the grouped weight layout (DevWeight).
// vaddvq_f32(sumv0) + vaddvq_f32(sumv1) across the 8 chains of a row: lane^1, lane^2 give
// (l0+l1)+(l2+l3), lane^16 adds the other parity.  IEEE addition is commutative, so every
// thread of the row ends with the same value.
__device__ __forceinline__ float reduce_row8(float a) {
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
    return a;
}

// ── GEMV: 8 warps = 8 row groups per CTA; x staged in shared memory ─────────
constexpr int GEMV_GROUPS = 8;

// One chain (p, r, l) of group `g` over the blocks of its parity.
template <int DT>
__device__ __forceinline__ float gemv_chain(const DevWeight& w, int g, int lane, const int* __restrict__ xq32,
                                            const float* __restrict__ xs) {
    const int nb = w.k / QK;
    const int p = lane >> 4, r = (lane >> 2) & 3, l = lane & 3;
    const __half* dg = w.d + (size_t)g * nb * 4 + r;
    const uint32_t* qg = reinterpret_cast<const uint32_t*>(w.q + (size_t)g * w.q_group_bytes());
    float acc = 0.0f;
    if (DT == DT_Q4_0) {
        const uint32_t* qp = qg + (lane & 15);
#pragma unroll 4
        for (int b = p; b < nb; b += 2) {
            uint32_t ww = __ldg(qp + b * 16);
            float d = __fmul_rn(__half2float(__ldg(dg + b * 4)), xs[b]);
            int s = lane_sum_q4(ww, xq32[b * 8 + l], xq32[b * 8 + 4 + l]);
            acc = __fadd_rn(acc, __fmul_rn((float)s, d));
        }
    } else {
        const uint32_t* qp = qg + lane;  // p*16 + r*4 + l inside a block pair's half
#pragma unroll 4
        for (int b = p; b < nb; b += 2) {
            int w_lo = (int)__ldg(qp + (b >> 1) * 64), w_hi = (int)__ldg(qp + (b >> 1) * 64 + 32);
            float d = __fmul_rn(__half2float(__ldg(dg + b * 4)), xs[b]);
            int s = lane_sum_q8(w_lo, w_hi, xq32[b * 8 + l], xq32[b * 8 + 4 + l]);
            acc = __fadd_rn(acc, __fmul_rn((float)s, d));
        }
    }
    return acc;
}

__global__ void __launch_bounds__(256) k_gemv(GemvJob job, const float* __restrict__ xs_g,
                                              const int8_t* __restrict__ xq_g) {
    extern __shared__ int smem_i[];
    const int k = job.w[0].k, nb = k / QK;
    int* xq32 = smem_i;                                   // k/4 words
    float* xs = reinterpret_cast<float*>(smem_i + k / 4);  // nb floats
    const int* src = reinterpret_cast<const int*>(xq_g);
    for (int i = threadIdx.x; i < k / 4; i += blockDim.x) xq32[i] = src[i];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) xs[i] = xs_g[i];
    __syncthreads();

    const int lane = threadIdx.x & 31;
    int g = blockIdx.x * GEMV_GROUPS + (threadIdx.x >> 5);
    int mi = 0;
    while (mi < job.count && g >= (job.w[mi].m + 3) / 4) {
        g -= (job.w[mi].m + 3) / 4;
        mi++;
    }
    if (mi >= job.count) return;  // whole warp leaves together
    const DevWeight& w = job.w[mi];
    float acc = w.dtype == DT_Q4_0 ? gemv_chain<DT_Q4_0>(w, g, lane, xq32, xs) : gemv_chain<DT_Q8_0>(w, g, lane, xq32, xs);
    acc = reduce_row8(acc);
    const int row = g * 4 + ((lane >> 2) & 3);
    if ((lane & 19) == 0 && row < w.m) job.y[mi][row] = acc;
}

void launch_gemv(cudaStream_t st, const GemvJob& job, const float* xs, const int8_t* xq) {
    int groups = 0;
    for (int i = 0; i < job.count; i++) groups += (job.w[i].m + 3) / 4;
    if (!groups) return;
    const int k = job.w[0].k;
    size_t smem = (size_t)k + (size_t)(k / QK) * 4;
    g_kernel_launches++;
    k_gemv<<<(groups + GEMV_GROUPS - 1) / GEMV_GROUPS, 256, smem, st>>>(job, xs, xq);
}

// ── block sums (parity tap) ────────────────────────────────────────────────
__global__ void k_block_sums(DevWeight w, const int8_t* __restrict__ xq, int32_t* __restrict__ S) {
    const int nb = w.k / QK;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)w.m * nb) return;
    int row = (int)(idx / nb), b = (int)(idx % nb);
    const int g = row >> 2, r = row & 3;
    const int* x32 = reinterpret_cast<const int*>(xq) + b * 8;
    const uint32_t* qg = reinterpret_cast<const uint32_t*>(w.q + (size_t)g * w.q_group_bytes());
    int s = 0;
    if (w.dtype == DT_Q4_0) {
        for (int l = 0; l < 4; l++) s += lane_sum_q4(qg[q4_word(b, r, l)], x32[l], x32[4 + l]);
    } else {
        for (int l = 0; l < 4; l++) s += lane_sum_q8((int)qg[q8_word(b, 0, r, l)], (int)qg[q8_word(b, 1, r, l)], x32[l], x32[4 + l]);
    }
    S[idx] = s;
}
void launch_block_sums(cudaStream_t st, const DevWeight& w, const int8_t* xq, int32_t* S) {
    size_t total = (size_t)w.m * (w.k / QK);
    if (!total) return;
    g_kernel_launches++;
    k_block_sums<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(w, xq, S);
}

// ── GEMM over n quantised tokens ───────────────────────────────────────────
// Same chains, TJ tokens per CTA sharing each weight word.  256 threads = 8 warps = 8 row
// groups (32 rows) x 8 chains; every thread keeps TJ accumulators.  Activation words are staged transposed,
// xt[(b*8 + word)][token], so one 128-bit shared load feeds four tokens.  K is walked in
// chunks of KC blocks so the staging buffer stays small; chains continue across chunks.
constexpr int GEMM_ROWS = 32;
constexpr int TJ = 32;
constexpr int TJP = TJ + 4;  // padded token stride (words) of the transposed tiles
constexpr int KC = 32;       // blocks per K chunk

template <int DT>
__global__ void __launch_bounds__(256) k_gemm(DevWeight w, const float* __restrict__ bs, const int8_t* __restrict__ bq,
                                              int n, float* __restrict__ out) {
    __shared__ __align__(16) int xt[KC * 8 * TJP];
    __shared__ __align__(16) float st[KC * TJP];
    const int k = w.k, nb = k / QK, m = w.m;
    const int j0 = blockIdx.y * TJ;
    const int lane = threadIdx.x & 31;
    const int p = lane >> 4, r = (lane >> 2) & 3, l = lane & 3;
    int g = blockIdx.x * (GEMM_ROWS / 4) + (threadIdx.x >> 5);
    const int row = g * 4 + r;
    const bool rvalid = row < m;
    if (g >= w.groups()) g = 0;  // keep the warp in the barriers below; results are not stored
    const __half* dr = w.d + (size_t)g * nb * 4 + r;
    const uint32_t* qg = reinterpret_cast<const uint32_t*>(w.q + (size_t)g * w.q_group_bytes());

    float acc[TJ];
#pragma unroll
    for (int t = 0; t < TJ; t++) acc[t] = 0.0f;

    for (int b0 = 0; b0 < nb; b0 += KC) {
        const int nbc = min(KC, nb - b0);
        __syncthreads();
        // stage activations: token t, words [b0*8, (b0+nbc)*8)
        for (int idx = threadIdx.x; idx < nbc * 8 * TJ; idx += blockDim.x) {
            int t = idx / (nbc * 8), wi = idx % (nbc * 8);
            int j = j0 + t;
            int v = 0;
            if (j < n) v = reinterpret_cast<const int*>(bq + (size_t)j * k)[b0 * 8 + wi];
            xt[wi * TJP + t] = v;
        }
        for (int idx = threadIdx.x; idx < nbc * TJ; idx += blockDim.x) {
            int t = idx / nbc, bi = idx % nbc;
            int j = j0 + t;
            st[bi * TJP + t] = j < n ? bs[(size_t)j * nb + b0 + bi] : 0.0f;
        }
        __syncthreads();
        // chain parity is that of the global block index
        for (int bi = (p - (b0 & 1)) & 1; bi < nbc; bi += 2) {
            const int b = b0 + bi;
            const float dw = __half2float(__ldg(dr + b * 4));
            uint32_t ww = 0;
            int w_lo = 0, w_hi = 0;
            if (DT == DT_Q4_0) ww = __ldg(qg + q4_word(b, r, l));
            else { w_lo = (int)__ldg(qg + q8_word(b, 0, r, l)); w_hi = (int)__ldg(qg + q8_word(b, 1, r, l)); }
            const int4* xlo = reinterpret_cast<const int4*>(xt + (bi * 8 + l) * TJP);
            const int4* xhi = reinterpret_cast<const int4*>(xt + (bi * 8 + 4 + l) * TJP);
            const float4* sx = reinterpret_cast<const float4*>(st + bi * TJP);
#pragma unroll
            for (int t4 = 0; t4 < TJ / 4; t4++) {
                int4 a = xlo[t4], c = xhi[t4];
                float4 s = sx[t4];
                int p0, p1, p2, p3;
                if (DT == DT_Q4_0) {
                    p0 = lane_sum_q4(ww, a.x, c.x); p1 = lane_sum_q4(ww, a.y, c.y);
                    p2 = lane_sum_q4(ww, a.z, c.z); p3 = lane_sum_q4(ww, a.w, c.w);
                } else {
                    p0 = lane_sum_q8(w_lo, w_hi, a.x, c.x); p1 = lane_sum_q8(w_lo, w_hi, a.y, c.y);
                    p2 = lane_sum_q8(w_lo, w_hi, a.z, c.z); p3 = lane_sum_q8(w_lo, w_hi, a.w, c.w);
                }
                acc[t4 * 4 + 0] = __fadd_rn(acc[t4 * 4 + 0], __fmul_rn((float)p0, __fmul_rn(dw, s.x)));
                acc[t4 * 4 + 1] = __fadd_rn(acc[t4 * 4 + 1], __fmul_rn((float)p1, __fmul_rn(dw, s.y)));
                acc[t4 * 4 + 2] = __fadd_rn(acc[t4 * 4 + 2], __fmul_rn((float)p2, __fmul_rn(dw, s.z)));
                acc[t4 * 4 + 3] = __fadd_rn(acc[t4 * 4 + 3], __fmul_rn((float)p3, __fmul_rn(dw, s.w)));
            }
        }
    }
    const int sub = (lane & 3) | ((lane >> 2) & 4);  // 0..7 over the row's eight chains
#pragma unroll
    for (int t = 0; t < TJ; t++) {
        float v = reduce_row8(acc[t]);
        int j = j0 + t;
        if ((t & 7) == sub && rvalid && j < n) out[(size_t)j * m + row] = v;
    }
}

void launch_gemm(cudaStream_t st, const DevWeight& w, const float* bs, const int8_t* bq, int n, float* out) {
    if (!n || !w.m) return;
    dim3 grid((w.m + GEMM_ROWS - 1) / GEMM_ROWS, (n + TJ - 1) / TJ);
    if (w.dtype == DT_Q4_0) g_kernel_launches++, k_gemm<DT_Q4_0><<<grid, 256, 0, st>>>(w, bs, bq, n, out);
    else g_kernel_launches++, k_gemm<DT_Q8_0><<<grid, 256, 0, st>>>(w, bs, bq, n, out);
}

}  // namespace wick
