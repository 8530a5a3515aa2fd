// Kernels of the multi-sequence decode step (wick_cuda_decode_batch): row j of the batch is the next token of
// sequence j, with its own position, KV caches and rolling conv buffer.  wick keeps ONE sequence per model
// (wick/src/model/mod.rs:56-71); these kernels lift that limit for serving many independent sequences from one
// copy of the weights.  The mat-vecs of the step are the batched integer GEMMs of the prefill path (weights read
// once for all rows); everything sequence-specific is here, with the arithmetic of the single-sequence kernels
// (kernels_basic.cu, kernels_attn.cu) so that every row equals the same sequence decoded alone, bit for bit.
#include "attn_common.cuh"
#include "kernels.cuh"

namespace wick {

// ── gated short conv, one step per row (lfm2.rs:688-725) ───────────────────
// A warp owns 32 consecutive channels of one row = one Q8_0 block of the out_proj input.  The row's rolling
// buffer [d_conv][hs] is read, used and advanced by the thread that owns the channel.
__global__ void k_shortconv_rows(const float* __restrict__ proj, const float* __restrict__ conv_w, float* const* __restrict__ states,
                                 int n, int hs, int ks, float* __restrict__ q8s, int8_t* __restrict__ q8q) {
    const int dc = ks - 1;
    const size_t gw = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int bpr = hs / QK;
    if (gw >= (size_t)n * bpr) return;
    const int j = (int)(gw / bpr), ch = (int)(gw % bpr) * QK + lane;
    const float* pj = proj + (size_t)j * 3 * hs;
    float* state = states[j];
    float sum = 0.0f, prev[8];
#pragma unroll
    for (int k = 0; k < 8; k++)
        if (k < dc) {
            prev[k] = state[(size_t)k * hs + ch];
            sum = __fadd_rn(sum, __fmul_rn(prev[k], conv_w[ch * ks + k]));
        }
    const float bx = __fmul_rn(pj[ch], pj[2 * hs + ch]);
    sum = __fadd_rn(sum, __fmul_rn(bx, conv_w[ch * ks + dc]));
    const float o = __fmul_rn(pj[hs + ch], sum);
#pragma unroll
    for (int k = 0; k < 8; k++)
        if (k + 1 < dc) state[(size_t)k * hs + ch] = prev[k + 1];
    if (dc > 0) state[(size_t)(dc - 1) * hs + ch] = bx;
    float sc;
    const int8_t q = quantize_lane(o, &sc);
    q8q[(size_t)j * hs + ch] = q;
    if (lane == 0) q8s[gw] = sc;
}

void launch_shortconv_rows(cudaStream_t st, const float* proj, const float* conv_w, float* const* states, int n, int hs, int ks,
                           float* q8s, int8_t* q8q) {
    const size_t warps = (size_t)n * (hs / QK);
    if (!warps) return;
    g_kernel_launches++;
    k_shortconv_rows<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(proj, conv_w, states, n, hs, ks, q8s, q8q);
}

// ── per-head QK RMSNorm + RoPE + KV append, per-row position and caches (lfm2.rs:783-855) ──
// One warp per (row, head); same steps as k_qknorm_rope_kv.
__global__ void __launch_bounds__(32) k_qknorm_rope_kv_rows(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                           const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                                           const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                                                           float* const* __restrict__ k_caches, float* const* __restrict__ v_caches,
                                                           const uint32_t* __restrict__ positions, int n_heads, int n_kv_heads, int hd) {
    __shared__ float xs[256];
    const int j = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int hs = n_heads * hd, kv_dim = n_kv_heads * hd, half = hd / 2;
    const int pos = (int)positions[j];
    const bool is_q = head < n_heads;
    const int h = is_q ? head : head - n_heads;
    const float* src = is_q ? q + (size_t)j * hs + h * hd : k + (size_t)j * kv_dim + h * hd;
    const float* w = is_q ? q_norm : k_norm;
    for (int i = lane; i < hd; i += 32) xs[i] = src[i];
    __syncwarp();
    double sum_sq = 0.0;
    for (int i = 0; i < hd; i++) {
        double x = (double)xs[i];
        sum_sq += x * x;
    }
    const float inv = (float)(1.0 / sqrt(sum_sq / (double)hd + (double)eps));
    float* dst = is_q ? q + (size_t)j * hs + h * hd : k_caches[j] + (size_t)pos * kv_dim + h * hd;
    for (int i = lane; i < half; i += 32) {
        const float x0 = __fmul_rn(__fmul_rn(xs[i], inv), w[i]);
        const float x1 = __fmul_rn(__fmul_rn(xs[i + half], inv), w[i + half]);
        const float c = rope_cos[(size_t)pos * half + i], s = rope_sin[(size_t)pos * half + i];
        dst[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        dst[i + half] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    if (!is_q) {
        const float* vs = v + (size_t)j * kv_dim + h * hd;
        float* vd = v_caches[j] + (size_t)pos * kv_dim + h * hd;
        for (int i = lane; i < hd; i += 32) vd[i] = vs[i];
    }
}

void launch_qknorm_rope_kv_rows(cudaStream_t st, float* q, const float* k, const float* v, const float* q_norm, const float* k_norm,
                                float eps, const float* rope_cos, const float* rope_sin, float* const* k_caches, float* const* v_caches,
                                const uint32_t* positions, int n, int n_heads, int n_kv_heads, int head_dim) {
    dim3 grid(n, n_heads + n_kv_heads);
    g_kernel_launches++;
    k_qknorm_rope_kv_rows<<<grid, 32, 0, st>>>(q, k, v, q_norm, k_norm, eps, rope_cos, rope_sin, k_caches, v_caches, positions, n_heads,
                                               n_kv_heads, head_dim);
}

// ── single-query attention per (head, row), per-row cache and length ───────
// attn_scores / softmax_inplace / attn_values (cpu.rs:1404-1509, :715-731) exactly as k_attention_naive does them:
// NEON-order dots, f64 denominator in the same fixed thread order, one fused chain per output dim in ascending t.
constexpr int ROWS_ATTN_THREADS = 128;

__device__ __forceinline__ float qk_dot_rows(const float* __restrict__ q, const float* __restrict__ kv, int hd) {
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < hd; d += 8) {
        const float4 ka = *reinterpret_cast<const float4*>(kv + d);
        const float4 kb = *reinterpret_cast<const float4*>(kv + d + 4);
        s0[0] = __fmaf_rn(q[d + 0], ka.x, s0[0]);
        s0[1] = __fmaf_rn(q[d + 1], ka.y, s0[1]);
        s0[2] = __fmaf_rn(q[d + 2], ka.z, s0[2]);
        s0[3] = __fmaf_rn(q[d + 3], ka.w, s0[3]);
        s1[0] = __fmaf_rn(q[d + 4], kb.x, s1[0]);
        s1[1] = __fmaf_rn(q[d + 5], kb.y, s1[1]);
        s1[2] = __fmaf_rn(q[d + 6], kb.z, s1[2]);
        s1[3] = __fmaf_rn(q[d + 7], kb.w, s1[3]);
    }
    const float v0 = __fadd_rn(s0[0], s1[0]), v1 = __fadd_rn(s0[1], s1[1]);
    const float v2 = __fadd_rn(s0[2], s1[2]), v3 = __fadd_rn(s0[3], s1[3]);
    return __fadd_rn(__fadd_rn(v0, v1), __fadd_rn(v2, v3));
}

__global__ void __launch_bounds__(ROWS_ATTN_THREADS) k_attention_rows(const float* __restrict__ q, float* const* __restrict__ k_caches,
                                                                      float* const* __restrict__ v_caches, const uint32_t* __restrict__ positions,
                                                                      float* __restrict__ out, int n_heads, int n_kv_heads, int hd, int max_seq) {
    extern __shared__ __align__(16) float sm[];
    __shared__ double red[32];
    __shared__ float redf[32];
    float* qs = sm;       // hd floats
    float* sc = sm + hd;  // seq floats
    const int h = blockIdx.x, j = blockIdx.y;
    const int hs = n_heads * hd, kv_dim = n_kv_heads * hd;
    const int seq = (int)positions[j] + 1;
    const int off = (h / (n_heads / n_kv_heads)) * hd;
    const float* k_cache = k_caches[j];
    const float* v_cache = v_caches[j];
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = ROWS_ATTN_THREADS / 32;

    for (int i = tid; i < hd; i += ROWS_ATTN_THREADS) qs[i] = q[(size_t)j * hs + h * hd + i];
    __syncthreads();
    float mx = __int_as_float(0xFF800000);
    for (int t = tid; t < seq; t += ROWS_ATTN_THREADS) {
        const float s = __fmul_rn(qk_dot_rows(qs, k_cache + (size_t)t * kv_dim + off, hd), scale);
        sc[t] = s;
        mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) redf[warp] = mx;
    __syncthreads();
    mx = redf[0];
    for (int i = 1; i < nw; i++) mx = fmaxf(mx, redf[i]);
    double sum = 0.0;
    for (int t = tid; t < seq; t += ROWS_ATTN_THREADS) {
        const float e = ggml_expf(__fsub_rn(sc[t], mx));
        sc[t] = e;
        sum += (double)e;
    }
    sum = warp_sum_f64(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    double tot = 0.0;
    for (int i = 0; i < nw; i++) tot += red[i];
    const float inv = (float)(1.0 / tot);
    for (int t = tid; t < seq; t += ROWS_ATTN_THREADS) sc[t] = __fmul_rn(sc[t], inv);
    __syncthreads();
    if (hd <= ROWS_ATTN_THREADS && hd % 4 == 0) {
        float* vt = sc + ((max_seq + 3) & ~3);
        attn_values_staged(sc, v_cache + off, kv_dim, hd, seq, vt, out + (size_t)j * hs + h * hd);
        return;
    }
    for (int d = tid; d < hd; d += ROWS_ATTN_THREADS) {
        const float* vp = v_cache + off + d;
        float acc = 0.0f;
#pragma unroll 8
        for (int t = 0; t < seq; t++) acc = __fmaf_rn(sc[t], vp[(size_t)t * kv_dim], acc);
        out[(size_t)j * hs + h * hd + d] = acc;
    }
}

cudaError_t launch_attention_rows(cudaStream_t st, const float* q, float* const* k_caches, float* const* v_caches, const uint32_t* positions,
                                  float* out, int n, int n_heads, int n_kv_heads, int head_dim, int max_seq) {
    static size_t granted[64] = {};  // opt-in shared-memory limit of this kernel per device: only ever raised
    const size_t smem = naive_attention_smem_bytes(head_dim, max_seq);
    if (smem > 48 * 1024) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64 || granted[dev] < smem) {
            e = cudaFuncSetAttribute(k_attention_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) granted[dev] = smem;
        }
    }
    dim3 grid(n_heads, n);
    g_kernel_launches++;
    k_attention_rows<<<grid, ROWS_ATTN_THREADS, smem, st>>>(q, k_caches, v_caches, positions, out, n_heads, n_kv_heads, head_dim, max_seq);
    return cudaSuccess;
}

// ── split-K single-query attention (opt-in) ────────────────────────────────
// The exact kernel above keeps the reference's one serial chain per output dim over ALL keys, which at thousands of
// cached keys is the whole cost of a decode step.  This pair splits the keys of every (row, head) into runs of
// SPLIT_KEYS: `k_attention_split` computes for each run its score maximum m, the sum l of exp(score - m) and the
// weighted V sum, `k_attention_merge` combines the runs as  out = sum_i acc_i e^(m_i - M) / sum_i l_i e^(m_i - M)
// (the scheme of wick's Metal split-K kernels, shaders/attention_splitk.metal:30, :162).  Inside a run the arithmetic
// is the reference's (NEON-order dots, ggml_expf, fused chains in ascending key order); ACROSS runs the summation
// order differs from the CPU path, so results agree within rounding (about 1e-6 relative), not bit for bit: this
// path is never the default.
constexpr int SPLIT_KEYS = 256;
constexpr int SPLIT_THREADS = 128;

// grid (heads, splits, rows); partial layout [row][head][split][hd + 2] = acc[hd], m, l
__global__ void __launch_bounds__(SPLIT_THREADS) k_attention_split(const float* __restrict__ q, float* const* __restrict__ k_caches,
                                                                   float* const* __restrict__ v_caches, const float* __restrict__ k_single,
                                                                   const float* __restrict__ v_single, const uint32_t* __restrict__ positions,
                                                                   float* __restrict__ partial, int n_heads, int n_kv_heads, int hd, int max_splits) {
    __shared__ float qs[256];
    __shared__ float sc[SPLIT_KEYS];
    __shared__ float redf[SPLIT_THREADS / 32];
    __shared__ double red[SPLIT_THREADS / 32];
    const int h = blockIdx.x, sp = blockIdx.y, j = blockIdx.z;
    const int seq = (int)positions[j] + 1;
    const int t0 = sp * SPLIT_KEYS;
    if (t0 >= seq) return;
    const int cnt = min(SPLIT_KEYS, seq - t0);
    const int hs = n_heads * hd, kv_dim = n_kv_heads * hd;
    const int off = (h / (n_heads / n_kv_heads)) * hd;
    const float* k_cache = k_caches ? k_caches[j] : k_single;
    const float* v_cache = v_caches ? v_caches[j] : v_single;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = SPLIT_THREADS / 32;
    for (int i = tid; i < hd; i += SPLIT_THREADS) qs[i] = q[(size_t)j * hs + h * hd + i];
    __syncthreads();
    float mx = __int_as_float(0xFF800000);
    for (int t = tid; t < cnt; t += SPLIT_THREADS) {
        const float s = __fmul_rn(qk_dot_rows(qs, k_cache + (size_t)(t0 + t) * kv_dim + off, hd), scale);
        sc[t] = s;
        mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) redf[warp] = mx;
    __syncthreads();
    mx = redf[0];
    for (int i = 1; i < nw; i++) mx = fmaxf(mx, redf[i]);
    double sum = 0.0;
    for (int t = tid; t < cnt; t += SPLIT_THREADS) {
        const float e = ggml_expf(__fsub_rn(sc[t], mx));
        sc[t] = e;
        sum += (double)e;
    }
    sum = warp_sum_f64(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    float* out = partial + (((size_t)j * n_heads + h) * max_splits + sp) * (hd + 2);
    for (int d = tid; d < hd; d += SPLIT_THREADS) {
        const float* vp = v_cache + (size_t)t0 * kv_dim + off + d;
        float acc = 0.0f;
#pragma unroll 8
        for (int t = 0; t < cnt; t++) acc = __fmaf_rn(sc[t], vp[(size_t)t * kv_dim], acc);
        out[d] = acc;
    }
    if (tid == 0) {
        double tot = 0.0;
        for (int i = 0; i < nw; i++) tot += red[i];
        out[hd] = mx;
        out[hd + 1] = (float)tot;
    }
}

// grid (heads, rows), one thread per output dim
__global__ void k_attention_merge(const float* __restrict__ partial, const uint32_t* __restrict__ positions, float* __restrict__ out, int n_heads,
                                  int hd, int max_splits) {
    const int h = blockIdx.x, j = blockIdx.y;
    const int seq = (int)positions[j] + 1;
    const int ns = (seq + SPLIT_KEYS - 1) / SPLIT_KEYS;
    const float* p = partial + ((size_t)j * n_heads + h) * max_splits * (hd + 2);
    float M = __int_as_float(0xFF800000);
    for (int i = 0; i < ns; i++) M = fmaxf(M, p[(size_t)i * (hd + 2) + hd]);
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float L = 0.0f, acc = 0.0f;
        for (int i = 0; i < ns; i++) {
            const float w = ggml_expf(__fsub_rn(p[(size_t)i * (hd + 2) + hd], M));
            L = __fmaf_rn(p[(size_t)i * (hd + 2) + hd + 1], w, L);
            acc = __fmaf_rn(p[(size_t)i * (hd + 2) + d], w, acc);
        }
        out[(size_t)j * n_heads * hd + h * hd + d] = __fdiv_rn(acc, L);
    }
}

size_t attention_splitk_scratch_floats(int n, int n_heads, int head_dim, int max_seq) {
    const int max_splits = (max_seq + SPLIT_KEYS - 1) / SPLIT_KEYS;
    return (size_t)n * n_heads * max_splits * (head_dim + 2);
}

void launch_attention_splitk(cudaStream_t st, const float* q, float* const* k_caches, float* const* v_caches, const float* k_single,
                             const float* v_single, const uint32_t* positions, float* out, float* scratch, int n, int n_heads, int n_kv_heads,
                             int head_dim, int max_seq) {
    if (!n) return;
    const int max_splits = (max_seq + SPLIT_KEYS - 1) / SPLIT_KEYS;
    g_kernel_launches += 2;
    k_attention_split<<<dim3(n_heads, max_splits, n), SPLIT_THREADS, 0, st>>>(q, k_caches, v_caches, k_single, v_single, positions, scratch, n_heads,
                                                                               n_kv_heads, head_dim, max_splits);
    k_attention_merge<<<dim3(n_heads, n), 64, 0, st>>>(scratch, positions, out, n_heads, head_dim, max_splits);
}

// ── cpu_argmax (sampler.rs:8-19) of every row of logits [n][count]; one CTA per row ──
__global__ void __launch_bounds__(1024) k_argmax_rows(const float* __restrict__ x, int count, uint32_t* __restrict__ out) {
    __shared__ unsigned long long sh[32];
    const float* row = x + (size_t)blockIdx.x * count;
    unsigned long long best = 0;
    for (int i = threadIdx.x; i < count; i += 1024) {
        const unsigned long long p = argmax_pack(row[i], (uint32_t)i);
        best = p > best ? p : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 32; i++) best = sh[i] > best ? sh[i] : best;
        out[blockIdx.x] = (uint32_t)(best & 0xffffffffull);
    }
}

void launch_argmax_rows(cudaStream_t st, const float* logits, int n, int count, uint32_t* out) {
    if (!n) return;
    g_kernel_launches++;
    k_argmax_rows<<<n, 1024, 0, st>>>(logits, count, out);
}

// End of a batched step kept on the device: the chosen tokens become the next step's inputs, every position
// advances by one, and the tokens are recorded in row `step` of the output table [steps][n].
__global__ void k_rows_advance(uint32_t* __restrict__ tokens, const uint32_t* __restrict__ next, uint32_t* __restrict__ positions,
                               uint32_t* __restrict__ out_table, int n, int step) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const uint32_t t = next[j];
    tokens[j] = t;
    positions[j] += 1;
    out_table[(size_t)step * n + j] = t;
}

void launch_rows_advance(cudaStream_t st, uint32_t* tokens, const uint32_t* next, uint32_t* positions, uint32_t* out_table, int n, int step) {
    if (!n) return;
    g_kernel_launches++;
    k_rows_advance<<<(n + 127) / 128, 128, 0, st>>>(tokens, next, positions, out_table, n, step);
}

}  // namespace wick
