// Attention kernels that reproduce the CPU path's operation order exactly.
#include "kernels.cuh"

namespace wick {

// q . k in the order of the NEON kernels (cpu.rs:1430-1456, :1778-1795): two 4-lane fused
// accumulators over alternating groups of four dims, added lane-wise, then (l0+l1)+(l2+l3).
template <int HD, class KP>
__device__ __forceinline__ float qk_dot(const float* __restrict__ q, KP kv) {
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < HD; d += 8) {
        float4 ka = *reinterpret_cast<const float4*>(kv + d);
        float4 kb = *reinterpret_cast<const float4*>(kv + d + 4);
        s0[0] = __fmaf_rn(q[d + 0], ka.x, s0[0]);
        s0[1] = __fmaf_rn(q[d + 1], ka.y, s0[1]);
        s0[2] = __fmaf_rn(q[d + 2], ka.z, s0[2]);
        s0[3] = __fmaf_rn(q[d + 3], ka.w, s0[3]);
        s1[0] = __fmaf_rn(q[d + 4], kb.x, s1[0]);
        s1[1] = __fmaf_rn(q[d + 5], kb.y, s1[1]);
        s1[2] = __fmaf_rn(q[d + 6], kb.z, s1[2]);
        s1[3] = __fmaf_rn(q[d + 7], kb.w, s1[3]);
    }
    float v0 = __fadd_rn(s0[0], s1[0]), v1 = __fadd_rn(s0[1], s1[1]);
    float v2 = __fadd_rn(s0[2], s1[2]), v3 = __fadd_rn(s0[3], s1[3]);
    return __fadd_rn(__fadd_rn(v0, v1), __fadd_rn(v2, v3));
}

// Generic head_dim version (multiple of 8) used by the naive kernel.
__device__ __forceinline__ float qk_dot_dyn(const float* __restrict__ q, const float* __restrict__ kv, int hd) {
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < hd; d += 8) {
        float4 ka = *reinterpret_cast<const float4*>(kv + d);
        float4 kb = *reinterpret_cast<const float4*>(kv + d + 4);
        s0[0] = __fmaf_rn(q[d + 0], ka.x, s0[0]);
        s0[1] = __fmaf_rn(q[d + 1], ka.y, s0[1]);
        s0[2] = __fmaf_rn(q[d + 2], ka.z, s0[2]);
        s0[3] = __fmaf_rn(q[d + 3], ka.w, s0[3]);
        s1[0] = __fmaf_rn(q[d + 4], kb.x, s1[0]);
        s1[1] = __fmaf_rn(q[d + 5], kb.y, s1[1]);
        s1[2] = __fmaf_rn(q[d + 6], kb.z, s1[2]);
        s1[3] = __fmaf_rn(q[d + 7], kb.w, s1[3]);
    }
    float v0 = __fadd_rn(s0[0], s1[0]), v1 = __fadd_rn(s0[1], s1[1]);
    float v2 = __fadd_rn(s0[2], s1[2]), v3 = __fadd_rn(s0[3], s1[3]);
    return __fadd_rn(__fadd_rn(v0, v1), __fadd_rn(v2, v3));
}

// ── per-token attention: scores -> softmax -> weighted V ───────────────────
// lfm2.rs:982-1006: attn_scores (cpu.rs:1404-1458), softmax_inplace (cpu.rs:715-731),
// attn_values (cpu.rs:1463-1509).  One CTA per (head, query).  The f64 softmax denominator
// is added per thread in stride order and combined in a fixed tree (the reference adds in
// element order; the two agree unless an f64 rounding occurs, see block_sum_sq_f64).  The
// weighted V sum is one fused chain per output dim in ascending t, as in the reference.
constexpr int NAIVE_THREADS = 128;

__global__ void __launch_bounds__(NAIVE_THREADS) k_attention_naive(const float* __restrict__ q,
                                                                    const float* __restrict__ k_cache,
                                                                    const float* __restrict__ v_cache,
                                                                    float* __restrict__ out, int start_pos,
                                                                    const DecodeCtl* __restrict__ ctl, int n_heads,
                                                                    int n_kv_heads, int hd) {
    extern __shared__ float sm[];
    __shared__ double red[32];
    __shared__ float redf[32];
    float* qs = sm;           // hd floats
    float* sc = sm + hd;      // seq floats
    const int h = blockIdx.x, j = blockIdx.y;
    const int hs = n_heads * hd, kv_dim = n_kv_heads * hd;
    const int seq = (start_pos >= 0 ? start_pos : (int)ctl->pos) + j + 1;
    const int off = (h / (n_heads / n_kv_heads)) * hd;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = NAIVE_THREADS / 32;

    for (int i = tid; i < hd; i += NAIVE_THREADS) qs[i] = q[(size_t)j * hs + h * hd + i];
    __syncthreads();

    float mx = __int_as_float(0xFF800000);
    for (int t = tid; t < seq; t += NAIVE_THREADS) {
        float s = __fmul_rn(qk_dot_dyn(qs, k_cache + (size_t)t * kv_dim + off, hd), scale);
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
    for (int t = tid; t < seq; t += NAIVE_THREADS) {
        float e = ggml_expf(__fsub_rn(sc[t], mx));
        sc[t] = e;
        sum += (double)e;
    }
    sum = warp_sum_f64(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    double tot = 0.0;
    for (int i = 0; i < nw; i++) tot += red[i];
    const float inv = (float)(1.0 / tot);
    for (int t = tid; t < seq; t += NAIVE_THREADS) sc[t] = __fmul_rn(sc[t], inv);
    __syncthreads();

    for (int d = tid; d < hd; d += NAIVE_THREADS) {
        const float* vp = v_cache + off + d;
        float acc = 0.0f;
#pragma unroll 8
        for (int t = 0; t < seq; t++) acc = __fmaf_rn(sc[t], vp[(size_t)t * kv_dim], acc);
        out[(size_t)j * hs + h * hd + d] = acc;
    }
}

// The opt-in limit is a property of the kernel on a device, shared by every model and operator call: it is only
// ever raised (a second model with a shorter context, or an operator call with a shorter sequence, must not
// lower the limit under a model that still launches with its own, larger size).
static cudaError_t raise_naive_attention_smem(size_t bytes) {
    constexpr int MAX_DEV = 64;
    static size_t granted[MAX_DEV] = {};  // written under the callers' own serialisation (one handle = one thread at a time);
                                          // a lost update only repeats an idempotent cudaFuncSetAttribute
    if (bytes <= 48 * 1024) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < MAX_DEV && granted[dev] >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(k_attention_naive, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && dev >= 0 && dev < MAX_DEV) granted[dev] = bytes;
    return e;
}

void configure_naive_attention_smem(size_t bytes) { raise_naive_attention_smem(bytes); }

void launch_attention_naive(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out,
                            int n, int start_pos, const DecodeCtl* ctl, int n_heads, int n_kv_heads, int head_dim,
                            int max_seq) {
    dim3 grid(n_heads, n);
    size_t smem = (size_t)(head_dim + max_seq) * sizeof(float);
    raise_naive_attention_smem(smem);  // no-op once granted; a failure surfaces as the launch error
    g_kernel_launches++;
    k_attention_naive<<<grid, NAIVE_THREADS, smem, st>>>(q, k_cache, v_cache, out, start_pos, ctl, n_heads, n_kv_heads,
                                                        head_dim);
}

// ── tiled online-softmax prefill attention ─────────────────────────────────
// flash_attention_gqa_neon (cpu.rs:1696-1850).  One thread runs the reference's loop for
// one (query head, query): 32-key tiles, tile max, rescale by ggml_expf(old_max - new_max),
// f64 tile sum in order, acc *= rescale, fused acc += p * v in ascending key order,
// running_sum = running_sum * rescale + tile_sum in f64, one normalisation at the end.
// A CTA holds the `group` query heads of ONE KV head for a run of queries, so every thread
// reads the same K / V tile from shared memory (broadcast).
constexpr int FLASH_THREADS = 128;
constexpr int FLASH_TILE = 32;  // FLASH_TILE_KV, cpu.rs:1513

template <int HD>
__global__ void __launch_bounds__(FLASH_THREADS) k_attention_flash(const float* __restrict__ q,
                                                                    const float* __restrict__ k_cache,
                                                                    const float* __restrict__ v_cache,
                                                                    float* __restrict__ out, int n, int start_pos,
                                                                    int n_heads, int n_kv_heads) {
    __shared__ __align__(16) float Ks[FLASH_TILE * HD];
    __shared__ __align__(16) float Vs[FLASH_TILE * HD];
    const int group = n_heads / n_kv_heads;
    const int qb = FLASH_THREADS / group;  // queries per CTA
    const int kvh = blockIdx.x;
    const int g = threadIdx.x % group, jq = threadIdx.x / group;
    const int j = blockIdx.y * qb + jq;
    const int h = kvh * group + g;
    const int hs = n_heads * HD, kv_dim = n_kv_heads * HD;
    const bool active = jq < qb && j < n;
    const int my_max = active ? start_pos + j + 1 : 0;
    int cta_last = min(n, (int)(blockIdx.y + 1) * qb) - 1;
    const int cta_max = start_pos + cta_last + 1;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)HD));

    float qr[HD], acc[HD];
#pragma unroll
    for (int d = 0; d < HD; d++) {
        qr[d] = active ? q[(size_t)j * hs + h * HD + d] : 0.0f;
        acc[d] = 0.0f;
    }
    float running_max = __int_as_float(0xFF800000);
    double running_sum = 0.0;

    for (int kv0 = 0; kv0 < cta_max; kv0 += FLASH_TILE) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < FLASH_TILE * HD / 4; idx += FLASH_THREADS) {
            int r = idx / (HD / 4), c4 = idx % (HD / 4);
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (kv0 + r < cta_max) {
                size_t o = (size_t)(kv0 + r) * kv_dim + kvh * HD + c4 * 4;
                kk = *reinterpret_cast<const float4*>(k_cache + o);
                vv = *reinterpret_cast<const float4*>(v_cache + o);
            }
            reinterpret_cast<float4*>(Ks)[idx] = kk;
            reinterpret_cast<float4*>(Vs)[idx] = vv;
        }
        __syncthreads();
        const int len = min(FLASH_TILE, my_max - kv0);
        if (len <= 0) continue;

        float ts[FLASH_TILE];
        float tmax = __int_as_float(0xFF800000);
#pragma unroll
        for (int ti = 0; ti < FLASH_TILE; ti++) {
            if (ti < len) {
                float s = __fmul_rn(qk_dot<HD>(qr, Ks + ti * HD), scale);
                ts[ti] = s;
                if (s > tmax) tmax = s;
            }
        }
        const float new_max = fmaxf(running_max, tmax);
        const float rescale = running_max > __int_as_float(0xFF800000) ? ggml_expf(__fsub_rn(running_max, new_max)) : 0.0f;
        double tsum = 0.0;
#pragma unroll
        for (int ti = 0; ti < FLASH_TILE; ti++) {
            if (ti < len) {
                float e = ggml_expf(__fsub_rn(ts[ti], new_max));
                ts[ti] = e;
                tsum += (double)e;
            }
        }
#pragma unroll
        for (int d = 0; d < HD; d++) acc[d] = __fmul_rn(acc[d], rescale);
#pragma unroll
        for (int ti = 0; ti < FLASH_TILE; ti++) {
            if (ti < len) {
                const float s = ts[ti];
#pragma unroll
                for (int d = 0; d < HD; d += 4) {
                    float4 vv = *reinterpret_cast<const float4*>(Vs + ti * HD + d);
                    acc[d + 0] = __fmaf_rn(s, vv.x, acc[d + 0]);
                    acc[d + 1] = __fmaf_rn(s, vv.y, acc[d + 1]);
                    acc[d + 2] = __fmaf_rn(s, vv.z, acc[d + 2]);
                    acc[d + 3] = __fmaf_rn(s, vv.w, acc[d + 3]);
                }
            }
        }
        running_sum = running_sum * (double)rescale + tsum;
        running_max = new_max;
    }
    if (active) {
        const float inv = (float)(1.0 / running_sum);
#pragma unroll
        for (int d = 0; d < HD; d++) out[(size_t)j * hs + h * HD + d] = __fmul_rn(acc[d], inv);
    }
}

void launch_attention_flash(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out,
                            int n, int start_pos, int n_heads, int n_kv_heads, int head_dim) {
    const int group = n_heads / n_kv_heads;
    const int qb = FLASH_THREADS / group;
    dim3 grid(n_kv_heads, (n + qb - 1) / qb);
    g_kernel_launches++;
    if (head_dim == 64)
        k_attention_flash<64><<<grid, FLASH_THREADS, 0, st>>>(q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads);
    else if (head_dim == 32)
        k_attention_flash<32><<<grid, FLASH_THREADS, 0, st>>>(q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads);
}

}  // namespace wick
