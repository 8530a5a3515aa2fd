// Stochastic token sampling on the device: Sampler::sample (wick/src/sampler.rs:64-158) for logits that already live in
// GPU memory, so a sampled decode step reads back 4 bytes instead of the whole vocabulary row.  The uniform draw `r`
// comes from the caller: wick draws it from the `rand` crate's StdRng on the host, and the generator stays there.
//
// One CTA of 1024 threads, in the reference's order of operations:
//   temperature scaling (one rounded product per logit); top-k: the k-th largest scaled value by an 8-bit radix
//   select over order-preserving keys, everything below it dropped (ties with it stay, as `*l < threshold` drops only
//   smaller ones); the survivors are compacted in index order; top-p: survivors sorted by descending value (bitonic,
//   equal values by ascending index - wick's unstable sort leaves that order open), their exp / sum / cumulative sum
//   run serially in f32 exactly as written in apply_top_p, the tail beyond the cut dropped; softmax_inplace
//   (cpu.rs:715-731: max, ggml_expf, f64 sum in element order, one f32 reciprocal) and the f32 cumulative sum of
//   weighted_sample, both serial over the kept entries in index order (dropped entries are exact zeros and change
//   neither sum).
// The only step that is not bit-pinned is `f32::exp` inside top-p (the platform libm in wick; here exp in f64 rounded to
// f32); it can move the cut only when the cumulative sum lands within an ulp of top_p.
// Limit: top-p needs the survivors in shared memory, at most SAMPLE_MAX_SORT of them (top_k <= 4096, or top_p == 1);
// otherwise *status is set and nothing is written, and the caller samples on the host from a logits read-back.
#include "kernels.cuh"

namespace wick {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_MAX_SORT = 4096;

__device__ __forceinline__ uint32_t sample_key(float f) {  // ascending order of floats as unsigned integers
    const uint32_t b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) k_sample(const float* __restrict__ logits, int n, float temperature, int top_k, float top_p,
                                                           float r, float* __restrict__ val, int* __restrict__ idx, uint32_t* __restrict__ out,
                                                           uint32_t* __restrict__ status) {
    __shared__ unsigned int hist[256];
    __shared__ int warp_tot[32];
    __shared__ unsigned int sh_prefix, sh_remaining;
    __shared__ int sh_count, sh_cut;
    __shared__ float sh_max;
    __shared__ float s_val[SAMPLE_MAX_SORT];
    __shared__ int s_pos[SAMPLE_MAX_SORT];
    __shared__ unsigned char s_keep[SAMPLE_MAX_SORT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float inv_temp = __fdiv_rn(1.0f, temperature);
    const float NEG_INF = __int_as_float(0xFF800000);

    // ── top-k threshold: the k-th largest scaled value ──
    const bool use_k = top_k > 0 && top_k < n;
    uint32_t thr_key = 0;
    if (use_k) {
        if (tid == 0) {
            sh_prefix = 0;
            sh_remaining = (unsigned)top_k;
        }
        for (int pass = 3; pass >= 0; pass--) {
            for (int i = tid; i < 256; i += SAMPLE_THREADS) hist[i] = 0;
            __syncthreads();
            const uint32_t prefix = sh_prefix;
            const uint32_t hi_mask = pass == 3 ? 0u : 0xFFFFFFFFu << (8 * (pass + 1));
            for (int i = tid; i < n; i += SAMPLE_THREADS) {
                const uint32_t k = sample_key(__fmul_rn(logits[i], inv_temp));
                if ((k & hi_mask) == prefix) atomicAdd(&hist[(k >> (8 * pass)) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned remaining = sh_remaining;
                int b = 255;
                for (; b > 0; b--) {
                    if (hist[b] >= remaining) break;
                    remaining -= hist[b];
                }
                sh_prefix = prefix | ((uint32_t)b << (8 * pass));
                sh_remaining = remaining;
            }
            __syncthreads();
        }
        thr_key = sh_prefix;
    }

    // ── survivors, compacted in index order ──
    if (tid == 0) sh_count = 0;
    __syncthreads();
    for (int base = 0; base < n; base += SAMPLE_THREADS) {
        const int i = base + tid;
        float s = NEG_INF;
        if (i < n) s = __fmul_rn(logits[i], inv_temp);
        const bool alive = i < n && s > NEG_INF && s == s && (!use_k || sample_key(s) >= thr_key);
        const unsigned ballot = __ballot_sync(0xffffffffu, alive);
        if (lane == 0) warp_tot[warp] = __popc(ballot);
        __syncthreads();
        int before = sh_count;
        for (int w = 0; w < warp; w++) before += warp_tot[w];
        if (alive) {
            const int p = before + __popc(ballot & ((1u << lane) - 1u));
            val[p] = s;
            idx[p] = i;
        }
        __syncthreads();
        if (tid == 0) {
            int t = 0;
            for (int w = 0; w < 32; w++) t += warp_tot[w];
            sh_count += t;
        }
        __syncthreads();
    }
    const int S = sh_count;
    if (S == 0) {  // every logit is -inf (or NaN): softmax of that is NaN everywhere and no cumulative sum reaches r
        if (tid == 0) *out = (uint32_t)(n - 1);
        return;
    }

    // ── top-p over the survivors ──
    const bool use_p = top_p < 1.0f;
    if (use_p) {
        if (S > SAMPLE_MAX_SORT) {
            if (tid == 0) atomicOr(status, 1u);
            return;
        }
        int P = 1;
        while (P < S) P <<= 1;
        for (int j = tid; j < P; j += SAMPLE_THREADS) {
            s_val[j] = j < S ? val[j] : NEG_INF;
            s_pos[j] = j < S ? j : 0x7FFFFFFF;
            if (j < S) s_keep[j] = 1;
        }
        __syncthreads();
        // bitonic sort: descending value, equal values by ascending position
        for (int k = 2; k <= P; k <<= 1) {
            for (int jj = k >> 1; jj > 0; jj >>= 1) {
                for (int a = tid; a < P; a += SAMPLE_THREADS) {
                    const int b = a ^ jj;
                    if (b > a) {
                        const float va = s_val[a], vb = s_val[b];
                        const int pa = s_pos[a], pb = s_pos[b];
                        const bool a_first = va > vb || (va == vb && pa < pb);   // a belongs before b in the final order
                        const bool up = (a & k) == 0;                          // this pair is ordered "first .. last"
                        if (a_first != up) {
                            s_val[a] = vb;
                            s_val[b] = va;
                            s_pos[a] = pb;
                            s_pos[b] = pa;
                        }
                    }
                }
                __syncthreads();
            }
        }
        if (tid == 0) {
            const float max_val = s_val[0];
            float sum = 0.0f;
            for (int j = 0; j < S; j++) sum = __fadd_rn(sum, (float)exp((double)__fsub_rn(s_val[j], max_val)));
            int cut = S;
            float cumsum = 0.0f;
            for (int j = 0; j < S; j++) {
                const float p = __fdiv_rn((float)exp((double)__fsub_rn(s_val[j], max_val)), sum);
                cumsum = __fadd_rn(cumsum, p);
                if (cumsum >= top_p) {
                    cut = j + 1;
                    break;
                }
            }
            sh_cut = cut;
        }
        __syncthreads();
        for (int j = sh_cut + tid; j < S; j += SAMPLE_THREADS) s_keep[s_pos[j]] = 0;
        __syncthreads();
    }

    // ── softmax over what is left, then the weighted pick ──
    float mx = NEG_INF;
    for (int j = tid; j < S; j += SAMPLE_THREADS)
        if (!use_p || s_keep[j]) mx = fmaxf(mx, val[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __shared__ float wmax[32];
    if (lane == 0) wmax[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        float m2 = wmax[0];
        for (int w = 1; w < 32; w++) m2 = fmaxf(m2, wmax[w]);
        sh_max = m2;
    }
    __syncthreads();
    mx = sh_max;
    for (int j = tid; j < S; j += SAMPLE_THREADS) val[j] = (!use_p || s_keep[j]) ? ggml_expf(__fsub_rn(val[j], mx)) : 0.0f;
    __syncthreads();
    if (tid == 0) {
        double sum = 0.0;
        for (int j = 0; j < S; j++) sum += (double)val[j];
        const float inv = (float)(1.0 / sum);
        float cumsum = 0.0f;
        uint32_t pick = (uint32_t)(n - 1);
        if (r <= 0.0f) {
            pick = 0;  // the reference's loop stops at element 0 whatever its probability (0 + p >= r)
        } else {
            for (int j = 0; j < S; j++) {
                cumsum = __fadd_rn(cumsum, __fmul_rn(val[j], inv));
                if (cumsum >= r) {
                    pick = (uint32_t)idx[j];
                    break;
                }
            }
        }
        *out = pick;
    }
}

void launch_sample(cudaStream_t st, const float* logits, int n, float temperature, int top_k, float top_p, float r, float* val, int* idx,
                   uint32_t* out, uint32_t* status) {
    g_kernel_launches++;
    k_sample<<<1, SAMPLE_THREADS, 0, st>>>(logits, n, temperature, top_k, top_p, r, val, idx, out, status);
}

}  // namespace wick
