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
// flash_attention_gqa_neon (cpu.rs:1696-1850): per (query head, query) 32-key tiles, tile max, rescale by
// ggml_expf(old_max - new_max), f64 tile sum in key order, acc *= rescale, fused acc += p * v in ascending key
// order, running_sum = running_sum * rescale + tile_sum in f64, one normalisation at the end.
//
// Mapping.  A CTA serves ONE KV head and a run of QB consecutive queries for every query head of its group, so
// a K / V tile is fetched once for all of them.  A producer warp streams the tiles with bulk asynchronous copies
// (cp.async.bulk, one per cache row, completion counted on an mbarrier) into a two-deep ring of shared memory;
// rows are padded to HD + 4 floats so that the accesses below are free of bank conflicts.  A consumer warp owns
// 8 queries of one head; lane = (query jq = lane / 4, part s = lane % 4):
//   * q.k: the lane holds its query row in registers and computes the dots of keys t = 4 i + s (i = 0..7) of the
//     tile with the reference's eight fused chains; the four parts of a query read four different rows (one
//     128-byte wavefront per 16-byte load, each value feeding 8 queries);
//   * softmax: tile max over the lane's 8 scores and its three partner lanes; each lane exponentiates its own 8;
//   * the probabilities travel by warp shuffle, in key order: every lane adds all 32 to the f64 tile sum in the
//     reference's order and applies them to its quarter of the output dims (acc chains in ascending key order).
// Keys at or beyond a query's causal limit are skipped by predicate (they may hold anything).
// Every wait is bounded: on expiry the CTA sets *err, stops waiting and returns.
constexpr int FLASH_TILE = 32;  // FLASH_TILE_KV, cpu.rs:1513
constexpr unsigned FLASH_SPIN_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t fa_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool fa_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(fa_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// false: the wait ran out (or another wait of this CTA did): *err is set and the caller must stop
__device__ __forceinline__ bool fa_wait(uint64_t* bar, uint32_t parity, volatile int* abort, uint32_t* err, uint32_t code) {
    unsigned spins = 0;
    while (!fa_try_wait(bar, parity)) {
        if (*abort) return false;
        if (++spins > FLASH_SPIN_LIMIT) {
            atomicOr(err, code);
            *abort = 1;
            return false;
        }
    }
    return !*abort;
}

#ifndef WICK_FA_MIN_CTAS
#define WICK_FA_MIN_CTAS 2
#endif
#ifndef WICK_FA_KB
#define WICK_FA_KB 2
#endif
template <int HD>
__global__ void __launch_bounds__(288, HD <= 64 ? WICK_FA_MIN_CTAS : 1) k_attention_flash(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                          const float* __restrict__ v_cache, float* __restrict__ out, int n, int start_pos,
                                                          int n_heads, int n_kv_heads, int qb, uint32_t* __restrict__ err) {
    constexpr int ROW = HD + 4;          // padded row, floats
    constexpr int DPL = HD / 4;          // output dims per lane
    constexpr int KB = WICK_FA_KB;       // keys whose dots share one pass over the query row
    extern __shared__ __align__(128) uint8_t fa_smem[];
    float* Ks = reinterpret_cast<float*>(fa_smem);                   // [2][32][ROW]
    float* Vs = Ks + 2 * FLASH_TILE * ROW;                            // [2][32][ROW]
    float* Qs = Vs + 2 * FLASH_TILE * ROW;                            // [consumer warps][8][ROW]
    uint64_t* full = reinterpret_cast<uint64_t*>(Qs + 8 * 8 * ROW);   // [2]
    uint64_t* empty = full + 2;                                       // [2]
    volatile int* abort = reinterpret_cast<volatile int*>(empty + 2);

    const int group = n_heads / n_kv_heads;
    const int n_cw = group * (qb / 8);  // consumer warps
    const int kvh = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hs = n_heads * HD, kv_dim = n_kv_heads * HD;
    const int j_first = blockIdx.y * qb;
    const int j_last = min(n, j_first + qb) - 1;
    const int cta_max = start_pos + j_last + 1;  // keys this CTA needs
    const int n_tiles = (cta_max + FLASH_TILE - 1) / FLASH_TILE;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_smem_u32(&full[i])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_smem_u32(&empty[i])), "r"(n_cw));
        }
        *abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == n_cw) {
        // producer: tile `it` goes to buffer it & 1 once its previous user has been released by every consumer warp
        for (int it = 0; it < n_tiles; it++) {
            const int buf = it & 1;
            if (it >= 2 && !fa_wait(&empty[buf], ((it >> 1) - 1) & 1, abort, err, 0x100u)) break;
            const int kv0 = it * FLASH_TILE;
            const int rows = min(FLASH_TILE, cta_max - kv0);
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fa_smem_u32(&full[buf])), "r"(rows * HD * 8) : "memory");
            __syncwarp();
            if (lane < rows) {
                const size_t src = (size_t)(kv0 + lane) * kv_dim + (size_t)kvh * HD;
                const uint32_t bar = fa_smem_u32(&full[buf]);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 fa_smem_u32(Ks + (buf * FLASH_TILE + lane) * ROW)),
                             "l"(k_cache + src), "r"(HD * 4), "r"(bar)
                             : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 fa_smem_u32(Vs + (buf * FLASH_TILE + lane) * ROW)),
                             "l"(v_cache + src), "r"(HD * 4), "r"(bar)
                             : "memory");
            }
        }
        // never leave with a copy in flight: the last two tiles' bytes must have landed (bounded)
        for (int it = max(0, n_tiles - 2); it < n_tiles; it++) {
            unsigned spins = 0;
            while (!fa_try_wait(&full[it & 1], (it >> 1) & 1) && ++spins < FLASH_SPIN_LIMIT) {
            }
        }
        return;
    }
    if (warp > n_cw) return;

    const int g = warp % group, oct = warp / group;
    const int jq = lane >> 2, s = lane & 3;
    const int j = j_first + oct * 8 + jq;
    const int h = kvh * group + g;
    const bool active = j < n;
    const int my_max = active ? start_pos + j + 1 : 0;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)HD));

    // the warp's 8 query rows in shared memory (padded like the K rows: the 8 queries of a 16-byte load hit 8
    // different bank groups); lane L copies 16-byte pieces L, L + 32, ...
    float* qw = Qs + warp * 8 * ROW;
    for (int i = lane; i < 8 * (HD / 4); i += 32) {
        const int r = i / (HD / 4), c = i % (HD / 4);
        const int jr = j_first + oct * 8 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (jr < n) v = __ldg(reinterpret_cast<const float4*>(q + (size_t)jr * hs + h * HD) + c);
        reinterpret_cast<float4*>(qw + r * ROW)[c] = v;
    }
    __syncwarp();
    const float* qrow = qw + jq * ROW;
    float acc[DPL];
#pragma unroll
    for (int d = 0; d < DPL; d++) acc[d] = 0.0f;
    float running_max = __int_as_float(0xFF800000);
    double running_sum = 0.0;
    const int src_base = lane & ~3;

    for (int it = 0; it < n_tiles; it++) {
        const int buf = it & 1, kv0 = it * FLASH_TILE;
        if (!fa_wait(&full[buf], (it >> 1) & 1, abort, err, 0x200u)) return;
        const int len = min(FLASH_TILE, my_max - kv0);  // keys of this tile the lane's query attends (<= 0: none)
        if (__reduce_max_sync(0xffffffffu, len) > 0) {
            const float* Kt = Ks + buf * FLASH_TILE * ROW;
            const float* Vt = Vs + buf * FLASH_TILE * ROW;
            float e[8];
            float tmax = __int_as_float(0xFF800000);
            // the lane's 8 keys in blocks of KB: a 16-byte piece of the query row is loaded once per block
#pragma unroll
            for (int i0 = 0; i0 < 8; i0 += KB) {
                if (4 * i0 + s < len) {  // (keys of a block ascend: if the first is out of range, all are)
                    float s0[KB][4], s1[KB][4];
#pragma unroll
                    for (int u = 0; u < KB; u++)
#pragma unroll
                        for (int l = 0; l < 4; l++) s0[u][l] = s1[u][l] = 0.0f;
#pragma unroll
                    for (int d = 0; d < HD; d += 8) {
                        const float4 qa = *reinterpret_cast<const float4*>(qrow + d);
                        const float4 qb4 = *reinterpret_cast<const float4*>(qrow + d + 4);
#pragma unroll
                        for (int u = 0; u < KB; u++) {
                            const float* kr = Kt + (4 * (i0 + u) + s) * ROW + d;
                            const float4 ka = *reinterpret_cast<const float4*>(kr);
                            const float4 kb = *reinterpret_cast<const float4*>(kr + 4);
                            s0[u][0] = __fmaf_rn(qa.x, ka.x, s0[u][0]);
                            s0[u][1] = __fmaf_rn(qa.y, ka.y, s0[u][1]);
                            s0[u][2] = __fmaf_rn(qa.z, ka.z, s0[u][2]);
                            s0[u][3] = __fmaf_rn(qa.w, ka.w, s0[u][3]);
                            s1[u][0] = __fmaf_rn(qb4.x, kb.x, s1[u][0]);
                            s1[u][1] = __fmaf_rn(qb4.y, kb.y, s1[u][1]);
                            s1[u][2] = __fmaf_rn(qb4.z, kb.z, s1[u][2]);
                            s1[u][3] = __fmaf_rn(qb4.w, kb.w, s1[u][3]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < KB; u++) {
                        const float v0 = __fadd_rn(s0[u][0], s1[u][0]), v1 = __fadd_rn(s0[u][1], s1[u][1]);
                        const float v2 = __fadd_rn(s0[u][2], s1[u][2]), v3 = __fadd_rn(s0[u][3], s1[u][3]);
                        const float sc = __fmul_rn(__fadd_rn(__fadd_rn(v0, v1), __fadd_rn(v2, v3)), scale);
                        const bool in = 4 * (i0 + u) + s < len;
                        e[i0 + u] = in ? sc : __int_as_float(0xFF800000);
                        if (in && sc > tmax) tmax = sc;
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < KB; u++) e[i0 + u] = __int_as_float(0xFF800000);
                }
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float new_max = fmaxf(running_max, tmax);
            const float rescale = running_max > __int_as_float(0xFF800000) ? ggml_expf(__fsub_rn(running_max, new_max)) : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = (4 * i + s < len) ? ggml_expf(__fsub_rn(e[i], new_max)) : 0.0f;
#pragma unroll
            for (int d = 0; d < DPL; d++) acc[d] = __fmul_rn(acc[d], rescale);
            double tsum = 0.0;
#pragma unroll
            for (int t = 0; t < FLASH_TILE; t++) {
                const float p = __shfl_sync(0xffffffffu, e[t >> 2], src_base | (t & 3));
                if (t < len) {
                    tsum += (double)p;
                    const float4* vp = reinterpret_cast<const float4*>(Vt + t * ROW + s * DPL);
#pragma unroll
                    for (int c = 0; c < DPL / 4; c++) {
                        const float4 vv = vp[c];
                        acc[4 * c + 0] = __fmaf_rn(p, vv.x, acc[4 * c + 0]);
                        acc[4 * c + 1] = __fmaf_rn(p, vv.y, acc[4 * c + 1]);
                        acc[4 * c + 2] = __fmaf_rn(p, vv.z, acc[4 * c + 2]);
                        acc[4 * c + 3] = __fmaf_rn(p, vv.w, acc[4 * c + 3]);
                    }
                }
            }
            if (len > 0) {
                running_sum = running_sum * (double)rescale + tsum;
                running_max = new_max;
            }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fa_smem_u32(&empty[buf])) : "memory");
    }
    if (active) {
        const float inv = (float)(1.0 / running_sum);
        float4* op = reinterpret_cast<float4*>(out + (size_t)j * hs + h * HD + s * DPL);
#pragma unroll
        for (int c = 0; c < DPL / 4; c++)
            op[c] = make_float4(__fmul_rn(acc[4 * c + 0], inv), __fmul_rn(acc[4 * c + 1], inv), __fmul_rn(acc[4 * c + 2], inv),
                                __fmul_rn(acc[4 * c + 3], inv));
    }
}

bool attention_flash_supported(int n_heads, int n_kv_heads, int head_dim) {
    if (head_dim != 32 && head_dim != 64 && head_dim != 128) return false;
    return n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= 8;
}

template <int HD>
static cudaError_t launch_flash_hd(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out, int n,
                                   int start_pos, int n_heads, int n_kv_heads, uint32_t* err) {
    const int group = n_heads / n_kv_heads;
    const int qb = group <= 4 ? 16 : 8;  // queries per CTA: 8 per consumer warp, at most 8 consumer warps
    const size_t smem = (size_t)(4 * FLASH_TILE + 64) * (HD + 4) * sizeof(float) + 4 * sizeof(uint64_t) + 16;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
        e = cudaFuncSetAttribute(k_attention_flash<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid(n_kv_heads, (n + qb - 1) / qb);
    const int threads = (group * (qb / 8) + 1) * 32;
    g_kernel_launches++;
    k_attention_flash<HD><<<grid, threads, smem, st>>>(q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads, qb, err);
    return cudaSuccess;
}

cudaError_t launch_attention_flash(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out,
                                   int n, int start_pos, int n_heads, int n_kv_heads, int head_dim, uint32_t* err) {
    if (!attention_flash_supported(n_heads, n_kv_heads, head_dim)) return cudaErrorInvalidValue;
    if (head_dim == 64) return launch_flash_hd<64>(st, q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads, err);
    if (head_dim == 32) return launch_flash_hd<32>(st, q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads, err);
    return launch_flash_hd<128>(st, q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads, err);
}

}  // namespace wick
