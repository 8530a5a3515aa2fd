// Attention kernels that reproduce the CPU path's operation order exactly.
#include "attn_common.cuh"
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
                                                                    int n_kv_heads, int hd, int max_seq) {
    extern __shared__ __align__(16) float sm[];
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

    if (hd <= NAIVE_THREADS && hd % 4 == 0) {
        float* vt = sc + ((max_seq + 3) & ~3);  // staging area behind the scores (16-byte aligned: hd is a multiple of 4)
        attn_values_staged(sc, v_cache + off, kv_dim, hd, seq, vt, out + (size_t)j * hs + h * hd);
        return;
    }
    for (int d = tid; d < hd; d += NAIVE_THREADS) {  // heads wider than the CTA: rows straight from global memory
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

// q row, scores of up to max_seq keys (padded to a multiple of 4), two staged V tiles
size_t naive_attention_smem_bytes(int head_dim, int max_seq) {
    return (size_t)(head_dim + ((max_seq + 3) & ~3) + 2 * ATTN_V_TILE * head_dim) * sizeof(float);
}

void launch_attention_naive(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out,
                            int n, int start_pos, const DecodeCtl* ctl, int n_heads, int n_kv_heads, int head_dim,
                            int max_seq) {
    dim3 grid(n_heads, n);
    size_t smem = naive_attention_smem_bytes(head_dim, max_seq);
    raise_naive_attention_smem(smem);  // no-op once granted; a failure surfaces as the launch error
    g_kernel_launches++;
    k_attention_naive<<<grid, NAIVE_THREADS, smem, st>>>(q, k_cache, v_cache, out, start_pos, ctl, n_heads, n_kv_heads,
                                                        head_dim, max_seq);
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
// 8 * BQ consecutive queries of one head (their rows sit in shared memory too); lane = (part g = lane / 8, chain /
// slot c = lane % 8):
//   * q.k: in passes of 8 queries x the 8 keys of the part, lane c runs chain c (dims c, c + 8, ...) of all 64 dots,
//     so a loaded query or key value feeds 8 multiply-adds (the first version, one lane per dot, was bound by
//     shared-memory wavefronts); the 8 chains of a dot are then added across lanes in the reference's order by three
//     halving exchanges, which leave lane c with the 8 scores of query c of the pass;
//   * softmax: tile max over the lane's 8 scores and the three lanes holding the same query's other parts; each
//     lane exponentiates its own 8;
//   * the probabilities travel by warp shuffle, in key order: every lane adds all 32 to the f64 tile sum in the
//     reference's order and applies them to its 4-float pieces of the output (acc chains in ascending key order); a
//     piece of a V row serves the lane's BQ queries.
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
#define WICK_FA_MIN_CTAS 4
#endif
#ifndef WICK_FA_BQ
#define WICK_FA_BQ 1
#endif
template <int HD, int BQ, int MAXW>  // MAXW: the most consumer warps a launch of this instance has (4 or 8)
__global__ void __launch_bounds__((MAXW + 1) * 32, MAXW == 4 ? (HD <= 64 ? WICK_FA_MIN_CTAS : 2) : 1) k_attention_flash(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                          const float* __restrict__ v_cache, float* __restrict__ out, int n, int start_pos,
                                                          int n_heads, int n_kv_heads, int qb, int wave_size, uint32_t* __restrict__ err) {
    constexpr int ROW = HD + 4;          // padded row, floats
    constexpr int DPL = HD / 4;          // output dims per lane
    extern __shared__ __align__(128) uint8_t fa_smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(fa_smem);           // [2]
    uint64_t* empty = full + 2;                                       // [2]
    volatile int* abort = reinterpret_cast<volatile int*>(empty + 2);
    float* Ks = reinterpret_cast<float*>(fa_smem + 64);              // [2][32][ROW]
    float* Vs = Ks + 2 * FLASH_TILE * ROW;                            // [2][32][ROW]
    float* Qs = Vs + 2 * FLASH_TILE * ROW;                            // [consumer warps][8 * BQ][ROW]

    const int group = n_heads / n_kv_heads;
    const int n_cw = group * (qb / (8 * BQ));  // consumer warps (<= MAXW)
    // Which (KV head, query block) this CTA takes.  All CTAs of a launch are resident together, 3 or 4 to an SM, and a
    // CTA's work grows with its query block (causal), so the launch ends when the SM with the heaviest set ends.  The
    // items are ranked by descending work and dealt to the block indices in waves of one block per SM, forwards in
    // even waves and backwards in odd ones: with the usual placement (blocks b, b + #SMs, b + 2 #SMs, ... on one SM)
    // every SM then holds about the same work.  Any placement is correct; only the balance depends on it.
    const int n_qblocks = (n + qb - 1) / qb;
    int kvh, qblock;
    {
        const int b = blockIdx.x, total = gridDim.x;
        const int wave = b / wave_size, pos = b % wave_size;
        const int lo = wave * wave_size, hi = min(lo + wave_size, total);
        const int r = (wave & 1) ? hi - 1 - pos : lo + pos;
        qblock = n_qblocks - 1 - r / n_kv_heads;
        kvh = r % n_kv_heads;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hs = n_heads * HD, kv_dim = n_kv_heads * HD;
    const int j_first = qblock * qb;
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

    // A consumer warp owns QPW = 8 * BQ consecutive queries of one head.  lane = (part g = lane / 8, chain c = lane % 8).
    //   q.k: part g owns keys t = 8 (u / 2) + 2 g + (u % 2), u = 0..7, of the tile (rows two apart for neighbouring
    //   parts: with the padded rows their 8-word reads fall into four different bank octets).  A pass handles 8 queries
    //   x the part's 8 keys; lane c runs chain c of all 64 dots (dims c, c + 8, ...: chains 0..3 are the reference's sum0
    //   lanes, 4..7 its sum1 lanes), so every loaded query or key value feeds 8 multiply-adds.  The chains of a dot are then
    //   added across the 8 lanes in the reference's order - (sum0[l] + sum1[l]) by an exchange with lane c ^ 4, then
    //   lanes c ^ 1, then c ^ 2 - each exchange halving what a lane keeps, so that lane c ends with the 8 scores of
    //   query c of the pass (a + b == b + a bit for bit, so both partners hold the same sums).
    //   softmax and weighted V: lane (g, c) is "slot c, part g": it owns the scores of queries c, c + 8, ... for its part's
    //   keys and, of those queries' outputs, the 4-float pieces g, g + 4, g + 8, ... of the head.
    constexpr int QPW = 8 * BQ;
    const int g = warp % group, run = warp / group;
    const int part = lane >> 3, c = lane & 7;
    const int h = kvh * group + g;
    const int j0 = j_first + run * QPW;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)HD));
    int my_max[BQ];
#pragma unroll
    for (int u = 0; u < BQ; u++) {
        const int j = j0 + u * 8 + c;
        my_max[u] = j < n ? start_pos + j + 1 : 0;
    }

    // the warp's query rows in shared memory (padded like the K rows); lane L copies 16-byte pieces L, L + 32, ...
    float* qw = Qs + warp * QPW * ROW;
    for (int i = lane; i < QPW * (HD / 4); i += 32) {
        const int r = i / (HD / 4), cc = i % (HD / 4);
        const int jr = j0 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (jr < n) v = __ldg(reinterpret_cast<const float4*>(q + (size_t)jr * hs + h * HD) + cc);
        reinterpret_cast<float4*>(qw + r * ROW)[cc] = v;
    }
    __syncwarp();
    float acc[BQ][DPL];
    float running_max[BQ];
    double running_sum[BQ];
#pragma unroll
    for (int u = 0; u < BQ; u++) {
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[u][d] = 0.0f;
        running_max[u] = __int_as_float(0xFF800000);
        running_sum[u] = 0.0;
    }
    // key index of the part's u-th key, and where the probability of key t of this lane's queries lives
    auto part_key = [&](int u) { return 8 * (u >> 1) + 2 * part + (u & 1); };

    for (int it = 0; it < n_tiles; it++) {
        const int buf = it & 1, kv0 = it * FLASH_TILE;
        if (!fa_wait(&full[buf], (it >> 1) & 1, abort, err, 0x200u)) return;
        int len[BQ], len_max = 0;  // keys of this tile each of the lane's queries attends (<= 0: none)
#pragma unroll
        for (int u = 0; u < BQ; u++) {
            len[u] = min(FLASH_TILE, my_max[u] - kv0);
            len_max = max(len_max, len[u]);
        }
        if (__reduce_max_sync(0xffffffffu, len_max) > 0) {
            const float* Kt = Ks + buf * FLASH_TILE * ROW;
            const float* Vt = Vs + buf * FLASH_TILE * ROW;
            float e[BQ][8];
            float tmax[BQ];
#pragma unroll
            for (int pass = 0; pass < BQ; pass++) {
                // chain c of the 8 x 8 dots of this pass
                float d8[8][8];
#pragma unroll
                for (int j = 0; j < 8; j++)
#pragma unroll
                    for (int u = 0; u < 8; u++) d8[j][u] = 0.0f;
                const float* qp = qw + (pass * 8) * ROW + c;
                const float* kp = Kt + (2 * part) * ROW + c;
#pragma unroll 2
                for (int i = 0; i < HD; i += 8) {
                    float qv[8], kv[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) qv[j] = qp[j * ROW + i];
#pragma unroll
                    for (int u = 0; u < 8; u++) kv[u] = kp[(8 * (u >> 1) + (u & 1)) * ROW + i];
#pragma unroll
                    for (int j = 0; j < 8; j++)
#pragma unroll
                        for (int u = 0; u < 8; u++) d8[j][u] = __fmaf_rn(qv[j], kv[u], d8[j][u]);
                }
                // sum0[l] + sum1[l]: exchange with lane c ^ 4, keeping the queries whose bit 2 equals this lane's
                float r1[4][8];
                const bool hi4 = (c & 4) != 0;
#pragma unroll
                for (int jj = 0; jj < 4; jj++)
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const float mine = hi4 ? d8[jj + 4][u] : d8[jj][u];
                        const float other = hi4 ? d8[jj][u] : d8[jj + 4][u];
                        r1[jj][u] = __fadd_rn(mine, __shfl_xor_sync(0xffffffffu, other, 4));
                    }
                // (v0 + v1), (v2 + v3): exchange with lane c ^ 1, keeping the queries whose bit 0 equals this lane's
                float r2[2][8];
                const bool hi1 = (c & 1) != 0;
#pragma unroll
                for (int m = 0; m < 2; m++)
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const float mine = hi1 ? r1[2 * m + 1][u] : r1[2 * m][u];
                        const float other = hi1 ? r1[2 * m][u] : r1[2 * m + 1][u];
                        r2[m][u] = __fadd_rn(mine, __shfl_xor_sync(0xffffffffu, other, 1));
                    }
                // (v0 + v1) + (v2 + v3): exchange with lane c ^ 2: query c of the pass remains
                const bool hi2 = (c & 2) != 0;
                float mx = __int_as_float(0xFF800000);
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float mine = hi2 ? r2[1][u] : r2[0][u];
                    const float other = hi2 ? r2[0][u] : r2[1][u];
                    const float sc = __fmul_rn(__fadd_rn(mine, __shfl_xor_sync(0xffffffffu, other, 2)), scale);
                    const bool in = part_key(u) < len[pass];
                    e[pass][u] = in ? sc : __int_as_float(0xFF800000);
                    if (in && sc > mx) mx = sc;
                }
                tmax[pass] = mx;
            }
            float new_max[BQ];
#pragma unroll
            for (int u = 0; u < BQ; u++) {
                tmax[u] = fmaxf(tmax[u], __shfl_xor_sync(0xffffffffu, tmax[u], 8));
                tmax[u] = fmaxf(tmax[u], __shfl_xor_sync(0xffffffffu, tmax[u], 16));
                new_max[u] = fmaxf(running_max[u], tmax[u]);
                const float rescale = running_max[u] > __int_as_float(0xFF800000) ? ggml_expf(__fsub_rn(running_max[u], new_max[u])) : 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) e[u][i] = (part_key(i) < len[u]) ? ggml_expf(__fsub_rn(e[u][i], new_max[u])) : 0.0f;
#pragma unroll
                for (int d = 0; d < DPL; d++) acc[u][d] = __fmul_rn(acc[u][d], rescale);
                if (len[u] > 0) running_sum[u] = running_sum[u] * (double)rescale;  // (+ the tile sum, below)
            }
            double tsum[BQ];
#pragma unroll
            for (int u = 0; u < BQ; u++) tsum[u] = 0.0;
#pragma unroll
            for (int t = 0; t < FLASH_TILE; t++) {
                // key t belongs to part (t % 8) / 2, as its key number 2 (t / 8) + t % 2
                float p[BQ];
#pragma unroll
                for (int u = 0; u < BQ; u++) p[u] = __shfl_sync(0xffffffffu, e[u][2 * (t >> 3) + (t & 1)], (((t & 7) >> 1) << 3) | c);
                if (t < len_max) {
                    float4 vv[DPL / 4];
                    const float4* vp = reinterpret_cast<const float4*>(Vt + t * ROW) + part;
#pragma unroll
                    for (int cc = 0; cc < DPL / 4; cc++) vv[cc] = vp[4 * cc];  // the four parts read 64 consecutive bytes
#pragma unroll
                    for (int u = 0; u < BQ; u++)
                        if (t < len[u]) {
                            tsum[u] += (double)p[u];
#pragma unroll
                            for (int cc = 0; cc < DPL / 4; cc++) {
                                acc[u][4 * cc + 0] = __fmaf_rn(p[u], vv[cc].x, acc[u][4 * cc + 0]);
                                acc[u][4 * cc + 1] = __fmaf_rn(p[u], vv[cc].y, acc[u][4 * cc + 1]);
                                acc[u][4 * cc + 2] = __fmaf_rn(p[u], vv[cc].z, acc[u][4 * cc + 2]);
                                acc[u][4 * cc + 3] = __fmaf_rn(p[u], vv[cc].w, acc[u][4 * cc + 3]);
                            }
                        }
                }
            }
#pragma unroll
            for (int u = 0; u < BQ; u++)
                if (len[u] > 0) {
                    running_sum[u] = running_sum[u] + tsum[u];
                    running_max[u] = new_max[u];
                }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fa_smem_u32(&empty[buf])) : "memory");
    }
#pragma unroll
    for (int u = 0; u < BQ; u++) {
        const int j = j0 + u * 8 + c;
        if (j < n) {
            const float inv = (float)(1.0 / running_sum[u]);
            float4* op = reinterpret_cast<float4*>(out + (size_t)j * hs + h * HD) + part;
#pragma unroll
            for (int cc = 0; cc < DPL / 4; cc++)
                op[4 * cc] = make_float4(__fmul_rn(acc[u][4 * cc + 0], inv), __fmul_rn(acc[u][4 * cc + 1], inv), __fmul_rn(acc[u][4 * cc + 2], inv),
                                     __fmul_rn(acc[u][4 * cc + 3], inv));
        }
    }
}

bool attention_flash_supported(int n_heads, int n_kv_heads, int head_dim) {
    if (head_dim != 32 && head_dim != 64 && head_dim != 128) return false;
    return n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= 8;
}

template <int HD>
static cudaError_t launch_flash_hd(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out, int n,
                                   int start_pos, int n_heads, int n_kv_heads, uint32_t* err) {
    constexpr int BQ = WICK_FA_BQ;
    const int group = n_heads / n_kv_heads;
    const int runs = group >= 4 ? 1 : 4 / group;  // runs of 8 * BQ queries per head and CTA: 4 consumer warps (8 when group is 5..8)
    const int qb = runs * 8 * BQ;                 // queries per CTA
    const int n_cw = group * runs;
    const size_t smem = 64 + (size_t)(4 * FLASH_TILE + n_cw * 8 * BQ) * (HD + 4) * sizeof(float);
    static size_t configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || configured[dev] < smem)) {
        e = cudaFuncSetAttribute(k_attention_flash<HD, BQ, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(k_attention_flash<HD, BQ, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    static bool carved[64] = {};
    if (dev >= 0 && dev < 64 && !carved[dev]) {  // several CTAs per SM only fit when the SM's L1/shared split favours shared memory
        cudaFuncSetAttribute(k_attention_flash<HD, BQ, 4>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(k_attention_flash<HD, BQ, 8>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carved[dev] = true;
    }
    static int sm_count[64] = {};
    if (dev >= 0 && dev < 64 && sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    const int wave = (dev >= 0 && dev < 64 && sm_count[dev] > 0) ? sm_count[dev] : 148;
    const unsigned grid = (unsigned)(n_kv_heads * ((n + qb - 1) / qb));
    const int threads = (n_cw + 1) * 32;
    g_kernel_launches++;
    if (n_cw <= 4) k_attention_flash<HD, BQ, 4><<<grid, threads, smem, st>>>(q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads, qb, wave, err);
    else k_attention_flash<HD, BQ, 8><<<grid, threads, smem, st>>>(q, k_cache, v_cache, out, n, start_pos, n_heads, n_kv_heads, qb, wave, err);
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
