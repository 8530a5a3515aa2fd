// Persistent decode kernel: one launch runs whole decode steps (all layers, the tied
// vocabulary head and the argmax), one CTA per SM.
//
// Why it exists: at batch 1 every decode step streams all quantised weights once
// (wick's run_layers, wick/src/model/lfm2.rs:1020-1124, is a chain of ~70 dependent
// mat-vecs of 0.4-12 us each at HBM speed), so a kernel per mat-vec spends most of its
// time draining and refilling the memory pipe.  Here
//   * warp 0 of every CTA streams that CTA's share of the weights with bulk async copies
//     (cp.async.bulk + mbarrier) into a ring of shared-memory slots.  The weights do not
//     depend on activations, so this producer runs AHEAD across phase boundaries: while the
//     grid waits for a dependency, HBM keeps streaming into the ring;
//   * 16 consumer warps take ring slots; a warp owns 4-row groups and its lanes are the
//     eight f32 accumulation chains of each row (see kernels_gemv.cu), reading weights and the
//     quantised input from shared memory without bank conflicts (grouped layout, DevWeight);
//   * the small operators between mat-vecs (RMSNorm + Q8_0 quantise, short-conv gating,
//     SwiGLU, attention-output quantise) are recomputed by every CTA as the prologue of the
//     phase that consumes them, so a phase boundary is exactly one grid-wide barrier;
//   * residual adds and the argmax are epilogues of the mat-vec that produces their input.
// Arithmetic and its order are those of the per-kernel path (and of the CPU reference).
//
// Every wait (mbarrier or grid barrier) is bounded; on expiry the kernel sets ctl->error,
// drains its own copies and returns.
#include <cooperative_groups.h>

#include "decode_mega.cuh"

namespace wick {
namespace {

constexpr int NC = MEGA_CONSUMER_WARPS;
constexpr int NCT = NC * 32;
constexpr unsigned SPIN_LIMIT = 1u << 22;  // x ~0.25-1 us of back-off per iteration

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.  Both addresses and
// the size are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }

struct Smem {
    uint8_t* ring;
    float* xf;     // f32 staging of a phase input (also attention scores)
    int8_t* xq;    // quantised phase input
    float* xs;     // its block scales
    float* xs16;   // scales / 16 (Q4_0 lane sums are kept multiplied by 16)
    double* red;   // [NC]
    float* redf;   // [NC]
    float* head;   // [4 * 256]: rotated q, rotated k, raw q, raw k of the attention phase
    unsigned long long* best;  // [NC]
    uint64_t* full;
    uint64_t* empty;
    volatile int* abort;
};

__device__ __forceinline__ Smem carve(uint8_t* base, const MegaParams& P) {
    Smem s;
    size_t o = 0;
    s.ring = base;
    o += (size_t)P.n_slots * P.slot_bytes;
    int nf = P.kmax > P.max_seq ? P.kmax : P.max_seq;
    s.xf = (float*)(base + o);
    o += (size_t)nf * 4;
    s.xs = (float*)(base + o);
    o += (size_t)(P.kmax / QK) * 4;
    s.xs16 = (float*)(base + o);
    o += (size_t)(P.kmax / QK) * 4;
    o = (o + 15) & ~(size_t)15;
    s.xq = (int8_t*)(base + o);
    o += (size_t)P.kmax;
    o = (o + 15) & ~(size_t)15;
    s.red = (double*)(base + o);
    o += NC * 8;
    s.best = (unsigned long long*)(base + o);
    o += NC * 8;
    s.full = (uint64_t*)(base + o);
    o += (size_t)P.n_slots * 8;
    s.empty = (uint64_t*)(base + o);
    o += (size_t)P.n_slots * 8;
    s.redf = (float*)(base + o);
    o += NC * 4;
    o = (o + 15) & ~(size_t)15;
    s.head = (float*)(base + o);
    o += 4 * 256 * 4;
    s.abort = (volatile int*)(base + o);
    return s;
}

// Work split of one phase for one CTA: a contiguous run [lo, hi) of the phase's row groups
// (all matrices of the phase concatenated), cut into stages of at most `rg` groups (one ring
// slot each).  EVERY consumer warp waits for EVERY stage in order and releases it, so a warp
// can never wait two uses of a slot ahead (mbarrier parity would alias); inside a stage the
// groups are dealt to the warps round-robin by their running index in the phase.
struct Plan {
    int lo, hi, rg;
};
__device__ __forceinline__ Plan plan_phase(const MegaPhase& ph, int cta, int ncta, int slot_bytes) {
    int gt = 0, gb = 1;
    for (int i = 0; i < ph.n_mat; i++) {
        gt += ph.mat[i].w.groups();
        int b = (int)(ph.mat[i].w.q_group_bytes() + ph.mat[i].w.d_group_bytes());
        gb = b > gb ? b : gb;
    }
    Plan p;
    p.lo = (int)((long long)cta * gt / ncta);
    p.hi = (int)((long long)(cta + 1) * gt / ncta);
    int cap = slot_bytes / gb;
    cap = cap < 1 ? 1 : cap;
    p.rg = cap > 4 ? 4 : cap;
    return p;
}

// ── producer ───────────────────────────────────────────────────────────────
// Returns the number of stages issued (the caller drains the last n_slots of them on abort).
__device__ unsigned long long producer(const MegaParams& P, const Smem& S, int cta, int ncta) {
    unsigned long long cnt = 0;
    for (int t = 0; t < P.n_tokens; t++) {
        for (int pi = 0; pi < P.n_phases; pi++) {
            const MegaPhase& ph = P.phases[pi];
            if (ph.kind == MPH_ATTN) continue;
            Plan pl = plan_phase(ph, cta, ncta, P.slot_bytes);
            int off = 0;
            for (int mi = 0; mi < ph.n_mat; mi++) {
                const DevWeight& w = ph.mat[mi].w;
                const int gm = w.groups();
                int a = (pl.lo > off ? pl.lo : off) - off, b = (pl.hi < off + gm ? pl.hi : off + gm) - off;
                const uint32_t qgb = (uint32_t)w.q_group_bytes(), dgb = (uint32_t)w.d_group_bytes();
                for (int g0 = a; g0 < b; g0 += pl.rg, cnt++) {
                    int ng = pl.rg < b - g0 ? pl.rg : b - g0;
                    int slot = (int)(cnt % P.n_slots);
                    uint32_t u = (uint32_t)(cnt / P.n_slots);
                    unsigned spins = 0;
                    while (!mbar_try_wait(&S.empty[slot], (u & 1) ^ 1)) {
                        if (*S.abort) return cnt;
                        if (++spins > SPIN_LIMIT) {
                            atomicOr(&P.ctl->error, 2u);
                            *S.abort = 1;
                            return cnt;
                        }
                        __nanosleep(64);
                    }
                    uint8_t* dst = S.ring + (size_t)slot * P.slot_bytes;
                    mbar_expect_tx(&S.full[slot], ng * (qgb + dgb));
                    bulk_g2s(dst, w.q + (size_t)g0 * qgb, ng * qgb, &S.full[slot]);
                    bulk_g2s(dst + (size_t)ng * qgb, (const uint8_t*)w.d + (size_t)g0 * dgb, ng * dgb, &S.full[slot]);
                }
                off += gm;
            }
        }
    }
    return cnt;
}

// ── consumer helpers ───────────────────────────────────────────────────────
struct Ctx {
    const MegaParams& P;
    const Smem& S;
    int cta, ncta, ct, cw, lane;
};

// Waits are "fail open": once a wait has expired (here or in any CTA, seen through ctl->error)
// the abort flag is set and every later wait returns at once, so all threads still walk the same
// barrier sequence and the kernel ends by itself with the error recorded.
__device__ void grid_wait(Ctx& c, unsigned long long target) {
    if (c.ct == 0 && !*c.S.abort) {
        unsigned spins = 0;
        while (ld_acquire_u64(c.P.bar_counter) < target) {
            if (++spins > SPIN_LIMIT || ((spins & 1023) == 0 && __ldcg(&c.P.ctl->error) != 0)) {
                atomicOr(&c.P.ctl->error, 1u);
                *c.S.abort = 1;
                break;
            }
            if (spins > 64) __nanosleep(32);
        }
    }
    consumer_sync();
}

__device__ void grid_arrive(Ctx& c) {
    consumer_sync();
    if (c.ct == 0) {
        __threadfence();
        atomicAdd(c.P.bar_counter, 1ull);
    }
}

// Quantise xf[0..k) to Q8_0 in shared memory (simd.rs:255-323), one block per warp step.
__device__ void quantize_input(Ctx& c, int k) {
    const int nb = k / QK;
    for (int b = c.cw; b < nb; b += NC) {
        float sc;
        int8_t q = quantize_lane(c.S.xf[b * QK + c.lane], &sc);
        c.S.xq[b * QK + c.lane] = q;
        if (c.lane == 0) {
            c.S.xs[b] = sc;
            c.S.xs16[b] = __fmul_rn(sc, 0.0625f);
        }
    }
    consumer_sync();
}

__device__ __forceinline__ float embed_elem(const DevWeight& w, uint32_t tok, int e) {
    const int nb = w.k / QK, g = tok >> 2, r = tok & 3, b = e >> 5, i = e & 31;
    float d = __half2float(w.d[(size_t)g * nb * 4 + b * 4 + r]);
    const uint8_t* qg = w.q + (size_t)g * w.q_group_bytes();
    int v;
    if (w.dtype == DT_Q4_0) {
        uint8_t byte = qg[q4_word(b, r, 0) * 4 + (i & 15)];
        v = (int)(i < 16 ? (byte & 0x0F) : (byte >> 4)) - 8;
    } else {
        v = (int)((const int8_t*)qg)[q8_word(b, i >> 4, r, 0) * 4 + (i & 15)];
    }
    return __fmul_rn((float)v, d);
}

// b * x of channel ch from the in_proj output (lfm2.rs:691-695)
__device__ __forceinline__ float conv_bx(const float* proj, int hs, int ch) {
    return __fmul_rn(__ldcg(proj + ch), __ldcg(proj + 2 * hs + ch));
}

__device__ void prologue_norm(Ctx& c, const MegaPhase& ph, uint32_t token) {
    const MegaParams& P = c.P;
    const int k = ph.k;
    if (ph.conv_commit >= 0) {
        // advance the conv rolling buffer of the layer whose gating ran one phase ago; every CTA
        // finished reading the old buffer before the barrier that was just passed
        const MegaLayer& L = P.layers[ph.conv_commit];
        const int dc = P.conv_ks - 1, hs = P.hs;
        int c0 = (int)((long long)c.cta * hs / c.ncta), c1 = (int)((long long)(c.cta + 1) * hs / c.ncta);
        for (int ch = c0 + c.ct; ch < c1; ch += NCT) {
            for (int kk = 0; kk + 1 < dc; kk++) L.conv_state[(size_t)kk * hs + ch] = __ldcg(L.conv_state + (size_t)(kk + 1) * hs + ch);
            if (dc > 0) L.conv_state[(size_t)(dc - 1) * hs + ch] = conv_bx(P.proj, hs, ch);
        }
    }
    if (ph.embed) {
        int e0 = (int)((long long)c.cta * k / c.ncta), e1 = (int)((long long)(c.cta + 1) * k / c.ncta);
        for (int e = c.ct; e < k; e += NCT) {
            float v = embed_elem(P.embd, token, e);
            c.S.xf[e] = v;
            if (e >= e0 && e < e1) P.hidden[e] = v;
        }
    } else {
        for (int e = c.ct; e < k; e += NCT) c.S.xf[e] = __ldcg(P.hidden + e);
    }
    // cpu::rmsnorm (cpu.rs:577-594); f64 partial sums combined in a fixed order
    double s = 0.0;
    for (int e = c.ct; e < k; e += NCT) {
        double v = (double)c.S.xf[e];
        s += v * v;
    }
    s = warp_sum_f64(s);
    if (c.lane == 0) c.S.red[c.cw] = s;
    consumer_sync();
    double tot = 0.0;
    for (int i = 0; i < NC; i++) tot += c.S.red[i];
    const float inv = (float)(1.0 / sqrt(tot / (double)k + (double)P.eps));
    for (int e = c.ct; e < k; e += NCT) c.S.xf[e] = __fmul_rn(__fmul_rn(c.S.xf[e], inv), __ldg(ph.norm_w + e));
    consumer_sync();
    quantize_input(c, k);
}

__device__ void prologue_conv(Ctx& c, const MegaPhase& ph) {
    const MegaParams& P = c.P;
    const MegaLayer& L = P.layers[ph.layer];
    const int hs = P.hs, ks = P.conv_ks, dc = ks - 1;
    for (int ch = c.ct; ch < hs; ch += NCT) {
        float sum = 0.0f;
        for (int kk = 0; kk < dc; kk++)
            sum = __fadd_rn(sum, __fmul_rn(__ldcg(L.conv_state + (size_t)kk * hs + ch), __ldg(L.conv_w + ch * ks + kk)));
        float bx = conv_bx(P.proj, hs, ch);
        sum = __fadd_rn(sum, __fmul_rn(bx, __ldg(L.conv_w + ch * ks + dc)));
        c.S.xf[ch] = __fmul_rn(__ldcg(P.proj + hs + ch), sum);
    }
    consumer_sync();
    quantize_input(c, hs);
}

__device__ void prologue_silu(Ctx& c, const MegaPhase& ph) {
    const MegaParams& P = c.P;
    for (int e = c.ct; e < ph.k; e += NCT) c.S.xf[e] = silu_mul_elem(__ldcg(P.gate + e), __ldcg(P.up + e));
    consumer_sync();
    quantize_input(c, ph.k);
}

__device__ void prologue_quant(Ctx& c, const MegaPhase& ph) {
    for (int e = c.ct; e < ph.k; e += NCT) c.S.xf[e] = __ldcg(c.P.attn_out + e);
    consumer_sync();
    quantize_input(c, ph.k);
}

// NEON-order dot (cpu.rs:1430-1456) of a shared-memory q with a key row.
template <bool GLOBAL>
__device__ __forceinline__ float qk_dot_row(const float* q, const float* kv, int hd) {
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < hd; d += 8) {
        float4 ka, kb;
        if (GLOBAL) {
            ka = __ldcg(reinterpret_cast<const float4*>(kv + d));
            kb = __ldcg(reinterpret_cast<const float4*>(kv + d + 4));
        } else {
            ka = *reinterpret_cast<const float4*>(kv + d);
            kb = *reinterpret_cast<const float4*>(kv + d + 4);
        }
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

// Per-head RMSNorm (sum in element order, f64) + RoPE of `src` into dst (lfm2.rs:783-802);
// executed by one warp, dst in shared memory.
__device__ void head_norm_rope(const float* src_g, const float* w, float eps, const float* cosr, const float* sinr, int hd,
                               float* raw, float* dst, int lane) {
    for (int i = lane; i < hd; i += 32) raw[i] = __ldcg(src_g + i);
    __syncwarp();
    double ss = 0.0;
    for (int i = 0; i < hd; i++) {
        double x = (double)raw[i];
        ss += x * x;
    }
    const float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)eps));
    const int half = hd / 2;
    for (int i = lane; i < half; i += 32) {
        float x0 = __fmul_rn(__fmul_rn(raw[i], inv), __ldg(w + i));
        float x1 = __fmul_rn(__fmul_rn(raw[i + half], inv), __ldg(w + i + half));
        float cs = __ldg(cosr + i), sn = __ldg(sinr + i);
        dst[i] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        dst[i + half] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
    }
    __syncwarp();
}

// forward_attn_block between the QKV and output projections (lfm2.rs:783-1007) for the
// heads this CTA owns.
__device__ void phase_attention(Ctx& c, const MegaPhase& ph, int pos) {
    const MegaParams& P = c.P;
    const MegaLayer& L = P.layers[ph.layer];
    const int hd = P.head_dim, n_heads = P.n_heads, n_kv = L.n_kv, kv_dim = n_kv * hd, group = n_heads / n_kv;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const float* cosr = P.rope_cos + (size_t)pos * (hd / 2);
    const float* sinr = P.rope_sin + (size_t)pos * (hd / 2);
    float* sc = c.S.xf;
    float *qs = c.S.head, *ks = c.S.head + 256, *raw = c.S.head + 512;  // raw: [512,768) q, [768,1024) k
    const int seq = pos + 1;
    for (int h = 0; h < n_heads; h++) {
        if ((int)((long long)h * c.ncta / n_heads) != c.cta) continue;
        const int kvh = h / group, off = kvh * hd;
        consumer_sync();
        if (c.cw == 0) head_norm_rope(P.qbuf + h * hd, L.q_norm, P.eps, cosr, sinr, hd, raw, qs, c.lane);
        if (c.cw == 1) {
            head_norm_rope(P.kbuf + off, L.k_norm, P.eps, cosr, sinr, hd, raw + 256, ks, c.lane);
            if (h % group == 0) {  // one writer per KV head appends to the caches
                for (int i = c.lane; i < hd; i += 32) {
                    L.k_cache[(size_t)pos * kv_dim + off + i] = ks[i];
                    L.v_cache[(size_t)pos * kv_dim + off + i] = __ldcg(P.vbuf + off + i);
                }
            }
        }
        consumer_sync();
        // scores + max (attn_scores, cpu.rs:1404-1458)
        float mx = __int_as_float(0xFF800000);
        for (int t = c.ct; t < seq; t += NCT) {
            float dot = t < pos ? qk_dot_row<true>(qs, L.k_cache + (size_t)t * kv_dim + off, hd) : qk_dot_row<false>(qs, ks, hd);
            float s = __fmul_rn(dot, scale);
            sc[t] = s;
            mx = fmaxf(mx, s);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (c.lane == 0) c.S.redf[c.cw] = mx;
        consumer_sync();
        mx = c.S.redf[0];
        for (int i = 1; i < NC; i++) mx = fmaxf(mx, c.S.redf[i]);
        // softmax_inplace (cpu.rs:715-731)
        double sum = 0.0;
        for (int t = c.ct; t < seq; t += NCT) {
            float e = ggml_expf(__fsub_rn(sc[t], mx));
            sc[t] = e;
            sum += (double)e;
        }
        sum = warp_sum_f64(sum);
        if (c.lane == 0) c.S.red[c.cw] = sum;
        consumer_sync();
        double tot = 0.0;
        for (int i = 0; i < NC; i++) tot += c.S.red[i];
        const float inv = (float)(1.0 / tot);
        for (int t = c.ct; t < seq; t += NCT) sc[t] = __fmul_rn(sc[t], inv);
        consumer_sync();
        // attn_values (cpu.rs:1463-1509): one fused chain per output dim, ascending t
        if (c.ct < hd) {
            const float* vp = L.v_cache + off + c.ct;
            float acc = 0.0f;
#pragma unroll 8
            for (int t = 0; t < pos; t++) acc = __fmaf_rn(sc[t], __ldcg(vp + (size_t)t * kv_dim), acc);
            acc = __fmaf_rn(sc[pos], __ldcg(P.vbuf + off + c.ct), acc);
            P.attn_out[h * hd + c.ct] = acc;
        }
    }
}

__device__ __forceinline__ float reduce_row8(float a) {
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
    return a;
}

// One 4-row group from a ring slot: lane = p*16 + r*4 + l owns chain (p, l) of row r.
template <int DT>
__device__ __forceinline__ float group_chain(const uint32_t* __restrict__ qs, const __half* __restrict__ ds, int nb, int lane,
                                             const int* __restrict__ xq32, const float* __restrict__ xsc) {
    const int p = lane >> 4, r = (lane >> 2) & 3, l = lane & 3;
    float acc = 0.0f;
    if (DT == DT_Q4_0) {
        const uint32_t* qp = qs + (lane & 15);
#pragma unroll 4
        for (int b = p; b < nb; b += 2) {
            uint32_t w = qp[b * 16];
            float d = __fmul_rn(__half2float(ds[b * 4 + r]), xsc[b]);  // xsc = scale / 16
            int hi = (int)((w & 0xF0F0F0F0u) ^ 0x80808080u);
            int lo = (int)(((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u);
            int s16 = __dp4a(hi, xq32[b * 8 + 4 + l], __dp4a(lo, xq32[b * 8 + l], 0));  // 16 * lane sum
            acc = __fadd_rn(acc, __fmul_rn((float)s16, d));
        }
    } else {
        const uint32_t* qp = qs + lane;
#pragma unroll 4
        for (int b = p; b < nb; b += 2) {
            int w_lo = (int)qp[(b >> 1) * 64], w_hi = (int)qp[(b >> 1) * 64 + 32];
            float d = __fmul_rn(__half2float(ds[b * 4 + r]), xsc[b]);
            int s = __dp4a(w_hi, xq32[b * 8 + 4 + l], __dp4a(w_lo, xq32[b * 8 + l], 0));
            acc = __fadd_rn(acc, __fmul_rn((float)s, d));
        }
    }
    return acc;
}

__device__ void consumer(const MegaParams& P, const Smem& S, int cta, int ncta) {
    Ctx c{P, S, cta, ncta, (int)threadIdx.x - 32, ((int)threadIdx.x - 32) >> 5, (int)threadIdx.x & 31};
    unsigned long long cnt = 0;
    const uint32_t pos0 = __ldcg(&P.ctl->pos), step0 = __ldcg(&P.ctl->step);
    uint32_t token = __ldcg(&P.ctl->token);
    const int* xq32 = reinterpret_cast<const int*>(S.xq);
    for (int t = 0; t < P.n_tokens; t++) {
        const int pos = (int)pos0 + t;
        unsigned long long best = 0;
        for (int pi = 0; pi < P.n_phases; pi++) {
            const MegaPhase& ph = P.phases[pi];
            if (t > 0 || pi > 0) grid_wait(c, (P.bar_base + (unsigned long long)t * P.n_phases + pi) * (unsigned long long)ncta);
            const bool prof = P.prof && cta == 0 && c.ct == 0 && t == P.n_tokens - 1;
            if (prof) P.prof[pi * 4 + 0] = globaltimer_ns();
            if (pi == 0 && t > 0) {
                // argmax of the previous step is this step's input (Session::generate, session.rs:1251)
                token = (uint32_t)(__ldcg(&P.argmax_acc[(t - 1) & 1]) & 0xffffffffull);
                if (cta == 0 && c.ct == 0) P.ring[(step0 + t - 1) % (uint32_t)P.ring_len] = token;
            }
            if (pi == 1 && cta == 0 && c.ct == 0) P.argmax_acc[(t + 1) & 1] = 0;  // free for the next step
            switch (ph.kind) {
                case MPH_NORM: prologue_norm(c, ph, token); break;
                case MPH_CONV: prologue_conv(c, ph); break;
                case MPH_SILU: prologue_silu(c, ph); break;
                case MPH_QUANT: prologue_quant(c, ph); break;
                default: phase_attention(c, ph, pos); break;
            }
            if (prof) P.prof[pi * 4 + 1] = globaltimer_ns();
            if (ph.kind != MPH_ATTN) {
                Plan pl = plan_phase(ph, cta, ncta, P.slot_bytes);
                int off = 0, ls = 0;
                for (int mi = 0; mi < ph.n_mat; mi++) {
                    const MegaMat& M = ph.mat[mi];
                    const DevWeight& w = M.w;
                    const int gm = w.groups(), nb = w.k / QK;
                    int a = (pl.lo > off ? pl.lo : off) - off, b = (pl.hi < off + gm ? pl.hi : off + gm) - off;
                    const uint32_t qgb = (uint32_t)w.q_group_bytes();
                    for (int g0 = a; g0 < b; g0 += pl.rg, cnt++) {
                        int ng = pl.rg < b - g0 ? pl.rg : b - g0;
                        int slot = (int)(cnt % P.n_slots);
                        uint32_t u = (uint32_t)(cnt / P.n_slots);
                        unsigned spins = 0;
                        while (!*S.abort && !mbar_try_wait(&S.full[slot], u & 1)) {
                            if (++spins > SPIN_LIMIT) {
                                atomicOr(&P.ctl->error, 4u);
                                *S.abort = 1;
                                break;
                            }
                            if (spins > 32) __nanosleep(32);
                        }
                        const uint8_t* base = S.ring + (size_t)slot * P.slot_bytes;
                        const __half* dbase = reinterpret_cast<const __half*>(base + (size_t)ng * qgb);
                        for (int gi = 0; gi < ng; gi++, ls++) {
                            if (ls % NC != c.cw) continue;
                            const uint32_t* qs = reinterpret_cast<const uint32_t*>(base + (size_t)gi * qgb);
                            const __half* ds = dbase + (size_t)gi * nb * 4;
                            float acc = w.dtype == DT_Q4_0 ? group_chain<DT_Q4_0>(qs, ds, nb, c.lane, xq32, S.xs16)
                                                           : group_chain<DT_Q8_0>(qs, ds, nb, c.lane, xq32, S.xs);
                            acc = reduce_row8(acc);
                            const int row = (g0 + gi) * 4 + ((c.lane >> 2) & 3);
                            if ((c.lane & 19) == 0 && row < w.m) {
                                if (M.epi == MEP_ADD) {
                                    M.y[row] = __fadd_rn(__ldcg(M.y + row), acc);
                                } else if (M.epi == MEP_STORE) {
                                    M.y[row] = acc;
                                } else {
                                    if (!P.greedy) M.y[row] = acc;
                                    unsigned long long pk = argmax_pack(acc, (uint32_t)row);
                                    best = pk > best ? pk : best;
                                }
                            }
                        }
                        __syncwarp();
                        if (c.lane == 0) mbar_arrive(&S.empty[slot]);
                    }
                    off += gm;
                }
            }
            if (pi == P.n_phases - 1 && P.greedy) {
                // cpu_argmax (sampler.rs:8-19): CTA-level max, then one atomic per CTA
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    unsigned long long v = __shfl_xor_sync(0xffffffffu, best, o);
                    best = v > best ? v : best;
                }
                if (c.lane == 0) S.best[c.cw] = best;
                consumer_sync();
                if (c.ct == 0) {
                    unsigned long long b = 0;
                    for (int i = 0; i < NC; i++) b = S.best[i] > b ? S.best[i] : b;
                    atomicMax(&P.argmax_acc[t & 1], b);
                }
            }
            if (prof) P.prof[pi * 4 + 2] = globaltimer_ns();
            grid_arrive(c);
            if (prof) P.prof[pi * 4 + 3] = globaltimer_ns();
        }
    }
    // last step's result and the control block
    if (cta == 0) {
        const int n = P.n_tokens;
        grid_wait(c, (P.bar_base + (unsigned long long)n * P.n_phases) * (unsigned long long)ncta);
        if (c.ct == 0 && !*S.abort) {
            if (P.greedy) {
                uint32_t tok = (uint32_t)(__ldcg(&P.argmax_acc[(n - 1) & 1]) & 0xffffffffull);
                P.ring[(step0 + n - 1) % (uint32_t)P.ring_len] = tok;
                P.ctl->token = tok;
                P.argmax_acc[0] = 0;
                P.argmax_acc[1] = 0;
            }
            P.ctl->pos = pos0 + n;
            P.ctl->step = step0 + n;
        }
    }
}

__global__ void __launch_bounds__(MEGA_THREADS, 1) k_decode_mega(const MegaParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem S = carve(smem_raw, P);
    if (threadIdx.x == 0) {
        for (int i = 0; i < P.n_slots; i++) {
            mbar_init(&S.full[i], 1);
            mbar_init(&S.empty[i], NC);  // every consumer warp releases every stage
        }
        *S.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        if (threadIdx.x == 0) {
            unsigned long long issued = producer(P, S, blockIdx.x, gridDim.x);
            if (*S.abort) {
                // never leave with a copy of ours still in flight: wait (bounded) for the bytes
                // already requested for the stages that may not have been consumed
                unsigned long long first = issued > (unsigned long long)P.n_slots ? issued - P.n_slots : 0;
                for (unsigned long long i = first; i < issued; i++) {
                    unsigned spins = 0;
                    while (!mbar_try_wait(&S.full[i % P.n_slots], (uint32_t)(i / P.n_slots) & 1) && ++spins < SPIN_LIMIT) __nanosleep(64);
                }
            }
        }
    } else {
        consumer(P, S, blockIdx.x, gridDim.x);
    }
    __syncthreads();
}

}  // namespace

size_t mega_smem_bytes(const MegaParams& P) {
    int nf = P.kmax > P.max_seq ? P.kmax : P.max_seq;
    size_t o = (size_t)P.n_slots * P.slot_bytes + (size_t)nf * 4 + (size_t)(P.kmax / QK) * 8;
    o = (o + 15) & ~(size_t)15;
    o += P.kmax;
    o = (o + 15) & ~(size_t)15;
    o += NC * 16 + (size_t)P.n_slots * 16 + NC * 4;
    o = (o + 15) & ~(size_t)15;
    o += 4 * 256 * 4 + 16;
    return o;
}

int mega_max_ctas(const MegaParams& P) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t smem = mega_smem_bytes(P);
    if (cudaFuncSetAttribute(k_decode_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_mega, MEGA_THREADS, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return per_sm > 0 ? sms : 0;  // one CTA per SM
}

cudaError_t launch_decode_mega(cudaStream_t st, const MegaParams& P, int n_ctas) {
    size_t smem = mega_smem_bytes(P);
    // the attribute is per function, not per model: models of different size share the kernel
    cudaError_t e = cudaFuncSetAttribute(k_decode_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    void* args[] = {(void*)&P};
    g_kernel_launches++;
    return cudaLaunchCooperativeKernel((const void*)k_decode_mega, dim3(n_ctas), dim3(MEGA_THREADS), args, smem, st);
}

}  // namespace wick
