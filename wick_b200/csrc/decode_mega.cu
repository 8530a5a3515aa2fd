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
//   * 15 consumer warps take ring slots; a warp owns 4-row groups and its lanes are the
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
constexpr int TEAM_WARPS = MEGA_TEAM_WARPS;  // consumer warps work on ring slots in teams
constexpr int NTEAMS = MEGA_TEAMS;
constexpr int TEAM_THREADS = TEAM_WARPS * 32;
constexpr unsigned SPIN_LIMIT = 1u << 22;  // x ~0.25-2 us per iteration
constexpr unsigned WAIT_NS = 2000;         // hardware suspend limit of one mbarrier test

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
// The same test with a time limit: the thread is suspended in hardware until the phase completes or `ns` have
// passed, so a waiting warp issues almost nothing and wakes as soon as the barrier flips.
__device__ __forceinline__ bool mbar_try_wait_for(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.  Both addresses and
// the size are multiples of 16.
// The weights are read once per step and are far larger than L2: they are fetched with an
// evict-first policy so that they do not push the activations, KV rows and norm weights out.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }

// floats of the attention staging area: normalised scores of up to max_seq keys plus at least
// 64 gathered V rows of 16 columns
// (xf_extra: whatever shared memory is left once the ring is sized; at long contexts the V rows are gathered in
// chunks of (staging floats) / 16 rows, one memory round trip per chunk, so a larger staging area is fewer trips)
__host__ __device__ __forceinline__ int xf_floats(const MegaParams& P) { return P.max_seq + 4 + 64 * 16 + P.xf_extra; }

// Work split of one phase for one CTA (see plan_phase); computed once per launch into shared memory: it depends on
// the phase and the CTA only, and working it out again in every phase of every token (two integer divisions per matrix,
// a chain of dependent descriptor loads) cost each of the ~65 mat-vec phases of a token 0.2-0.3 us (2046 -> 2114 tok/s).
struct Plan {
    int lo, hi, rg, pad;
};

struct Smem {
    Plan* plan;    // [n_phases]
    uint8_t* ring;
    float* xf;     // attention phase: normalised scores, then gathered V rows
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
    MegaPhase* ph;      // the phase list, copied from global memory when the kernel starts
    MegaLayer* layers;
};

__device__ __forceinline__ Smem carve(uint8_t* base, const MegaParams& P) {
    Smem s;
    size_t o = 0;
    s.ring = base;
    o += (size_t)P.n_slots * P.slot_bytes;
    int nf = xf_floats(P);
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
    o += 16;
    s.ph = (MegaPhase*)(base + o);
    o += (size_t)P.n_phases * sizeof(MegaPhase);
    s.layers = (MegaLayer*)(base + o);
    o += (size_t)P.n_layers * sizeof(MegaLayer);
    o = (o + 15) & ~(size_t)15;
    s.plan = (Plan*)(base + o);
    return s;
}

// floor(i * n / d) in 32-bit arithmetic (64-bit integer division is emulated and costs hundreds of
// cycles); every product here stays far below 2^32 (n < 2^21 elements or groups, i <= #SMs).
__device__ __forceinline__ int share(int i, int n, int d) { return (int)((unsigned)i * (unsigned)n / (unsigned)d); }

// Work split of one phase for one CTA: a contiguous run [lo, hi) of the phase's row groups
// (all matrices of the phase concatenated), cut into stages of at most `rg` groups (one ring
// slot each).  Stages are dealt to the consumer teams round-robin through their ring slot.
__device__ __forceinline__ Plan plan_phase(const MegaPhase& ph, int cta, int ncta, int slot_bytes) {
    int gt = 0, gb = 1;
    for (int i = 0; i < (ph.pair ? 1 : ph.n_mat); i++) {  // a paired phase is split by the rows of ONE of its matrices
        gt += ph.mat[i].w.groups();
        int b = (int)(ph.mat[i].w.q_group_bytes() + ph.mat[i].w.d_group_bytes());
        gb = b > gb ? b : gb;
    }
    Plan p;
    p.lo = share(cta, gt, ncta);
    p.hi = share(cta + 1, gt, ncta);
    int cap = slot_bytes / gb;
    cap = cap < 1 ? 1 : (cap > 4 ? 4 : cap);
    int rg = (p.hi - p.lo + NTEAMS - 1) / NTEAMS;  // spread a small phase over all teams
    rg = rg < 1 ? 1 : rg;
    p.rg = rg > cap ? cap : rg;
    p.pad = 0;
    return p;
}

// ── producer ───────────────────────────────────────────────────────────────
// Returns the number of stages issued (the caller drains the last n_slots of them on abort).
__device__ unsigned long long producer(const MegaParams& P, const Smem& S, int cta, int ncta) {
    unsigned long long cnt = 0;
    const uint64_t pol = l2_evict_first_policy();
    int slot = 0;      // cnt % n_slots and the parity of cnt / n_slots, kept incrementally
    uint32_t par = 0;  // (a 64-bit division per stage would cost more than issuing the copy)
    for (int t = 0; t < P.n_tokens; t++) {
        for (int pi = 0; pi < P.n_phases; pi++) {
            const MegaPhase& ph = S.ph[pi];
            if (ph.kind == MPH_ATTN || ph.kind == MPH_SCORES) continue;
            const Plan pl = S.plan[pi];
            // stage list: per matrix its chunks in order; a paired phase alternates the two matrices chunk by chunk
            const int n_seq = ph.pair ? 1 : ph.n_mat, n_alt = ph.pair ? 2 : 1;
            int off = 0;
            for (int mi = 0; mi < n_seq; mi++) {
                const int gm = ph.mat[mi].w.groups();
                int a = (pl.lo > off ? pl.lo : off) - off, b = (pl.hi < off + gm ? pl.hi : off + gm) - off;
                for (int g0 = a; g0 < b; g0 += pl.rg) {
                    for (int alt = 0; alt < n_alt; alt++, cnt++, slot = slot + 1 == P.n_slots ? 0 : slot + 1, par ^= (slot == 0)) {
                        const DevWeight& w = ph.mat[mi + alt].w;
                        const uint32_t qgb = (uint32_t)w.q_group_bytes(), dgb = (uint32_t)w.d_group_bytes();
                        int ng = pl.rg < b - g0 ? pl.rg : b - g0;
                        unsigned spins = 0;
                        while (!mbar_try_wait_for(&S.empty[slot], par ^ 1, WAIT_NS)) {
                            if (*S.abort) return cnt;
                            if (++spins > SPIN_LIMIT) {
                                atomicOr(&P.ctl->error, 2u);
                                *S.abort = 1;
                                return cnt;
                            }
                        }
                        uint8_t* dst = S.ring + (size_t)slot * P.slot_bytes;
                        mbar_expect_tx(&S.full[slot], ng * (qgb + dgb));
                        bulk_g2s(dst, w.q + (size_t)g0 * qgb, ng * qgb, &S.full[slot], pol);
                        bulk_g2s(dst + (size_t)ng * qgb, (const uint8_t*)w.d + (size_t)g0 * dgb, ng * dgb, &S.full[slot], pol);
                    }
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
    unsigned long long* stamp;  // fine-grained timeline of one selected phase (debug), or NULL
};
#define STAMP(c, i)                                             \
    do {                                                        \
        if ((c).stamp) (c).stamp[i] = globaltimer_ns();          \
    } while (0)

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

// `count` = 1 + the arrivals of the flag_out phases passed since the last one (those phases hand their rows over
// through flagged words and skip the barrier), so the counter stays one arrival per phase and CTA.
__device__ void grid_arrive(Ctx& c, unsigned count) {
    consumer_sync();
    if (c.ct == 0)  // release: orders the CTA's writes (made visible to this thread by the barrier) before the count
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(c.P.bar_counter), "l"((unsigned long long)count) : "memory");
}

// Phase inputs are produced block-wise: consumer warp cw owns the 32-element blocks
// cw, cw + NC, ... and lane `lane` element `lane` of each, so a value is computed, quantised
// (simd.rs:255-323) and stored by the same thread with no staging pass.
constexpr int MAXJ = 16;  // blocks per warp: inputs up to NC * MAXJ * 32 = 7680 elements
constexpr int FASTJ = 5;  // inputs of up to NC * FASTJ * 32 = 2400 elements take the short path

// Quantises blocks cw + j*NC (j < J, those below nb) whose element `lane` is v[j].
// The J block maxima are reduced "transposed": in every halving round a lane keeps half of its
// values and hands the other half to its partner, so after log2(JP) rounds lane L holds the
// maximum of block L >> SH only.  That costs JP + log2(32/JP) - 1 shuffles instead of 5 * J, and
// each lane then performs the two IEEE divisions of ONE block instead of all J (the inverse
// scales travel back by one shuffle per block).  max is exact, so the order does not matter.
template <int J>
__device__ __forceinline__ void quantize_blocks(Ctx& c, const float (&v)[J], int j0, int nb) {
    static_assert(J >= 1 && J <= 16, "at most 16 blocks per call");
    constexpr int JP = J <= 4 ? 4 : (J <= 8 ? 8 : 16);
    constexpr int LOG = JP == 4 ? 2 : (JP == 8 ? 3 : 4);
    constexpr int SH = 5 - LOG;  // lanes per block after the halving rounds: 1 << SH
    // Block maxima: |v| >= 0, so the IEEE bit patterns order like unsigned integers and one warp-wide integer
    // max per block (independent of one another) replaces the dependent shuffle rounds.  max is exact, so the order
    // does not matter.  Lane L then performs the two IEEE divisions of block L >> SH only.
    float a[1] = {0.0f};
#pragma unroll
    for (int j = 0; j < J; j++) {
        const float mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(v[j]))));
        a[0] = (c.lane >> SH) == j ? mx : a[0];
    }
    // this lane's block
    const int jm = c.lane >> SH;
    // d = amax / 127 and id = 1 / d, both correctly rounded (simd.rs:255-323) but without the generic division
    // routine: with r = RN(1/127), q0 = RN(a * r) and rem = RN(fma(-q0, 127, a)), fma(rem, r, q0) equals RN(a / 127)
    // for EVERY finite a >= 0 (checked exhaustively over all 2^31 - 2^23 bit patterns on the host, subnormals
    // included); the reciprocal intrinsic is the correctly rounded 1 / d by definition.
    constexpr float R127 = 1.0f / 127.0f;
    const float q0 = __fmul_rn(a[0], R127);
    float d = __fmaf_rn(__fmaf_rn(-q0, 127.0f, a[0]), R127, q0);
    if (!(a[0] < __int_as_float(0x7f800000))) d = __fdiv_rn(a[0], 127.0f);  // infinity / NaN: the plain division
    const float id = d != 0.0f ? __frcp_rn(d) : 0.0f;
    {
        const int b = c.cw + (j0 + jm) * NC;
        if ((c.lane & ((1 << SH) - 1)) == 0 && jm < J && b < nb) {
            const float sc = __half2float(__float2half_rn(d));
            c.S.xs[b] = sc;
            c.S.xs16[b] = __fmul_rn(sc, 0.0625f);
        }
    }
#pragma unroll
    for (int j = 0; j < J; j++) {
        const float idj = __shfl_sync(0xffffffffu, id, j << SH);
        const int b = c.cw + (j0 + j) * NC;
        if (b < nb) c.S.xq[b * QK + c.lane] = (int8_t)__float2int_rn(__fmul_rn(v[j], idj));
    }
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

// Norm weights of the thread's elements; static data, fetched BEFORE the dependency wait.
__device__ __forceinline__ void load_norm_w(const Ctx& c, const MegaPhase& ph, float (&w)[MAXJ]) {
    const int nb = ph.k / QK;
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
        const int b = c.cw + j * NC;
        w[j] = b < nb ? __ldg(ph.norm_w + b * QK + c.lane) : 0.0f;
    }
}

// Identifier a flag_out phase stamps on the rows it writes: unique among the values a word of the flagged copy
// can still hold (its previous writer ran at most a few phases earlier) and never 0, the cleared state.
__device__ __forceinline__ uint32_t phase_id(const MegaParams& P, int t, int pi) {
    return (uint32_t)(P.bar_base + (unsigned long long)t * P.n_phases + pi) | 0x80000000u;
}

// Sum of the NC per-warp partial sums as a balanced tree (depth 4 instead of 15 dependent f64 additions).
__device__ __forceinline__ double sum_warp_partials(const double* red) {
    static_assert(NC <= 16, "tree of 16 leaves");
    double t[16];
#pragma unroll
    for (int i = 0; i < 16; i++) t[i] = i < NC ? red[i] : 0.0;
#pragma unroll
    for (int w = 8; w >= 1; w >>= 1)
#pragma unroll
        for (int i = 0; i < w; i++) t[i] += t[i + w];
    return t[0];
}

__device__ void prologue_norm(Ctx& c, const MegaPhase& ph, uint32_t token, const float (&w)[MAXJ], uint32_t id_in) {
    const MegaParams& P = c.P;
    const int k = ph.k, nb = k / QK;
    // Conv state of the layer whose gating ran one phase ago (lfm2.rs:691-695).  The values are fetched now; the
    // rolling buffer is overwritten further down, once every CTA is known to have finished reading the old one.
    const MegaLayer* CL = ph.conv_commit >= 0 ? &c.S.layers[ph.conv_commit] : nullptr;
    const int dc = P.conv_ks - 1, hs = P.hs;
    const int cc0 = CL ? share(c.cta, hs, c.ncta) : 0, cc1 = CL ? share(c.cta + 1, hs, c.ncta) : 0;
    float cst[3] = {0.0f, 0.0f, 0.0f};  // conv_ks <= 4
    if (cc0 + c.ct < cc1) {
        const int ch = cc0 + c.ct;
#pragma unroll
        for (int kk = 0; kk < 2; kk++)
            if (kk + 1 < dc) cst[kk] = __ldcg(CL->conv_state + (size_t)(kk + 1) * hs + ch);
        cst[2] = conv_bx(P.proj, hs, ch);
    }
    STAMP(c, 0);
    float v[MAXJ];
    const int e0 = ph.embed ? share(c.cta, k, c.ncta) : 0, e1 = ph.embed ? share(c.cta + 1, k, c.ncta) : 0;
    if (ph.flag_in) {
        // The previous phase wrote every row as (its id, value) in one 64-bit word: a word that carries the id holds
        // the new value, so the row is consumed element by element as it arrives and no grid barrier is needed.
        // Seeing all words also proves that every team of every CTA has finished the previous mat-vec.
#pragma unroll
        for (int j = 0; j < MAXJ; j++) v[j] = 0.0f;
        uint32_t pending = 0;
#pragma unroll
        for (int j = 0; j < FASTJ; j++) pending |= (c.cw + j * NC < nb) ? 1u << j : 0u;
        unsigned spins = 0;
        while (pending && !*c.S.abort) {
            unsigned long long x[FASTJ];
#pragma unroll
            for (int j = 0; j < FASTJ; j++)
                if (pending >> j & 1) x[j] = ld_relaxed_u64(P.hidden_flagged + (c.cw + j * NC) * QK + c.lane);
#pragma unroll
            for (int j = 0; j < FASTJ; j++)
                if ((pending >> j & 1) && (uint32_t)(x[j] >> 32) == id_in) {
                    v[j] = __uint_as_float((uint32_t)x[j]);
                    pending &= ~(1u << j);
                }
            if (pending && ++spins > SPIN_LIMIT) {
                atomicOr(&P.ctl->error, 8u);
                *c.S.abort = 1;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int b = c.cw + j * NC, e = b * QK + c.lane;
            v[j] = 0.0f;
            if (b < nb) {
                if (ph.embed) {
                    v[j] = P.embd_q6k ? q6k_elem(P.embd6, token, e) : embed_elem(P.embd, token, e);
                    if (e >= e0 && e < e1) P.hidden[e] = v[j];
                } else {
                    v[j] = __ldcg(P.hidden + e);
                }
            }
        }
    }
    // cpu::rmsnorm (cpu.rs:577-594); f64 partial sums combined in a fixed order
    // (rows of up to FASTJ blocks per warp skip the other blocks' terms: they would add +0.0, which changes nothing,
    // but the additions are dependent f64 operations on the critical path)
    const bool short_row = nb <= FASTJ * NC;
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < FASTJ; j++) {
        double x = (double)v[j];
        s += x * x;  // absent blocks add +0.0
    }
    if (!short_row) {
#pragma unroll
        for (int j = FASTJ; j < MAXJ; j++) {
            double x = (double)v[j];
            s += x * x;
        }
    }
    STAMP(c, 1);
    s = warp_sum_f64(s);
    if (c.lane == 0) c.S.red[c.cw] = s;
    consumer_sync();
    STAMP(c, 2);
    if (CL) {
        // every CTA has passed the gating prologue that read the old buffer: either a grid barrier lies in between,
        // or (flag_in) all rows of the mat-vec that followed that prologue have been seen by this CTA
        for (int ch = cc0 + c.ct; ch < cc1; ch += NCT) {
            if (ch != cc0 + c.ct) {  // rows beyond the first of this thread (hidden sizes above 480 x CTAs)
#pragma unroll
                for (int kk = 0; kk < 2; kk++)
                    if (kk + 1 < dc) cst[kk] = __ldcg(CL->conv_state + (size_t)(kk + 1) * hs + ch);
                cst[2] = conv_bx(P.proj, hs, ch);
            }
#pragma unroll
            for (int kk = 0; kk < 2; kk++)
                if (kk + 1 < dc) CL->conv_state[(size_t)kk * hs + ch] = cst[kk];
            if (dc > 0) CL->conv_state[(size_t)(dc - 1) * hs + ch] = cst[2];
        }
    }
    const double tot = sum_warp_partials(c.S.red);
    // (for a power-of-two length the division is an exact scaling, as is the multiplication by its reciprocal)
    const double mean = (k & (k - 1)) == 0 ? tot * (1.0 / (double)k) : tot / (double)k;
    const float inv = (float)(1.0 / sqrt(mean + (double)P.eps));
    STAMP(c, 3);
    if (short_row) {
        float vf[FASTJ];  // (a cast to a sub-array would force v into local memory)
#pragma unroll
        for (int j = 0; j < FASTJ; j++) vf[j] = __fmul_rn(__fmul_rn(v[j], inv), w[j]);
        quantize_blocks<FASTJ>(c, vf, 0, nb);
    } else {
#pragma unroll
        for (int j = 0; j < MAXJ; j++) v[j] = __fmul_rn(__fmul_rn(v[j], inv), w[j]);
        quantize_blocks<MAXJ>(c, v, 0, nb);
    }
    STAMP(c, 4);
    consumer_sync();
    STAMP(c, 5);
}

__device__ void prologue_conv(Ctx& c, const MegaPhase& ph) {
    const MegaParams& P = c.P;
    const MegaLayer& L = c.S.layers[ph.layer];
    const int hs = P.hs, ks = P.conv_ks, dc = ks - 1, nb = hs / QK;
    constexpr int MAXKS = 4;  // kernel sizes up to 4 (LFM2 uses 3); larger ones take the per-kernel path
    // five blocks per warp and pass: hidden sizes up to 2400 are done in one pass (one memory round trip)
    constexpr int CJ = FASTJ;
    for (int j0 = 0; j0 * NC < nb; j0 += CJ) {
        float st[CJ][MAXKS - 1], pb[CJ], pc[CJ], px[CJ], cw[CJ][MAXKS];
#pragma unroll
        for (int j = 0; j < CJ; j++) {  // every load of the blocks first
            const int b = c.cw + (j0 + j) * NC;
            const int chs = (b < nb ? b : 0) * QK + c.lane;
            pb[j] = __ldcg(P.proj + chs);
            pc[j] = __ldcg(P.proj + hs + chs);
            px[j] = __ldcg(P.proj + 2 * hs + chs);
#pragma unroll
            for (int kk = 0; kk < MAXKS - 1; kk++) st[j][kk] = kk < dc ? __ldcg(L.conv_state + (size_t)kk * hs + chs) : 0.0f;
#pragma unroll
            for (int kk = 0; kk < MAXKS; kk++) cw[j][kk] = kk < ks ? __ldg(L.conv_w + chs * ks + kk) : 0.0f;
        }
        float o[CJ];
#pragma unroll
        for (int j = 0; j < CJ; j++) {
            float sum = 0.0f;
#pragma unroll
            for (int kk = 0; kk < MAXKS - 1; kk++)
                if (kk < dc) sum = __fadd_rn(sum, __fmul_rn(st[j][kk], cw[j][kk]));
            const float bx = __fmul_rn(pb[j], px[j]);
            float wl = cw[j][0];
#pragma unroll
            for (int kk = 1; kk < MAXKS; kk++) wl = kk == dc ? cw[j][kk] : wl;
            sum = __fadd_rn(sum, __fmul_rn(bx, wl));
            o[j] = __fmul_rn(pc[j], sum);
        }
        quantize_blocks<CJ>(c, o, j0, nb);
    }
    consumer_sync();
}

__device__ void prologue_silu(Ctx& c, const MegaPhase& ph) {
    const MegaParams& P = c.P;
    const int nb = ph.k / QK;
    float g[MAXJ], u[MAXJ];
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
        const int b = c.cw + j * NC, e = (b < nb ? b : 0) * QK + c.lane;
        g[j] = __ldcg(P.gate + e);
        u[j] = __ldcg(P.up + e);
    }
#pragma unroll
    for (int j = 0; j < MAXJ; j++) g[j] = silu_mul_elem(g[j], u[j]);
    quantize_blocks<MAXJ>(c, g, 0, nb);
    consumer_sync();
}

__device__ void prologue_quant(Ctx& c, const MegaPhase& ph) {
    const int nb = ph.k / QK;
    if (nb <= FASTJ * NC) {
        float v[FASTJ];
#pragma unroll
        for (int j = 0; j < FASTJ; j++) {
            const int b = c.cw + j * NC;
            v[j] = __ldcg(ph.src + (b < nb ? b : 0) * QK + c.lane);
        }
        quantize_blocks<FASTJ>(c, v, 0, nb);
    } else {
        float v[MAXJ];
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int b = c.cw + j * NC;
            v[j] = __ldcg(ph.src + (b < nb ? b : 0) * QK + c.lane);
        }
        quantize_blocks<MAXJ>(c, v, 0, nb);
    }
    consumer_sync();
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

// Per-head RMSNorm + RoPE of `src` into dst (lfm2.rs:783-802), by one warp; dst in shared memory.
// Lane i holds the RoPE pair (i, i + hd/2) (hd <= 64: one pair per lane; larger heads loop).  The
// f64 sum of squares is combined in a fixed tree (the reference adds in element order; the sums
// agree to ~1e-16 relative, far below the f32 rounding of the result it feeds).
__device__ void head_norm_rope(const float* src_g, const float* w, float eps, const float* cosr, const float* sinr, int hd,
                               float* dst, int lane) {
    const int half = hd / 2;
    if (half <= 64) {
        // heads up to 128 wide: every operand (values, norm weights, rotation table) is requested before the first
        // use, so the whole step costs one memory round trip; the arithmetic and its order are those of the loop below
        float a[2], b[2], wa[2], wb[2], cs[2], sn[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int i = lane + 32 * r, ii = i < half ? i : 0;
            a[r] = __ldcg(src_g + ii);
            b[r] = __ldcg(src_g + ii + half);
            wa[r] = __ldg(w + ii);
            wb[r] = __ldg(w + ii + half);
            cs[r] = __ldg(cosr + ii);
            sn[r] = __ldg(sinr + ii);
        }
        double ss = 0.0;
#pragma unroll
        for (int r = 0; r < 2; r++)
            if (lane + 32 * r < half) {
                ss += (double)a[r] * (double)a[r];
                ss += (double)b[r] * (double)b[r];
            }
        ss = warp_sum_f64(ss);
        const double mean = (hd & (hd - 1)) == 0 ? ss * (1.0 / (double)hd) : ss / (double)hd;  // exact scaling either way
        const float inv = (float)(1.0 / sqrt(mean + (double)eps));
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int i = lane + 32 * r;
            if (i < half) {
                const float x0 = __fmul_rn(__fmul_rn(a[r], inv), wa[r]);
                const float x1 = __fmul_rn(__fmul_rn(b[r], inv), wb[r]);
                dst[i] = __fsub_rn(__fmul_rn(x0, cs[r]), __fmul_rn(x1, sn[r]));
                dst[i + half] = __fadd_rn(__fmul_rn(x0, sn[r]), __fmul_rn(x1, cs[r]));
            }
        }
        __syncwarp();
        return;
    }
    double ss = 0.0;
    for (int i = lane; i < half; i += 32) {
        double a = (double)__ldcg(src_g + i), b = (double)__ldcg(src_g + i + half);
        ss += a * a;
        ss += b * b;
    }
    ss = warp_sum_f64(ss);
    const float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)eps));
    for (int i = lane; i < half; i += 32) {
        float x0 = __fmul_rn(__fmul_rn(__ldcg(src_g + i), inv), __ldg(w + i));
        float x1 = __fmul_rn(__fmul_rn(__ldcg(src_g + i + half), inv), __ldg(w + i + half));
        float cs = __ldg(cosr + i), sn = __ldg(sinr + i);
        dst[i] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        dst[i + half] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
    }
    __syncwarp();
}

// Long contexts: the q.k scores of the cached keys, for the phase_attention that follows.  In phase_attention
// every (head, slice) item recomputes its head's scores, which is cheap while the context is short; at thousands
// of keys it dominates the step (each CTA can only keep a few hundred small loads in flight).  Here the work
// items are (head, block of KEYS_PER_ITEM keys), dealt to ALL CTAs, and each score is computed once, with the
// arithmetic of the in-phase loop (attn_scores, cpu.rs:1404-1458), and stored to P.scores_g.
__device__ void phase_scores(Ctx& c, const MegaPhase& ph, int pos) {
    const MegaParams& P = c.P;
    const MegaLayer& L = c.S.layers[ph.layer];
    const int hd = P.head_dim, n_heads = P.n_heads, n_kv = L.n_kv, kv_dim = n_kv * hd, group = n_heads / n_kv;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const float* cosr = P.rope_cos + (size_t)pos * (hd / 2);
    const float* sinr = P.rope_sin + (size_t)pos * (hd / 2);
    float* qs = c.S.head;
    constexpr int KU = 4;
    constexpr int KPR = NCT / 8;
    constexpr int KEYS_PER_ITEM = KPR * KU;
    const int nblk = (pos + KEYS_PER_ITEM - 1) / KEYS_PER_ITEM;
    const int items = n_heads * nblk;
    const int it0 = share(c.cta, items, c.ncta), it1 = share(c.cta + 1, items, c.ncta);
    const int ch = c.ct & 7, kslot = c.ct >> 3;
    const int nd8 = hd >> 3;
    int cur_h = -1;
    float qreg[8];
    for (int it = it0; it < it1; it++) {
        const int h = it / nblk, tb = (it - h * nblk) * KEYS_PER_ITEM;
        const int off = (h / group) * hd;
        if (h != cur_h) {
            consumer_sync();  // everyone is done with the previous head's q
            if (c.cw == 0) head_norm_rope(P.qbuf + h * hd, L.q_norm, P.eps, cosr, sinr, hd, qs, c.lane);
            consumer_sync();
#pragma unroll
            for (int j = 0; j < 8; j++) qreg[j] = j < nd8 ? qs[ch + j * 8] : 0.0f;
            cur_h = h;
        }
        float kv[KU][8];
#pragma unroll
        for (int u = 0; u < KU; u++) {
            const int t = tb + u * KPR + kslot;
            const float* kp = L.k_cache + (size_t)(t < pos ? t : 0) * kv_dim + off + ch;
#pragma unroll
            for (int j = 0; j < 8; j++) kv[u][j] = __ldcg(kp + (j < nd8 ? j : 0) * 8);
        }
#pragma unroll
        for (int u = 0; u < KU; u++) {
            const int t = tb + u * KPR + kslot;
            float a = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (j < nd8) a = __fmaf_rn(qreg[j], kv[u][j], a);
            for (int j = 8; j < nd8; j++)  // heads wider than 64
                a = __fmaf_rn(qs[ch + j * 8], __ldcg(L.k_cache + (size_t)(t < pos ? t : 0) * kv_dim + off + ch + j * 8), a);
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
            if (t < pos && ch == 0) P.scores_g[(size_t)h * P.max_seq + t] = __fmul_rn(a, scale);
        }
    }
}

// forward_attn_block between the QKV and output projections (lfm2.rs:783-1007).  A work item is
// (query head, 16-wide slice of the head's output dims); items are spread over the CTAs.  Every
// item recomputes its head's scores and softmax (cheap), then the slice's weighted V sum: the
// needed V columns are first gathered into shared memory by all threads (one memory latency per
// chunk), and 16 threads run the fused chains in ascending t, the reference's order.
template <bool LONG>
__device__ void phase_attention(Ctx& c, const MegaPhase& ph, int pos) {
    const MegaParams& P = c.P;
    const MegaLayer& L = c.S.layers[ph.layer];
    const int hd = P.head_dim, n_heads = P.n_heads, n_kv = L.n_kv, kv_dim = n_kv * hd, group = n_heads / n_kv;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const float* cosr = P.rope_cos + (size_t)pos * (hd / 2);
    const float* sinr = P.rope_sin + (size_t)pos * (hd / 2);
    float* sc = c.S.xf;
    float *qs = c.S.head, *ks = c.S.head + 256;
    const int seq = pos + 1;
    const int nq = hd / 16, items = n_heads * nq;
    const int nf = xf_floats(P);
    const int sc_pad = (seq + 3) & ~3;
    float* Vs = sc + sc_pad;                 // [rows][16]
    int chunk = (nf - sc_pad) / 16;
    chunk = chunk > seq ? seq : chunk;
    // items it with floor(it * ncta / items) == cta, i.e. ceil(cta * items / ncta) <= it < ceil((cta+1) * items / ncta)
    const int it0 = (int)(((unsigned)c.cta * items + c.ncta - 1) / c.ncta);
    const int it1 = (int)(((unsigned)(c.cta + 1) * items + c.ncta - 1) / c.ncta);
    for (int it = it0; it < it1 && it < items; it++) {
        const int h = it / nq, d0 = (it % nq) * 16;
        const int kvh = h / group, off = kvh * hd;
        STAMP(c, 0);
        consumer_sync();
        {   // The V columns of the first chunk do not depend on the scores: they are fetched now with asynchronous
            // global -> shared copies (no registers held) and land while the scores and the softmax are computed.
            const int rows = chunk < seq ? chunk : seq;
            for (int i = c.ct; i < rows * 4; i += NCT) {
                const float* src = (i >> 2) < pos ? L.v_cache + (size_t)(i >> 2) * kv_dim + off + d0 + (i & 3) * 4 : P.vbuf + off + d0 + (i & 3) * 4;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(Vs + i * 4)), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        if (c.cw == 0) head_norm_rope(P.qbuf + h * hd, L.q_norm, P.eps, cosr, sinr, hd, qs, c.lane);
        if (c.cw == 1) {
            head_norm_rope(P.kbuf + off, L.k_norm, P.eps, cosr, sinr, hd, ks, c.lane);
            if (h % group == 0 && d0 == 0) {  // one writer per KV head appends to the caches
                for (int i = c.lane; i < hd; i += 32) {
                    L.k_cache[(size_t)pos * kv_dim + off + i] = ks[i];
                    L.v_cache[(size_t)pos * kv_dim + off + i] = __ldcg(P.vbuf + off + i);
                }
            }
        }
        STAMP(c, 1);
        consumer_sync();
        STAMP(c, 2);
        // scores + max (attn_scores, cpu.rs:1404-1458).  The NEON dot keeps 8 fused chains: chain
        // ch = 0..3 is lane ch of sum0 (dims ch, ch+8, ...), chain 4..7 lane ch-4 of sum1 (dims ch, ch+8,
        // ...), then v[l] = sum0[l] + sum1[l] and (v0+v1)+(v2+v3).  Eight threads share a key, one chain
        // each, and every thread issues the loads of KU keys before any arithmetic.
        float mx = __int_as_float(0xFF800000);
        {
            constexpr int KU = 4;
            constexpr int KPR = NCT / 8;                   // keys per round of the consumer threads
            const int ch = c.ct & 7, kslot = c.ct >> 3;
            const int nd8 = hd >> 3;
            float qreg[8];
#pragma unroll
            for (int j = 0; j < 8; j++) qreg[j] = j < nd8 ? qs[ch + j * 8] : 0.0f;
            // long contexts: the cached keys' scores were computed once by the MPH_SCORES phase
            if (LONG) {
                for (int t = c.ct; t < pos; t += NCT) {
                    const float sv = __ldcg(P.scores_g + (size_t)h * P.max_seq + t);
                    sc[t] = sv;
                    mx = fmaxf(mx, sv);
                }
            }
            // cached keys t < pos: branch-free loads (out-of-range keys read row 0 and are dropped)
            for (int tb = 0; tb < pos && !LONG; tb += KPR * KU) {
                float kv[KU][8];
#pragma unroll
                for (int u = 0; u < KU; u++) {
                    const int t = tb + u * KPR + kslot;
                    const float* kp = L.k_cache + (size_t)(t < pos ? t : 0) * kv_dim + off + ch;
#pragma unroll
                    for (int j = 0; j < 8; j++) kv[u][j] = __ldcg(kp + (j < nd8 ? j : 0) * 8);
                }
#pragma unroll
                for (int u = 0; u < KU; u++) {
                    const int t = tb + u * KPR + kslot;
                    float a = 0.0f;
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        if (j < nd8) a = __fmaf_rn(qreg[j], kv[u][j], a);
                    for (int j = 8; j < nd8; j++)  // heads wider than 64
                        a = __fmaf_rn(qs[ch + j * 8], __ldcg(L.k_cache + (size_t)(t < pos ? t : 0) * kv_dim + off + ch + j * 8), a);
                    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));  // sum0[l] + sum1[l]
                    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
                    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
                    if (t < pos) {
                        float sv = __fmul_rn(a, scale);
                        if (ch == 0) sc[t] = sv;
                        mx = fmaxf(mx, sv);
                    }
                }
            }
            // the key of this step is still in shared memory
            if (c.cw == 0) {
                float a = 0.0f;
                for (int j = 0; j < nd8; j++) a = __fmaf_rn(qs[ch + j * 8], ks[ch + j * 8], a);
                a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));
                a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
                a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
                float sv = __fmul_rn(a, scale);
                if (c.lane == 0) sc[pos] = sv;
                mx = fmaxf(mx, sv);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        STAMP(c, 3);
        if (c.lane == 0) c.S.redf[c.cw] = mx;
        consumer_sync();
        STAMP(c, 4);
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
        const double tot = sum_warp_partials(c.S.red);
        const float inv = (float)(1.0 / tot);
        for (int t = c.ct; t < seq; t += NCT) sc[t] = __fmul_rn(sc[t], inv);
        STAMP(c, 5);
        // attn_values (cpu.rs:1463-1509): one fused chain per output dim, ascending t
        float acc = 0.0f;
        for (int t0 = 0; t0 < seq; t0 += chunk) {
            const int rows = chunk < seq - t0 ? chunk : seq - t0;
            consumer_sync();  // scores normalised / previous chunk consumed
            if (t0 == 0) STAMP(c, 8);
            if (t0 == 0) asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's copies of the first chunk
            // later chunks: four independent 16-byte loads in flight per thread (a load -> store pair per iteration
            // pays one memory latency per iteration)
            for (int idx0 = c.ct; idx0 < rows * 4 && t0 > 0; idx0 += NCT * 4) {
                float4 g0, g1, g2, g3;
                const int n4 = rows * 4;
                const int i0 = idx0, i1 = idx0 + NCT, i2 = idx0 + 2 * NCT, i3 = idx0 + 3 * NCT;
#define WICK_VSRC(i) ((t0 + ((i) >> 2)) < pos ? L.v_cache + (size_t)(t0 + ((i) >> 2)) * kv_dim + off + d0 + ((i)&3) * 4 \
                                              : P.vbuf + off + d0 + ((i)&3) * 4)
                g0 = __ldcg(reinterpret_cast<const float4*>(WICK_VSRC(i0)));
                g1 = __ldcg(reinterpret_cast<const float4*>(WICK_VSRC(i1 < n4 ? i1 : i0)));
                g2 = __ldcg(reinterpret_cast<const float4*>(WICK_VSRC(i2 < n4 ? i2 : i0)));
                g3 = __ldcg(reinterpret_cast<const float4*>(WICK_VSRC(i3 < n4 ? i3 : i0)));
#undef WICK_VSRC
                float4* V4 = reinterpret_cast<float4*>(Vs);
                V4[i0] = g0;
                if (i1 < n4) V4[i1] = g1;
                if (i2 < n4) V4[i2] = g2;
                if (i3 < n4) V4[i3] = g3;
            }
            consumer_sync();
            if (t0 == 0) STAMP(c, 9);
            if (c.ct < 16) {
                // the chain is serial, its operands are not: 16 steps' operands are loaded before their FMAs
                const float* scp = sc + t0;
                const float* vp = Vs + c.ct;
                int tl = 0;
                for (; tl + 16 <= rows; tl += 16) {
                    float sv[16], vv[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        sv[i] = scp[tl + i];
                        vv[i] = vp[(tl + i) * 16];
                    }
#pragma unroll
                    for (int i = 0; i < 16; i++) acc = __fmaf_rn(sv[i], vv[i], acc);
                }
                for (; tl < rows; tl++) acc = __fmaf_rn(scp[tl], vp[tl * 16], acc);
            }
            if (t0 == 0) STAMP(c, 10);
        }
        STAMP(c, 6);
        if (c.ct < 16) P.attn_out[h * hd + d0 + c.ct] = acc;
    }
    STAMP(c, 7);
}

__device__ __forceinline__ float reduce_row8(float a) {
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
    return a;
}

// The mat-vec over one ring slot is done by a TEAM of three consumer warps in two steps.
//  1. products: every (row, block, lane-word) term  float(p) * (f16(d_w) * d_x)  is independent of
//     every other one, so the team's 96 threads compute them all in parallel and write each one
//     over the weight word it came from (same size: 4 bytes; for Q8_0 over the low word of the pair);
//  2. chains: one warp per 4-row group, lane = p*16 + r*4 + l, adds its chain's products in block
//     order (the only part of the reference's arithmetic that is serial), then the three shuffle-adds.
// Both steps touch shared memory as 32 consecutive words per warp access (no bank conflicts).
__device__ __forceinline__ void team_sync(int team) {
    asm volatile("bar.sync %0, %1;" ::"r"(2 + team), "n"(TEAM_THREADS) : "memory");
}

// One thread takes one (block, row) of the group per step: its four lane-words are 16 contiguous
// bytes (as are the matching input words), so weights, inputs and products move as 128-bit
// shared-memory accesses and the scale product is formed once per four terms.
template <int DT, int U = (DT == DT_Q4_0 ? 3 : 2)>
__device__ __forceinline__ void stage_products(uint32_t* __restrict__ qs, const __half* __restrict__ ds, int nb, int tt,
                                               const int* __restrict__ xq32, const float* __restrict__ xsc) {
    const int ni = nb * 4;  // (block, row) items of the group
    for (int i0 = tt; i0 < ni; i0 += TEAM_THREADS * U) {
        uint4 wa[U], wb[U];
        int4 xl[U], xh[U];
        float d[U];
        int at[U];
#pragma unroll
        for (int u = 0; u < U; u++) {  // every load of the U independent items first
            const int i = i0 + u * TEAM_THREADS, is = i < ni ? i : i0;
            const int b = is >> 2, r = is & 3;
            at[u] = DT == DT_Q4_0 ? q4_word(b, r, 0) : q8_word(b, 0, r, 0);
            wa[u] = *reinterpret_cast<const uint4*>(qs + at[u]);
            if (DT == DT_Q8_0) wb[u] = *reinterpret_cast<const uint4*>(qs + at[u] + 32);
            xl[u] = *reinterpret_cast<const int4*>(xq32 + b * 8);
            xh[u] = *reinterpret_cast<const int4*>(xq32 + b * 8 + 4);
            d[u] = __fmul_rn(__half2float(ds[is]), xsc[b]);  // scale plane index b*4 + r == item index
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            int s0, s1, s2, s3;
            if (DT == DT_Q4_0) {  // 16 * lane sum; xsc already carries the 1/16
#define WICK_Q4_TERM(w, lo_x, hi_x) \
    __dp4a((int)(((w)&0xF0F0F0F0u) ^ 0x80808080u), hi_x, __dp4a((int)((((w) << 4) & 0xF0F0F0F0u) ^ 0x80808080u), lo_x, 0))
                s0 = WICK_Q4_TERM(wa[u].x, xl[u].x, xh[u].x);
                s1 = WICK_Q4_TERM(wa[u].y, xl[u].y, xh[u].y);
                s2 = WICK_Q4_TERM(wa[u].z, xl[u].z, xh[u].z);
                s3 = WICK_Q4_TERM(wa[u].w, xl[u].w, xh[u].w);
#undef WICK_Q4_TERM
            } else {
                s0 = __dp4a((int)wb[u].x, xh[u].x, __dp4a((int)wa[u].x, xl[u].x, 0));
                s1 = __dp4a((int)wb[u].y, xh[u].y, __dp4a((int)wa[u].y, xl[u].y, 0));
                s2 = __dp4a((int)wb[u].z, xh[u].z, __dp4a((int)wa[u].z, xl[u].z, 0));
                s3 = __dp4a((int)wb[u].w, xh[u].w, __dp4a((int)wa[u].w, xl[u].w, 0));
            }
            if (i0 + u * TEAM_THREADS < ni) {
                uint4 o;
                o.x = __float_as_uint(__fmul_rn((float)s0, d[u]));
                o.y = __float_as_uint(__fmul_rn((float)s1, d[u]));
                o.z = __float_as_uint(__fmul_rn((float)s2, d[u]));
                o.w = __float_as_uint(__fmul_rn((float)s3, d[u]));
                *reinterpret_cast<uint4*>(qs + at[u]) = o;
            }
        }
    }
}

template <int DT, int U>
__device__ __forceinline__ void chain_batches(const uint32_t* __restrict__ pp, int nb, int& b, float& acc) {
    for (; b + 2 * (U - 1) < nb; b += 2 * U) {
        float t[U];
#pragma unroll
        for (int u = 0; u < U; u++) t[u] = __uint_as_float(DT == DT_Q4_0 ? pp[(b + 2 * u) * 16] : pp[((b + 2 * u) >> 1) * 64]);
#pragma unroll
        for (int u = 0; u < U; u++) acc = __fadd_rn(acc, t[u]);
    }
}

// The chain of one (row, parity, lane group): its products in block order.  The additions are serial by contract; the
// operand loads are not, so they are issued 32 at a time (then 8 at a time for what is left) ahead of the additions:
// with 8 at a time the 32 terms of a 2048-long row took ~620 cycles, most of it shared-memory latency between batches.
template <int DT>
__device__ __forceinline__ float group_chain_sum(const uint32_t* __restrict__ qs, int nb, int lane) {
    const int p = lane >> 4;
    const uint32_t* pp = DT == DT_Q4_0 ? qs + (lane & 15) : qs + lane;
    float acc = 0.0f;
    int b = p;
    chain_batches<DT, 32>(pp, nb, b, acc);
    chain_batches<DT, 8>(pp, nb, b, acc);
    for (; b < nb; b += 2) acc = __fadd_rn(acc, __uint_as_float(DT == DT_Q4_0 ? pp[b * 16] : pp[(b >> 1) * 64]));
    return acc;
}

// DTK: the quantisation type every streamed matrix of the model has (DT_Q4_0 or DT_Q8_0), or 0 when they differ
// and the type is looked up per matrix.  Specialising removes the other type's product / chain code from the
// kernel: the kernel walks ~70 short phases per token, and its speed turned out to depend on its code size.
template <int DTK>
__device__ __forceinline__ bool is_q4(int dtype) { return DTK ? DTK == DT_Q4_0 : dtype == DT_Q4_0; }

// LONG: the launch uses the long-context phase list (MPH_SCORES phases present).  A separate instantiation, so
// that the short-context kernel does not carry that code (see the note on code size above).
template <int DTK, bool LONG>
__device__ void consumer(const MegaParams& P, const Smem& S, int cta, int ncta) {
    Ctx c{P, S, cta, ncta, (int)threadIdx.x - 32, ((int)threadIdx.x - 32) >> 5, (int)threadIdx.x & 31, nullptr};
    int slot = 0;
    uint32_t par = 0;
    const int team = c.cw / TEAM_WARPS, tw = c.cw % TEAM_WARPS, tt = tw * 32 + c.lane;
    const uint32_t pos0 = __ldcg(&P.ctl->pos), step0 = __ldcg(&P.ctl->step);
    uint32_t token = __ldcg(&P.ctl->token);
    unsigned owed = 0;  // arrivals of flag_out phases not yet added to the barrier counter
    const int* xq32 = reinterpret_cast<const int*>(S.xq);
    for (int t = 0; t < P.n_tokens; t++) {
        const int pos = (int)pos0 + t;
        unsigned long long best = 0;
        for (int pi = 0; pi < P.n_phases; pi++) {
            const MegaPhase& ph = S.ph[pi];
            const uint32_t id_out = phase_id(P, t, pi);
            // the descriptor fields the phase branches on, and its work split, are fetched here, ahead of the dependency
            // wait (as register copies: through the reference every use after a barrier is another shared-memory load,
            // and those loads sat between the prologue and the first stage)
            const int kind = ph.kind, pair = ph.pair, n_mat = ph.n_mat, flag_out = ph.flag_out;
            const Plan pl = S.plan[pi];
            float nw[MAXJ];
            if (kind == MPH_NORM) load_norm_w(c, ph, nw);
            if ((t > 0 || pi > 0) && !ph.flag_in) grid_wait(c, (P.bar_base + (unsigned long long)t * P.n_phases + pi) * (unsigned long long)ncta);
            const bool prof = P.prof && cta == 0 && c.ct == 0 && t == P.n_tokens - 1;
            c.stamp = (prof && pi == P.prof_phase) ? P.prof + (size_t)P.n_phases * 4 : nullptr;
            if (prof) P.prof[pi * 4 + 0] = globaltimer_ns();
            if (pi == 0 && t > 0) {
                // argmax of the previous step is this step's input (Session::generate, session.rs:1251)
                token = (uint32_t)(__ldcg(&P.argmax_acc[(t - 1) & 1]) & 0xffffffffull);
                if (cta == 0 && c.ct == 0) P.ring[(step0 + t - 1) % (uint32_t)P.ring_len] = token;
            }
            if (pi == 1 && cta == 0 && c.ct == 0) P.argmax_acc[(t + 1) & 1] = 0;  // free for the next step
            switch (kind) {
                case MPH_NORM: prologue_norm(c, ph, token, nw, phase_id(P, t, pi - 1)); break;
                case MPH_CONV: prologue_conv(c, ph); break;
                case MPH_SILU: prologue_silu(c, ph); break;
                case MPH_QUANT: prologue_quant(c, ph); break;
                case MPH_SCORES:
                    if (LONG) phase_scores(c, ph, pos);
                    break;
                default: phase_attention<LONG>(c, ph, pos); break;
            }
            if (prof) P.prof[pi * 4 + 1] = globaltimer_ns();
            if (kind != MPH_ATTN && kind != MPH_SCORES && pair) {
                // gate / up as alternating stages: stage pair j goes to team j % NTEAMS, which keeps both
                // slots until it has the two sums of each row and can apply SwiGLU (n_slots is a multiple of
                // 2 * NTEAMS, so within the phase a slot always returns to the same team)
                const DevWeight& wg = ph.mat[0].w;
                const DevWeight& wu = ph.mat[1].w;
                const int nb = wg.k / QK;
                const uint32_t qgb = (uint32_t)wg.q_group_bytes();
                float* act = ph.mat[0].y;
                int pj = 0;
                for (int g0 = pl.lo; g0 < pl.hi; g0 += pl.rg, pj++) {
                    const int slot_a = slot;
                    const uint32_t par_a = par;
                    slot = slot + 1 == P.n_slots ? 0 : slot + 1;
                    par ^= (slot == 0);
                    const int slot_b = slot;
                    const uint32_t par_b = par;
                    slot = slot + 1 == P.n_slots ? 0 : slot + 1;
                    par ^= (slot == 0);
                    if (pj % NTEAMS != team) continue;
                    const int ng = pl.rg < pl.hi - g0 ? pl.rg : pl.hi - g0;
                    uint8_t* bases[2] = {S.ring + (size_t)slot_a * P.slot_bytes, S.ring + (size_t)slot_b * P.slot_bytes};
                    for (int half = 0; half < 2; half++) {
                        unsigned spins = 0;
                        while (!mbar_try_wait_for(&S.full[half ? slot_b : slot_a], half ? par_b : par_a, WAIT_NS) && !*S.abort) {
                            if (++spins > SPIN_LIMIT) {
                                atomicOr(&P.ctl->error, 4u);
                                *S.abort = 1;
                                break;
                            }
                        }
                        const DevWeight& w = half ? wu : wg;
                        const __half* dbase = reinterpret_cast<const __half*>(bases[half] + (size_t)ng * qgb);
                        for (int gi = 0; gi < ng; gi++) {
                            uint32_t* qs = reinterpret_cast<uint32_t*>(bases[half] + (size_t)gi * qgb);
                            if (is_q4<DTK>(w.dtype)) stage_products<DT_Q4_0>(qs, dbase + (size_t)gi * nb * 4, nb, tt, xq32, S.xs16);
                            else stage_products<DT_Q8_0>(qs, dbase + (size_t)gi * nb * 4, nb, tt, xq32, S.xs);
                        }
                    }
                    team_sync(team);
                    for (int gi = tw; gi < ng; gi += TEAM_WARPS) {
                        const uint32_t* qa = reinterpret_cast<const uint32_t*>(bases[0] + (size_t)gi * qgb);
                        const uint32_t* qb = reinterpret_cast<const uint32_t*>(bases[1] + (size_t)gi * qgb);
                        float ga = is_q4<DTK>(wg.dtype) ? group_chain_sum<DT_Q4_0>(qa, nb, c.lane) : group_chain_sum<DT_Q8_0>(qa, nb, c.lane);
                        float ua = is_q4<DTK>(wu.dtype) ? group_chain_sum<DT_Q4_0>(qb, nb, c.lane) : group_chain_sum<DT_Q8_0>(qb, nb, c.lane);
                        ga = reduce_row8(ga);
                        ua = reduce_row8(ua);
                        const int row = (g0 + gi) * 4 + ((c.lane >> 2) & 3);
                        if ((c.lane & 19) == 0 && row < wg.m) act[row] = silu_mul_elem(ga, ua);  // cpu.rs:668-673
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    team_sync(team);
                    if (tt == 0) {
                        mbar_arrive(&S.empty[slot_a]);
                        mbar_arrive(&S.empty[slot_b]);
                    }
                }
            } else if (kind != MPH_ATTN && kind != MPH_SCORES) {
                int off = 0, nst = 0;
                for (int mi = 0; mi < n_mat; mi++) {
                    const MegaMat& M = ph.mat[mi];
                    const DevWeight& w = M.w;
                    const int gm = w.groups(), nb = w.k / QK;
                    int a = (pl.lo > off ? pl.lo : off) - off, b = (pl.hi < off + gm ? pl.hi : off + gm) - off;
                    const uint32_t qgb = (uint32_t)w.q_group_bytes();
                    const int epi = M.epi, wm = w.m;  // (register copies: read again after every barrier otherwise)
                    float* const y = M.y;
                    for (int g0 = a; g0 < b; g0 += pl.rg, slot = slot + 1 == P.n_slots ? 0 : slot + 1, par ^= (slot == 0)) {
                        // a slot always belongs to the same team (n_slots is a multiple of NTEAMS), so a team
                        // never waits two uses of a slot ahead and mbarrier parity cannot alias
                        if (slot % NTEAMS != team) continue;
                        int ng = pl.rg < b - g0 ? pl.rg : b - g0;
                        if (c.stamp && nst < 4) c.stamp[nst * 4 + 0] = globaltimer_ns();
                        unsigned spins = 0;
                        while (!mbar_try_wait_for(&S.full[slot], par, WAIT_NS) && !*S.abort) {
                            if (++spins > SPIN_LIMIT) {
                                atomicOr(&P.ctl->error, 4u);
                                *S.abort = 1;
                                break;
                            }
                        }
                        if (c.stamp && nst < 4) c.stamp[nst * 4 + 1] = globaltimer_ns();
                        uint8_t* base = S.ring + (size_t)slot * P.slot_bytes;
                        const __half* dbase = reinterpret_cast<const __half*>(base + (size_t)ng * qgb);
                        for (int gi = 0; gi < ng; gi++) {
                            uint32_t* qs = reinterpret_cast<uint32_t*>(base + (size_t)gi * qgb);
                            if (is_q4<DTK>(w.dtype)) stage_products<DT_Q4_0>(qs, dbase + (size_t)gi * nb * 4, nb, tt, xq32, S.xs16);
                            else stage_products<DT_Q8_0>(qs, dbase + (size_t)gi * nb * 4, nb, tt, xq32, S.xs);
                        }
                        // residual-add epilogue: the old value of the row is fetched now, so that its latency runs
                        // under the chain step instead of after it (a warp owns at most two groups of a slot)
                        float resid[2] = {0.0f, 0.0f};
                        if (epi == MEP_ADD && (c.lane & 19) == 0) {
#pragma unroll
                            for (int q = 0; q < 2; q++) {
                                const int gi = tw + q * TEAM_WARPS, row = (g0 + gi) * 4 + ((c.lane >> 2) & 3);
                                if (gi < ng && row < wm) resid[q] = __ldcg(y + row);
                            }
                        }
                        team_sync(team);
                        if (c.stamp && nst < 4) c.stamp[nst * 4 + 2] = globaltimer_ns();
                        for (int gi = tw; gi < ng; gi += TEAM_WARPS) {
                            const uint32_t* qs = reinterpret_cast<const uint32_t*>(base + (size_t)gi * qgb);
                            float acc = is_q4<DTK>(w.dtype) ? group_chain_sum<DT_Q4_0>(qs, nb, c.lane) : group_chain_sum<DT_Q8_0>(qs, nb, c.lane);
                            acc = reduce_row8(acc);
                            const int row = (g0 + gi) * 4 + ((c.lane >> 2) & 3);
                            if ((c.lane & 19) == 0 && row < wm) {
                                if (epi == MEP_ADD) {
                                    const float hv = __fadd_rn(gi == tw ? resid[0] : resid[1], acc);
                                    y[row] = hv;
                                    if (flag_out) st_relaxed_u64(P.hidden_flagged + row, (unsigned long long)id_out << 32 | __float_as_uint(hv));
                                } else if (epi == MEP_STORE) {
                                    y[row] = acc;
                                } else {
                                    if (!P.greedy) y[row] = acc;
                                    unsigned long long pk = argmax_pack(acc, (uint32_t)row);
                                    best = pk > best ? pk : best;
                                }
                            }
                        }
                        // the slot was written through the generic proxy (products); order that before the
                        // bulk copy (async proxy) that will refill it
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        team_sync(team);
                        if (c.stamp && nst < 4) c.stamp[nst * 4 + 3] = globaltimer_ns();
                        nst++;
                        if (tt == 0) mbar_arrive(&S.empty[slot]);
                    }
                    off += gm;
                }
            }
            if (pi == P.n_phases - 1 && P.greedy && !P.skip_logits) {
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
            if (flag_out) {
                owed++;
            } else {
                grid_arrive(c, 1 + owed);
                owed = 0;
            }
            if (prof) P.prof[pi * 4 + 3] = globaltimer_ns();
        }
    }
    // last step's result and the control block
    if (cta == 0 && !P.skip_logits) {
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

template <int DTK, bool LONG>
__global__ void __launch_bounds__(MEGA_THREADS, 1) k_decode_mega(const MegaParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem S = carve(smem_raw, P);
    {   // phase and layer descriptors into shared memory (word copies; both are multiples of 8 bytes)
        const uint32_t* src = reinterpret_cast<const uint32_t*>(P.phases);
        uint32_t* dst = reinterpret_cast<uint32_t*>(S.ph);
        for (int i = threadIdx.x; i < (int)(P.n_phases * sizeof(MegaPhase) / 4); i += blockDim.x) dst[i] = __ldg(src + i);
        src = reinterpret_cast<const uint32_t*>(P.layers);
        dst = reinterpret_cast<uint32_t*>(S.layers);
        for (int i = threadIdx.x; i < (int)(P.n_layers * sizeof(MegaLayer) / 4); i += blockDim.x) dst[i] = __ldg(src + i);
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < P.n_slots; i++) {
            mbar_init(&S.full[i], 1);
            mbar_init(&S.empty[i], 1);  // released by the team that owns the slot
        }
        *S.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P.n_phases; i += blockDim.x) {
        Plan pl{0, 0, 1, 0};
        if (S.ph[i].kind != MPH_ATTN && S.ph[i].kind != MPH_SCORES) pl = plan_phase(S.ph[i], blockIdx.x, gridDim.x, P.slot_bytes);
        S.plan[i] = pl;
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
        consumer<DTK, LONG>(P, S, blockIdx.x, gridDim.x);
    }
    __syncthreads();
}

}  // namespace

size_t mega_smem_bytes(const MegaParams& P) {
    int nf = xf_floats(P);
    size_t o = (size_t)P.n_slots * P.slot_bytes + (size_t)nf * 4 + (size_t)(P.kmax / QK) * 8;
    o = (o + 15) & ~(size_t)15;
    o += P.kmax;
    o = (o + 15) & ~(size_t)15;
    o += NC * 16 + (size_t)P.n_slots * 16 + NC * 4;
    o = (o + 15) & ~(size_t)15;
    o += 4 * 256 * 4 + 16;
    o += (size_t)P.n_phases * sizeof(MegaPhase) + (size_t)P.n_layers * sizeof(MegaLayer);
    o = (o + 15) & ~(size_t)15;
    o += (size_t)P.n_phases * sizeof(Plan);
    return o;
}

namespace {
const void* mega_kernel(const MegaParams& P) {
    if (P.long_ctx) {
        switch (P.uniform_dtype) {
            case DT_Q4_0: return (const void*)k_decode_mega<DT_Q4_0, true>;
            case DT_Q8_0: return (const void*)k_decode_mega<DT_Q8_0, true>;
            default: return (const void*)k_decode_mega<0, true>;
        }
    }
    switch (P.uniform_dtype) {
        case DT_Q4_0: return (const void*)k_decode_mega<DT_Q4_0, false>;
        case DT_Q8_0: return (const void*)k_decode_mega<DT_Q8_0, false>;
        default: return (const void*)k_decode_mega<0, false>;
    }
}
}  // namespace

int mega_max_ctas(const MegaParams& P) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t smem = mega_smem_bytes(P);
    if (cudaFuncSetAttribute(mega_kernel(P), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mega_kernel(P), MEGA_THREADS, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return per_sm > 0 ? sms : 0;  // one CTA per SM
}

cudaError_t launch_decode_mega(cudaStream_t st, const MegaParams& P, int n_ctas) {
    size_t smem = mega_smem_bytes(P);
    // the attribute is per function, not per model: models of different size share the kernel
    cudaError_t e = cudaFuncSetAttribute(mega_kernel(P), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    void* args[] = {(void*)&P};
    g_kernel_launches++;
    return cudaLaunchCooperativeKernel(mega_kernel(P), dim3(n_ctas), dim3(MEGA_THREADS), args, smem, st);
}

}  // namespace wick
