// Tensor-core prefill GEMM for sm_100a: int8 x int8 -> int32 block sums on tcgen05 with the
// accumulator in tensor memory, operands staged by TMA, per-block f32 scaling in the epilogue warps.
//
// What it computes, for a weight matrix W [m rows][k] in Q4_0 / Q8_0 and n activation rows
// quantised to Q8_0 (simd.rs:255-323):
//     S_b[i][j]  = sum over the 32 elements of block b of  w_int[i][.] * x_int[j][.]        (int32, exact)
//     out[j][i]  = sum over b, in ascending b, of  fma(float(S_b[i][j]), f16->f32(d_w[i][b]) * d_x[j][b], acc)
// S_b is the same integer the NEON kernels produce per block (simd.rs:696-1019, the four lane
// partials added up); what differs from them is the f32 accumulation: one fused chain per output in
// block order instead of 2 x 4 unfused lane chains, so outputs agree to f32 rounding (~1e-6 relative),
// not bit for bit.  The bit-exact order lives in k_gemm (kernels_gemv.cu); this kernel is the
// throughput path of forward_prefill.
//
// One MMA instruction covers exactly one quantisation block (K = 32 int8), writes a fresh 128 x BN
// int32 tile into one of 512/BN tensor-memory buffers and never accumulates across blocks, because
// each block has its own scale pair.  The epilogue warps drain a buffer (tcgen05.ld), hand it back,
// and apply the scales on the CUDA cores: 3 instructions per (output, block), which is what bounds the
// kernel (the tensor pipe needs about 1/6 of that time).
//
// Roles in a CTA of 20 warps (one CTA per SM, persistent over output tiles):
//   warp 0  lane 0: TMA producer, one K=128 stage (4 blocks) of W rows and activation rows per step
//   warp 1  lane 0: issues tcgen05.mma / tcgen05.commit; the whole warp owns the TMEM allocation
//   warp 2        : copies the stage's weight scales and (transposed) activation scales into smem (cp.async)
//   warps 4..19   : epilogue; warp w reads TMEM lanes 32*(w%4).. and columns (w-4)/4 * BN/4 ..; four
//                   warps per scheduler hide the tensor-memory load and barrier latencies
// Every wait is bounded: on expiry the kernel records an error code, all roles leave their loops and
// the CTA frees its tensor memory and exits.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstring>
#include <mutex>

#include "gemm_tc.cuh"

namespace wick {

namespace {

constexpr int TC_BM = 128;          // weight rows per tile == TMEM lanes
constexpr int TC_KSTAGE = 128;      // int8 elements (bytes) per row per stage == one 128B swizzle atom
constexpr int TC_KB_PER_STAGE = TC_KSTAGE / QK;  // 4 quantisation blocks per stage
// Shared-memory stages: as many as fit (27.6 KB each for 64-column tiles, 36.9 KB for 128).  A stage is
// only refilled after the epilogue has finished with its scales, and the refill has to be back from L2 before
// the MMA issuer needs it; with four stages that left about one microsecond, less than a loaded L2 round trip.
template <int BN>
__host__ __device__ constexpr int tc_stages() { return BN <= 64 ? 8 : 6; }
constexpr int TC_COL_GROUPS = 4;    // epilogue warps per TMEM lane quarter; each takes BN/4 columns
constexpr int TC_EPI_WARPS = 4 * TC_COL_GROUPS;
constexpr int TC_THREADS = 32 * (4 + TC_EPI_WARPS);
constexpr uint32_t TC_SPIN_LIMIT = 1u << 18;  // try_wait itself suspends for a while, so this is of the order of a second

template <int BN>
struct alignas(1024) TcStage {
    int8_t a[TC_BM * TC_KSTAGE];              // 16 KB, rows of 128 B, 128B-swizzled by TMA
    int8_t b[BN * TC_KSTAGE];                 // BN rows of 128 B
    float sw[TC_KB_PER_STAGE][TC_BM];         // weight scales of the stage's blocks
    float sx[TC_KB_PER_STAGE][BN];            // activation scales, transposed to [block][token]
};

template <int BN>
struct TcSmem {
    TcStage<BN> stage[tc_stages<BN>()];
    unsigned long long full[tc_stages<BN>()];   // TMA bytes landed + scales written
    unsigned long long empty[tc_stages<BN>()];  // MMAs of the stage retired + epilogue done with its scales
    unsigned long long tmem_full[512 / BN];   // block sums of one k-block are in the buffer
    unsigned long long tmem_empty[512 / BN];  // all epilogue warps have read the buffer
    uint32_t tmem_base;
    volatile uint32_t abort;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait.  Returns false once the limit is hit or another role has already given up.
// SLEEP_NS > 0 is for the producer, MMA and scale-loader roles: they run stages ahead of the epilogue, and a
// tight poll loop in those warps would take issue slots from the epilogue warps that bound the kernel.
template <int BN, unsigned SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(TcSmem<BN>* sm, uint32_t bar, uint32_t parity, uint32_t* err, uint32_t code) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (SLEEP_NS) __nanosleep(SLEEP_NS);
        if ((i & 1023u) == 1023u && sm->abort) return false;
    }
    sm->abort = 1;
    atomicCAS(err, 0u, code);
    return false;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// K-major operand tile, rows of 128 bytes, 128B swizzle: 8-row atoms 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc_sw128(uint32_t smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr >> 4) & 0x3FFF);  // start address
    d |= 1ull << 16;                                        // leading byte offset (unused for swizzled K-major)
    d |= (unsigned long long)(1024 >> 4) << 32;             // stride byte offset between 8-row atoms
    d |= 1ull << 46;                                        // descriptor version of this architecture
    d |= 2ull << 61;                                        // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, unsigned long long da, unsigned long long db, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
template <int COLS>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int32_t* r) {
    static_assert(COLS == 8 || COLS == 16 || COLS == 32, "one tcgen05.ld per k-block");
    if constexpr (COLS == 8) tmem_ld8(taddr, r);
    else if constexpr (COLS == 16) tmem_ld16(taddr, r);
    else tmem_ld32(taddr, r);
}
// Two f32 lanes per instruction (sm_100 packed f32x2 arithmetic), used by the fused-chain epilogue,
// which is bound by instruction issue: each half of a packed multiply or fused multiply-add is rounded
// like the scalar instruction.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace


namespace {

// Which matrix and which 128 x BN output tile a linear tile index means.  Tiles of one matrix are
// consecutive, token tiles fastest, so CTAs running side by side share a weight tile in L2.
struct TcTile {
    int mat, m0, n0;
};
__device__ __forceinline__ TcTile tc_decode_tile(const TcJob& job, int t, int tiles_n, int bn) {
    TcTile r;
    r.mat = (t >= job.tile_start[1] ? 1 : 0) + (t >= job.tile_start[2] ? 1 : 0);
    const int local = t - job.tile_start[r.mat];
    r.m0 = (local / tiles_n) * TC_BM;
    r.n0 = (local % tiles_n) * bn;
    return r;
}

template <int BN, bool SUMS, bool EXACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_gemm_tc(const __grid_constant__ TcJob job, const __grid_constant__ CUtensorMap map_x,
          const float* __restrict__ x_scales,  // [n][k/32]
          int32_t* __restrict__ sums,          // optional [n][m][k/32] (single-matrix jobs only)
          int n, int k, uint32_t* err) {
    extern __shared__ uint8_t tc_smem_raw[];
    TcSmem<BN>* sm = reinterpret_cast<TcSmem<BN>*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int NBUF = 512 / BN;
    constexpr int UNIT = NBUF / 2 < TC_KB_PER_STAGE ? NBUF / 2 : TC_KB_PER_STAGE;  // blocks per hand-over: two units in flight
    constexpr int NB2 = 2 * UNIT;  // buffers in use (32-column tiles leave half of tensor memory unused)
    static_assert(TC_KB_PER_STAGE % UNIT == 0 && NBUF >= NB2, "two hand-over units that tile a stage");
    constexpr int TC_STAGES = tc_stages<BN>();
    constexpr int COLS = BN / TC_COL_GROUPS;  // columns per epilogue thread
    // EXACT: a column is (token, NEON lane group); the activation rows arrive masked to one lane group
    // each (tc_mask_expand), so a tile covers BN/4 tokens and the MMA yields the four lane partials
    constexpr int TOK = EXACT ? BN / 4 : BN;  // tokens per tile
    constexpr int XROWS = EXACT ? 4 : 1;      // rows of the activation operand per token
    static_assert(!EXACT || ((COLS == 16 || COLS == 8) && !SUMS), "exact epilogue: 4 (or 2) tokens x 4 lane groups per thread");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = k / QK;
    const int k_stages = k / TC_KSTAGE;
    const int tiles_n = (n + TOK - 1) / TOK;
    const int tiles = job.tile_start[job.count];

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(smem_u32(&sm->full[s]), 1 + 32);            // producer (with tx bytes) + every lane of the scale warp
            mbar_init(smem_u32(&sm->empty[s]), 1 + TC_EPI_WARPS);  // MMA commit + epilogue warps
        }
        for (int b = 0; b < NBUF; b++) {
            mbar_init(smem_u32(&sm->tmem_full[b]), 1);
            mbar_init(smem_u32(&sm->tmem_empty[b]), TC_EPI_WARPS);
        }
        sm->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm->tmem_base;

    if (warp == 0) {
        // ── TMA producer ─────────────────────────────────────────────────────
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TcTile tl = tc_decode_tile(job, t, tiles_n, TOK);
                const CUtensorMap* mw = &job.map_w[tl.mat];
                for (int ks = 0; ks < k_stages; ks++, g++) {
                    const int s = g % TC_STAGES;
                    const uint32_t u = g / TC_STAGES;
                    ok = mbar_wait<BN, 256>(sm, smem_u32(&sm->empty[s]), (u & 1) ^ 1, err, 1);
                    if (!ok) break;
                    const uint32_t bar = smem_u32(&sm->full[s]);
                    mbar_arrive_expect_tx(bar, (TC_BM + BN) * TC_KSTAGE);
                    tma_load_2d(smem_u32(sm->stage[s].a), mw, bar, ks * TC_KSTAGE, tl.m0);
                    tma_load_2d(smem_u32(sm->stage[s].b), &map_x, bar, ks * TC_KSTAGE, tl.n0 * XROWS);
                }
            }
        }
    } else if (warp == 1) {
        // ── MMA issuer ───────────────────────────────────────────────────────
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            uint32_t g = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % TC_STAGES;
                    const uint32_t u = g / TC_STAGES;
                    ok = mbar_wait<BN, 128>(sm, smem_u32(&sm->full[s]), u & 1, err, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned long long da = umma_desc_sw128(smem_u32(sm->stage[s].a));
                    const unsigned long long db = umma_desc_sw128(smem_u32(sm->stage[s].b));
#pragma unroll
                    for (int kk = 0; kk < TC_KB_PER_STAGE; kk++) {
                        const uint32_t j = g * TC_KB_PER_STAGE + kk;
                        const uint32_t buf = j % NB2;
                        if (kk % UNIT == 0) {
                            // Buffers are handed over half of tensor memory (UNIT blocks) at a time: every hand-over
                            // costs each epilogue warp a barrier wait and an arrival, both long dependent steps of its
                            // loop, and that loop - not the tensor pipe - sets the pace of the kernel
                            const uint32_t un = j / UNIT;
                            ok = mbar_wait<BN, 64>(sm, smem_u32(&sm->tmem_empty[un & 1u]), ((un >> 1) & 1) ^ 1, err, 3);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        // 32 bytes further along K inside the swizzle atom: +2 in the 16-byte address field
                        umma_i8(tmem_base + buf * BN, da + (unsigned long long)(kk * 2), db + (unsigned long long)(kk * 2), idesc);
                        if (kk % UNIT == UNIT - 1) umma_commit(smem_u32(&sm->tmem_full[(j / UNIT) & 1u]));
                    }
                    if (ok) umma_commit(smem_u32(&sm->empty[s]));
                }
            }
        }
    } else if (warp == 2) {
        // ── scale loader ─────────────────────────────────────────────────────
        uint32_t g = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            const TcTile tl = tc_decode_tile(job, t, tiles_n, TOK);
            const float* wst = job.scales_t[tl.mat];
            const int m_pad = job.m_pad[tl.mat];
            for (int ks = 0; ks < k_stages; ks++, g++) {
                const int s = g % TC_STAGES;
                const uint32_t u = g / TC_STAGES;
                ok = mbar_wait<BN, 256>(sm, smem_u32(&sm->empty[s]), (u & 1) ^ 1, err, 4);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                TcStage<BN>& st = sm->stage[s];
                const int b0 = ks * TC_KB_PER_STAGE;
                // Asynchronous copies (cp.async), each lane's arrival on the stage's barrier deferred until its own copies
                // have landed: the warp never waits for a load, so the scales of as many stages as the ring has free are
                // in flight at once (with plain loads every stage cost this warp one dependent trip to L2).
#pragma unroll
                for (int kk = 0; kk < TC_KB_PER_STAGE; kk++)
                    cp_async_16(smem_u32(reinterpret_cast<float4*>(st.sw[kk]) + lane),
                                reinterpret_cast<const float4*>(wst + (size_t)(b0 + kk) * m_pad + tl.m0) + lane);
#pragma unroll
                for (int c = lane; c < TOK; c += 32) {
                    if (tl.n0 + c < n) {
                        const float* src = x_scales + (size_t)(tl.n0 + c) * nb + b0;
#pragma unroll
                        for (int kk = 0; kk < TC_KB_PER_STAGE; kk++) cp_async_4(smem_u32(&st.sx[kk][c]), src + kk);
                    } else {
#pragma unroll
                        for (int kk = 0; kk < TC_KB_PER_STAGE; kk++) st.sx[kk][c] = 0.0f;
                    }
                }
                // .noinc: the arrival was counted when the barrier was initialised (33 = producer + 32 lanes)
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&sm->full[s])) : "memory");
            }
        }
    } else if (warp >= 4) {
        // ── epilogue ─────────────────────────────────────────────────────────
        const int quarter = warp & 3, cg = (warp - 4) >> 2;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cg * COLS);
        uint32_t g = 0;
        bool ok = true;
        if constexpr (!EXACT) {
            f32x2 acc[COLS / 2];
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TcTile tl = tc_decode_tile(job, t, tiles_n, TOK);
                const int m = job.m[tl.mat];
                const int row = tl.m0 + row_in_tile;
#pragma unroll
                for (int c = 0; c < COLS / 2; c++) acc[c] = pack2(0.f, 0.f);
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % TC_STAGES;
                    const uint32_t u = g / TC_STAGES;
                    // (every lane of a warp runs the same wait on the same barrier and gets the same answer)
                    ok = mbar_wait(sm, smem_u32(&sm->full[s]), u & 1, err, 5);
                    if (!ok) break;
                    const TcStage<BN>& st = sm->stage[s];
#pragma unroll(BN == 64 && !SUMS ? TC_KB_PER_STAGE : 1)
                    for (int kk = 0; kk < TC_KB_PER_STAGE; kk++) {
                        const uint32_t j = g * TC_KB_PER_STAGE + kk;
                        const uint32_t buf = j % NB2, un = j / UNIT;
                        if (kk % UNIT == 0) {
                            ok = mbar_wait(sm, smem_u32(&sm->tmem_full[un & 1u]), (un >> 1) & 1, err, 6);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        int32_t S[COLS];
                        tmem_ld<COLS>(lane_base + buf * BN, S);
                        tmem_ld_wait();
                        if (kk % UNIT == UNIT - 1) {  // the unit's blocks are all in registers or consumed
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&sm->tmem_empty[un & 1u]));
                        }
                        const float sw = st.sw[kk][row_in_tile];
                        const f32x2 sw2 = pack2(sw, sw);
                        const float4* sx4 = reinterpret_cast<const float4*>(&st.sx[kk][cg * COLS]);
#pragma unroll
                        for (int c = 0; c < COLS; c += 4) {
                            const float4 x = sx4[c >> 2];
                            acc[c / 2 + 0] = fma2(pack2(__int2float_rn(S[c + 0]), __int2float_rn(S[c + 1])), mul2(sw2, pack2(x.x, x.y)), acc[c / 2 + 0]);
                            acc[c / 2 + 1] = fma2(pack2(__int2float_rn(S[c + 2]), __int2float_rn(S[c + 3])), mul2(sw2, pack2(x.z, x.w)), acc[c / 2 + 1]);
                        }
                        if (SUMS && row < m) {
                            const int b = ks * TC_KB_PER_STAGE + kk;
#pragma unroll
                            for (int c = 0; c < COLS; c++) {
                                const int tok = tl.n0 + cg * COLS + c;
                                if (tok < n) sums[((size_t)tok * m + row) * nb + b] = S[c];
                            }
                        }
                    }
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
                }
                if (ok && row < m) {
                    float* out = job.out[tl.mat];
#pragma unroll
                    for (int c = 0; c < COLS; c += 2) {
                        const int tok = tl.n0 + cg * COLS + c;
                        float a0, a1;
                        unpack2(acc[c / 2], a0, a1);
                        if (tok < n) out[(size_t)tok * m + row] = a0;
                        if (tok + 1 < n) out[(size_t)(tok + 1) * m + row] = a1;
                    }
                }
            }
        } else {
            // The arithmetic of gemm_q*_q8_0_neon (simd.rs:696-1019) bit for bit: per output eight unfused
            // chains acc[parity of the block][lane group] += float(lane partial) * (f16(d_w) * d_x), blocks
            // in ascending order, combined at the end as ((a0+a1)+(a2+a3)) per parity, even + odd.
            constexpr int TPT = COLS / 4;  // tokens per thread
            // The products are formed one by one; the chain additions go out two lanes at a time (add.rn.f32x2).  A packed
            // multiply feeding a packed add directly is turned into a fused multiply-add by the assembler, whatever the
            // rounding modifiers say (wrong rounding for this contract); scalar products into a packed add are left alone.
            f32x2 acc2[TPT][2][2];
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TcTile tl = tc_decode_tile(job, t, tiles_n, TOK);
                const int m = job.m[tl.mat];
                const int row = tl.m0 + row_in_tile;
#pragma unroll
                for (int i = 0; i < TPT; i++)
#pragma unroll
                    for (int l = 0; l < 4; l++) {
                        acc2[i][0][l >> 1] = acc2[i][1][l >> 1] = pack2(0.f, 0.f);
                    }
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % TC_STAGES;
                    const uint32_t u = g / TC_STAGES;
                    // (every lane of a warp runs the same wait on the same barrier and gets the same answer)
                    ok = mbar_wait(sm, smem_u32(&sm->full[s]), u & 1, err, 5);  // the stage's scales
                    if (!ok) break;
                    static_assert(UNIT == TC_KB_PER_STAGE, "the exact epilogue takes a whole stage per hand-over");
                    const uint32_t unit = g & 1u;                                // the half of tensor memory with its 4 blocks
                    ok = mbar_wait(sm, smem_u32(&sm->tmem_full[unit]), (g >> 1) & 1, err, 6);
                    if (!ok) break;
                    tc_fence_after();
                    const TcStage<BN>& st = sm->stage[s];
                    {
                        // the load of block kk + 1 is in flight while the chains of block kk run
                        int32_t SA[COLS], SB[COLS];
                        auto chains = [&](const int32_t (&S)[COLS], const int kk) {
                            const float sw = st.sw[kk][row_in_tile];
                            float xs[TPT];
                            if constexpr (TPT == 4) {
                                const float4 x = *reinterpret_cast<const float4*>(&st.sx[kk][cg * TPT]);
                                xs[0] = x.x, xs[1] = x.y, xs[2] = x.z, xs[3] = x.w;
                            } else {
                                const float2 x = *reinterpret_cast<const float2*>(&st.sx[kk][cg * TPT]);
                                xs[0] = x.x, xs[1] = x.y;
                            }
#pragma unroll
                            for (int i = 0; i < TPT; i++) {
                                const float d = __fmul_rn(sw, xs[i]);
#pragma unroll
                                for (int l = 0; l < 4; l += 2)
                                    acc2[i][kk & 1][l >> 1] = add2(acc2[i][kk & 1][l >> 1], pack2(__fmul_rn(__int2float_rn(S[i * 4 + l]), d),
                                                                                                 __fmul_rn(__int2float_rn(S[i * 4 + l + 1]), d)));
                            }
                        };
                        const uint32_t t0 = lane_base + (unit * TC_KB_PER_STAGE) * BN;
                        tmem_ld<COLS>(t0, SA);
                        tmem_ld_wait();
                        tmem_ld<COLS>(t0 + BN, SB);
                        chains(SA, 0);
                        tmem_ld_wait();
                        tmem_ld<COLS>(t0 + 2 * BN, SA);
                        chains(SB, 1);
                        tmem_ld_wait();
                        tmem_ld<COLS>(t0 + 3 * BN, SB);
                        chains(SA, 2);
                        tmem_ld_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&sm->tmem_empty[unit]));
                        chains(SB, 3);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
                }
                if (ok && row < m) {
                    float* out = job.out[tl.mat];
#pragma unroll
                    for (int i = 0; i < TPT; i++) {
                        const int tok = tl.n0 + cg * TPT + i;
                        float acc[1][2][4];
                        unpack2(acc2[i][0][0], acc[0][0][0], acc[0][0][1]);
                        unpack2(acc2[i][0][1], acc[0][0][2], acc[0][0][3]);
                        unpack2(acc2[i][1][0], acc[0][1][0], acc[0][1][1]);
                        unpack2(acc2[i][1][1], acc[0][1][2], acc[0][1][3]);
#define WICK_ACC(p, l) acc[0][p][l]
                        const float e = __fadd_rn(__fadd_rn(WICK_ACC(0, 0), WICK_ACC(0, 1)), __fadd_rn(WICK_ACC(0, 2), WICK_ACC(0, 3)));
                        const float o = __fadd_rn(__fadd_rn(WICK_ACC(1, 0), WICK_ACC(1, 1)), __fadd_rn(WICK_ACC(1, 2), WICK_ACC(1, 3)));
#undef WICK_ACC
                        if (tok < n) out[(size_t)tok * m + row] = __fadd_rn(e, o);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (sm->abort) {
            // copies issued before the failure may still be landing in this CTA's shared memory
            for (int i = 0; i < 64; i++) __nanosleep(1000);
        }
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

// ── host side ────────────────────────────────────────────────────────────────
namespace {

// One thread per (row, block): widen the block's quants to int8 and store its scale.
__global__ void k_tc_unpack(DevWeight w, int8_t* __restrict__ q, float* __restrict__ scales_t, int m_pad) {
    const int nb = w.k / QK;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)w.m * nb) return;
    const int row = (int)(idx / nb), b = (int)(idx % nb);
    const int g = row >> 2, r = row & 3;
    const __half* dg = w.d + (size_t)g * nb * 4;
    const uint32_t* qg = reinterpret_cast<const uint32_t*>(w.q + (size_t)g * w.q_group_bytes());
    scales_t[(size_t)b * m_pad + row] = __half2float(dg[b * 4 + r]);
    uint32_t o[8];
    if (w.dtype == DT_Q4_0) {
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t v = qg[q4_word(b, r, l)];
            // bytes of v: elements 4l..4l+3 in the low nibbles, 16+4l.. in the high nibbles
            const uint32_t lo = v & 0x0F0F0F0Fu, hi = (v >> 4) & 0x0F0F0F0Fu;
            o[l] = __vsub4(lo, 0x08080808u);
            o[4 + l] = __vsub4(hi, 0x08080808u);
        }
    } else {
#pragma unroll
        for (int l = 0; l < 4; l++) {
            o[l] = qg[q8_word(b, 0, r, l)];
            o[4 + l] = qg[q8_word(b, 1, r, l)];
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(q + (size_t)row * w.k + (size_t)b * QK);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// int8 matrix [rows][k] row-major; box = 128 bytes along k x box_rows rows; 128B swizzle.
cudaError_t encode_rows_map(const void* base, int rows, int k, int box_rows, CUtensorMap* out) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k};
    cuuint32_t box[2] = {(cuuint32_t)TC_KSTAGE, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int BN, bool EXACT>
cudaError_t launch_tc(cudaStream_t st, const TcJob& job, const CUtensorMap& map_x, const float* x_scales, int n, int k,
                      int32_t* sums, uint32_t* err) {
    static int sm_count = 0;
    static bool configured = false;
    const size_t smem = sizeof(TcSmem<BN>) + 1024;
    if (!configured) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(k_gemm_tc<BN, false, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if constexpr (!EXACT) {
            e = cudaFuncSetAttribute(k_gemm_tc<BN, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        configured = true;
    }
    const int tiles = job.tile_start[job.count];
    const int grid = tiles < sm_count ? tiles : sm_count;
    g_kernel_launches++;
    if constexpr (!EXACT) {
        if (sums) {
            k_gemm_tc<BN, true, false><<<grid, TC_THREADS, smem, st>>>(job, map_x, x_scales, sums, n, k, err);
            return cudaGetLastError();
        }
    }
    k_gemm_tc<BN, false, EXACT><<<grid, TC_THREADS, smem, st>>>(job, map_x, x_scales, nullptr, n, k, err);
    return cudaGetLastError();
}

// One thread per 16 input bytes (half a quantisation block): NEON lane group l owns bytes 4l..4l+3
// of each half (simd.rs:381-383: vdotq_s32 lane l), so output row 4*j + l keeps word l and zeroes the rest.
__global__ void k_tc_mask_expand(const uint4* __restrict__ xq, uint4* __restrict__ xm, size_t n_chunks, int chunks_per_row) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_chunks) return;
    const uint4 v = xq[i];
    const size_t row = i / chunks_per_row, c = i % chunks_per_row;
    uint4* o = xm + (row * 4) * chunks_per_row + c;
    o[0] = make_uint4(v.x, 0u, 0u, 0u);
    o[(size_t)chunks_per_row] = make_uint4(0u, v.y, 0u, 0u);
    o[(size_t)2 * chunks_per_row] = make_uint4(0u, 0u, v.z, 0u);
    o[(size_t)3 * chunks_per_row] = make_uint4(0u, 0u, 0u, v.w);
}

cudaError_t fill_job(TcJob& job, const TcWeight* const* w, float* const* out, int count, int tiles_n) {
    memset(&job, 0, sizeof(job));
    job.count = count;
    int t = 0;
    for (int i = 0; i < 3; i++) {
        job.tile_start[i] = t;
        if (i >= count) continue;
        if (w[i]->k != w[0]->k) return cudaErrorInvalidValue;
        job.map_w[i] = w[i]->map;
        job.scales_t[i] = w[i]->scales_t;
        job.out[i] = out[i];
        job.m[i] = w[i]->m;
        job.m_pad[i] = w[i]->m_pad;
        t += (w[i]->m_pad / TC_BM) * tiles_n;
    }
    job.tile_start[3] = t;
    for (int i = count; i < 3; i++) job.tile_start[i] = t;  // unused matrices own no tiles
    return cudaSuccess;
}

}  // namespace

bool tc_gemm_supported(int m, int k) { return m > 0 && k > 0 && k % TC_KSTAGE == 0; }

int tc_gemm_bn(int n, int row_tiles) {
    // 128-token tiles halve the weight-tile traffic; 64-token tiles are used while the wider ones
    // would leave the grid at less than two tiles per SM
    if (n <= 64) return 64;
    return row_tiles * ((n + 127) / 128) < 2 * 148 ? 64 : 128;
}

cudaError_t tc_weight_fill(cudaStream_t st, const DevWeight& w, TcWeight* out) {
    out->m = w.m;
    out->k = w.k;
    out->m_pad = (w.m + TC_BM - 1) / TC_BM * TC_BM;
    cudaError_t e = cudaMemsetAsync(out->q, 0, out->q_bytes(), st);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(out->scales_t, 0, out->s_bytes(), st);
    if (e != cudaSuccess) return e;
    const size_t n_blocks = (size_t)w.m * (w.k / QK);
    g_kernel_launches++;
    k_tc_unpack<<<(unsigned)((n_blocks + 255) / 256), 256, 0, st>>>(w, out->q, out->scales_t, out->m_pad);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return encode_rows_map(out->q, out->m_pad, out->k, TC_BM, &out->map);
}

cudaError_t tc_make_activation_map(const int8_t* xq, int rows_cap, int k, int bn, CUtensorMap* out) {
    return encode_rows_map(xq, rows_cap, k, bn, out);
}

cudaError_t launch_gemm_tc(cudaStream_t st, const TcWeight* const* w, float* const* out, int count, const CUtensorMap* map_x,
                           const float* x_scales, int n, int32_t* sums, uint32_t* err) {
    if (n <= 0 || count <= 0) return cudaSuccess;
    if (count > 3 || (sums && count != 1)) return cudaErrorInvalidValue;
    int rows = 0;
    for (int i = 0; i < count; i++) rows += w[i]->m_pad / TC_BM;
    const int bn = tc_gemm_bn(n, rows);
    TcJob job;
    cudaError_t e = fill_job(job, w, out, count, (n + bn - 1) / bn);
    if (e != cudaSuccess) return e;
    return bn == 64 ? launch_tc<64, false>(st, job, map_x[0], x_scales, n, w[0]->k, sums, err)
                    : launch_tc<128, false>(st, job, map_x[1], x_scales, n, w[0]->k, sums, err);
}

void launch_tc_mask_expand(cudaStream_t st, const int8_t* xq, int n, int k, int8_t* xm) {
    const size_t chunks = (size_t)n * (k / 16);
    if (!chunks) return;
    g_kernel_launches++;
    k_tc_mask_expand<<<(unsigned)((chunks + 255) / 256), 256, 0, st>>>(reinterpret_cast<const uint4*>(xq), reinterpret_cast<uint4*>(xm),
                                                                         chunks, k / 16);
}

cudaError_t launch_gemm_tc_exact(cudaStream_t st, const TcWeight* const* w, float* const* out, int count, const CUtensorMap& map_xm,
                                 const float* x_scales, int n, uint32_t* err, const CUtensorMap* map_xm_narrow) {
    if (n <= 0 || count <= 0) return cudaSuccess;
    if (count > 3) return cudaErrorInvalidValue;
    TcJob job;
    // 8-token tiles while twice the 16-token tiles still fit one wave (few rows and a narrow matrix: the multi-sequence
    // decode step): a tile's time is set by its K loop, so more, smaller tiles only pay when they run side by side
    int row_tiles = 0;
    for (int i = 0; i < count; i++) row_tiles += w[i]->m_pad / TC_BM;
    if (map_xm_narrow && 2 * row_tiles * ((n + TC_EXACT_TOKENS - 1) / TC_EXACT_TOKENS) <= 148) {
        cudaError_t e = fill_job(job, w, out, count, (n + TC_EXACT_TOKENS / 2 - 1) / (TC_EXACT_TOKENS / 2));
        if (e != cudaSuccess) return e;
        return launch_tc<2 * TC_EXACT_TOKENS, true>(st, job, *map_xm_narrow, x_scales, n, w[0]->k, nullptr, err);
    }
    cudaError_t e = fill_job(job, w, out, count, (n + TC_EXACT_TOKENS - 1) / TC_EXACT_TOKENS);
    if (e != cudaSuccess) return e;
    return launch_tc<4 * TC_EXACT_TOKENS, true>(st, job, map_xm, x_scales, n, w[0]->k, nullptr, err);
}

}  // namespace wick
