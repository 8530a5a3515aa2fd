// CPU oracle: a C++ restatement of the arithmetic of wick's own CPU path
// (aarch64 / NEON integer flavour) for the LFM2 decode + prefill hot path.
//
// THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are
// compared against and the timed CPU baseline of the benchmark.  Nothing in
// the product library links, imports or calls it.
//
// Parity status: wick is Rust and cannot be compiled where this was written
// (no cargo / rustc), so the restatement is pinned against the closed-form
// and self-consistency checks of wick's own unit tests (tests/ of this repo
// re-create those inputs), not against outputs of a running wick.  Whole-model
// logits are therefore "parity unpinned": they follow the cited source lines
// but were never compared with a wick binary.  Platform libm (`powf`, `sinf`,
// `cosf` inside RoPE) is a further unpinned input: wick calls the host libm.
//
// Every function cites the wick source it follows (path:line inside the wick
// repository).  Floating-point contraction must be OFF when compiling this file
// (-ffp-contract=off): Rust never fuses `a * b + c`, and NEON `vmlaq_n_f32`
// is a separate multiply and add.  Where wick uses a fused NEON FMA
// (`vfmaq_f32`) this file calls fmaf() explicitly.
//
// Layout note: wick's batched prefill keeps activations column-major
// [dim x n]; here they are token-major [n][dim].  Only addressing differs, the
// per-element arithmetic and its order are the same.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#if defined(__AVX2__) && defined(__F16C__)
#include <immintrin.h>
#define ORC_AVX2 1
#else
#define ORC_AVX2 0
#endif

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int QK = 32;
constexpr int DT_Q4_0 = 2;  // GGML type ids, wick/src/gguf.rs:36-44
constexpr int DT_Q8_0 = 8;
constexpr int DT_Q6_K = 14;
constexpr int QK_K = 256;       // elements of a Q6_K super-block
constexpr int Q6_K_BYTES = 210;  // ql[128] qh[64] scales[16] d (quant.rs:63-70)
constexpr int GEMV_PAR_THRESHOLD = 256;  // wick/src/backend/cpu.rs:310

int g_use_simd = 1;

// ── f16 <-> f32 (IEEE, round to nearest even; the `half` crate's behaviour) ─

inline float f16_to_f32(uint16_t h) {
#if ORC_AVX2
    return _cvtsh_ss(h);
#else
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FF;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f; memcpy(&f, &bits, 4); return f;
#endif
}

inline uint16_t f32_to_f16(float f) {
#if ORC_AVX2
    return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
#else
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000;
    int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFF;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00 | (man ? 0x200 : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000;
        int shift = 14 - exp;
        uint32_t r = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) r++;
        return (uint16_t)(sign | r);
    }
    uint32_t r = (uint32_t)(exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFF;
    if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) r++;
    return (uint16_t)(sign | r);
#endif
}

inline uint16_t load_u16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }

inline int block_bytes(int dtype) { return dtype == DT_Q4_0 ? 18 : 34; }
// bytes of one row of k elements
inline size_t row_bytes(int dtype, int k) {
    return dtype == DT_Q6_K ? (size_t)(k / QK_K) * Q6_K_BYTES : (size_t)(k / QK) * block_bytes(dtype);
}

template <class F>
inline void par_for(int n, bool parallel, F f) {
#ifdef _OPENMP
    if (parallel) {
#pragma omp parallel for schedule(static)
        for (int i = 0; i < n; i++) f(i);
        return;
    }
#endif
    for (int i = 0; i < n; i++) f(i);
}

// ── Activation quantiser ───────────────────────────────────────────────────
// wick/src/backend/simd.rs:255-323 (quantize_f32_to_q8_0_neon): per 32-block
// amax; d = amax / 127; id = d != 0 ? 1/d : 0; q = round-to-nearest-even(x*id)
// (vcvtnq_s32_f32) then a truncating cast to i8; the scale handed downstream is
// d after a round trip through f16.
void quantize_q8_0(const float* x, int k, float* scales, int8_t* quants) {
    int nb = k / QK;
    for (int b = 0; b < nb; b++) {
        const float* xb = x + b * QK;
        float amax = 0.0f;
        for (int i = 0; i < QK; i++) amax = std::max(amax, std::fabs(xb[i]));
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        scales[b] = f16_to_f32(f32_to_f16(d));
        for (int i = 0; i < QK; i++) {
            float v = xb[i] * id;
            // nearbyintf under the default rounding mode = ties to even
            quants[b * QK + i] = (int8_t)(int32_t)nearbyintf(v);
        }
    }
}

// ── Integer block dot, lane-structured ─────────────────────────────────────
// simd.rs:369-383 / :478-492: p = vdotq_s32(vdotq_s32(0, w_lo, x_lo), w_hi, x_hi)
// with w_lo = elements 0..15 and w_hi = elements 16..31 of the block, so lane l
// of p sums elements {4l..4l+3} and {16+4l..16+4l+3}.
inline void lane_sums_q4_0(const uint8_t* blk, const int8_t* xq, int32_t p[4]) {
    const uint8_t* qs = blk + 2;
    for (int l = 0; l < 4; l++) {
        int32_t s = 0;
        for (int i = 4 * l; i < 4 * l + 4; i++) {
            s += ((int)(qs[i] & 0x0F) - 8) * (int)xq[i];
            s += ((int)(qs[i] >> 4) - 8) * (int)xq[16 + i];
        }
        p[l] = s;
    }
}

inline void lane_sums_q8_0(const uint8_t* blk, const int8_t* xq, int32_t p[4]) {
    const int8_t* w = (const int8_t*)(blk + 2);
    for (int l = 0; l < 4; l++) {
        int32_t s = 0;
        for (int i = 4 * l; i < 4 * l + 4; i++) {
            s += (int)w[i] * (int)xq[i];
            s += (int)w[16 + i] * (int)xq[16 + i];
        }
        p[l] = s;
    }
}

// One output element of the integer GEMV / GEMM.  simd.rs:346-407 (Q4_0),
// :458-516 (Q8_0), shared by the batched kernels through gemm_dot_pair! /
// gemm_dot_single! (simd.rs:59-86): even blocks accumulate into sumv0, odd into
// sumv1, each `acc[l] = acc[l] + float(p[l]) * (f16(d_w) * d_x)` with the multiply
// and the add rounded separately; result = vaddvq(sumv0) + vaddvq(sumv1) with
// vaddvq = (l0 + l1) + (l2 + l3).
template <int DT>
float row_dot_scalar(const uint8_t* row, const float* xs, const int8_t* xq, int nb) {
    float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    const int bb = DT == DT_Q4_0 ? 18 : 34;
    for (int b = 0; b < nb; b++) {
        const uint8_t* blk = row + (size_t)b * bb;
        int32_t p[4];
        if (DT == DT_Q4_0) lane_sums_q4_0(blk, xq + b * QK, p);
        else lane_sums_q8_0(blk, xq + b * QK, p);
        float d = f16_to_f32(load_u16(blk)) * xs[b];
        float* a = acc[b & 1];
        for (int l = 0; l < 4; l++) {
            float prod = (float)p[l] * d;
            a[l] = a[l] + prod;
        }
    }
    float s0 = (acc[0][0] + acc[0][1]) + (acc[0][2] + acc[0][3]);
    float s1 = (acc[1][0] + acc[1][1]) + (acc[1][2] + acc[1][3]);
    return s0 + s1;
}

#if ORC_AVX2
// Same arithmetic, vectorised: one __m256 holds [sumv0 | sumv1].  Integer sums
// are exact in any order; the f32 multiply and add are separate instructions
// (this translation unit is built with -ffp-contract=off).
template <int DT>
inline __m256i pair_sums_epi32(const uint8_t* blk, const int8_t* xq) {
    // returns 8 x int32: t[i] = sum over byte pair (2i, 2i+1) of lo + hi halves
    __m128i w_lo, w_hi;
    if (DT == DT_Q4_0) {
        __m128i q = _mm_loadu_si128((const __m128i*)(blk + 2));
        const __m128i m = _mm_set1_epi8(0x0F), e = _mm_set1_epi8(8);
        w_lo = _mm_sub_epi8(_mm_and_si128(q, m), e);
        w_hi = _mm_sub_epi8(_mm_and_si128(_mm_srli_epi16(q, 4), m), e);
    } else {
        w_lo = _mm_loadu_si128((const __m128i*)(blk + 2));
        w_hi = _mm_loadu_si128((const __m128i*)(blk + 18));
    }
    __m128i x_lo = _mm_loadu_si128((const __m128i*)xq);
    __m128i x_hi = _mm_loadu_si128((const __m128i*)(xq + 16));
    __m256i a = _mm256_madd_epi16(_mm256_cvtepi8_epi16(w_lo), _mm256_cvtepi8_epi16(x_lo));
    __m256i b = _mm256_madd_epi16(_mm256_cvtepi8_epi16(w_hi), _mm256_cvtepi8_epi16(x_hi));
    return _mm256_add_epi32(a, b);
}

template <int DT>
float row_dot_avx2(const uint8_t* row, const float* xs, const int8_t* xq, int nb) {
    const int bb = DT == DT_Q4_0 ? 18 : 34;
    __m256 acc = _mm256_setzero_ps();
    int b = 0;
    for (; b + 1 < nb; b += 2) {
        const uint8_t* b0 = row + (size_t)b * bb;
        const uint8_t* b1 = b0 + bb;
        __m256i t0 = pair_sums_epi32<DT>(b0, xq + b * QK);
        __m256i t1 = pair_sums_epi32<DT>(b1, xq + (b + 1) * QK);
        // hadd: [p0_0 p0_1 p1_0 p1_1 | p0_2 p0_3 p1_2 p1_3] -> [p0_0..3 | p1_0..3]
        __m256i h = _mm256_permute4x64_epi64(_mm256_hadd_epi32(t0, t1), 0xD8);
        float d0 = f16_to_f32(load_u16(b0)) * xs[b];
        float d1 = f16_to_f32(load_u16(b1)) * xs[b + 1];
        __m256 dv = _mm256_set_m128(_mm_set1_ps(d1), _mm_set1_ps(d0));
        __m256 prod = _mm256_mul_ps(_mm256_cvtepi32_ps(h), dv);
        acc = _mm256_add_ps(acc, prod);
    }
    float a[8];
    _mm256_storeu_ps(a, acc);
    if (b < nb) {
        const uint8_t* blk = row + (size_t)b * bb;
        int32_t p[4];
        if (DT == DT_Q4_0) lane_sums_q4_0(blk, xq + b * QK, p);
        else lane_sums_q8_0(blk, xq + b * QK, p);
        float d = f16_to_f32(load_u16(blk)) * xs[b];
        for (int l = 0; l < 4; l++) {
            float prod = (float)p[l] * d;
            a[l] = a[l] + prod;
        }
    }
    float s0 = (a[0] + a[1]) + (a[2] + a[3]);
    float s1 = (a[4] + a[5]) + (a[6] + a[7]);
    return s0 + s1;
}
#endif

template <int DT>
inline float row_dot(const uint8_t* row, const float* xs, const int8_t* xq, int nb) {
#if ORC_AVX2
    if (g_use_simd) return row_dot_avx2<DT>(row, xs, xq, nb);
#endif
    return row_dot_scalar<DT>(row, xs, xq, nb);
}

// gemv_q4_0_q8_0_neon / gemv_q8_0_q8_0_neon (simd.rs:328-415, :440-524); rows in
// parallel once m >= 256 (cpu.rs:310), which does not change any result.
// gemv_q6k_q8_0_neon (simd.rs:552-672): one serial f32 sum per row over 16-element sub-blocks in the
// order (super-block, pass, half, {+0, +32, +64, +96}); each term is (d * scale * d_x) * float(int dot),
// products evaluated left to right, the term's product and the add unfused.
float row_dot_q6_k(const uint8_t* row, const float* xs, const int8_t* xq, int k) {
    float sumf = 0.0f;
    for (int bi = 0; bi < k / QK_K; bi++) {
        const uint8_t* blk = row + (size_t)bi * Q6_K_BYTES;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t* sc = (const int8_t*)(blk + 192);
        const float d = f16_to_f32(load_u16(blk + 208));
        const int xq_off = bi * QK_K;
        int sc_idx = 0, ql_p = 0, qh_p = 0, y_p = 0;
        for (int pass = 0; pass < 2; pass++) {
            for (int half = 0; half < 2; half++) {
                const int l_off = half * 16;
                for (int j = 0; j < 4; j++) {  // q1..q4
                    int32_t dot = 0;
                    for (int l = 0; l < 16; l++) {
                        const uint8_t lo = ql[ql_p + l_off + l + (j & 1 ? 32 : 0)];
                        const uint8_t h = qh[qh_p + l_off + l];
                        const int nib = j < 2 ? (lo & 0x0F) : (lo >> 4);
                        const int hi2 = (h >> (2 * j)) & 3;
                        const int q = (nib | (hi2 << 4)) - 32;
                        dot += q * (int)xq[xq_off + y_p + l_off + 32 * j + l];
                    }
                    const int q8_bi = (xq_off + y_p + l_off + 32 * j) / 32;
                    const float dj = d * (float)sc[sc_idx + 2 * j] * xs[q8_bi];
                    sumf += dj * (float)dot;
                }
                sc_idx += 1;
            }
            y_p += 128;
            ql_p += 64;
            qh_p += 32;
            sc_idx = 8;
        }
    }
    return sumf;
}

void gemv_preq(int dtype, const uint8_t* a, const float* xs, const int8_t* xq, float* y, int m, int k) {
    if (dtype == DT_Q6_K) {
        const size_t rb6 = row_bytes(dtype, k);
        par_for(m, m >= GEMV_PAR_THRESHOLD, [&](int i) { y[i] = row_dot_q6_k(a + i * rb6, xs, xq, k); });
        return;
    }
    int nb = k / QK;
    size_t rb = (size_t)nb * block_bytes(dtype);
    par_for(m, m >= GEMV_PAR_THRESHOLD, [&](int i) {
        y[i] = dtype == DT_Q4_0 ? row_dot<DT_Q4_0>(a + i * rb, xs, xq, nb)
                                : row_dot<DT_Q8_0>(a + i * rb, xs, xq, nb);
    });
}

// gemm_q4_0_q8_0_neon / gemm_q8_0_q8_0_neon (simd.rs:696-925, :937-1019):
// out[i*n + j] = the GEMV result of row i against pre-quantised column j
// (b_quants[j*k..], b_scales[j*nb..]).  The 8/4/1-column grouping of the NEON
// code only shares the weight decode; each (i, j) runs the same chain.
void gemm_preq(int dtype, const uint8_t* a, const float* bs, const int8_t* bq, float* out, int m, int n, int k,
               size_t out_row_stride, size_t out_col_stride) {
    int nb = k / QK;
    size_t rb = (size_t)nb * block_bytes(dtype);
    par_for(m, m >= 8, [&](int i) {
        const uint8_t* row = a + i * rb;
        for (int j = 0; j < n; j++) {
            float v = dtype == DT_Q4_0 ? row_dot<DT_Q4_0>(row, bs + (size_t)j * nb, bq + (size_t)j * k, nb)
                                       : row_dot<DT_Q8_0>(row, bs + (size_t)j * nb, bq + (size_t)j * k, nb);
            out[i * out_row_stride + j * out_col_stride] = v;
        }
    });
}

// ── Norm, exp, activations, softmax ────────────────────────────────────────

// cpu.rs:577-594: f64 sum of squares in element order, inv = (1/sqrt(mean+eps)) as f32,
// x[i] = x[i] * inv * w[i] (two f32 multiplies, left to right).
void rmsnorm(float* x, const float* w, int n, float eps) {
    double sum_sq = 0.0;
    for (int i = 0; i < n; i++) sum_sq += (double)x[i] * (double)x[i];
    double mean = sum_sq / (double)n;
    double rms = std::sqrt(mean + (double)eps);
    float inv = (float)(1.0 / rms);
    for (int i = 0; i < n; i++) x[i] = x[i] * inv * w[i];
}

inline float from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
inline uint32_t to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

// cpu.rs:602-642 (ggml_expf): magic-number rounding, Cody-Waite reduction,
// degree-5 polynomial, three range branches; all plain f32 mul/add, no FMA.
float ggml_expf(float x) {
    const float R = from_bits(0x4B400000u);
    const float LOG2E = from_bits(0x3FB8AA3Bu);
    const float LN2_HI = from_bits(0x3F317200u);
    const float LN2_LO = from_bits(0x35BFBE8Eu);
    const float C1 = from_bits(0x3F7FFFF6u);
    const float C2 = from_bits(0x3EFFFEDBu);
    const float C3 = from_bits(0x3E2AAF33u);
    const float C4 = from_bits(0x3D2B9F17u);
    const float C5 = from_bits(0x3C072010u);
    float z = R + x * LOG2E;
    float n = z - R;
    float b = x - n * LN2_HI - n * LN2_LO;
    uint32_t e = to_bits(z) << 23;
    float k = from_bits(e + to_bits(1.0f));
    float u = b * b;
    float j = C1 * b + (C2 + C3 * b + (C4 + C5 * b) * u) * u;
    float abs_n = from_bits(to_bits(n) & 0x7FFFFFFFu);
    if (abs_n <= 126.0f) {
        return k + j * k;
    } else if (abs_n > 192.0f) {
        return n > 0.0f ? std::numeric_limits<float>::infinity() : 0.0f;
    } else {
        uint32_t d = n <= 0.0f ? 0x82000000u : 0u;
        float s1 = from_bits(d + 0x7f000000u);
        float s2 = from_bits(e - d);
        return (s2 + s2 * j) * s1;
    }
}

// cpu.rs:668-673
void silu_mul(float* gate, const float* up, size_t n) {
    for (size_t i = 0; i < n; i++) gate[i] = gate[i] / (1.0f + ggml_expf(-gate[i])) * up[i];
}

// cpu.rs:715-731: f32 max, ggml_expf(x - max), f64 sum in element order,
// multiply by (1/sum) as f32.
void softmax(float* x, int n) {
    float mx = -std::numeric_limits<float>::infinity();
    for (int i = 0; i < n; i++) mx = std::max(mx, x[i]);
    double sum = 0.0;
    for (int i = 0; i < n; i++) {
        x[i] = ggml_expf(x[i] - mx);
        sum += (double)x[i];
    }
    float inv = (float)(1.0 / sum);
    for (int i = 0; i < n; i++) x[i] *= inv;
}

// ── RoPE ───────────────────────────────────────────────────────────────────
// cpu.rs:2145-2158: theta_scale = powf(base, -2/hd); theta starts at pos as f32 and
// is multiplied by theta_scale after each pair; pairs are (i, i + hd/2).
void rope_head(float* head, int pos, int hd, float base) {
    int half = hd / 2;
    float theta_scale = powf(base, -2.0f / (float)hd);
    float theta = (float)pos;
    for (int i = 0; i < half; i++) {
        float s = sinf(theta), c = cosf(theta);
        float x0 = head[i], x1 = head[i + half];
        head[i] = x0 * c - x1 * s;
        head[i + half] = x0 * s + x1 * c;
        theta *= theta_scale;
    }
}

// ── Attention ──────────────────────────────────────────────────────────────

// vaddvq_f32(vaddq_f32(sum0, sum1)) of the NEON dot (cpu.rs:1430-1456, :1778-1795):
// sum0 lane l fuses dims {l, 8+l, 16+l, ...}, sum1 lane l dims {4+l, 12+l, ...}.
// head_dim % 8 == 0 assumed (64 here).
inline float qk_dot_neon_order(const float* q, const float* kv, int hd) {
    float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
    for (int d = 0; d + 8 <= hd; d += 8) {
        for (int l = 0; l < 4; l++) {
            s0[l] = fmaf(q[d + l], kv[d + l], s0[l]);
            s1[l] = fmaf(q[d + 4 + l], kv[d + 4 + l], s1[l]);
        }
    }
    float v[4];
    for (int l = 0; l < 4; l++) v[l] = s0[l] + s1[l];
    return (v[0] + v[1]) + (v[2] + v[3]);
}

// attn_scores_neon, cpu.rs:1404-1458
void attn_scores(const float* q, const float* kc, float* scores, int kv_dim, int off, int hd, float scale, int seq) {
    for (int t = 0; t < seq; t++) scores[t] = qk_dot_neon_order(q, kc + (size_t)t * kv_dim + off, hd) * scale;
}

// attn_values_neon, cpu.rs:1463-1509: acc[d] = fma(s[t], v[t][d], acc[d]), t ascending.
void attn_values(const float* scores, const float* vc, float* out, int kv_dim, int off, int hd, int seq) {
    for (int d = 0; d < hd; d++) out[d] = 0.0f;
    for (int t = 0; t < seq; t++) {
        float s = scores[t];
        const float* v = vc + (size_t)t * kv_dim + off;
        for (int d = 0; d < hd; d++) out[d] = fmaf(s, v[d], out[d]);
    }
}

// flash_attention_gqa_neon, cpu.rs:1696-1850, for one (head, query): KV tiles of
// 32, online softmax with ggml_expf, f64 running sum, accumulator rescale, one
// normalisation at the end.  q is the contiguous head vector.
void flash_one(const float* q, const float* kc, const float* vc, float* out, int kv_dim, int off, int hd,
               float scale, int max_kv) {
    const int TILE = 32;  // FLASH_TILE_KV, cpu.rs:1513
    float acc[256];
    float ts[TILE];
    for (int d = 0; d < hd; d++) acc[d] = 0.0f;
    float running_max = -std::numeric_limits<float>::infinity();
    double running_sum = 0.0;
    for (int kv0 = 0; kv0 < max_kv; kv0 += TILE) {
        int len = std::min(TILE, max_kv - kv0);
        for (int ti = 0; ti < len; ti++) ts[ti] = qk_dot_neon_order(q, kc + (size_t)(kv0 + ti) * kv_dim + off, hd) * scale;
        float tmax = -std::numeric_limits<float>::infinity();
        for (int ti = 0; ti < len; ti++)
            if (ts[ti] > tmax) tmax = ts[ti];
        float new_max = std::max(running_max, tmax);
        float rescale = running_max > -std::numeric_limits<float>::infinity() ? ggml_expf(running_max - new_max) : 0.0f;
        double tsum = 0.0;
        for (int ti = 0; ti < len; ti++) {
            ts[ti] = ggml_expf(ts[ti] - new_max);
            tsum += (double)ts[ti];
        }
        for (int d = 0; d < hd; d++) acc[d] = acc[d] * rescale;
        for (int ti = 0; ti < len; ti++) {
            float s = ts[ti];
            const float* v = vc + (size_t)(kv0 + ti) * kv_dim + off;
            for (int d = 0; d < hd; d++) acc[d] = fmaf(s, v[d], acc[d]);
        }
        running_sum = running_sum * (double)rescale + tsum;
        running_max = new_max;
    }
    float inv = (float)(1.0 / running_sum);
    for (int d = 0; d < hd; d++) out[d] = acc[d] * inv;
}

// sampler.rs:8-19: max_by + total_cmp, NaN treated as -inf; the LAST of equal
// maxima wins and +0.0 ranks above -0.0.
inline int32_t total_key(float f) {
    if (f != f) f = -std::numeric_limits<float>::infinity();
    int32_t b; memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
uint32_t argmax(const float* x, int n) {
    int best = 0;
    int32_t bk = 0;
    for (int i = 0; i < n; i++) {
        int32_t k = total_key(x[i]);
        if (i == 0 || k >= bk) { bk = k; best = i; }
    }
    return (uint32_t)best;
}

// quant.rs:78-105, :154-177 (dequantize rows; the embedding lookup lfm2.rs:621-643)
void dequant_row(int dtype, const uint8_t* row, int k, float* out) {
    if (dtype == DT_Q6_K) {  // dequantize_q6_k_block, quant.rs:380-413: d * scale * q, left to right
        for (int bi = 0; bi < k / QK_K; bi++) {
            const uint8_t* blk = row + (size_t)bi * Q6_K_BYTES;
            const uint8_t *ql = blk, *qh = blk + 128;
            const int8_t* sc = (const int8_t*)(blk + 192);
            const float d = f16_to_f32(load_u16(blk + 208));
            float* o = out + (size_t)bi * QK_K;
            for (int n = 0; n < 2; n++)
                for (int l = 0; l < 32; l++) {
                    const int is = l / 16;
                    const uint8_t a = ql[64 * n + l], b = ql[64 * n + l + 32], h = qh[32 * n + l];
                    const int q1 = ((a & 0xF) | ((h & 3) << 4)) - 32, q2 = ((b & 0xF) | (((h >> 2) & 3) << 4)) - 32;
                    const int q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32, q4 = ((b >> 4) | (((h >> 6) & 3) << 4)) - 32;
                    o[128 * n + l] = d * (float)sc[8 * n + is] * (float)q1;
                    o[128 * n + l + 32] = d * (float)sc[8 * n + is + 2] * (float)q2;
                    o[128 * n + l + 64] = d * (float)sc[8 * n + is + 4] * (float)q3;
                    o[128 * n + l + 96] = d * (float)sc[8 * n + is + 6] * (float)q4;
                }
        }
        return;
    }
    int nb = k / QK;
    for (int b = 0; b < nb; b++) {
        const uint8_t* blk = row + (size_t)b * block_bytes(dtype);
        float d = f16_to_f32(load_u16(blk));
        if (dtype == DT_Q4_0) {
            for (int i = 0; i < 16; i++) {
                int lo = (int)(blk[2 + i] & 0x0F) - 8, hi = (int)(blk[2 + i] >> 4) - 8;
                out[b * QK + i] = (float)lo * d;
                out[b * QK + i + 16] = (float)hi * d;
            }
        } else {
            const int8_t* q = (const int8_t*)(blk + 2);
            for (int i = 0; i < QK; i++) out[b * QK + i] = (float)q[i] * d;
        }
    }
}

}  // namespace

// ── Model ──────────────────────────────────────────────────────────────────

extern "C" {
struct OrcWeight {
    const uint8_t* data;
    int32_t dtype, m, k;
};
struct OrcLayer {
    int32_t is_attn, n_kv_heads;
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;
    const float* k_norm;
    const float* conv_w;  // [hidden][kernel]
    OrcWeight in_proj, out_proj, q, k, v, o, gate, up, down;
};
struct OrcModelDesc {
    int32_t n_layers, hidden, ffn, n_heads, vocab, max_seq_len, conv_kernel;
    float rope_theta, eps;
    const float* output_norm;
    OrcWeight embd;
    const OrcLayer* layers;
};
}

namespace {

struct OrcModel {
    OrcModelDesc d;
    std::vector<OrcLayer> layers;
    int seq_len = 0;
    // InferenceState (kv_cache.rs:62-130): f32 K/V per attention layer, time-major
    // [seq][kv_dim]; conv rolling buffer [d_conv][hidden].
    std::vector<std::vector<float>> kc, vc, conv;
    // scratch
    std::vector<float> q8s;
    std::vector<int8_t> q8q;

    int head_dim() const { return d.hidden / d.n_heads; }
};

void gemv_own_quant(OrcModel& M, const OrcWeight& w, const float* x, float* y) {
    // lfm2.rs:469-472 -> cpu::gemv_dispatch(.., None) -> gemv_q*_f32_neon
    // (simd.rs:420-436): quantise x, then the integer GEMV.
    std::vector<float> s(w.k / QK);
    std::vector<int8_t> q(w.k);
    quantize_q8_0(x, w.k, s.data(), q.data());
    gemv_preq(w.dtype, w.data, s.data(), q.data(), y, w.m, w.k);
}

// forward_conv_block, lfm2.rs:646-730.  `M.q8*` hold the quantised normed input.
void conv_block(OrcModel& M, int li, float* out) {
    const OrcLayer& L = M.layers[li];
    int hs = M.d.hidden, ks = M.d.conv_kernel, dc = ks - 1;
    std::vector<float> proj(3 * hs), bx(hs), y(hs);
    gemv_preq(L.in_proj.dtype, L.in_proj.data, M.q8s.data(), M.q8q.data(), proj.data(), L.in_proj.m, L.in_proj.k);
    const float *b = proj.data(), *c = b + hs, *x = c + hs;
    for (int i = 0; i < hs; i++) bx[i] = b[i] * x[i];
    std::vector<float>& buf = M.conv[li];
    for (int ch = 0; ch < hs; ch++) {
        float sum = 0.0f;
        for (int k = 0; k < dc; k++) sum += buf[(size_t)k * hs + ch] * L.conv_w[ch * ks + k];
        sum += bx[ch] * L.conv_w[ch * ks + dc];
        y[ch] = sum;
    }
    if (dc > 0) {
        if (dc > 1) memmove(buf.data(), buf.data() + hs, (size_t)(dc - 1) * hs * sizeof(float));
        memcpy(buf.data() + (size_t)(dc - 1) * hs, bx.data(), hs * sizeof(float));
    }
    for (int i = 0; i < hs; i++) bx[i] = c[i] * y[i];
    gemv_own_quant(M, L.out_proj, bx.data(), out);
}

// Per-head QK RMSNorm + RoPE of one token's q [hs] and k [kv_dim]
// (lfm2.rs:783-802, :1557-1574).
void qk_norm_rope(OrcModel& M, const OrcLayer& L, float* q, float* k, int pos) {
    int hd = M.head_dim();
    for (int h = 0; h < M.d.n_heads; h++) rmsnorm(q + h * hd, L.q_norm, hd, M.d.eps);
    for (int h = 0; h < L.n_kv_heads; h++) rmsnorm(k + h * hd, L.k_norm, hd, M.d.eps);
    for (int h = 0; h < M.d.n_heads; h++) rope_head(q + h * hd, pos, hd, M.d.rope_theta);
    for (int h = 0; h < L.n_kv_heads; h++) rope_head(k + h * hd, pos, hd, M.d.rope_theta);
}

// The naive per-head attention of lfm2.rs:980-1007 / :1857-1897 over the first
// `seq` cached positions.
void naive_attention(OrcModel& M, int li, const float* q, float* attn_out, int seq) {
    const OrcLayer& L = M.layers[li];
    int hd = M.head_dim(), kv_dim = L.n_kv_heads * hd, group = M.d.n_heads / L.n_kv_heads;
    float scale = 1.0f / std::sqrt((float)hd);
    std::vector<float> scores(seq);
    for (int h = 0; h < M.d.n_heads; h++) {
        int off = (h / group) * hd;
        attn_scores(q + h * hd, M.kc[li].data(), scores.data(), kv_dim, off, hd, scale, seq);
        softmax(scores.data(), seq);
        attn_values(scores.data(), M.vc[li].data(), attn_out + h * hd, kv_dim, off, hd, seq);
    }
}

// forward_attn_block, lfm2.rs:733-1017 (f32 KV, no TurboQuant).
void attn_block(OrcModel& M, int li, int pos, float* out) {
    const OrcLayer& L = M.layers[li];
    int hs = M.d.hidden, hd = M.head_dim(), kv_dim = L.n_kv_heads * hd;
    std::vector<float> q(hs), k(kv_dim), v(kv_dim), ao(hs);
    gemv_preq(L.q.dtype, L.q.data, M.q8s.data(), M.q8q.data(), q.data(), L.q.m, L.q.k);
    gemv_preq(L.k.dtype, L.k.data, M.q8s.data(), M.q8q.data(), k.data(), L.k.m, L.k.k);
    gemv_preq(L.v.dtype, L.v.data, M.q8s.data(), M.q8q.data(), v.data(), L.v.m, L.v.k);
    qk_norm_rope(M, L, q.data(), k.data(), pos);
    M.kc[li].insert(M.kc[li].end(), k.begin(), k.end());
    M.vc[li].insert(M.vc[li].end(), v.begin(), v.end());
    int seq = (int)(M.kc[li].size() / kv_dim);
    naive_attention(M, li, q.data(), ao.data(), seq);
    gemv_own_quant(M, L.o, ao.data(), out);
}

void quantize_scratch(OrcModel& M, const float* x, int k) {
    M.q8s.resize(k / QK);
    M.q8q.resize(k);
    quantize_q8_0(x, k, M.q8s.data(), M.q8q.data());
}

// run_layers, lfm2.rs:1020-1124 (aarch64 branch), then the tied-embedding logits
// GEMV of forward(), lfm2.rs:2268-2288.
// `emb` != NULL: forward_from_embedding / forward_hidden_from_embedding (lfm2.rs:2295-2350), the
// input vector replaces the embedding row.
void forward_token(OrcModel& M, uint32_t token, float* logits, float* hidden_out, const float* emb = nullptr) {
    int hs = M.d.hidden, is = M.d.ffn;
    std::vector<float> hidden(hs), normed(hs), out(hs), gate(is), up(is);
    if (emb) memcpy(hidden.data(), emb, hs * sizeof(float));
    else dequant_row(M.d.embd.dtype, M.d.embd.data + (size_t)token * row_bytes(M.d.embd.dtype, hs), hs, hidden.data());
    int pos = M.seq_len;
    for (int i = 0; i < M.d.n_layers; i++) {
        const OrcLayer& L = M.layers[i];
        normed = hidden;
        rmsnorm(normed.data(), L.attn_norm, hs, M.d.eps);
        quantize_scratch(M, normed.data(), hs);
        if (L.is_attn) attn_block(M, i, pos, out.data());
        else conv_block(M, i, out.data());
        for (int j = 0; j < hs; j++) hidden[j] += out[j];
        normed = hidden;
        rmsnorm(normed.data(), L.ffn_norm, hs, M.d.eps);
        quantize_scratch(M, normed.data(), hs);
        gemv_preq(L.gate.dtype, L.gate.data, M.q8s.data(), M.q8q.data(), gate.data(), L.gate.m, L.gate.k);
        gemv_preq(L.up.dtype, L.up.data, M.q8s.data(), M.q8q.data(), up.data(), L.up.m, L.up.k);
        silu_mul(gate.data(), up.data(), is);
        quantize_scratch(M, gate.data(), is);
        gemv_preq(L.down.dtype, L.down.data, M.q8s.data(), M.q8q.data(), out.data(), L.down.m, L.down.k);
        for (int j = 0; j < hs; j++) hidden[j] += out[j];
    }
    rmsnorm(hidden.data(), M.d.output_norm, hs, M.d.eps);
    M.seq_len += 1;
    if (hidden_out) memcpy(hidden_out, hidden.data(), hs * sizeof(float));
    if (logits) {
        quantize_scratch(M, hidden.data(), hs);
        gemv_preq(M.d.embd.dtype, M.d.embd.data, M.q8s.data(), M.q8q.data(), logits, M.d.embd.m, M.d.embd.k);
    }
}

// quantize_columns, lfm2.rs:571-592: every token's vector quantised on its own.
void quantize_tokens(const float* mat, int dim, int n, std::vector<float>& s, std::vector<int8_t>& q) {
    int nb = dim / QK;
    s.resize((size_t)n * nb);
    q.resize((size_t)n * dim);
    par_for(n, n >= 16, [&](int j) { quantize_q8_0(mat + (size_t)j * dim, dim, s.data() + (size_t)j * nb, q.data() + (size_t)j * dim); });
}

// C[n][m] token-major = gemm_preq with swapped output strides.
void gemm_tokens(const OrcWeight& w, const std::vector<float>& s, const std::vector<int8_t>& q, float* out, int n) {
    gemm_preq(w.dtype, w.data, s.data(), q.data(), out, w.m, n, w.k, /*row stride*/ 1, /*col stride*/ (size_t)w.m);
}

// prefill_layers_and_logits, lfm2.rs:1139-2213, aarch64 / non-BLAS branch.
// `emb` != NULL: forward_prefill_from_embeddings (lfm2.rs:2452-2500), row-major frames [n][hs].
void forward_prefill(OrcModel& M, const uint32_t* tokens, int n, int start_pos, float* logits, const float* emb = nullptr) {
    int hs = M.d.hidden, is = M.d.ffn, hd = M.head_dim();
    std::vector<float> hidden((size_t)n * hs), normed((size_t)n * hs), block_out((size_t)n * hs);
    std::vector<float> bs;
    std::vector<int8_t> bq;
    const size_t erb = row_bytes(M.d.embd.dtype, hs);
    // forward_prefill_inner, lfm2.rs:2238-2251
    if (emb) memcpy(hidden.data(), emb, (size_t)n * hs * sizeof(float));
    else
        for (int j = 0; j < n; j++)
            dequant_row(M.d.embd.dtype, M.d.embd.data + (size_t)tokens[j] * erb, hs, hidden.data() + (size_t)j * hs);

    for (int li = 0; li < M.d.n_layers; li++) {
        const OrcLayer& L = M.layers[li];
        normed = hidden;
        par_for(n, n >= 16, [&](int j) { rmsnorm(normed.data() + (size_t)j * hs, L.attn_norm, hs, M.d.eps); });
        quantize_tokens(normed.data(), hs, n, bs, bq);
        std::vector<float> opi((size_t)n * hs);  // out_proj_input
        if (!L.is_attn) {
            // lfm2.rs:1277-1379
            int ks = M.d.conv_kernel, dc = ks - 1;
            std::vector<float> proj((size_t)n * 3 * hs);
            gemm_tokens(L.in_proj, bs, bq, proj.data(), n);
            std::vector<float>& buf = M.conv[li];
            std::vector<float> bx(hs);
            for (int j = 0; j < n; j++) {
                const float *b = proj.data() + (size_t)j * 3 * hs, *c = b + hs, *x = c + hs;
                for (int i = 0; i < hs; i++) bx[i] = b[i] * x[i];
                float* o = opi.data() + (size_t)j * hs;
                for (int ch = 0; ch < hs; ch++) {
                    float sum = 0.0f;
                    for (int k = 0; k < dc; k++) sum += buf[(size_t)k * hs + ch] * L.conv_w[ch * ks + k];
                    sum += bx[ch] * L.conv_w[ch * ks + dc];
                    o[ch] = sum;
                }
                if (dc > 0) {
                    if (dc > 1) memmove(buf.data(), buf.data() + hs, (size_t)(dc - 1) * hs * sizeof(float));
                    memcpy(buf.data() + (size_t)(dc - 1) * hs, bx.data(), hs * sizeof(float));
                }
                for (int i = 0; i < hs; i++) o[i] = c[i] * o[i];
            }
            quantize_tokens(opi.data(), hs, n, bs, bq);
            gemm_tokens(L.out_proj, bs, bq, block_out.data(), n);
        } else {
            // lfm2.rs:1398-1931
            int kv_dim = L.n_kv_heads * hd, group = M.d.n_heads / L.n_kv_heads;
            float scale = 1.0f / std::sqrt((float)hd);
            std::vector<float> qm((size_t)n * hs), km((size_t)n * kv_dim), vm((size_t)n * kv_dim);
            gemm_tokens(L.q, bs, bq, qm.data(), n);
            gemm_tokens(L.k, bs, bq, km.data(), n);
            gemm_tokens(L.v, bs, bq, vm.data(), n);
            // Pass A (lfm2.rs:1544-1623): norm + RoPE, append ALL n tokens to the cache
            for (int j = 0; j < n; j++)
                qk_norm_rope(M, L, qm.data() + (size_t)j * hs, km.data() + (size_t)j * kv_dim, start_pos + j);
            M.kc[li].insert(M.kc[li].end(), km.begin(), km.end());
            M.vc[li].insert(M.vc[li].end(), vm.begin(), vm.end());
            const float* kc = M.kc[li].data();
            const float* vc = M.vc[li].data();
            // Pass B: flash for chunks of >= 256 tokens (lfm2.rs:1646-1647), else naive
            if (n >= 256) {
                par_for(n * M.d.n_heads, true, [&](int idx) {
                    int j = idx / M.d.n_heads, h = idx % M.d.n_heads;
                    flash_one(qm.data() + (size_t)j * hs + h * hd, kc, vc, opi.data() + (size_t)j * hs + h * hd, kv_dim,
                              (h / group) * hd, hd, scale, start_pos + j + 1);
                });
            } else {
                int cached = (int)(M.kc[li].size() / kv_dim);
                par_for(n, n >= 8, [&](int j) {
                    int seq = std::min(start_pos + j + 1, cached);
                    std::vector<float> scores(seq);
                    for (int h = 0; h < M.d.n_heads; h++) {
                        int off = (h / group) * hd;
                        attn_scores(qm.data() + (size_t)j * hs + h * hd, kc, scores.data(), kv_dim, off, hd, scale, seq);
                        softmax(scores.data(), seq);
                        attn_values(scores.data(), vc, opi.data() + (size_t)j * hs + h * hd, kv_dim, off, hd, seq);
                    }
                });
            }
            quantize_tokens(opi.data(), hs, n, bs, bq);
            gemm_tokens(L.o, bs, bq, block_out.data(), n);
        }
        for (size_t i = 0; i < (size_t)n * hs; i++) hidden[i] += block_out[i];

        // FFN, lfm2.rs:2001-2177
        normed = hidden;
        par_for(n, n >= 16, [&](int j) { rmsnorm(normed.data() + (size_t)j * hs, L.ffn_norm, hs, M.d.eps); });
        quantize_tokens(normed.data(), hs, n, bs, bq);
        std::vector<float> gate((size_t)n * is), up((size_t)n * is);
        gemm_tokens(L.gate, bs, bq, gate.data(), n);
        gemm_tokens(L.up, bs, bq, up.data(), n);
        par_for(n, n >= 16, [&](int j) { silu_mul(gate.data() + (size_t)j * is, up.data() + (size_t)j * is, is); });
        quantize_tokens(gate.data(), is, n, bs, bq);
        gemm_tokens(L.down, bs, bq, block_out.data(), n);
        for (size_t i = 0; i < (size_t)n * hs; i++) hidden[i] += block_out[i];
    }
    M.seq_len = start_pos + n;
    // lfm2.rs:2190-2212
    std::vector<float> last(hidden.begin() + (size_t)(n - 1) * hs, hidden.end());
    rmsnorm(last.data(), M.d.output_norm, hs, M.d.eps);
    quantize_scratch(M, last.data(), hs);
    gemv_preq(M.d.embd.dtype, M.d.embd.data, M.q8s.data(), M.q8q.data(), logits, M.d.embd.m, M.d.embd.k);
}

void reset(OrcModel& M) {
    M.seq_len = 0;
    int hs = M.d.hidden;
    for (int i = 0; i < M.d.n_layers; i++) {
        M.kc[i].clear();
        M.vc[i].clear();
        if (!M.layers[i].is_attn) M.conv[i].assign((size_t)(M.d.conv_kernel - 1) * hs, 0.0f);
    }
}

}  // namespace

// ── C ABI (used from Python through ctypes) ────────────────────────────────

ORC_API void orc_set_simd(int on) { g_use_simd = on; }
ORC_API int orc_has_avx2() { return ORC_AVX2; }
ORC_API int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
ORC_API float orc_f16_round(float x) { return f16_to_f32(f32_to_f16(x)); }
ORC_API void orc_quantize_q8_0(const float* x, int k, float* scales, int8_t* quants) { quantize_q8_0(x, k, scales, quants); }
ORC_API void orc_quantize_q8_0_rows(const float* x, int n, int k, float* scales, int8_t* quants) {
    for (int j = 0; j < n; j++) quantize_q8_0(x + (size_t)j * k, k, scales + (size_t)j * (k / QK), quants + (size_t)j * k);
}
ORC_API void orc_gemv(int dtype, const uint8_t* a, const float* xs, const int8_t* xq, float* y, int m, int k) {
    gemv_preq(dtype, a, xs, xq, y, m, k);
}
// out[i*n + j] as in the reference GEMM
ORC_API void orc_gemm(int dtype, const uint8_t* a, const float* bs, const int8_t* bq, float* out, int m, int n, int k) {
    gemm_preq(dtype, a, bs, bq, out, m, n, k, (size_t)n, 1);
}
// whole-block int32 sums S[i][b] and lane sums P[i][b][4] of row i against one column
ORC_API void orc_block_sums(int dtype, const uint8_t* a, const int8_t* xq, int m, int k, int32_t* S, int32_t* P) {
    int nb = k / QK;
    size_t rb = (size_t)nb * block_bytes(dtype);
    for (int i = 0; i < m; i++)
        for (int b = 0; b < nb; b++) {
            int32_t p[4];
            const uint8_t* blk = a + i * rb + (size_t)b * block_bytes(dtype);
            if (dtype == DT_Q4_0) lane_sums_q4_0(blk, xq + b * QK, p);
            else lane_sums_q8_0(blk, xq + b * QK, p);
            if (S) S[(size_t)i * nb + b] = p[0] + p[1] + p[2] + p[3];
            if (P) memcpy(P + ((size_t)i * nb + b) * 4, p, 16);
        }
}
ORC_API void orc_rmsnorm(float* x, const float* w, int n, float eps) { rmsnorm(x, w, n, eps); }
ORC_API void orc_expf(const float* x, float* y, int n) { for (int i = 0; i < n; i++) y[i] = ggml_expf(x[i]); }
ORC_API void orc_silu_mul(float* gate, const float* up, int n) { silu_mul(gate, up, n); }
ORC_API void orc_softmax(float* x, int n) { softmax(x, n); }
ORC_API void orc_rope(float* q, float* k, int pos, int n_heads, int n_kv_heads, int hd, float base) {
    for (int h = 0; h < n_heads; h++) rope_head(q + h * hd, pos, hd, base);
    for (int h = 0; h < n_kv_heads; h++) rope_head(k + h * hd, pos, hd, base);
}
// cos/sin table exactly as rope_head evaluates them: tab[pos][i] = (cos, sin)
ORC_API void orc_rope_table(int n_pos, int hd, float base, float* cos_out, float* sin_out) {
    int half = hd / 2;
    float theta_scale = powf(base, -2.0f / (float)hd);
    for (int p = 0; p < n_pos; p++) {
        float theta = (float)p;
        for (int i = 0; i < half; i++) {
            cos_out[(size_t)p * half + i] = cosf(theta);
            sin_out[(size_t)p * half + i] = sinf(theta);
            theta *= theta_scale;
        }
    }
}
ORC_API void orc_attn_scores(const float* q, const float* kc, float* scores, int kv_dim, int off, int hd, float scale, int seq) {
    attn_scores(q, kc, scores, kv_dim, off, hd, scale, seq);
}
ORC_API void orc_attn_values(const float* scores, const float* vc, float* out, int kv_dim, int off, int hd, int seq) {
    attn_values(scores, vc, out, kv_dim, off, hd, seq);
}
// One head, single query, naive path: scores -> softmax -> values
ORC_API void orc_attention_naive(const float* q, const float* kc, const float* vc, float* out, int kv_dim, int off, int hd,
                                 float scale, int seq) {
    std::vector<float> s(seq);
    attn_scores(q, kc, s.data(), kv_dim, off, hd, scale, seq);
    softmax(s.data(), seq);
    attn_values(s.data(), vc, out, kv_dim, off, hd, seq);
}
// Signature of flash_attention_gqa_cpu (cpu.rs:1538-1552): q_mat is [hs x n] with
// stride q_stride, out is [group][n_queries][hd].
ORC_API void orc_flash_attention_gqa(const float* q_mat, const float* kc, const float* vc, float* out, int n_heads_start,
                                     int group_size, int n_queries, int q_stride, int kv_dim, int kv_h_offset, int hd,
                                     float scale, int start_pos) {
    for (int g = 0; g < group_size; g++) {
        int h = n_heads_start + g;
        for (int j = 0; j < n_queries; j++) {
            float q[256];
            for (int d = 0; d < hd; d++) q[d] = q_mat[(size_t)(h * hd + d) * q_stride + j];
            flash_one(q, kc, vc, out + ((size_t)g * n_queries + j) * hd, kv_dim, kv_h_offset, hd, scale, start_pos + j + 1);
        }
    }
}
ORC_API uint32_t orc_argmax(const float* x, int n) { return argmax(x, n); }
// Sampler::sample (sampler.rs:64-158) with the uniform draw `r` supplied by the caller (wick draws it from `rand`'s
// StdRng; the generator is outside this path).  Works on a copy of the logits.  Ties: top-k keeps every value equal to
// the k-th largest (`*l < threshold` is what gets dropped); top-p orders equal values by ascending index (wick's
// unstable sort leaves their order unspecified, which can only change WHICH of several equal logits is cut).
ORC_API uint32_t orc_sample(const float* logits_in, int n, float temperature, int top_k, float top_p, float r) {
    std::vector<float> logits(logits_in, logits_in + n);
    if (temperature <= 0.0f || top_k == 1) return argmax(logits.data(), n);
    const float inv_temp = 1.0f / temperature;
    for (float& l : logits) l *= inv_temp;
    if (top_k > 0 && top_k < n) {  // apply_top_k, sampler.rs:100-111
        std::vector<float> sorted(logits);
        std::nth_element(sorted.begin(), sorted.begin() + (top_k - 1), sorted.end(), [](float a, float b) { return a > b; });
        const float threshold = sorted[top_k - 1];
        for (float& l : logits)
            if (l < threshold) l = -std::numeric_limits<float>::infinity();
    }
    if (top_p < 1.0f) {  // apply_top_p, sampler.rs:113-145
        std::vector<int> idx;
        for (int i = 0; i < n; i++)
            if (std::isfinite(logits[i])) idx.push_back(i);
        if (!idx.empty()) {
            std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return logits[a] > logits[b]; });
            const float max_val = logits[idx[0]];
            std::vector<float> probs(idx.size());
            for (size_t j = 0; j < idx.size(); j++) probs[j] = expf(logits[idx[j]] - max_val);
            float sum = 0.0f;
            for (float p : probs) sum += p;
            for (float& p : probs) p /= sum;
            size_t cutoff = probs.size();
            float cumsum = 0.0f;
            for (size_t j = 0; j < probs.size(); j++) {
                cumsum += probs[j];
                if (cumsum >= top_p) {
                    cutoff = j + 1;
                    break;
                }
            }
            for (size_t j = cutoff; j < idx.size(); j++) logits[idx[j]] = -std::numeric_limits<float>::infinity();
        }
    }
    softmax(logits.data(), n);  // cpu::softmax_inplace
    float cumsum = 0.0f;          // weighted_sample, sampler.rs:147-158
    for (int i = 0; i < n; i++) {
        cumsum += logits[i];
        if (cumsum >= r) return (uint32_t)i;
    }
    return (uint32_t)(n - 1);
}

ORC_API void orc_dequant_row(int dtype, const uint8_t* row, int k, float* out) { dequant_row(dtype, row, k, out); }

ORC_API void* orc_model_create(const OrcModelDesc* d) {
    OrcModel* M = new OrcModel();
    M->d = *d;
    M->layers.assign(d->layers, d->layers + d->n_layers);
    M->d.layers = M->layers.data();
    M->kc.resize(d->n_layers);
    M->vc.resize(d->n_layers);
    M->conv.resize(d->n_layers);
    reset(*M);
    return M;
}
ORC_API void orc_model_free(void* m) { delete (OrcModel*)m; }
ORC_API void orc_model_reset(void* m) { reset(*(OrcModel*)m); }
ORC_API int orc_model_seq_len(void* m) { return ((OrcModel*)m)->seq_len; }
// Model::forward (lfm2.rs:2258-2289).  `logits` / `hidden` may be NULL.
ORC_API void orc_model_forward(void* m, uint32_t token, float* logits, float* hidden) {
    forward_token(*(OrcModel*)m, token, logits, hidden);
}
// Model::forward_prefill without the prefix cache (lfm2.rs:2220-2254); start_pos == 0
// does NOT reset here, the caller resets, as with a fresh InferenceState.
ORC_API void orc_model_forward_prefill(void* m, const uint32_t* tokens, int n, int start_pos, float* logits) {
    forward_prefill(*(OrcModel*)m, tokens, n, start_pos, logits);
}
// forward_from_embedding (logits) / forward_hidden_from_embedding (hidden), lfm2.rs:2295-2350; either output may be NULL.
ORC_API void orc_model_forward_from_embedding(void* m, const float* emb, float* logits, float* hidden) {
    forward_token(*(OrcModel*)m, 0, logits, hidden, emb);
}
// forward_prefill_from_embeddings, lfm2.rs:2452-2500.
ORC_API void orc_model_forward_prefill_from_embeddings(void* m, const float* emb, int n, int start_pos, float* logits) {
    forward_prefill(*(OrcModel*)m, nullptr, n, start_pos, logits, emb);
}
// Model::shift_kv -> InferenceState::shift_kv_with_rope (lfm2.rs:2507-2516, kv_cache.rs:601-715): drop rows
// [n_keep, n_keep + shift) of every attention layer's K and V, slide the tail down, and rotate the moved K
// rows by R(-shift) (apply_rope_delta_to_head, cpu.rs:2174-2187: iterative theta, libm sin / cos, unfused
// products).  Conv buffers are left alone.  Returns 0, or -1 when the preconditions the reference asserts fail.
ORC_API int orc_model_shift_kv(void* m, int n_keep, int shift) {
    OrcModel& M = *(OrcModel*)m;
    if (shift <= 0 || n_keep < 0 || n_keep + shift > M.seq_len) return -1;
    const int hd = M.head_dim(), half = hd / 2, new_len = M.seq_len - shift;
    const float theta_scale = powf(M.d.rope_theta, -2.0f / (float)hd);
    for (int li = 0; li < M.d.n_layers; li++) {
        const OrcLayer& L = M.layers[li];
        if (!L.is_attn) continue;
        const int kv_dim = L.n_kv_heads * hd;
        std::vector<float>& kc = M.kc[li];
        std::vector<float>& vc = M.vc[li];
        if (kc.empty() && vc.empty()) continue;
        kc.erase(kc.begin() + (size_t)n_keep * kv_dim, kc.begin() + (size_t)(n_keep + shift) * kv_dim);
        vc.erase(vc.begin() + (size_t)n_keep * kv_dim, vc.begin() + (size_t)(n_keep + shift) * kv_dim);
        for (int t = n_keep; t < new_len; t++)
            for (int h = 0; h < L.n_kv_heads; h++) {
                float* head = kc.data() + (size_t)t * kv_dim + (size_t)h * hd;
                float theta = (float)(-shift);
                for (int i = 0; i < half; i++) {
                    const float sn = sinf(theta), cs = cosf(theta);
                    const float x0 = head[i], x1 = head[i + half];
                    head[i] = x0 * cs - x1 * sn;
                    head[i + half] = x0 * sn + x1 * cs;
                    theta *= theta_scale;
                }
            }
    }
    M.seq_len = new_len;
    return 0;
}
// Greedy decode loop as Session::generate drives it (session.rs:1186-1257): feeds
// `first`, writes n_steps argmax tokens.
ORC_API void orc_model_generate_greedy(void* m, uint32_t first, int n_steps, uint32_t* out_tokens) {
    OrcModel& M = *(OrcModel*)m;
    std::vector<float> logits(M.d.vocab);
    uint32_t tok = first;
    for (int i = 0; i < n_steps; i++) {
        forward_token(M, tok, logits.data(), nullptr);
        tok = argmax(logits.data(), M.d.vocab);
        out_tokens[i] = tok;
    }
}
ORC_API int orc_model_kv_rows(void* m, int layer) {
    OrcModel& M = *(OrcModel*)m;
    const OrcLayer& L = M.layers[layer];
    if (!L.is_attn) return 0;
    return (int)(M.kc[layer].size() / (L.n_kv_heads * M.head_dim()));
}
ORC_API void orc_model_get_kv(void* m, int layer, float* k_out, float* v_out) {
    OrcModel& M = *(OrcModel*)m;
    memcpy(k_out, M.kc[layer].data(), M.kc[layer].size() * sizeof(float));
    memcpy(v_out, M.vc[layer].data(), M.vc[layer].size() * sizeof(float));
}
ORC_API void orc_model_get_conv_state(void* m, int layer, float* out) {
    OrcModel& M = *(OrcModel*)m;
    memcpy(out, M.conv[layer].data(), M.conv[layer].size() * sizeof(float));
}
