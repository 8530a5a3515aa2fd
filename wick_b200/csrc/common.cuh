// Shared device helpers.  This library is compiled with --fmad=false: the CPU path
// it must agree with bit for bit never contracts a*b+c, so every fused multiply-add
// in these kernels is an explicit fmaf()/__fmaf_rn() that mirrors an explicit NEON
// vfmaq_f32 in wick (wick/src/backend/cpu.rs:1440-1441, :1491, :1831).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wick {

constexpr int QK = 32;         // elements per quantised block
constexpr int DT_Q4_0 = 2;     // ggml type ids (wick/src/gguf.rs:38, :42)
constexpr int DT_Q8_0 = 8;

// A quantised matrix in the library's device layout.  Same bytes as the GGUF blocks
// (wick/src/quant.rs:13-34: f16 scale + 16 nibble bytes, or + 32 int8), re-ordered once at
// load time so that the eight accumulation chains of four consecutive rows sit next to each
// other: rows are taken in groups of four and, inside a group, the quant words are stored
// block-major.  With (r = row in group, l = 32-bit word of the lane, p = block parity):
//   Q4_0 quant plane : word  b*16 + r*4 + l                    (16 bytes per row per block)
//   Q8_0 quant plane : word  (b/2)*64 + half*32 + p*16 + r*4 + l   (half 0 = elements 0..15)
//   scale plane      : f16   b*4 + r
// A warp whose lanes are (p, r, l) therefore reads 128 contiguous bytes per step, from
// global or shared memory alike (no bank conflicts), and any run of whole groups is one
// contiguous, 16-byte aligned byte range that a single bulk copy can fetch.
// m is padded to a multiple of 4 with zero rows; for Q8_0 an odd block count is padded to even.
struct DevWeight {
    const uint8_t* q = nullptr;
    const __half* d = nullptr;
    int m = 0, k = 0, dtype = 0;
    __host__ __device__ int nb() const { return k / QK; }
    __host__ __device__ int groups() const { return (m + 3) / 4; }
    // bytes of one 4-row group in each plane
    __host__ __device__ size_t q_group_bytes() const {
        return dtype == DT_Q4_0 ? (size_t)nb() * 64 : (size_t)((nb() + 1) / 2) * 256;
    }
    __host__ __device__ size_t d_group_bytes() const { return (size_t)nb() * 8; }
    size_t q_bytes() const { return (size_t)groups() * q_group_bytes(); }
    size_t d_bytes() const { return (size_t)groups() * d_group_bytes(); }
};

// token_embd stored as Q6_K (ggml type 14; BlockQ6K, wick/src/quant.rs:63-70: 256 elements in ql[128] low
// nibbles, qh[64] high bit pairs, 16 int8 sub-block scales, f16 d).  The 210-byte blocks are only 2-byte
// aligned, so the four fields are split into planes at load; every row of every plane then starts on a
// 16-byte boundary (k is a multiple of 256).
constexpr int DT_Q6_K = 14;
constexpr int QK_K = 256;
struct DevQ6K {
    const uint8_t* ql = nullptr;  // [m][k/2]
    const uint8_t* qh = nullptr;  // [m][k/4]
    const int8_t* sc = nullptr;   // [m][k/16]
    const __half* d = nullptr;    // [m][k/256]
    int m = 0, k = 0;
    size_t bytes() const { return (size_t)m * (k / 2 + k / 4 + k / 16 + k / 256 * 2); }
};

// Element e of a row: quant.rs:393-410.  Within a super-block, pass n = (e % 256) / 128, r = e % 128,
// j = r / 32 selects (ql half, nibble, qh bit pair), l = r % 32; scale index 8n + l/16 + 2j.
__device__ __forceinline__ float q6k_elem(const DevQ6K& w, size_t row, int e) {
    const int k = w.k, bi = e >> 8, n = (e >> 7) & 1, r = e & 127, j = r >> 5, l = r & 31;
    const uint8_t* ql = w.ql + row * (size_t)(k / 2) + (size_t)bi * 128 + 64 * n + l + ((j & 1) ? 32 : 0);
    const uint8_t h = w.qh[row * (size_t)(k / 4) + (size_t)bi * 64 + 32 * n + l];
    const int nib = j < 2 ? (*ql & 0x0F) : (*ql >> 4);
    const int q = (nib | (((h >> (2 * j)) & 3) << 4)) - 32;
    const float d = __half2float(w.d[row * (size_t)(k / QK_K) + bi]);
    const float s = (float)w.sc[row * (size_t)(k / 16) + (size_t)bi * 16 + 8 * n + (l >> 4) + 2 * j];
    return __fmul_rn(__fmul_rn(d, s), (float)q);
}

// Word offsets inside a group (see DevWeight).
__host__ __device__ __forceinline__ int q4_word(int b, int r, int l) { return b * 16 + r * 4 + l; }
__host__ __device__ __forceinline__ int q8_word(int b, int half, int r, int l) {
    return (b >> 1) * 64 + half * 32 + (b & 1) * 16 + r * 4 + l;
}

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }

// ggml_expf, wick/src/backend/cpu.rs:602-642.  Plain f32 mul/add (the file is built
// without FMA contraction).
__device__ __forceinline__ float ggml_expf(float x) {
    const float R = __uint_as_float(0x4B400000u);
    const float LOG2E = __uint_as_float(0x3FB8AA3Bu);
    const float LN2_HI = __uint_as_float(0x3F317200u);
    const float LN2_LO = __uint_as_float(0x35BFBE8Eu);
    const float C1 = __uint_as_float(0x3F7FFFF6u);
    const float C2 = __uint_as_float(0x3EFFFEDBu);
    const float C3 = __uint_as_float(0x3E2AAF33u);
    const float C4 = __uint_as_float(0x3D2B9F17u);
    const float C5 = __uint_as_float(0x3C072010u);
    float z = __fadd_rn(R, __fmul_rn(x, LOG2E));
    float n = __fsub_rn(z, R);
    float b = __fsub_rn(__fsub_rn(x, __fmul_rn(n, LN2_HI)), __fmul_rn(n, LN2_LO));
    uint32_t e = __float_as_uint(z) << 23;
    float k = __uint_as_float(e + 0x3F800000u);
    float u = __fmul_rn(b, b);
    float t45 = __fadd_rn(C4, __fmul_rn(C5, b));
    float t23 = __fadd_rn(__fadd_rn(C2, __fmul_rn(C3, b)), __fmul_rn(t45, u));
    float j = __fadd_rn(__fmul_rn(C1, b), __fmul_rn(t23, u));
    float abs_n = fabsf(n);
    if (abs_n <= 126.0f) {
        return __fadd_rn(k, __fmul_rn(j, k));
    } else if (abs_n > 192.0f) {
        return n > 0.0f ? __int_as_float(0x7F800000) : 0.0f;
    } else {
        uint32_t d = n <= 0.0f ? 0x82000000u : 0u;
        float s1 = __uint_as_float(d + 0x7f000000u);
        float s2 = __uint_as_float(e - d);
        return __fmul_rn(__fadd_rn(s2, __fmul_rn(s2, j)), s1);
    }
}

// silu_mul_inplace element, cpu.rs:668-673: g / (1 + expf(-g)) * u
__device__ __forceinline__ float silu_mul_elem(float g, float u) {
    float e = ggml_expf(-g);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
}

// The Q8_0 activation quantiser for one 32-element block held one element per lane
// (wick/src/backend/simd.rs:255-323).  Returns the quant; *scale is the f16-rounded d.
__device__ __forceinline__ int8_t quantize_lane(float v, float* scale) {
    float a = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float d = __fdiv_rn(a, 127.0f);
    float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    *scale = __half2float(__float2half_rn(d));
    return (int8_t)__float2int_rn(__fmul_rn(v, id));
}

// The same quantiser with four consecutive elements per lane: a block is held by 8 consecutive lanes (lane & ~7 ..),
// a warp carries four blocks.  Every lane of the warp must call it (full-mask shuffles); returns the four quants
// packed little-endian.  One pair of IEEE divisions serves four elements instead of one.
__device__ __forceinline__ uint32_t quantize_lane4(float4 v, float* scale) {
    float a = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    const float d = __fdiv_rn(a, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    *scale = __half2float(__float2half_rn(d));
    const uint32_t q0 = (uint32_t)__float2int_rn(__fmul_rn(v.x, id)) & 0xFFu, q1 = (uint32_t)__float2int_rn(__fmul_rn(v.y, id)) & 0xFFu;
    const uint32_t q2 = (uint32_t)__float2int_rn(__fmul_rn(v.z, id)) & 0xFFu, q3 = (uint32_t)__float2int_rn(__fmul_rn(v.w, id)) & 0xFFu;
    return q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
}

// cpu_argmax ordering (wick/src/sampler.rs:8-19): total_cmp with NaN as -inf; packing the
// index below the key makes "largest key, then largest index" a plain u64 max.
__device__ __forceinline__ unsigned long long argmax_pack(float f, uint32_t idx) {
    if (f != f) f = __int_as_float(0xFF800000);
    int32_t b = __float_as_int(f);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    uint32_t key = (uint32_t)b ^ 0x80000000u;
    return ((unsigned long long)key << 32) | idx;
}

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum of squares of x[0..n) in f64 (cpu::rmsnorm, cpu.rs:583-586).  The reference adds
// in element order; here each thread adds its strided share in order and the partials are
// combined in a fixed tree, which can differ from the serial sum by a few f64 ulps (~1e-15
// relative) -- far below the f32 rounding of the result it feeds.  All threads get the sum.
__device__ __forceinline__ double block_sum_sq_f64(const float* x, int n, double* red /*>=32*/) {
    double s = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        double v = (double)x[i];
        s += v * v;
    }
    s = warp_sum_f64(s);
    int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if ((threadIdx.x & 31) == 0) red[w] = s;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; i++) t += red[i];
    __syncthreads();
    return t;
}

}  // namespace wick
