// Element-wise / normalisation / short-conv / argmax kernels of the LFM2 hot path.
#include "kernels.cuh"

namespace wick {

thread_local unsigned long long g_kernel_launches = 0;

// ── weight re-layout ───────────────────────────────────────────────────────
// GGUF block = f16 d followed by 16 (Q4_0) or 32 (Q8_0) quant bytes, 18 / 34 bytes,
// only 2-byte aligned (wick/src/quant.rs:13-34).  One thread moves one block of one row into
// the grouped layout described at DevWeight.  The planes are zero-filled first (padding rows).
__global__ void k_repack(DevWeight w, const uint8_t* __restrict__ raw, uint8_t* __restrict__ q, __half* __restrict__ d) {
    const int nb = w.k / QK;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)w.m * nb) return;
    const int row = (int)(idx / nb), b = (int)(idx % nb);
    const int g = row >> 2, r = row & 3;
    const int qb = w.dtype == DT_Q4_0 ? 16 : 32;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(raw + idx * (size_t)(qb + 2));
    reinterpret_cast<uint16_t*>(d)[(size_t)g * nb * 4 + b * 4 + r] = src[0];
    uint16_t* qg = reinterpret_cast<uint16_t*>(q + (size_t)g * w.q_group_bytes());
    if (w.dtype == DT_Q4_0) {
        for (int i = 0; i < 8; i++) qg[q4_word(b, r, 0) * 2 + i] = src[1 + i];
    } else {
        for (int i = 0; i < 8; i++) qg[q8_word(b, 0, r, 0) * 2 + i] = src[1 + i];
        for (int i = 0; i < 8; i++) qg[q8_word(b, 1, r, 0) * 2 + i] = src[9 + i];
    }
}

void launch_repack(cudaStream_t st, const DevWeight& w, const uint8_t* raw, uint8_t* q, __half* d) {
    size_t n_blocks = (size_t)w.m * (w.k / QK);
    if (!n_blocks) return;
    cudaMemsetAsync(q, 0, w.q_bytes(), st);
    cudaMemsetAsync(d, 0, w.d_bytes(), st);
    unsigned grid = (unsigned)((n_blocks + 255) / 256);
    g_kernel_launches++;
    k_repack<<<grid, 256, 0, st>>>(w, raw, q, d);
}

// ── embedding ──────────────────────────────────────────────────────────────
__global__ void k_embed(DevWeight w, const uint32_t* __restrict__ tokens, const DecodeCtl* __restrict__ ctl,
                        float* __restrict__ out) {
    int j = blockIdx.x;
    uint32_t tok = tokens ? tokens[j] : ctl->token;
    if (tok >= (uint32_t)w.m) tok = 0;  // host validates ids; never index outside the table
    const int k = w.k, nb = k / QK;
    const int g = tok >> 2, r = tok & 3;
    const __half* dg = w.d + (size_t)g * nb * 4;
    const uint8_t* qg = w.q + (size_t)g * w.q_group_bytes();
    for (int e = threadIdx.x; e < k; e += blockDim.x) {
        int b = e >> 5, i = e & 31;
        float d = __half2float(dg[b * 4 + r]);
        int v;
        if (w.dtype == DT_Q4_0) {
            uint8_t byte = qg[q4_word(b, r, 0) * 4 + (i & 15)];
            v = (int)(i < 16 ? (byte & 0x0F) : (byte >> 4)) - 8;
        } else {
            v = (int)((const int8_t*)qg)[q8_word(b, i >> 4, r, 0) * 4 + (i & 15)];
        }
        out[(size_t)j * k + e] = __fmul_rn((float)v, d);
    }
}

void launch_embed(cudaStream_t st, const DevWeight& w, const uint32_t* tokens, const DecodeCtl* ctl, float* out, int n) {
    g_kernel_launches++;
    k_embed<<<n, 256, 0, st>>>(w, tokens, ctl, out);
}

// ── residual add + RMSNorm + Q8_0 quantise ─────────────────────────────────
__global__ void __launch_bounds__(256) k_add_rmsnorm_quant(float* __restrict__ hidden, const float* __restrict__ add,
                                                          const float* __restrict__ weight, float eps, int dim,
                                                          float* __restrict__ q8s, int8_t* __restrict__ q8q,
                                                          float* __restrict__ normed_out) {
    extern __shared__ float xs[];
    __shared__ double red[32];
    const int row = blockIdx.x;
    float* h = hidden + (size_t)row * dim;
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {  // dim is a multiple of 32
        float4 v = *reinterpret_cast<const float4*>(h + i);
        if (add) {
            const float4 a = *reinterpret_cast<const float4*>(add + (size_t)row * dim + i);  // cpu::add_inplace, cpu.rs:2230-2235
            v = make_float4(__fadd_rn(v.x, a.x), __fadd_rn(v.y, a.y), __fadd_rn(v.z, a.z), __fadd_rn(v.w, a.w));
            *reinterpret_cast<float4*>(h + i) = v;
        }
        *reinterpret_cast<float4*>(xs + i) = v;
    }
    __syncthreads();
    double sum_sq = block_sum_sq_f64(xs, dim, red);
    double mean = sum_sq / (double)dim;
    float inv = (float)(1.0 / sqrt(mean + (double)eps));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int nb = dim / QK;
    // four blocks per warp and pass: 8 lanes per block, 4 consecutive elements per lane
    for (int b0 = warp * 4; b0 < nb; b0 += nw * 4) {
        const int b = b0 + (lane >> 3);
        const bool in = b < nb;
        const int i = b * QK + (lane & 7) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in) {
            const float4 x = *reinterpret_cast<const float4*>(xs + i);
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight + i));
            v = make_float4(__fmul_rn(__fmul_rn(x.x, inv), w.x), __fmul_rn(__fmul_rn(x.y, inv), w.y), __fmul_rn(__fmul_rn(x.z, inv), w.z),
                            __fmul_rn(__fmul_rn(x.w, inv), w.w));
            if (normed_out) *reinterpret_cast<float4*>(normed_out + (size_t)row * dim + i) = v;
        }
        if (q8q) {
            float sc;
            const uint32_t q = quantize_lane4(v, &sc);
            if (in) {
                *reinterpret_cast<uint32_t*>(q8q + (size_t)row * dim + i) = q;
                if ((lane & 7) == 0) q8s[(size_t)row * nb + b] = sc;
            }
        }
    }
}

void launch_add_rmsnorm_quant(cudaStream_t st, float* hidden, const float* add, const float* weight, float eps, int n,
                              int dim, float* q8s, int8_t* q8q, float* normed_out) {
    g_kernel_launches++;
    k_add_rmsnorm_quant<<<n, 256, dim * sizeof(float), st>>>(hidden, add, weight, eps, dim, q8s, q8q, normed_out);
}

__global__ void __launch_bounds__(256) k_rmsnorm_generic(float* __restrict__ x, const float* __restrict__ weight, int dim,
                                                        float eps) {
    __shared__ double red[32];
    float* h = x + (size_t)blockIdx.x * dim;
    double sum_sq = block_sum_sq_f64(h, dim, red);
    float inv = (float)(1.0 / sqrt(sum_sq / (double)dim + (double)eps));
    for (int i = threadIdx.x; i < dim; i += blockDim.x) h[i] = __fmul_rn(__fmul_rn(h[i], inv), weight[i]);
}

void launch_rmsnorm(cudaStream_t st, float* x, const float* weight, int n, int dim, float eps) {
    g_kernel_launches++;
    k_rmsnorm_generic<<<n, 256, 0, st>>>(x, weight, dim, eps);
}

// ── plain Q8_0 quantisation of rows ────────────────────────────────────────
__global__ void k_quant_rows(const float* __restrict__ x, size_t total_blocks, float* __restrict__ q8s,
                             int8_t* __restrict__ q8q) {
    // 8 lanes per block, 4 consecutive elements per lane; lanes past the end still take part in the shuffles
    const size_t gt = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t b = gt >> 3;
    const bool in = b < total_blocks;
    const size_t i = gt * 4;
    const float4 v = in ? *reinterpret_cast<const float4*>(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    float sc;
    const uint32_t q = quantize_lane4(v, &sc);
    if (in) {
        *reinterpret_cast<uint32_t*>(q8q + i) = q;
        if ((threadIdx.x & 7) == 0) q8s[b] = sc;
    }
}

void launch_quant_rows(cudaStream_t st, const float* x, int n, int k, float* q8s, int8_t* q8q) {
    size_t total = (size_t)n * (k / QK);
    if (!total) return;
    unsigned grid = (unsigned)((total * 8 + 255) / 256);
    g_kernel_launches++;
    k_quant_rows<<<grid, 256, 0, st>>>(x, total, q8s, q8q);
}

// ── SwiGLU + quantise ──────────────────────────────────────────────────────
__global__ void k_silu_mul_quant(const float* __restrict__ gate, const float* __restrict__ up, size_t total_blocks,
                                 float* __restrict__ q8s, int8_t* __restrict__ q8q, float* __restrict__ act_out) {
    const size_t gt = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t b = gt >> 3;
    const bool in = b < total_blocks;
    const size_t i = gt * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (in) {
        const float4 g = *reinterpret_cast<const float4*>(gate + i), u = *reinterpret_cast<const float4*>(up + i);
        a = make_float4(silu_mul_elem(g.x, u.x), silu_mul_elem(g.y, u.y), silu_mul_elem(g.z, u.z), silu_mul_elem(g.w, u.w));
        if (act_out) *reinterpret_cast<float4*>(act_out + i) = a;
    }
    float sc;
    const uint32_t q = quantize_lane4(a, &sc);
    if (in) {
        *reinterpret_cast<uint32_t*>(q8q + i) = q;
        if ((threadIdx.x & 7) == 0) q8s[b] = sc;
    }
}

void launch_silu_mul_quant(cudaStream_t st, const float* gate, const float* up, int n, int dim, float* q8s, int8_t* q8q,
                           float* act_out) {
    size_t total = (size_t)n * (dim / QK);
    if (!total) return;
    unsigned grid = (unsigned)((total * 8 + 255) / 256);
    g_kernel_launches++;
    k_silu_mul_quant<<<grid, 256, 0, st>>>(gate, up, total, q8s, q8q, act_out);
}

__global__ void k_silu_mul(float* __restrict__ gate, const float* __restrict__ up, size_t count) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) gate[i] = silu_mul_elem(gate[i], up[i]);
}
void launch_silu_mul(cudaStream_t st, float* gate, const float* up, size_t count) {
    if (!count) return;
    g_kernel_launches++;
    k_silu_mul<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(gate, up, count);
}
__global__ void k_expf(const float* __restrict__ x, float* __restrict__ y, size_t count) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) y[i] = ggml_expf(x[i]);
}
void launch_expf(cudaStream_t st, const float* x, float* y, size_t count) {
    if (!count) return;
    g_kernel_launches++;
    k_expf<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(x, y, count);
}

// ── gated short conv ───────────────────────────────────────────────────────
// forward_conv_block core, lfm2.rs:688-725 (batched twin :1316-1354).  For token j the
// rolling buffer slot k holds bx[j - d_conv + k], or the incoming state for the first
// d_conv tokens, so every (token, channel) is independent given the incoming state:
//   y = 0 + S_0*w_0 + ... + S_{dc-1}*w_{dc-1} + bx_j*w_dc     (products and adds rounded one by one)
//   out = c * y
// A warp owns 32 consecutive channels of one token = one Q8_0 block of the out_proj input.
__global__ void k_shortconv(const float* __restrict__ proj, const float* __restrict__ conv_w,
                            const float* __restrict__ state, int n, int hs, int ks, float* __restrict__ out,
                            float* __restrict__ q8s, int8_t* __restrict__ q8q) {
    const int dc = ks - 1;
    size_t gw = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    int bpr = hs / QK;
    if (gw >= (size_t)n * bpr) return;
    int j = (int)(gw / bpr), ch = (int)(gw % bpr) * QK + lane;
    const float* pj = proj + (size_t)j * 3 * hs;
    float sum = 0.0f;
    for (int k = 0; k < dc; k++) {
        int src = j - dc + k;
        float s;
        if (src >= 0) {
            const float* ps = proj + (size_t)src * 3 * hs;
            s = __fmul_rn(ps[ch], ps[2 * hs + ch]);
        } else {
            s = state[(size_t)(k + j) * hs + ch];
        }
        sum = __fadd_rn(sum, __fmul_rn(s, conv_w[ch * ks + k]));
    }
    float bx = __fmul_rn(pj[ch], pj[2 * hs + ch]);
    sum = __fadd_rn(sum, __fmul_rn(bx, conv_w[ch * ks + dc]));
    float o = __fmul_rn(pj[hs + ch], sum);
    if (out) out[(size_t)j * hs + ch] = o;
    if (q8q) {
        float sc;
        int8_t q = quantize_lane(o, &sc);
        q8q[(size_t)j * hs + ch] = q;
        if (lane == 0) q8s[gw] = sc;
    }
}

// State after n tokens: slot k <- bx[n - dc + k], or the old slot k + n while that is still
// inside the old buffer (n < d_conv).  One thread per channel, ascending k, so the in-place
// shift never reads a slot it already overwrote.
__global__ void k_shortconv_state(const float* __restrict__ proj, float* __restrict__ state, int n, int hs, int ks) {
    const int dc = ks - 1;
    int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= hs) return;
    for (int k = 0; k < dc; k++) {
        int src = n - dc + k;
        float s;
        if (src >= 0) {
            const float* ps = proj + (size_t)src * 3 * hs;
            s = __fmul_rn(ps[ch], ps[2 * hs + ch]);
        } else {
            s = state[(size_t)(k + n) * hs + ch];
        }
        state[(size_t)k * hs + ch] = s;
    }
}

void launch_shortconv(cudaStream_t st, const float* proj, const float* conv_w, float* state, int n, int hs, int ks,
                      float* out, float* q8s, int8_t* q8q) {
    size_t warps = (size_t)n * (hs / QK);
    if (!warps) return;
    g_kernel_launches++;
    k_shortconv<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(proj, conv_w, state, n, hs, ks, out, q8s, q8q);
    if (ks > 1) g_kernel_launches++, k_shortconv_state<<<(hs + 255) / 256, 256, 0, st>>>(proj, state, n, hs, ks);
}

// ── per-head QK RMSNorm + RoPE + KV append ─────────────────────────────────
// lfm2.rs:783-855.  One warp per (token, head).  The 64-element sum of squares is added
// in element order in f64 exactly like cpu::rmsnorm (every lane does it redundantly).
// RoPE pairs are (i, i + hd/2) with cos/sin from a table the host fills with libm in the
// reference's iteration order (cpu.rs:2145-2158).
__global__ void __launch_bounds__(32) k_qknorm_rope_kv(float* __restrict__ q, const float* __restrict__ k,
                                                      const float* __restrict__ v, const float* __restrict__ q_norm,
                                                      const float* __restrict__ k_norm, float eps,
                                                      const float* __restrict__ rope_cos,
                                                      const float* __restrict__ rope_sin, float* __restrict__ k_cache,
                                                      float* __restrict__ v_cache, int start_pos,
                                                      const DecodeCtl* __restrict__ ctl, int n_heads, int n_kv_heads,
                                                      int hd) {
    __shared__ float xs[256];
    const int j = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int hs = n_heads * hd, kv_dim = n_kv_heads * hd, half = hd / 2;
    const int pos = (start_pos >= 0 ? start_pos : (int)ctl->pos) + j;
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
    float inv = (float)(1.0 / sqrt(sum_sq / (double)hd + (double)eps));
    float* dst = is_q ? q + (size_t)j * hs + h * hd : k_cache + (size_t)pos * kv_dim + h * hd;
    for (int i = lane; i < half; i += 32) {
        float x0 = __fmul_rn(__fmul_rn(xs[i], inv), w[i]);
        float x1 = __fmul_rn(__fmul_rn(xs[i + half], inv), w[i + half]);
        float c = rope_cos[(size_t)pos * half + i], s = rope_sin[(size_t)pos * half + i];
        dst[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        dst[i + half] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    if (!is_q) {
        const float* vs = v + (size_t)j * kv_dim + h * hd;
        float* vd = v_cache + (size_t)pos * kv_dim + h * hd;
        for (int i = lane; i < hd; i += 32) vd[i] = vs[i];
    }
}

void launch_qknorm_rope_kv(cudaStream_t st, float* q, const float* k, const float* v, const float* q_norm,
                           const float* k_norm, float eps, const float* rope_cos, const float* rope_sin, float* k_cache,
                           float* v_cache, int n, int start_pos, const DecodeCtl* ctl, int n_heads, int n_kv_heads,
                           int head_dim) {
    dim3 grid(n, n_heads + n_kv_heads);
    g_kernel_launches++;
    k_qknorm_rope_kv<<<grid, 32, 0, st>>>(q, k, v, q_norm, k_norm, eps, rope_cos, rope_sin, k_cache, v_cache, start_pos,
                                          ctl, n_heads, n_kv_heads, head_dim);
}

__global__ void k_rope(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ cos_row,
                       const float* __restrict__ sin_row, int n_heads, int hd) {
    int head = blockIdx.x, half = hd / 2;
    float* p = head < n_heads ? q + (size_t)head * hd : k + (size_t)(head - n_heads) * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float x0 = p[i], x1 = p[i + half], c = cos_row[i], s = sin_row[i];
        p[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        p[i + half] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
}
void launch_rope(cudaStream_t st, float* q, float* k, const float* cos_row, const float* sin_row, int n_heads,
                 int n_kv_heads, int head_dim) {
    g_kernel_launches++;
    k_rope<<<n_heads + n_kv_heads, 32, 0, st>>>(q, k, cos_row, sin_row, n_heads, head_dim);
}

// ── argmax ─────────────────────────────────────────────────────────────────
__global__ void k_argmax_partial(const float* __restrict__ x, int count, unsigned long long* __restrict__ acc) {
    unsigned long long best = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
        unsigned long long p = argmax_pack(x[i], (uint32_t)i);
        best = p > best ? p : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) atomicMax(acc, best);
}
__global__ void k_argmax_finish(unsigned long long* __restrict__ acc, uint32_t* __restrict__ out) {
    *out = (uint32_t)(*acc & 0xffffffffull);
    *acc = 0;
}
void launch_argmax(cudaStream_t st, const float* logits, int count, unsigned long long* scratch, uint32_t* out) {
    int grid = (count + 1023) / 1024;
    if (grid > 148) grid = 148;
    if (grid < 1) grid = 1;
    g_kernel_launches++;
    k_argmax_partial<<<grid, 256, 0, st>>>(logits, count, scratch);
    g_kernel_launches++;
    k_argmax_finish<<<1, 1, 0, st>>>(scratch, out);
}

__global__ void k_decode_advance(DecodeCtl* __restrict__ ctl, const uint32_t* __restrict__ argmax_tok,
                                 uint32_t* __restrict__ ring, int ring_len) {
    uint32_t t = *argmax_tok;
    ctl->token = t;
    ctl->pos += 1;
    if (ring) ring[ctl->step % (uint32_t)ring_len] = t;
    ctl->step += 1;
}
void launch_decode_advance(cudaStream_t st, DecodeCtl* ctl, const uint32_t* argmax_tok, uint32_t* ring, int ring_len) {
    g_kernel_launches++;
    k_decode_advance<<<1, 1, 0, st>>>(ctl, argmax_tok, ring, ring_len);
}

// ── n_keep context shift ────────────────────────────────────────────────────
// Rows [row0, row0 + rows) of a K or V cache, read `shift` rows further up, into a dense scratch
// [rows][kv_dim]; K rows are rotated by R(-shift) on the way (apply_rope_delta_to_head, cpu.rs:2174-2187:
// unfused products, pair (i, i + hd/2)); cd / sd == NULL: plain copy (V).
__global__ void k_kv_shift_gather(const float* __restrict__ cache, float* __restrict__ scratch, int row0, int rows, int shift,
                                  int kv_dim, int hd, const float* __restrict__ cd, const float* __restrict__ sd) {
    const int half = hd / 2, pairs_per_row = kv_dim / 2;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * pairs_per_row) return;
    const int r = (int)(idx / pairs_per_row), pr = (int)(idx % pairs_per_row);
    const int h = pr / half, i = pr % half;
    const float* src = cache + (size_t)(row0 + r + shift) * kv_dim + (size_t)h * hd;
    float* dst = scratch + (size_t)r * kv_dim + (size_t)h * hd;
    const float x0 = src[i], x1 = src[i + half];
    if (cd) {
        const float c = cd[i], sn = sd[i];
        dst[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
        dst[i + half] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
    } else {
        dst[i] = x0;
        dst[i + half] = x1;
    }
}

void launch_kv_shift_gather(cudaStream_t st, const float* cache, float* scratch, int row0, int rows, int shift, int kv_dim, int hd,
                            const float* cos_delta, const float* sin_delta) {
    const size_t n = (size_t)rows * (kv_dim / 2);
    if (!n) return;
    g_kernel_launches++;
    k_kv_shift_gather<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(cache, scratch, row0, rows, shift, kv_dim, hd, cos_delta, sin_delta);
}

}  // namespace wick
