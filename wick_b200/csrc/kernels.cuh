// Launch wrappers of the CUDA kernels (definitions in kernels_*.cu).  All are
// asynchronous on `st`.  Activations are token-major: [n tokens][dim].
#pragma once
#include "common.cuh"

namespace wick {

// Number of kernels launched by the launch_* wrappers on this host thread (also counts launches
// recorded into a stream capture).
extern thread_local unsigned long long g_kernel_launches;

// Device-resident control block of the decode step: lets one captured CUDA graph
// serve every position (kernels read the token and position from here).
struct DecodeCtl {
    uint32_t token;      // token to embed this step
    uint32_t pos;        // its position == number of cached rows before the step
    uint32_t step;       // index into the generated-token ring
    uint32_t error;      // sticky device-side error flags
    unsigned long long argmax;  // packed (key, index) accumulator of the argmax kernels
};

// Re-layout of GGUF block rows into the quant / scale planes of DevWeight.
void launch_repack(cudaStream_t st, const DevWeight& w, const uint8_t* raw, uint8_t* q, __half* d);

// Embedding rows: out[j][:] = dequantised row tokens[j] (quant.rs:78-105, :154-177).
// tokens may be a device array, or NULL to read the single token from ctl.
void launch_embed(cudaStream_t st, const DevWeight& w, const uint32_t* tokens, const DecodeCtl* ctl, float* out, int n);

// Optional residual add (hidden += add), RMSNorm (cpu.rs:577-594) and Q8_0 quantisation
// (simd.rs:255-323) of n rows.  normed_out (f32) is optional.
void launch_add_rmsnorm_quant(cudaStream_t st, float* hidden, const float* add, const float* weight, float eps,
                              int n, int dim, float* q8s, int8_t* q8q, float* normed_out);
// In-place RMSNorm of n rows (operator entry point).
void launch_rmsnorm(cudaStream_t st, float* x, const float* weight, int n, int dim, float eps);
// Q8_0 quantisation of n rows.
void launch_quant_rows(cudaStream_t st, const float* x, int n, int k, float* q8s, int8_t* q8q);
// gate = silu(gate) * up (cpu.rs:668-673) over n rows of dim, then quantise -> q8; `act_out`
// optional f32 copy.
void launch_silu_mul_quant(cudaStream_t st, const float* gate, const float* up, int n, int dim, float* q8s,
                           int8_t* q8q, float* act_out);
void launch_silu_mul(cudaStream_t st, float* gate, const float* up, size_t count);
void launch_expf(cudaStream_t st, const float* x, float* y, size_t count);

// Gated short conv (lfm2.rs:688-725, :1316-1354) over n tokens, state [d_conv][hs] updated;
// writes f32 out [n][hs] (optional) and its Q8_0 quantisation (optional).
void launch_shortconv(cudaStream_t st, const float* proj, const float* conv_w, float* state, int n, int hs,
                      int ksize, float* out, float* q8s, int8_t* q8q);

// Per-head QK RMSNorm + RoPE + KV append (lfm2.rs:783-855, :1544-1623).  q [n][hs] in place;
// k, v [n][kv_dim] read; rows start_pos+j of the caches written.  start_pos < 0: read from ctl.
void launch_qknorm_rope_kv(cudaStream_t st, float* q, const float* k, const float* v, const float* q_norm,
                           const float* k_norm, float eps, const float* rope_cos, const float* rope_sin,
                           float* k_cache, float* v_cache, int n, int start_pos, const DecodeCtl* ctl, int n_heads,
                           int n_kv_heads, int head_dim);
void launch_rope(cudaStream_t st, float* q, float* k, const float* cos_row, const float* sin_row, int n_heads,
                 int n_kv_heads, int head_dim);

// Exact single-query / per-token attention (lfm2.rs:980-1007; cpu.rs:1404-1509, :715-731).
// Query j attends rows [0, start_pos + j]; start_pos < 0: read from ctl.  smem grows with seq.
void launch_attention_naive(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out,
                            int n, int start_pos, const DecodeCtl* ctl, int n_heads, int n_kv_heads, int head_dim,
                            int max_seq);
// Opt-in to more than 48 KB of dynamic shared memory for the kernel above; call before any
// stream capture that contains it.
void configure_naive_attention_smem(size_t bytes);
// Dynamic shared memory the kernel needs for this head size and longest sequence.
size_t naive_attention_smem_bytes(int head_dim, int max_seq);
// Exact tiled online-softmax attention (cpu.rs:1696-1850) for head_dim 32, 64 or 128 and up to 8 query heads per
// KV head (attention_flash_supported); other shapes return cudaErrorInvalidValue without launching.  `err` is a
// device word that receives a non-zero code if a bounded wait inside the kernel runs out.
bool attention_flash_supported(int n_heads, int n_kv_heads, int head_dim);
cudaError_t launch_attention_flash(cudaStream_t st, const float* q, const float* k_cache, const float* v_cache, float* out,
                                   int n, int start_pos, int n_heads, int n_kv_heads, int head_dim, uint32_t* err);

// Q6_K vocabulary matrix (kernels_q6k.cu): re-layout of raw GGUF blocks into the planes of `w` (already
// pointing at device memory), embedding rows, and the logits mat-vec y[m] (simd.rs:552-672).  The mat-vec
// uses gemv_q6k_smem(k) bytes of dynamic shared memory (k <= 6144 stays under the 48 KB default).
void launch_repack_q6k(cudaStream_t st, const uint8_t* raw, const DevQ6K& w);
void launch_embed_q6k(cudaStream_t st, const DevQ6K& w, const uint32_t* tokens, const DecodeCtl* ctl, float* out, int n);
size_t gemv_q6k_smem(int k);
void launch_gemv_q6k(cudaStream_t st, const DevQ6K& w, const float* xs, const int8_t* xq, float* y);

// n_keep context shift (kv_cache.rs:601-715): gathers cache rows [row0 + shift, row0 + shift + rows) into a
// dense scratch, K rows rotated by the delta table (cos_delta / sin_delta of hd/2 entries), V rows as they are (NULL tables).
void launch_kv_shift_gather(cudaStream_t st, const float* cache, float* scratch, int row0, int rows, int shift, int kv_dim, int hd,
                            const float* cos_delta, const float* sin_delta);

// Integer GEMV, up to three matrices sharing one quantised input (simd.rs:328-415, :440-524).
struct GemvJob {
    DevWeight w[3];
    float* y[3];
    int count;
};
void launch_gemv(cudaStream_t st, const GemvJob& job, const float* xs, const int8_t* xq);
// Integer GEMM over n quantised tokens, out[j*m + i] (simd.rs:696-1019).
void launch_gemm(cudaStream_t st, const DevWeight& w, const float* bs, const int8_t* bq, int n, float* out);
void launch_block_sums(cudaStream_t st, const DevWeight& w, const int8_t* xq, int32_t* S);

// Multi-sequence decode step (kernels_batch.cu): row j of n is the next token of its own sequence, with its own
// position and state.  `states`, `k_caches`, `v_caches` are device arrays of n per-row pointers.
void launch_shortconv_rows(cudaStream_t st, const float* proj, const float* conv_w, float* const* states, int n, int hs, int ks,
                           float* q8s, int8_t* q8q);
void launch_qknorm_rope_kv_rows(cudaStream_t st, float* q, const float* k, const float* v, const float* q_norm, const float* k_norm,
                                float eps, const float* rope_cos, const float* rope_sin, float* const* k_caches, float* const* v_caches,
                                const uint32_t* positions, int n, int n_heads, int n_kv_heads, int head_dim);
cudaError_t launch_attention_rows(cudaStream_t st, const float* q, float* const* k_caches, float* const* v_caches, const uint32_t* positions,
                                  float* out, int n, int n_heads, int n_kv_heads, int head_dim, int max_seq);
// Opt-in split-K form of the single-query attention (keys of every (row, head) in runs of 256 + a merge pass; rounding
// differs from the exact kernel).  Caches per row (k_caches / v_caches) or one pair for all rows (k_single / v_single);
// positions[j] = cached rows before row j's token.  scratch: attention_splitk_scratch_floats() floats.
size_t attention_splitk_scratch_floats(int n, int n_heads, int head_dim, int max_seq);
void launch_attention_splitk(cudaStream_t st, const float* q, float* const* k_caches, float* const* v_caches, const float* k_single,
                             const float* v_single, const uint32_t* positions, float* out, float* scratch, int n, int n_heads, int n_kv_heads,
                             int head_dim, int max_seq);
void launch_argmax_rows(cudaStream_t st, const float* logits, int n, int count, uint32_t* out);
void launch_rows_advance(cudaStream_t st, uint32_t* tokens, const uint32_t* next, uint32_t* positions, uint32_t* out_table, int n, int step);

// Sampler::sample (sampler.rs:64-158) of n device logits with the uniform draw r; val / idx are n-element work arrays.
// *status gets bit 0 when top-p would need more than 4096 survivors sorted (nothing is written to *out then).
void launch_sample(cudaStream_t st, const float* logits, int n, float temperature, int top_k, float top_p, float r, float* val, int* idx,
                   uint32_t* out, uint32_t* status);

// cpu_argmax (sampler.rs:8-19).  Uses ctl->argmax as scratch when ctl != NULL, else `scratch`.
void launch_argmax(cudaStream_t st, const float* logits, int count, unsigned long long* scratch, uint32_t* out);
// End of a decode step on the device: token <- argmax, pos += 1, ring[step++] = token.
void launch_decode_advance(cudaStream_t st, DecodeCtl* ctl, const uint32_t* argmax_tok, uint32_t* ring, int ring_len);

}  // namespace wick
