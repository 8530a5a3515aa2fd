/*
 * wick_cuda.h -- C ABI of libwick_cuda, a CUDA (sm_100a) backend for the LFM2
 * decode / prefill hot path of the wick inference engine.
 *
 * The entry points are what a `wick/src/backend/cuda.rs` + `wick/src/model/cuda_lfm2.rs`
 * pair would bind with `extern "C"`: one opaque model handle that plays the role
 * MetalLfm2Model plays for `--device metal` (wick/src/model/metal_lfm2.rs:170-277),
 * i.e. weights, KV cache, conv state and scratch are resident on the GPU and ONE
 * sequence lives in the model.  Each function cites the wick interface it stands
 * in for (path:line inside the wick repository).
 *
 * Conventions
 *  - every function returns a status code (0 = ok, negative = error) and never
 *    throws or aborts; wick_cuda_last_error() returns the calling thread's last
 *    message.  wick's trait methods are infallible (they assert), so the Rust side
 *    panics after a non-zero status; load failures map to anyhow errors.
 *  - pointers named *_host are host memory, *_dev are device memory on the
 *    model's / current device.  The caller owns every buffer it passes.
 *  - calls on one handle must not overlap (the Rust side holds `infer_lock`,
 *    metal_lfm2.rs:254-267); different handles may be used from different threads.
 *  - functions that return results in host memory block until they are there.
 */
#ifndef WICK_CUDA_H
#define WICK_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WICK_CUDA_OK 0
#define WICK_CUDA_ERR_BAD_ARG (-1)
#define WICK_CUDA_ERR_CUDA (-2)
#define WICK_CUDA_ERR_OOM (-3)
#define WICK_CUDA_ERR_UNSUPPORTED_DTYPE (-4)
#define WICK_CUDA_ERR_CONTEXT_FULL (-5)
#define WICK_CUDA_ERR_TIMEOUT (-6)
#define WICK_CUDA_ERR_BAD_GGUF (-7)

/* GGML tensor type ids of the two supported weight formats (wick/src/gguf.rs:38, :42). */
#define WICK_DTYPE_Q4_0 2
#define WICK_DTYPE_Q8_0 8

typedef struct wick_cuda_model wick_cuda_model;
typedef struct wick_cuda_weight wick_cuda_weight;

/* Mirror of wick::model::ModelConfig (wick/src/model/mod.rs:28-46). */
typedef struct wick_cuda_config {
    uint32_t n_layers;
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t n_heads;
    uint32_t n_kv_heads;       /* max over layers */
    uint32_t vocab_size;
    uint32_t max_seq_len;      /* min(context_size, gguf context_length), lfm2.rs:120-127 */
    uint32_t conv_kernel_size;
    float rope_theta;
    float rms_norm_eps;
} wick_cuda_config;

/* ---- library ---------------------------------------------------------- */

/* Number of CUDA devices; backs `--device cuda[:N]` (wick/src/engine.rs:65-89). */
int32_t wick_cuda_device_count(int32_t* count);
/* Last error message of the calling thread (valid until its next failing call). */
const char* wick_cuda_last_error(void);

/* ---- model lifetime: load_model_metal / MetalLfm2Model::from_gguf
 *      (wick/src/model/mod.rs:386-403, metal_lfm2.rs:280-610) --------------- */

/* Parses a GGUF v3 image (the bytes of GgufFile::mmap_data(), gguf.rs:662), uploads and
 * re-lays-out the weights, allocates KV cache / conv state / scratch for
 * min(context_size, lfm2.context_length) positions.  The image may be freed on return. */
int32_t wick_cuda_model_create(const uint8_t* gguf_host, size_t gguf_len, uint32_t context_size,
                               int32_t device, wick_cuda_model** out);
/* Same, reading the file itself (GgufFile::open, gguf.rs:336-360). */
int32_t wick_cuda_model_create_from_file(const char* path, uint32_t context_size, int32_t device,
                                         wick_cuda_model** out);
/* Drop. NULL is allowed. */
void wick_cuda_model_destroy(wick_cuda_model* m);

/* Model::config (model/mod.rs:143). */
int32_t wick_cuda_model_config(const wick_cuda_model* m, wick_cuda_config* out);
/* ModelConfig::block_types / kv_heads_per_layer: out[i] = 0 for a gated-conv layer, else
 * that attention layer's KV head count.  `n` must equal n_layers. */
int32_t wick_cuda_model_kv_heads_per_layer(const wick_cuda_model* m, uint32_t* out, uint32_t n);
/* Model::gpu_memory_bytes (model/mod.rs:280). */
int32_t wick_cuda_gpu_memory_bytes(const wick_cuda_model* m, uint64_t* out);

/* ---- the Model trait (model/mod.rs:72-323) ---------------------------- */

/* Model::forward (mod.rs:74; Metal precedent metal_lfm2.rs:2078-2148): one token in, logits
 * [vocab_size] out.  As in the Metal backend the position is the model's own counter; `pos`
 * is checked against it and a mismatch is WICK_CUDA_ERR_BAD_ARG.  CONTEXT_FULL once
 * seq_len == max_seq_len. */
int32_t wick_cuda_forward(wick_cuda_model* m, uint32_t token, uint32_t pos, float* logits_host);
/* Model::forward_greedy (mod.rs:274; metal_lfm2.rs:2151-2203): same step, argmax on the GPU
 * with cpu_argmax's rule (sampler.rs:8-19: NaN = -inf, last of equal maxima), 4-byte readback. */
int32_t wick_cuda_forward_greedy(wick_cuda_model* m, uint32_t token, uint32_t pos, uint32_t* next_token);
/* Model::forward_prefill (mod.rs:79; lfm2.rs:2351, metal_lfm2.rs:2350): n >= 1 tokens at
 * positions start_pos.., logits of the LAST token out.  start_pos == 0 starts a new sequence
 * (resets seq_len, zeroes conv state); otherwise start_pos must equal seq_len.  Like the CPU
 * path, a call with n >= 256 uses the tiled online-softmax attention and a shorter one the
 * per-token attention (lfm2.rs:1646-1647).  Callers chunk long prompts themselves
 * (forward_prefill_chunked, mod.rs:111-140). */
int32_t wick_cuda_forward_prefill(wick_cuda_model* m, const uint32_t* tokens_host, uint32_t n,
                                  uint32_t start_pos, float* logits_host);

/* Embedding-input methods of the trait (model/mod.rs:172-267; CPU model lfm2.rs:2291-2350, :2452-2500);
 * supports_embedding_input() is true for this backend.  Inputs are host f32.
 *  - forward_prefill_from_embeddings: frames [n][hidden] row-major instead of token ids; logits of the
 *    last frame; same start_pos rules as forward_prefill.
 *  - forward_from_embedding: one frame at the model's own position (`pos` is ignored, like forward) -> logits.
 *  - forward_hidden_from_embedding / forward_embedding: one frame / one token id -> the output-normed
 *    hidden row [hidden] (the vector the logit projection would read), no logits.
 * All four advance seq_len and run the one-row or n-row prefill pipeline. */
int32_t wick_cuda_forward_prefill_from_embeddings(wick_cuda_model* m, const float* embeddings_host, uint32_t n,
                                                  uint32_t start_pos, float* logits_host);
int32_t wick_cuda_forward_from_embedding(wick_cuda_model* m, const float* embedding_host, uint32_t pos,
                                         float* logits_host);
int32_t wick_cuda_forward_hidden_from_embedding(wick_cuda_model* m, const float* embedding_host, uint32_t pos,
                                                float* hidden_host);
int32_t wick_cuda_forward_embedding(wick_cuda_model* m, uint32_t token, uint32_t pos, float* hidden_host);

/* Model::shift_kv, the n_keep context shift (model/mod.rs:145-170; CPU model lfm2.rs:2500-2516 ->
 * InferenceState::shift_kv_with_rope, kv_cache.rs:601-715); supports_kv_shift() is true for this backend.
 * Drops rows [n_keep, n_keep + shift) of every attention layer's K and V caches, slides the tail down and
 * rotates the moved K rows by R(-shift) (apply_rope_delta_to_head, cpu.rs:2174-2187); conv buffers are left
 * alone; seq_len -= shift.  The reference asserts shift > 0 and n_keep + shift <= seq_len; here those are
 * WICK_CUDA_ERR_BAD_ARG. */
int32_t wick_cuda_shift_kv(wick_cuda_model* m, uint32_t n_keep, uint32_t shift);

/* Which GEMM forward_prefill uses for chunks of >= 16 tokens (shorter chunks always take the
 * CUDA-core kernel).  Decode is not affected.
 * EXACT (default): the arithmetic of gemm_q*_q8_0_neon (simd.rs:696-1019) bit for bit, so logits and
 *   greedy tokens equal wick's CPU path.  When hidden and feed-forward sizes are multiples of 128 it
 *   runs on the tensor cores: tcgen05 int8 MMAs against lane-group-masked activations produce the
 *   four int32 lane partials of every block, and the epilogue keeps the reference's eight unfused f32
 *   chains per output; otherwise on the CUDA-core kernel.
 * EXACT_CUDA_CORES (env WICK_CUDA_PREFILL=exact-cuda-cores): always the CUDA-core kernel (same bits).
 * TENSOR (env WICK_CUDA_PREFILL=tensor; needs the multiples of 128): the kernel described at
 *   wick_cuda_gemm_q8_tc.  Each product agrees with EXACT to f32 rounding, but the first last-bit
 *   difference that flips one Q8_0 rounding of a later activation (simd.rs:285-300) moves that
 *   activation by a whole quantisation step, so over a long prompt the logits end up one
 *   quantisation-noise realisation away from the CPU path's (a few 1e-2 on logits of order 1), like
 *   wick's own GPU backends. */
#define WICK_CUDA_PREFILL_EXACT 0
#define WICK_CUDA_PREFILL_TENSOR 1
#define WICK_CUDA_PREFILL_EXACT_CUDA_CORES 2
int32_t wick_cuda_set_prefill_mode(wick_cuda_model* m, int32_t mode);
int32_t wick_cuda_prefill_mode(const wick_cuda_model* m, int32_t* mode);
/* 1 when the selected mode runs its GEMMs on the tensor cores for this model. */
int32_t wick_cuda_prefill_uses_tensor_cores(const wick_cuda_model* m, int32_t* yes);
/* Greedy decode loop of Session::generate (wick/src/session.rs:1186-1257) kept on the GPU:
 * feeds `first_token`, then each step's argmax, for n_steps steps; out_tokens_host[i] is the
 * token chosen by step i.  Equivalent to n_steps wick_cuda_forward_greedy calls without the
 * per-token host round trip. */
int32_t wick_cuda_generate_greedy(wick_cuda_model* m, uint32_t first_token, uint32_t n_steps,
                                  uint32_t* out_tokens_host);
/* New sequence without a prefill (InferenceState::from_config, kv_cache.rs:183). */
int32_t wick_cuda_reset(wick_cuda_model* m);
/* InferenceState::seq_len (kv_cache.rs:115-130). */
int32_t wick_cuda_seq_len(const wick_cuda_model* m, uint32_t* out);

/* Model::snapshot_state / restore_state (mod.rs:301-313; metal_lfm2.rs:2535-2650): KV rows
 * [0, seq_len) of every attention layer, conv rolling buffers and seq_len as one byte image. */
int32_t wick_cuda_snapshot_size(const wick_cuda_model* m, uint64_t* bytes);
int32_t wick_cuda_snapshot(wick_cuda_model* m, uint8_t* out_host, uint64_t capacity);
int32_t wick_cuda_restore(wick_cuda_model* m, const uint8_t* snap_host, uint64_t len);

/* Profiling hooks in the spirit of wick's GPU timers (WICK_PROFILE=gpu, metal_lfm2.rs:3922-3984):
 * device time, from CUDA events on the model's stream, of the GPU work of the last forward /
 * forward_greedy / forward_prefill / generate_greedy call (host<->device copies included), and the
 * number of kernels this model has launched since it was created (graph replays count their nodes). */
int32_t wick_cuda_last_elapsed_ms(wick_cuda_model* m, float* ms);
int32_t wick_cuda_kernel_launches(const wick_cuda_model* m, uint64_t* count);

/* Per-phase timeline of the most recent decode step run by the persistent kernel, in the spirit of
 * wick's per-category timers (WICK_PROFILE=timing, metal_lfm2.rs:3986-4035): for each phase four
 * device timestamps in ns (dependency barrier passed, input prologue done, mat-vec done, arrived at
 * the next barrier) taken by one CTA, and the phase kind (0 norm, 1 short-conv, 2 attention,
 * 3 attention-output quantise, 4 SwiGLU).  *n_phases is always set; the arrays are filled when
 * capacity >= *n_phases (ns_out holds 4 values per phase). */
int32_t wick_cuda_decode_profile(wick_cuda_model* m, uint64_t* ns_out, int32_t* kinds_out, uint32_t capacity,
                                 uint32_t* n_phases);
/* Test hook for the bounded waits of the persistent decode kernel: shifts the barrier sequence
 * number the NEXT decode call waits for by `delta` arrivals, so that its grid-wide waits expire
 * (about a second) and the call returns WICK_CUDA_ERR_TIMEOUT with the device context intact.
 * Returns WICK_CUDA_ERR_BAD_ARG when the model decodes through captured graphs instead. */
int32_t wick_cuda_debug_skew_barrier(wick_cuda_model* m, int64_t delta);
/* 1 if decode steps run in the persistent kernel, 0 if through the captured per-kernel graph
 * (models whose row length is not a multiple of 64, or WICK_CUDA_DECODE=graph in the environment). */
int32_t wick_cuda_decode_path(const wick_cuda_model* m, int32_t* persistent);

/* Debug / parity taps: f32 K and V rows [0, seq_len) x kv_dim of an attention layer
 * (LayerState::Attention, kv_cache.rs:62-70) or the [d_conv][hidden] rolling buffer of a conv
 * layer (LayerState::Conv, kv_cache.rs:72-74). */
int32_t wick_cuda_read_kv(wick_cuda_model* m, uint32_t layer, float* k_host, float* v_host);
int32_t wick_cuda_read_conv_state(wick_cuda_model* m, uint32_t layer, float* out_host);

/* ---- operators on device buffers ------------------------------------------
 * The free functions of wick/src/backend/{simd,cpu}.rs that the model is built
 * from, exposed so each kernel can be checked on its own.  All pointers are device
 * pointers; `stream` is a cudaStream_t (NULL = default stream); calls are
 * asynchronous on that stream. */

/* Uploads GGUF-layout quantised rows [m][k/32 blocks] (host memory) into the library's device
 * layout (quants plane + f16 scale plane, same byte count).  WeightRef, lfm2.rs:19-25. */
int32_t wick_cuda_weight_create(int32_t dtype, const uint8_t* raw_host, uint32_t m, uint32_t k,
                                wick_cuda_weight** out);
void wick_cuda_weight_destroy(wick_cuda_weight* w);

/* quantize_f32_to_q8_0_neon over n rows of k (simd.rs:255-323; quantize_columns lfm2.rs:571-592):
 * scales [n][k/32] f32 (f16-rounded), quants [n][k] i8.  x must be 16-byte aligned, quants 4-byte aligned. */
int32_t wick_cuda_quantize_q8_0(const float* x_dev, uint32_t n, uint32_t k, float* scales_dev,
                                int8_t* quants_dev, void* stream);
/* gemv_q4_0_q8_0_neon / gemv_q8_0_q8_0_neon (simd.rs:328-415, :440-524): y[m]. */
int32_t wick_cuda_gemv_q8(const wick_cuda_weight* w, const float* xs_dev, const int8_t* xq_dev,
                          float* y_dev, void* stream);
/* gemm_q4_0_q8_0_neon / gemm_q8_0_q8_0_neon (simd.rs:696-925, :937-1019) over n pre-quantised
 * columns; the result is token-major out[j*m + i] (the reference writes out[i*n + j]). */
int32_t wick_cuda_gemm_q8(const wick_cuda_weight* w, const float* bs_dev, const int8_t* bq_dev,
                          uint32_t n, float* out_dev, void* stream);
/* The same product on the tensor cores (tcgen05 int8 MMA, one instruction per 32-element block, int32
 * block sums in tensor memory, f32 scaling in the epilogue): the throughput path of forward_prefill.
 * Block sums are the exact integers of simd.rs:806-842; the f32 accumulation is one fused chain per
 * output in ascending block order, so `out` agrees with wick_cuda_gemm_q8 to f32 rounding, not bit for
 * bit.  Needs k % 128 == 0.  block_sums_dev: optional [n][m][k/32] int32.  Unlike the other operator
 * entry points this one synchronises `stream` before returning (it reports expired device waits as
 * WICK_CUDA_ERR_TIMEOUT) and, on its first call for a weight, allocates that weight's int8 copy. */
int32_t wick_cuda_gemm_q8_tc(wick_cuda_weight* w, const float* bs_dev, const int8_t* bq_dev, uint32_t n,
                             float* out_dev, int32_t* block_sums_dev, void* stream);
/* The bit-exact product on the tensor cores (the default GEMM of forward_prefill): same result as
 * wick_cuda_gemm_q8, bit for bit.  Needs k % 128 == 0.  Allocates a temporary for the masked
 * activations and synchronises `stream` (operator entry point for tests). */
int32_t wick_cuda_gemm_q8_tc_exact(wick_cuda_weight* w, const float* bs_dev, const int8_t* bq_dev, uint32_t n,
                                   float* out_dev, void* stream);
/* int32 block dot sums S[i][b] = sum over the 32 elements of block b of row i (the vdotq_s32
 * lanes of simd.rs:381-383 added up) against one quantised column. */
int32_t wick_cuda_block_sums(const wick_cuda_weight* w, const int8_t* xq_dev, int32_t* s_dev, void* stream);
/* cpu::rmsnorm over n rows of `dim` (cpu.rs:577-594), in place. */
int32_t wick_cuda_rmsnorm(float* x_dev, const float* weight_dev, uint32_t n, uint32_t dim, float eps, void* stream);
/* cpu::silu_mul_inplace (cpu.rs:668-673): gate = silu(gate) * up, `count` elements. */
int32_t wick_cuda_silu_mul(float* gate_dev, const float* up_dev, uint64_t count, void* stream);
/* ggml_expf (cpu.rs:602-642), element-wise. */
int32_t wick_cuda_expf(const float* x_dev, float* y_dev, uint64_t count, void* stream);
/* cpu::rope (cpu.rs:2113-2158) for one position; cos/sin are evaluated on the host with libm
 * exactly as the reference does and uploaded by this call. */
int32_t wick_cuda_rope(float* q_dev, float* k_dev, uint32_t pos, uint32_t n_heads, uint32_t n_kv_heads,
                       uint32_t head_dim, float freq_base, void* stream);
/* Per-head RMSNorm of Q and K (shared head_dim-long weights), NeoX RoPE and the KV append of forward_attn_block
 * (lfm2.rs:783-855) for n rows at positions start_pos..: q [n][n_heads*head_dim] is rotated in place; the rotated K rows
 * and the V rows go to rows start_pos + j of the caches [rows][n_kv_heads*head_dim].  rope_cos / rope_sin are
 * [positions][head_dim/2] tables (cpu.rs:2145-2158 gives the values: theta starts at the position and is multiplied
 * by base^(-2/head_dim) pair by pair). */
int32_t wick_cuda_qknorm_rope_kv(float* q_dev, const float* k_dev, const float* v_dev, const float* q_norm_dev,
                                 const float* k_norm_dev, float eps, const float* rope_cos_dev, const float* rope_sin_dev,
                                 float* k_cache_dev, float* v_cache_dev, uint32_t n, uint32_t start_pos, uint32_t n_heads,
                                 uint32_t n_kv_heads, uint32_t head_dim, void* stream);
/* Single-query attention of forward_attn_block (lfm2.rs:980-1007): attn_scores, softmax_inplace,
 * attn_values (cpu.rs:1320-1509, :715-731) for all heads over `seq` cached rows. */
int32_t wick_cuda_attention_decode(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                                   float* out_dev, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                   uint32_t seq, void* stream);
/* Causal GQA prefill attention: query j of n attends rows [0, start_pos + j].  flash != 0 selects
 * flash_attention_gqa_cpu (cpu.rs:1538-1850), else the per-token path (lfm2.rs:1857-1897).
 * q / out are token-major [n][n_heads*head_dim]. */
int32_t wick_cuda_attention_prefill(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                                    float* out_dev, uint32_t n, uint32_t start_pos, uint32_t n_heads,
                                    uint32_t n_kv_heads, uint32_t head_dim, int32_t flash, void* stream);
/* The gated short-conv core of forward_conv_block (lfm2.rs:688-725) over n tokens: proj is
 * token-major [n][3*hidden] (b, c, x thirds), state [d_conv][hidden] is read and updated,
 * out [n][hidden] = c * conv(b * x). */
int32_t wick_cuda_shortconv(const float* proj_dev, const float* conv_w_dev, float* state_dev, float* out_dev,
                            uint32_t n, uint32_t hidden, uint32_t kernel_size, void* stream);
/* cpu_argmax (sampler.rs:8-19) of `count` logits -> *out_dev. */
int32_t wick_cuda_argmax(const float* logits_dev, uint32_t count, uint32_t* out_dev, void* stream);

/* Split-K decode attention (opt-in).  The default single-query attention keeps the CPU path's one serial accumulation per
 * output dim over all cached keys (attn_values, cpu.rs:1463-1509), which is bit-exact and, at thousands of keys, slow.
 * WICK_CUDA_DECODE_ATTENTION_SPLITK splits the keys of every head into runs of 256 and merges the runs' (max, sum,
 * weighted V) partials, the scheme of wick's Metal kernels (shaders/attention_splitk.metal:30 attention_split_compute,
 * :162 attention_split_merge).  Results then agree with the CPU path within rounding (about 1e-6 relative on the attention
 * output), not bit for bit, so greedy tokens can differ where two logits are close.  It applies to the multi-sequence
 * step (wick_cuda_decode_batch*) and to single-sequence decode when that runs as captured graphs; the persistent decode
 * kernel always uses the exact form.  Also selectable with WICK_CUDA_DECODE_ATTENTION=splitk in the environment at model
 * creation.  wick_cuda_attention_decode_splitk is the operator form (q [n_heads*head_dim], caches [seq][n_kv_heads*head_dim]). */
#define WICK_CUDA_DECODE_ATTENTION_EXACT 0
#define WICK_CUDA_DECODE_ATTENTION_SPLITK 1
int32_t wick_cuda_set_decode_attention(wick_cuda_model* m, int32_t mode);
int32_t wick_cuda_attention_decode_splitk(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                                          float* out_dev, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                          uint32_t seq, void* stream);

/* Per-category device timers of forward_prefill: the counterpart of wick's WICK_PROFILE=timing / gpu switches
 * (wick/src/model/metal_lfm2.rs:529-533, :596-600).  Enabled with the environment variable WICK_CUDA_PROFILE=events at model
 * creation or with wick_cuda_profile_enable (which also clears the totals); while enabled, every prefill chunk records
 * a CUDA event after each group of kernels of one kind and adds the differences to a running total per category
 * (milliseconds since the last enable).  wick_cuda_profile_category_name(i), i < WICK_CUDA_PROFILE_CATEGORIES, names them:
 * embedding, rmsnorm+quantise, gemm, short-conv, qk-norm+rope+kv-append, attention, activation+quantise,
 * output-norm+logits.  (The persistent decode kernel has its own per-phase timeline: wick_cuda_decode_profile.) */
#define WICK_CUDA_PROFILE_CATEGORIES 8
int32_t wick_cuda_profile_enable(wick_cuda_model* m, int32_t on);
int32_t wick_cuda_profile_read(wick_cuda_model* m, double* ms_out, uint32_t capacity);
const char* wick_cuda_profile_category_name(uint32_t i);

/* Model::forward followed by Sampler::sample (wick/src/sampler.rs:64-158) with the logits kept on the device: temperature
 * scaling, top-k, top-p, softmax_inplace and the weighted pick, in the reference's order; 4 bytes come back.  `r` is the
 * uniform draw in [0, 1) that wick takes from its `rand` StdRng (`self.rng.gen::<f32>()`, sampler.rs:151): the generator
 * stays with the caller.  temperature <= 0 or top_k == 1 is the greedy path.  top_p < 1 needs 1 <= top_k <= 4096
 * (BAD_ARG otherwise, and when more than 4096 logits tie at the threshold): read the logits back with
 * wick_cuda_forward and sample on the host in that case.  wick_cuda_sample_logits is the same sampler on any device
 * logits (operator form, *out_dev on the device; synchronises the stream). */
int32_t wick_cuda_forward_sample(wick_cuda_model* m, uint32_t token, uint32_t pos, float temperature, uint32_t top_k,
                                 float top_p, float r, uint32_t* next_token);
int32_t wick_cuda_sample_logits(const float* logits_dev, uint32_t count, float temperature, uint32_t top_k, float top_p,
                                float r, uint32_t* out_dev, void* stream);

/* ---- many sequences on one model (extension) --------------------------------
 * wick's Model trait keeps ONE sequence per model instance, serialised behind `infer_lock`
 * (wick/src/model/mod.rs:56-71; the GPU backends keep that sequence's state inside the model,
 * metal_lfm2.rs:2146-2147), so these entry points are not reachable from the trait: they are for a
 * serving loop that decodes many independent sequences from one copy of the weights.  A slot holds one
 * more sequence's state (K / V caches, rolling conv buffers, length); the model's own sequence, the one
 * every entry point above uses, is not a slot and is left untouched.
 *
 * wick_cuda_decode_batch advances `bs` different slots by one token each in ONE pass over the weights:
 * row j feeds tokens_host[j] to slot seq_ids_host[j] at that slot's own position and returns its greedy
 * choice (cpu_argmax, sampler.rs:8-19) in next_tokens_host[j].  The mat-vecs of the step run as the batched
 * integer GEMMs of the prefill path, which are bit-identical to the mat-vec per row (simd.rs:1440-1623), so every
 * row's result equals the same sequence decoded alone through wick_cuda_forward_greedy.  A slot may appear at
 * most once per batch (BAD_ARG); CONTEXT_FULL when a slot has no room left.
 * wick_cuda_decode_batch_steps keeps n_steps such steps on the device (row j's token of step s comes back in
 * out_tokens_host[s * bs + j]); wick_cuda_decode_batch_logits is the one-step form of wick_cuda_forward:
 * logits_host[j * vocab ..] instead of the argmax.  wick_cuda_seq_prefill is wick_cuda_forward_prefill on a
 * slot (same chunk rule, start_pos == 0 starts the slot's sequence anew). */
int32_t wick_cuda_seq_create(wick_cuda_model* m, uint32_t* seq_id);
int32_t wick_cuda_seq_destroy(wick_cuda_model* m, uint32_t seq_id);
int32_t wick_cuda_seq_length(const wick_cuda_model* m, uint32_t seq_id, uint32_t* out);
int32_t wick_cuda_seq_prefill(wick_cuda_model* m, uint32_t seq_id, const uint32_t* tokens_host, uint32_t n,
                              uint32_t start_pos, float* logits_host);
int32_t wick_cuda_decode_batch(wick_cuda_model* m, const uint32_t* tokens_host, const uint32_t* seq_ids_host,
                               uint32_t bs, uint32_t* next_tokens_host);
int32_t wick_cuda_decode_batch_steps(wick_cuda_model* m, const uint32_t* first_tokens_host,
                                     const uint32_t* seq_ids_host, uint32_t bs, uint32_t n_steps,
                                     uint32_t* out_tokens_host);
int32_t wick_cuda_decode_batch_logits(wick_cuda_model* m, const uint32_t* tokens_host, const uint32_t* seq_ids_host,
                                      uint32_t bs, float* logits_host);

/* ---- tensor-parallel all-reduce over peer memory (extension) -----------------
 * wick runs on one device; there is no counterpart in its tree.  For a tensor-parallel split of the LFM2 layers over
 * the GPUs of one NVLink node (one process per GPU): after every row-split mat-vec (attention output, short-conv
 * out_proj, FFN down; the steps of run_layers, wick/src/model/lfm2.rs:1020-1124) each rank holds a partial sum of the
 * hidden row.  wick_cuda_tp_allreduce_add_rmsnorm_quant adds the partials of all ranks (in rank order, so every
 * rank gets the same bits), adds the sum to `hidden_dev` (16-byte aligned) in place, and - when norm_w_dev is given - applies
 * cpu::rmsnorm (cpu.rs:577-594) and the Q8_0 activation quantiser (simd.rs:255-323) for the next mat-vec, all in one
 * kernel that reads the peers' buffers directly (plain loads over NVLink, no multicast).
 *
 * Set-up, once per rank: create (allocates this rank's buffer), export its 64-byte IPC handle, gather the handles of
 * all ranks in rank order by any means (e.g. a host all-gather), connect.  Per call: the rank's partial [dim] must be
 * written to the address wick_cuda_tp_partial_buffer() returns (it alternates between two halves, ask before every
 * call) by work enqueued on `stream` before the call.  Every rank must make the same sequence of calls.
 * The call is asynchronous; device-side waits are bounded (about a second): wick_cuda_tp_status synchronises the
 * stream and returns WICK_CUDA_ERR_TIMEOUT with the mask of ranks that never arrived (outputs of that call are
 * then undefined, the context stays usable).  Messages: wick_cuda_tp_last_error(). */
#define WICK_CUDA_TP_HANDLE_BYTES 64
typedef struct wick_cuda_tp_comm wick_cuda_tp_comm;
int32_t wick_cuda_tp_comm_create(uint32_t world, uint32_t rank, uint32_t max_floats, wick_cuda_tp_comm** out);
int32_t wick_cuda_tp_comm_export(wick_cuda_tp_comm* c, uint8_t* handle_out /* WICK_CUDA_TP_HANDLE_BYTES */);
int32_t wick_cuda_tp_comm_connect(wick_cuda_tp_comm* c, const uint8_t* handles /* world * WICK_CUDA_TP_HANDLE_BYTES */);
int32_t wick_cuda_tp_partial_buffer(wick_cuda_tp_comm* c, float** partial_dev);
int32_t wick_cuda_tp_allreduce_add_rmsnorm_quant(wick_cuda_tp_comm* c, float* hidden_dev, const float* norm_w_dev, float eps,
                                                 uint32_t dim, float* q8s_dev, int8_t* q8q_dev, float* normed_out_dev,
                                                 void* stream);
int32_t wick_cuda_tp_status(wick_cuda_tp_comm* c, void* stream, uint32_t* gave_up_mask);
void wick_cuda_tp_comm_destroy(wick_cuda_tp_comm* c);
const char* wick_cuda_tp_last_error(void);

/* ---- allocation-free variant ------------------------------------------------
 * No counterpart in wick: this entry point exists for callers of this library that are not allowed
 * to allocate (a real-time audio or serving thread, a process that has given its whole device memory
 * pool away).  Same result as wick_cuda_argmax(), but the scratch it needs lives in a fixed 32 KB array
 * inside the library (held by every GPU that loads it, until the process exits); no CUDA allocation
 * routine is called and the host heap is not used either (error messages are formatted into a fixed
 * per-thread buffer).  At most WICK_CUDA_ARGMAX_NOALLOC_MAX logits; more is WICK_CUDA_ERR_BAD_ARG
 * (message from wick_cuda_argmax_noalloc_last_error()).  Every call takes a short process-wide mutex;
 * the FIRST call on each device additionally looks up the array's device address, which may load the
 * library's module onto that device: make that first call a warm-up, outside real-time sections and
 * outside any stream capture.  It must not be called from a cudaLaunchHostFunc callback (no CUDA API
 * call may).  All calls share the one array: two calls whose kernels can overlap on the GPU (different
 * streams) race; calls on one stream are safe, and nothing needs to be cleared between calls. */
#define WICK_CUDA_ARGMAX_NOALLOC_MAX (4096 * 1024)
int32_t wick_cuda_argmax_noalloc(const float* logits_dev, uint32_t count, uint32_t* out_dev, void* stream);
const char* wick_cuda_argmax_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* WICK_CUDA_H */
