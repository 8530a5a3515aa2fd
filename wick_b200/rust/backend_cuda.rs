//! wick/src/backend/cuda.rs: `extern "C"` bindings of libwick_cuda (include/wick_cuda.h).
//! Written against the header; not compiled where it was written (no Rust toolchain there).
#![allow(dead_code)]
use std::os::raw::c_char;

#[repr(C)]
pub struct WickCudaModel {
    _opaque: [u8; 0],
}

/// `wick_cuda_config`: plain-C mirror of `ModelConfig`.
#[repr(C)]
#[derive(Default, Clone, Copy, Debug)]
pub struct WickCudaConfig {
    pub n_layers: u32,
    pub hidden_size: u32,
    pub intermediate_size: u32,
    pub n_heads: u32,
    pub n_kv_heads: u32,
    pub vocab_size: u32,
    pub max_seq_len: u32,
    pub conv_kernel_size: u32,
    pub rope_theta: f32,
    pub rms_norm_eps: f32,
}

pub const WICK_CUDA_OK: i32 = 0;
pub const WICK_CUDA_PREFILL_EXACT: i32 = 0;
pub const WICK_CUDA_PREFILL_TENSOR: i32 = 1;
pub const WICK_CUDA_PREFILL_EXACT_CUDA_CORES: i32 = 2;

extern "C" {
    pub fn wick_cuda_device_count(count: *mut i32) -> i32;
    pub fn wick_cuda_last_error() -> *const c_char;
    pub fn wick_cuda_model_create(gguf: *const u8, len: usize, context_size: u32, device: i32, out: *mut *mut WickCudaModel) -> i32;
    pub fn wick_cuda_model_destroy(m: *mut WickCudaModel);
    pub fn wick_cuda_model_config(m: *const WickCudaModel, out: *mut WickCudaConfig) -> i32;
    pub fn wick_cuda_model_kv_heads_per_layer(m: *const WickCudaModel, out: *mut u32, n: u32) -> i32;
    pub fn wick_cuda_gpu_memory_bytes(m: *const WickCudaModel, out: *mut u64) -> i32;
    pub fn wick_cuda_forward(m: *mut WickCudaModel, token: u32, pos: u32, logits: *mut f32) -> i32;
    pub fn wick_cuda_forward_greedy(m: *mut WickCudaModel, token: u32, pos: u32, next: *mut u32) -> i32;
    pub fn wick_cuda_forward_prefill(m: *mut WickCudaModel, tokens: *const u32, n: u32, start_pos: u32, logits: *mut f32) -> i32;
    pub fn wick_cuda_forward_prefill_from_embeddings(m: *mut WickCudaModel, emb: *const f32, n: u32, start_pos: u32, logits: *mut f32) -> i32;
    pub fn wick_cuda_forward_from_embedding(m: *mut WickCudaModel, emb: *const f32, pos: u32, logits: *mut f32) -> i32;
    pub fn wick_cuda_forward_hidden_from_embedding(m: *mut WickCudaModel, emb: *const f32, pos: u32, hidden: *mut f32) -> i32;
    pub fn wick_cuda_forward_embedding(m: *mut WickCudaModel, token: u32, pos: u32, hidden: *mut f32) -> i32;
    pub fn wick_cuda_shift_kv(m: *mut WickCudaModel, n_keep: u32, shift: u32) -> i32;
    pub fn wick_cuda_reset(m: *mut WickCudaModel) -> i32;
    pub fn wick_cuda_seq_len(m: *const WickCudaModel, out: *mut u32) -> i32;
    pub fn wick_cuda_snapshot_size(m: *const WickCudaModel, bytes: *mut u64) -> i32;
    pub fn wick_cuda_snapshot(m: *mut WickCudaModel, out: *mut u8, capacity: u64) -> i32;
    pub fn wick_cuda_restore(m: *mut WickCudaModel, snap: *const u8, len: u64) -> i32;
    pub fn wick_cuda_set_prefill_mode(m: *mut WickCudaModel, mode: i32) -> i32;
    pub fn wick_cuda_generate_greedy(m: *mut WickCudaModel, first: u32, n_steps: u32, out: *mut u32) -> i32;
    pub fn wick_cuda_forward_sample(m: *mut WickCudaModel, token: u32, pos: u32, temperature: f32, top_k: u32, top_p: f32, r: f32, next: *mut u32) -> i32;
    // many sequences on one model (not part of `trait Model`)
    pub fn wick_cuda_seq_create(m: *mut WickCudaModel, seq_id: *mut u32) -> i32;
    pub fn wick_cuda_seq_destroy(m: *mut WickCudaModel, seq_id: u32) -> i32;
    pub fn wick_cuda_seq_length(m: *const WickCudaModel, seq_id: u32, out: *mut u32) -> i32;
    pub fn wick_cuda_seq_prefill(m: *mut WickCudaModel, seq_id: u32, tokens: *const u32, n: u32, start_pos: u32, logits: *mut f32) -> i32;
    pub fn wick_cuda_decode_batch(m: *mut WickCudaModel, tokens: *const u32, seq_ids: *const u32, bs: u32, next: *mut u32) -> i32;
    pub fn wick_cuda_decode_batch_steps(m: *mut WickCudaModel, first: *const u32, seq_ids: *const u32, bs: u32, n_steps: u32, out: *mut u32) -> i32;
    pub fn wick_cuda_decode_batch_logits(m: *mut WickCudaModel, tokens: *const u32, seq_ids: *const u32, bs: u32, logits: *mut f32) -> i32;
}

/// The calling thread's last error message.
pub fn last_error() -> String {
    // SAFETY: the library returns a NUL-terminated string owned by thread-local storage.
    unsafe { std::ffi::CStr::from_ptr(wick_cuda_last_error()) }.to_string_lossy().into_owned()
}

/// Trait methods are infallible in wick (the Metal backend asserts, metal_lfm2.rs:2085-2090): a non-zero status
/// after the C call has returned becomes a panic with the library's message.
pub fn check(code: i32) {
    if code != WICK_CUDA_OK {
        panic!("wick_cuda error {code}: {}", last_error());
    }
}

/// Number of CUDA devices visible to the process (0 when the runtime cannot be initialised).
pub fn device_count() -> usize {
    let mut n = 0i32;
    // SAFETY: plain out-parameter.
    if unsafe { wick_cuda_device_count(&mut n) } != WICK_CUDA_OK {
        return 0;
    }
    n.max(0) as usize
}
