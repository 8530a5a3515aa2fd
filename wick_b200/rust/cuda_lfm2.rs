//! wick/src/model/cuda_lfm2.rs: `CudaLfm2Model`, the `--device cuda` implementation of `trait Model`
//! (wick/src/model/mod.rs:72-323) over libwick_cuda.  It plays the role `MetalLfm2Model` plays for
//! `--device metal` (metal_lfm2.rs:170-277): the sequence state lives inside the model handle, every call also
//! updates the caller's `InferenceState::seq_len`, calls are serialised by `infer_lock`.
//! Written against the trait and the C header; not compiled where it was written (no Rust toolchain there).
use std::sync::Mutex;

use anyhow::{ensure, Result};

use crate::backend::cuda as ffi;
use crate::gguf::GgufFile;
use crate::kv_cache::{InferenceState, LayerSnapshot, StateSnapshot};
use crate::model::{BlockType, Model, ModelConfig};

pub struct CudaLfm2Model {
    h: *mut ffi::WickCudaModel,
    config: ModelConfig,
    infer_lock: Mutex<()>,
    /// Prefix-cache namespace; backend-unique so snapshots never cross backends (cf. lfm2.rs:287-291).
    #[allow(dead_code)]
    model_id: String,
}

// SAFETY: the handle is only used under `infer_lock`; the library allows any thread to call as long as calls on one
// handle do not overlap (include/wick_cuda.h, "Conventions").
unsafe impl Send for CudaLfm2Model {}
unsafe impl Sync for CudaLfm2Model {}

impl CudaLfm2Model {
    pub fn from_gguf_with_id(gguf: GgufFile, context_size: usize, device: i32, model_id: String) -> Result<Self> {
        let data = gguf.mmap_data(); // the library copies what it needs; the mapping may go away afterwards
        let mut h: *mut ffi::WickCudaModel = std::ptr::null_mut();
        // SAFETY: `data` outlives the call; `h` is a plain out-parameter.
        let rc = unsafe { ffi::wick_cuda_model_create(data.as_ptr(), data.len(), context_size as u32, device, &mut h) };
        ensure!(rc == ffi::WICK_CUDA_OK && !h.is_null(), "cuda backend: {}", ffi::last_error());
        let mut c = ffi::WickCudaConfig::default();
        // SAFETY: `h` is a live handle.
        ffi::check(unsafe { ffi::wick_cuda_model_config(h, &mut c) });
        let mut kv = vec![0u32; c.n_layers as usize];
        ffi::check(unsafe { ffi::wick_cuda_model_kv_heads_per_layer(h, kv.as_mut_ptr(), c.n_layers) });
        let config = ModelConfig {
            architecture: "lfm2".to_string(),
            n_layers: c.n_layers as usize,
            hidden_size: c.hidden_size as usize,
            intermediate_size: c.intermediate_size as usize,
            n_heads: c.n_heads as usize,
            n_kv_heads: c.n_kv_heads as usize,
            vocab_size: c.vocab_size as usize,
            max_seq_len: c.max_seq_len as usize,
            rope_theta: c.rope_theta,
            rms_norm_eps: c.rms_norm_eps,
            block_types: kv.iter().map(|&k| if k > 0 { BlockType::Attention } else { BlockType::GatedConv }).collect(),
            conv_kernel_size: Some(c.conv_kernel_size as usize),
            kv_heads_per_layer: kv.iter().map(|&k| k as usize).collect(),
        };
        Ok(Self { h, config, infer_lock: Mutex::new(()), model_id: format!("cuda:{model_id}") })
    }

    fn head_dim(&self) -> usize {
        self.config.hidden_size / self.config.n_heads
    }

    /// Bytes of one K (or V) plane of an attention layer at `seq_len` rows, and of a conv buffer.
    fn layer_bytes(&self, layer: usize, seq_len: usize) -> (usize, usize) {
        let kv = self.config.kv_heads_per_layer[layer];
        let d_conv = self.config.conv_kernel_size.unwrap_or(1).saturating_sub(1);
        (seq_len * kv * self.head_dim() * 4, d_conv * self.config.hidden_size * 4)
    }

    fn seq_len_locked(&self) -> usize {
        let mut n = 0u32;
        ffi::check(unsafe { ffi::wick_cuda_seq_len(self.h, &mut n) });
        n as usize
    }
}

impl Drop for CudaLfm2Model {
    fn drop(&mut self) {
        // SAFETY: the handle came from wick_cuda_model_create and is dropped once.
        unsafe { ffi::wick_cuda_model_destroy(self.h) }
    }
}

impl Model for CudaLfm2Model {
    fn forward(&self, tokens: &[u32], _pos: usize, state: &mut InferenceState) -> Vec<f32> {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert_eq!(tokens.len(), 1, "CUDA forward expects single token");
        let mut logits = vec![0f32; self.config.vocab_size];
        // like the Metal backend (metal_lfm2.rs:2098) the model's own counter is the position
        let pos = self.seq_len_locked() as u32;
        ffi::check(unsafe { ffi::wick_cuda_forward(self.h, tokens[0], pos, logits.as_mut_ptr()) });
        state.seq_len += 1; // metal_lfm2.rs:2146-2147
        logits
    }

    fn forward_greedy(&self, tokens: &[u32], _pos: usize, state: &mut InferenceState) -> u32 {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert_eq!(tokens.len(), 1, "CUDA forward expects single token");
        let mut next = 0u32;
        let pos = self.seq_len_locked() as u32;
        ffi::check(unsafe { ffi::wick_cuda_forward_greedy(self.h, tokens[0], pos, &mut next) });
        state.seq_len += 1;
        next
    }

    fn forward_prefill(&self, tokens: &[u32], start_pos: usize, state: &mut InferenceState) -> Vec<f32> {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert!(!tokens.is_empty(), "forward_prefill requires at least one token");
        let mut logits = vec![0f32; self.config.vocab_size];
        // start_pos == 0 starts a new sequence inside the library (reset + zeroed conv buffers, metal_lfm2.rs:2361-2397)
        ffi::check(unsafe {
            ffi::wick_cuda_forward_prefill(self.h, tokens.as_ptr(), tokens.len() as u32, start_pos as u32, logits.as_mut_ptr())
        });
        state.seq_len = start_pos + tokens.len();
        logits
    }

    // forward_prefill_chunked: the trait's default (mod.rs:111-140) is what the library expects.

    fn config(&self) -> &ModelConfig {
        &self.config
    }

    fn supports_kv_shift(&self) -> bool {
        true
    }

    fn shift_kv(&self, state: &mut InferenceState, n_keep: usize, shift: usize) {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        ffi::check(unsafe { ffi::wick_cuda_shift_kv(self.h, n_keep as u32, shift as u32) });
        state.seq_len -= shift;
    }

    fn supports_embedding_input(&self) -> bool {
        true
    }

    fn forward_embedding(&self, tokens: &[u32], _pos: usize, state: &mut InferenceState) -> Vec<f32> {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert_eq!(tokens.len(), 1, "CUDA forward expects single token");
        let mut hidden = vec![0f32; self.config.hidden_size];
        ffi::check(unsafe { ffi::wick_cuda_forward_embedding(self.h, tokens[0], 0, hidden.as_mut_ptr()) });
        state.seq_len += 1;
        hidden
    }

    fn forward_from_embedding(&self, embedding: &[f32], _pos: usize, state: &mut InferenceState) -> Vec<f32> {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert_eq!(embedding.len(), self.config.hidden_size, "embedding length != hidden_size");
        let mut logits = vec![0f32; self.config.vocab_size];
        ffi::check(unsafe { ffi::wick_cuda_forward_from_embedding(self.h, embedding.as_ptr(), 0, logits.as_mut_ptr()) });
        state.seq_len += 1;
        logits
    }

    fn forward_hidden_from_embedding(&self, embedding: &[f32], _pos: usize, state: &mut InferenceState) -> Vec<f32> {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert_eq!(embedding.len(), self.config.hidden_size, "embedding length != hidden_size");
        let mut hidden = vec![0f32; self.config.hidden_size];
        ffi::check(unsafe { ffi::wick_cuda_forward_hidden_from_embedding(self.h, embedding.as_ptr(), 0, hidden.as_mut_ptr()) });
        state.seq_len += 1;
        hidden
    }

    fn forward_prefill_from_embeddings(&self, embeddings: &[f32], n_tokens: usize, start_pos: usize, state: &mut InferenceState) -> Vec<f32> {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        assert!(n_tokens > 0, "forward_prefill_from_embeddings requires at least one frame");
        assert_eq!(embeddings.len(), n_tokens * self.config.hidden_size, "embeddings.len() != n_tokens * hidden_size");
        let mut logits = vec![0f32; self.config.vocab_size];
        ffi::check(unsafe {
            ffi::wick_cuda_forward_prefill_from_embeddings(self.h, embeddings.as_ptr(), n_tokens as u32, start_pos as u32, logits.as_mut_ptr())
        });
        state.seq_len = start_pos + n_tokens;
        logits
    }

    fn gpu_memory_bytes(&self) -> u64 {
        let mut b = 0u64;
        ffi::check(unsafe { ffi::wick_cuda_gpu_memory_bytes(self.h, &mut b) });
        b
    }

    /// The library hands out one flat image (8-byte header, then per layer K rows + V rows or the conv buffer, all
    /// f32); it is cut into the per-layer pieces of `StateSnapshot` here and glued back in `restore_state`.
    fn snapshot_state(&self) -> StateSnapshot {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        let mut size = 0u64;
        ffi::check(unsafe { ffi::wick_cuda_snapshot_size(self.h, &mut size) });
        let mut image = vec![0u8; size as usize];
        ffi::check(unsafe { ffi::wick_cuda_snapshot(self.h, image.as_mut_ptr(), size) });
        let seq_len = u32::from_le_bytes(image[4..8].try_into().unwrap()) as usize;
        let mut at = 8usize;
        let mut layers = Vec::with_capacity(self.config.n_layers);
        for li in 0..self.config.n_layers {
            let (kv_bytes, conv_bytes) = self.layer_bytes(li, seq_len);
            if self.config.kv_heads_per_layer[li] > 0 {
                let k_data = image[at..at + kv_bytes].to_vec();
                let v_data = image[at + kv_bytes..at + 2 * kv_bytes].to_vec();
                at += 2 * kv_bytes;
                layers.push(LayerSnapshot::Attention { k_data, v_data });
            } else {
                layers.push(LayerSnapshot::Conv { buffer: image[at..at + conv_bytes].to_vec() });
                at += conv_bytes;
            }
        }
        StateSnapshot { layers, seq_len }
    }

    fn restore_state(&self, snapshot: &StateSnapshot) {
        let _g = self.infer_lock.lock().expect("infer_lock poisoned");
        const SNAP_MAGIC: u32 = 0x534B_4357; // "WCKS"
        let mut image = Vec::with_capacity(8 + snapshot.byte_size());
        image.extend_from_slice(&SNAP_MAGIC.to_le_bytes());
        image.extend_from_slice(&(snapshot.seq_len as u32).to_le_bytes());
        for layer in &snapshot.layers {
            match layer {
                LayerSnapshot::Attention { k_data, v_data } => {
                    image.extend_from_slice(k_data);
                    image.extend_from_slice(v_data);
                }
                LayerSnapshot::Conv { buffer } => image.extend_from_slice(buffer),
                LayerSnapshot::AttentionCompressed { .. } => panic!("CUDA backend: compressed KV snapshots are not supported"),
            }
        }
        ffi::check(unsafe { ffi::wick_cuda_restore(self.h, image.as_ptr(), image.len() as u64) });
    }
}

/// `load_model_cuda`: the `BackendPreference::Cuda` arm of `engine::load_text_model` (engine.rs:1073-1102), to sit next
/// to `load_model_metal` in wick/src/model/mod.rs.
pub fn load_model_cuda(gguf: GgufFile, path: Option<&std::path::Path>, context_size: usize, device: i32) -> Result<Box<dyn Model>> {
    let arch = gguf.get_str("general.architecture").unwrap_or("unknown").to_string();
    let model_id = path.map(|p| p.to_string_lossy().into_owned()).unwrap_or_default();
    match arch.as_str() {
        "lfm2" => Ok(Box::new(CudaLfm2Model::from_gguf_with_id(gguf, context_size, device, model_id)?)),
        other => anyhow::bail!("unsupported architecture for CUDA: {other}"),
    }
}
