//! The pieces `--device cuda` adds to wick/src/engine.rs, as new code only (the surrounding wick code is not
//! reproduced here).  Not compiled where it was written (no Rust toolchain there).
//!
//! 1. `enum BackendPreference` (engine.rs:65-76) gains a variant that carries the device ordinal:
//!        /// CUDA (NVIDIA, sm_100a). Requires the `cuda` feature. `--device cuda` or `--device cuda:N`.
//!        Cuda(u32),
//! 2. `BackendPreference::parse_str` (engine.rs:78-88) gains the arm produced by `parse_cuda_label` below, placed
//!    before the catch-all arm, and its error text lists `cuda`.
//! 3. `load_text_model` (engine.rs:1073-1102) gains the two arms of `cuda_arms!` below.
//! 4. `load_text_model_auto` keeps its order (metal, gpu, cpu): CUDA is opt-in by name.
//! 5. wick-ffi (wick-ffi/src/lib.rs:219-250): the UniFFI enum gains `Cuda { device: u32 }` mapped to
//!    `BackendPreference::Cuda(device)`; the Kotlin / Swift bindings are regenerated with cargo.

/// "cuda" -> Some(0), "cuda:3" -> Some(3), anything else -> None.  Call with the lower-cased label.
pub fn parse_cuda_label(label: &str) -> Option<u32> {
    let rest = label.strip_prefix("cuda")?;
    if rest.is_empty() {
        return Some(0);
    }
    rest.strip_prefix(':')?.parse::<u32>().ok()
}

// In `parse_str`:
//     other if parse_cuda_label(other).is_some() => Ok(Self::Cuda(parse_cuda_label(other).unwrap())),

// In `load_text_model`:
//     #[cfg(feature = "cuda")]
//     BackendPreference::Cuda(device) => model::load_model_cuda(gguf, path, cfg.context_size, device as i32)
//         .map_err(|e| WickError::Backend(format!("CUDA model load failed: {e}"))),
//     #[cfg(not(feature = "cuda"))]
//     BackendPreference::Cuda(_) => Err(WickError::Backend(
//         "CUDA backend not available (compile with --features cuda)".into(),
//     )),

#[cfg(test)]
mod tests {
    use super::parse_cuda_label;

    #[test]
    fn labels() {
        assert_eq!(parse_cuda_label("cuda"), Some(0));
        assert_eq!(parse_cuda_label("cuda:7"), Some(7));
        assert_eq!(parse_cuda_label("cuda:"), None);
        assert_eq!(parse_cuda_label("cuda7"), None);
        assert_eq!(parse_cuda_label("metal"), None);
    }
}
