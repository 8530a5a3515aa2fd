// wick/build.rs (cargo feature `cuda`): compiles libwick_cuda from its CUDA sources with nvcc for sm_100a and links it
// statically into the wick crate.  Not compiled where it was written (no Rust toolchain there); the nvcc command
// line is the one wick_b200/build.py uses.
//
// Expects the sources under $WICK_CUDA_SRC (default: ../wick_b200/csrc relative to the crate) and the public header
// under $WICK_CUDA_INCLUDE (default: ../include).
use std::{env, path::PathBuf, process::Command};

const SOURCES: &[&str] = &[
    "kernels_basic.cu",
    "kernels_gemv.cu",
    "kernels_attn.cu",
    "kernels_q6k.cu",
    "kernels_batch.cu",
    "kernels_sample.cu",
    "tp_comm.cu",
    "decode_mega.cu",
    "gemm_tc.cu",
    "argmax_noalloc.cu",
    "wick_cuda.cu",
];

fn main() {
    if env::var("CARGO_FEATURE_CUDA").is_err() {
        return;
    }
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    let src_dir = env::var("WICK_CUDA_SRC").map(PathBuf::from).unwrap_or_else(|_| manifest.join("../wick_b200/csrc"));
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    let mut objects = Vec::new();
    for s in SOURCES {
        let src = src_dir.join(s);
        println!("cargo:rerun-if-changed={}", src.display());
        let obj = out.join(s.replace(".cu", ".o"));
        let status = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo"])
            .arg("--fmad=false") // numerics contract: a*b+c is never contracted; fused steps are explicit fmaf calls
            .args(["-Xcompiler", "-fPIC", "-c"])
            .arg(&src)
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("nvcc not found: set NVCC or put the CUDA toolkit on PATH");
        assert!(status.success(), "nvcc failed on {}", src.display());
        objects.push(obj);
    }
    let lib = out.join("libwick_cuda.a");
    let status = Command::new("ar").arg("crs").arg(&lib).args(&objects).status().expect("ar not found");
    assert!(status.success(), "ar failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=wick_cuda");
    let cuda_lib = env::var("CUDA_LIB_DIR").unwrap_or_else(|_| "/usr/local/cuda/lib64".into());
    println!("cargo:rustc-link-search=native={cuda_lib}");
    println!("cargo:rustc-link-lib=cudart"); // (the driver's tensor-map encoder is looked up at run time through the runtime)
    println!("cargo:rustc-link-lib=stdc++");
}
