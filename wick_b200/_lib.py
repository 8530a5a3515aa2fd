"""ctypes binding of libwick_cuda.so (the C ABI declared in include/wick_cuda.h).

There is no CPU fallback: if the shared library is missing the import fails with
instructions to build it, and on a machine without a CUDA device every model call
returns the library's CUDA error.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libwick_cuda.so")

OK = 0
ERR_BAD_ARG, ERR_CUDA, ERR_OOM, ERR_UNSUPPORTED_DTYPE, ERR_CONTEXT_FULL, ERR_TIMEOUT, ERR_BAD_GGUF = -1, -2, -3, -4, -5, -6, -7
ERR_NAMES = {
    ERR_BAD_ARG: "BAD_ARG", ERR_CUDA: "CUDA", ERR_OOM: "OOM", ERR_UNSUPPORTED_DTYPE: "UNSUPPORTED_DTYPE",
    ERR_CONTEXT_FULL: "CONTEXT_FULL", ERR_TIMEOUT: "TIMEOUT", ERR_BAD_GGUF: "BAD_GGUF",
}


class WickCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"wick_cuda error {ERR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class Config(C.Structure):
    """wick_cuda_config == wick::model::ModelConfig (wick/src/model/mod.rs:28-46)."""
    _fields_ = [("n_layers", C.c_uint32), ("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32),
                ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("vocab_size", C.c_uint32),
                ("max_seq_len", C.c_uint32), ("conv_kernel_size", C.c_uint32), ("rope_theta", C.c_float),
                ("rms_norm_eps", C.c_float)]


_vp, _u32, _i32, _u64, _f = C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64, C.c_float

# name -> argtypes; every function returns int32 except the three noted below
SIGNATURES = {
    "wick_cuda_device_count": [C.POINTER(_i32)],
    "wick_cuda_model_create": [_vp, C.c_size_t, _u32, _i32, C.POINTER(_vp)],
    "wick_cuda_model_create_from_file": [C.c_char_p, _u32, _i32, C.POINTER(_vp)],
    "wick_cuda_model_config": [_vp, C.POINTER(Config)],
    "wick_cuda_model_kv_heads_per_layer": [_vp, _vp, _u32],
    "wick_cuda_gpu_memory_bytes": [_vp, C.POINTER(_u64)],
    "wick_cuda_forward": [_vp, _u32, _u32, _vp],
    "wick_cuda_forward_greedy": [_vp, _u32, _u32, C.POINTER(_u32)],
    "wick_cuda_forward_prefill": [_vp, _vp, _u32, _u32, _vp],
    "wick_cuda_forward_prefill_from_embeddings": [_vp, _vp, _u32, _u32, _vp],
    "wick_cuda_forward_from_embedding": [_vp, _vp, _u32, _vp],
    "wick_cuda_forward_hidden_from_embedding": [_vp, _vp, _u32, _vp],
    "wick_cuda_forward_embedding": [_vp, _u32, _u32, _vp],
    "wick_cuda_shift_kv": [_vp, _u32, _u32],
    "wick_cuda_set_prefill_mode": [_vp, _i32],
    "wick_cuda_prefill_mode": [_vp, C.POINTER(_i32)],
    "wick_cuda_prefill_uses_tensor_cores": [_vp, C.POINTER(_i32)],
    "wick_cuda_generate_greedy": [_vp, _u32, _u32, _vp],
    "wick_cuda_reset": [_vp],
    "wick_cuda_seq_len": [_vp, C.POINTER(_u32)],
    "wick_cuda_snapshot_size": [_vp, C.POINTER(_u64)],
    "wick_cuda_snapshot": [_vp, _vp, _u64],
    "wick_cuda_restore": [_vp, _vp, _u64],
    "wick_cuda_last_elapsed_ms": [_vp, C.POINTER(_f)],
    "wick_cuda_kernel_launches": [_vp, C.POINTER(_u64)],
    "wick_cuda_set_decode_attention": [_vp, _i32],
    "wick_cuda_attention_decode_splitk": [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp],
    "wick_cuda_profile_enable": [_vp, _i32],
    "wick_cuda_profile_read": [_vp, _vp, _u32],
    "wick_cuda_decode_profile": [_vp, _vp, _vp, _u32, C.POINTER(_u32)],
    "wick_cuda_debug_skew_barrier": [_vp, C.c_int64],
    "wick_cuda_decode_path": [_vp, C.POINTER(_i32)],
    "wick_cuda_read_kv": [_vp, _u32, _vp, _vp],
    "wick_cuda_read_conv_state": [_vp, _u32, _vp],
    "wick_cuda_forward_sample": [_vp, _u32, _u32, _f, _u32, _f, _f, C.POINTER(_u32)],
    "wick_cuda_sample_logits": [_vp, _u32, _f, _u32, _f, _f, _vp, _vp],
    "wick_cuda_seq_create": [_vp, C.POINTER(_u32)],
    "wick_cuda_seq_destroy": [_vp, _u32],
    "wick_cuda_seq_length": [_vp, _u32, C.POINTER(_u32)],
    "wick_cuda_seq_prefill": [_vp, _u32, _vp, _u32, _u32, _vp],
    "wick_cuda_decode_batch": [_vp, _vp, _vp, _u32, _vp],
    "wick_cuda_decode_batch_steps": [_vp, _vp, _vp, _u32, _u32, _vp],
    "wick_cuda_decode_batch_logits": [_vp, _vp, _vp, _u32, _vp],
    "wick_cuda_tp_comm_create": [_u32, _u32, _u32, C.POINTER(_vp)],
    "wick_cuda_tp_comm_export": [_vp, _vp],
    "wick_cuda_tp_comm_connect": [_vp, _vp],
    "wick_cuda_tp_partial_buffer": [_vp, C.POINTER(_vp)],
    "wick_cuda_tp_allreduce_add_rmsnorm_quant": [_vp, _vp, _vp, _f, _u32, _vp, _vp, _vp, _vp],
    "wick_cuda_tp_status": [_vp, _vp, C.POINTER(_u32)],
    "wick_cuda_weight_create": [_i32, _vp, _u32, _u32, C.POINTER(_vp)],
    "wick_cuda_quantize_q8_0": [_vp, _u32, _u32, _vp, _vp, _vp],
    "wick_cuda_gemv_q8": [_vp, _vp, _vp, _vp, _vp],
    "wick_cuda_gemm_q8": [_vp, _vp, _vp, _u32, _vp, _vp],
    "wick_cuda_gemm_q8_tc": [_vp, _vp, _vp, _u32, _vp, _vp, _vp],
    "wick_cuda_gemm_q8_tc_exact": [_vp, _vp, _vp, _u32, _vp, _vp],
    "wick_cuda_block_sums": [_vp, _vp, _vp, _vp],
    "wick_cuda_rmsnorm": [_vp, _vp, _u32, _u32, _f, _vp],
    "wick_cuda_silu_mul": [_vp, _vp, _u64, _vp],
    "wick_cuda_expf": [_vp, _vp, _u64, _vp],
    "wick_cuda_rope": [_vp, _vp, _u32, _u32, _u32, _u32, _f, _vp],
    "wick_cuda_qknorm_rope_kv": [_vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp],
    "wick_cuda_attention_decode": [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp],
    "wick_cuda_attention_prefill": [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _i32, _vp],
    "wick_cuda_shortconv": [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp],
    "wick_cuda_argmax": [_vp, _u32, _vp, _vp],
    "wick_cuda_argmax_noalloc": [_vp, _u32, _vp, _vp],
}
VOID_FUNCS = {"wick_cuda_model_destroy": [_vp], "wick_cuda_weight_destroy": [_vp], "wick_cuda_tp_comm_destroy": [_vp]}
ALL_SYMBOLS = sorted(list(SIGNATURES) + list(VOID_FUNCS) + ["wick_cuda_last_error", "wick_cuda_argmax_noalloc_last_error",
                                                            "wick_cuda_tp_last_error", "wick_cuda_profile_category_name"])

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m wick_b200.build` (needs nvcc). "
            "wick_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = _i32
    for name, args in VOID_FUNCS.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = None
    lib.wick_cuda_last_error.argtypes = []
    lib.wick_cuda_last_error.restype = C.c_char_p
    lib.wick_cuda_argmax_noalloc_last_error.argtypes = []
    lib.wick_cuda_argmax_noalloc_last_error.restype = C.c_char_p
    lib.wick_cuda_tp_last_error.argtypes = []
    lib.wick_cuda_tp_last_error.restype = C.c_char_p
    lib.wick_cuda_profile_category_name.argtypes = [_u32]
    lib.wick_cuda_profile_category_name.restype = C.c_char_p
    _lib = lib
    return lib


def check(code: int, message=None) -> None:
    """Raises on a non-zero status; `message` (a callable returning str) overrides the library's general error text
    for entry points that keep their own (the tensor-parallel communicator)."""
    if code != OK:
        if message is not None:
            raise WickCudaError(code, message())
        msg = load().wick_cuda_last_error()
        raise WickCudaError(code, msg.decode("utf-8", "replace") if msg else "")
