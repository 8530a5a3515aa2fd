"""Operator-level entry points of libwick_cuda on torch CUDA tensors.

torch is only the device allocator here: every function hands raw device pointers to the
C ABI and launches on torch's current stream.  Names follow the wick functions they stand
in for (wick/src/backend/simd.rs, cpu.rs).
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import numpy as np
import torch

from . import _lib
from ._lib import check

DT_Q4_0, DT_Q8_0 = 2, 8
QTYPE_ID = {"q4_0": DT_Q4_0, "q8_0": DT_Q8_0}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor) -> int:
    assert t.is_cuda and t.is_contiguous()
    return t.data_ptr()


class QuantWeight:
    """A quantised [m, k] matrix resident on the GPU in the library's layout (WeightRef, lfm2.rs:19-25)."""

    def __init__(self, dtype: int, raw: np.ndarray, m: int, k: int):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        bb = 18 if dtype == DT_Q4_0 else 34
        assert raw.size == m * (k // 32) * bb, "raw block bytes do not match m x k"
        self._lib = _lib.load()
        self._h = C.c_void_p()
        self.dtype, self.m, self.k = dtype, m, k
        torch.cuda.init()
        check(self._lib.wick_cuda_weight_create(dtype, raw.ctypes.data, m, k, C.byref(self._h)))

    def close(self):
        if self._h.value:
            self._lib.wick_cuda_weight_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize_f32_to_q8_0(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """simd.rs:255-323 over the rows of x [n, k] -> (scales [n, k/32] f32, quants [n, k] i8)."""
    x = x.contiguous()
    n, k = (1, x.shape[0]) if x.dim() == 1 else x.shape
    s = torch.empty((n, k // 32), dtype=torch.float32, device=x.device)
    q = torch.empty((n, k), dtype=torch.int8, device=x.device)
    check(_lib.load().wick_cuda_quantize_q8_0(_ptr(x), n, k, _ptr(s), _ptr(q), _stream()))
    return s, q


def gemv_q8(w: QuantWeight, xs: torch.Tensor, xq: torch.Tensor) -> torch.Tensor:
    """gemv_q4_0_q8_0_neon / gemv_q8_0_q8_0_neon (simd.rs:328-415, :440-524)."""
    y = torch.empty(w.m, dtype=torch.float32, device=xq.device)
    check(_lib.load().wick_cuda_gemv_q8(w._h, _ptr(xs), _ptr(xq), _ptr(y), _stream()))
    return y


def gemm_q8(w: QuantWeight, bs: torch.Tensor, bq: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """gemm_q*_q8_0_neon (simd.rs:696-1019) over the n rows of bq; returns token-major [n, m]."""
    n = bq.shape[0]
    if out is None:
        out = torch.empty((n, w.m), dtype=torch.float32, device=bq.device)
    check(_lib.load().wick_cuda_gemm_q8(w._h, _ptr(bs), _ptr(bq), n, _ptr(out), _stream()))
    return out


def gemm_q8_tc(w: QuantWeight, bs: torch.Tensor, bq: torch.Tensor, want_sums: bool = False):
    """The tensor-core (tcgen05) form of gemm_q8: exact int32 block sums, one fused f32 chain per output
    in block order.  Returns out [n, m] (and the block sums [n, m, k/32] when asked).  Synchronises."""
    n = bq.shape[0]
    out = torch.empty((n, w.m), dtype=torch.float32, device=bq.device)
    sums = torch.empty((n, w.m, w.k // 32), dtype=torch.int32, device=bq.device) if want_sums else None
    check(_lib.load().wick_cuda_gemm_q8_tc(w._h, _ptr(bs), _ptr(bq), n, _ptr(out), _ptr(sums) if want_sums else None,
                                           _stream()))
    return (out, sums) if want_sums else out


def gemm_q8_tc_exact(w: QuantWeight, bs: torch.Tensor, bq: torch.Tensor) -> torch.Tensor:
    """gemm_q8 on the tensor cores with the reference's accumulation order: bit-identical to gemm_q8."""
    n = bq.shape[0]
    out = torch.empty((n, w.m), dtype=torch.float32, device=bq.device)
    check(_lib.load().wick_cuda_gemm_q8_tc_exact(w._h, _ptr(bs), _ptr(bq), n, _ptr(out), _stream()))
    return out


def block_sums(w: QuantWeight, xq: torch.Tensor) -> torch.Tensor:
    s = torch.empty((w.m, w.k // 32), dtype=torch.int32, device=xq.device)
    check(_lib.load().wick_cuda_block_sums(w._h, _ptr(xq), _ptr(s), _stream()))
    return s


def rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """cpu::rmsnorm (cpu.rs:577-594) on each row of x, in place."""
    n, dim = (1, x.shape[0]) if x.dim() == 1 else x.shape
    check(_lib.load().wick_cuda_rmsnorm(_ptr(x), _ptr(weight), n, dim, eps, _stream()))
    return x


def silu_mul_(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    check(_lib.load().wick_cuda_silu_mul(_ptr(gate), _ptr(up), gate.numel(), _stream()))
    return gate


def ggml_expf(x: torch.Tensor) -> torch.Tensor:
    y = torch.empty_like(x)
    check(_lib.load().wick_cuda_expf(_ptr(x), _ptr(y), x.numel(), _stream()))
    return y


def rope_(q: torch.Tensor, k: torch.Tensor, pos: int, n_heads: int, n_kv_heads: int, head_dim: int, freq_base: float):
    check(_lib.load().wick_cuda_rope(_ptr(q), _ptr(k), pos, n_heads, n_kv_heads, head_dim, freq_base, _stream()))
    return q, k


def qknorm_rope_kv_(q, k, v, q_norm, k_norm, eps: float, rope_cos, rope_sin, k_cache, v_cache, start_pos: int, n_heads: int,
                    n_kv_heads: int, head_dim: int):
    """Per-head RMSNorm of Q and K, RoPE from a (position, pair) cos / sin table, and the append of the rotated K rows
    and the V rows to the caches at rows start_pos.. (lfm2.rs:783-855) for the n rows of q [n, n_heads * head_dim]."""
    n = q.shape[0]
    check(_lib.load().wick_cuda_qknorm_rope_kv(_ptr(q), _ptr(k), _ptr(v), _ptr(q_norm), _ptr(k_norm), eps, _ptr(rope_cos), _ptr(rope_sin),
                                               _ptr(k_cache), _ptr(v_cache), n, start_pos, n_heads, n_kv_heads, head_dim, _stream()))
    return q


def attention_decode(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, seq) -> torch.Tensor:
    out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=q.device)
    check(_lib.load().wick_cuda_attention_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), n_heads, n_kv_heads,
                                                 head_dim, seq, _stream()))
    return out


def attention_decode_splitk(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, seq) -> torch.Tensor:
    """Opt-in split-K single-query attention (runs of 256 keys + merge); agrees with attention_decode within rounding."""
    out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=q.device)
    check(_lib.load().wick_cuda_attention_decode_splitk(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), n_heads, n_kv_heads,
                                                        head_dim, seq, _stream()))
    return out


def attention_prefill(q, k_cache, v_cache, n, start_pos, n_heads, n_kv_heads, head_dim, flash: bool) -> torch.Tensor:
    out = torch.empty((n, n_heads * head_dim), dtype=torch.float32, device=q.device)
    check(_lib.load().wick_cuda_attention_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), n, start_pos, n_heads,
                                                  n_kv_heads, head_dim, int(flash), _stream()))
    return out


def shortconv(proj: torch.Tensor, conv_w: torch.Tensor, state: torch.Tensor, kernel_size: int) -> torch.Tensor:
    n, three_hs = proj.shape
    hs = three_hs // 3
    out = torch.empty((n, hs), dtype=torch.float32, device=proj.device)
    check(_lib.load().wick_cuda_shortconv(_ptr(proj), _ptr(conv_w), _ptr(state), _ptr(out), n, hs, kernel_size, _stream()))
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    out = torch.empty(1, dtype=torch.int32, device=logits.device)
    check(_lib.load().wick_cuda_argmax(_ptr(logits), logits.numel(), _ptr(out), _stream()))
    return out


def sample_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, r: float) -> int:
    """Sampler::sample (sampler.rs:64-158) on device logits with the caller's uniform draw r."""
    out = torch.empty(1, dtype=torch.int32, device=logits.device)
    check(_lib.load().wick_cuda_sample_logits(_ptr(logits), logits.numel(), temperature, top_k, top_p, r, _ptr(out), _stream()))
    return int(out.item())


ARGMAX_NOALLOC_MAX = 4096 * 1024


def argmax_noalloc(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Same result as argmax() for callers that may not allocate: the scratch is a fixed array inside
    the library and the caller supplies `out` (one int32 on the device).  At most ARGMAX_NOALLOC_MAX
    logits.  Calls share that array, so keep them on one stream."""
    lib = _lib.load()
    code = lib.wick_cuda_argmax_noalloc(_ptr(logits), logits.numel(), _ptr(out), _stream())
    if code != 0:
        raise _lib.WickCudaError(code, lib.wick_cuda_argmax_noalloc_last_error().decode())
    return out
