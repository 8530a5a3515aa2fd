"""Host-side mirror of wick's `Model` trait for the CUDA backend.

`CudaLfm2Model` has the methods of `trait Model` (wick/src/model/mod.rs:72-323) with the
same names, argument meaning and failure behaviour as wick's GPU backends: the sequence
state lives in the model (metal_lfm2.rs:170-277), every call also updates the caller's
`InferenceState.seq_len` (metal_lfm2.rs:2146-2147), misuse raises (wick asserts), and only
loading can fail with a recoverable error.  It would be written in Rust inside wick; Rust
is not available where this was built, so the mirror is Python over the same C ABI the
Rust glue would bind.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import threading
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import WickCudaError, check


@dataclasses.dataclass
class InferenceState:
    """The slice of wick's InferenceState (kv_cache.rs:115-130) a GPU backend touches."""
    seq_len: int = 0


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """wick::model::ModelConfig (model/mod.rs:28-46)."""
    architecture: str
    n_layers: int
    hidden_size: int
    intermediate_size: int
    n_heads: int
    n_kv_heads: int
    vocab_size: int
    max_seq_len: int
    rope_theta: float
    rms_norm_eps: float
    block_types: Tuple[str, ...]
    conv_kernel_size: Optional[int]
    kv_heads_per_layer: Tuple[int, ...]


def device_count() -> int:
    n = C.c_int32(0)
    check(_lib.load().wick_cuda_device_count(C.byref(n)))
    return n.value


class CudaLfm2Model:
    """`load_model_cuda(gguf, path, context_size)`: the `--device cuda` arm of
    engine::load_text_model (wick/src/engine.rs:1073-1102)."""

    def __init__(self, path: str, context_size: int = 4096, device: int = 0):
        self._lib = _lib.load()
        self._h = C.c_void_p()
        self._lock = threading.Lock()  # infer_lock, metal_lfm2.rs:254-267
        check(self._lib.wick_cuda_model_create_from_file(path.encode(), context_size, device, C.byref(self._h)))
        cfg = _lib.Config()
        check(self._lib.wick_cuda_model_config(self._h, C.byref(cfg)))
        kv = np.zeros(cfg.n_layers, np.uint32)
        check(self._lib.wick_cuda_model_kv_heads_per_layer(self._h, kv.ctypes.data, cfg.n_layers))
        self._config = ModelConfig(
            "lfm2", cfg.n_layers, cfg.hidden_size, cfg.intermediate_size, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size,
            cfg.max_seq_len, cfg.rope_theta, cfg.rms_norm_eps,
            tuple("Attention" if k else "GatedConv" for k in kv), cfg.conv_kernel_size, tuple(int(k) for k in kv))
        self.device = device

    @classmethod
    def from_bytes(cls, data: bytes, context_size: int = 4096, device: int = 0) -> "CudaLfm2Model":
        """WickEngine::from_bytes path (engine.rs:224-363): the GGUF image is in memory."""
        self = cls.__new__(cls)
        self._lib = _lib.load()
        self._h = C.c_void_p()
        self._lock = threading.Lock()
        buf = (C.c_uint8 * len(data)).from_buffer_copy(data)
        check(self._lib.wick_cuda_model_create(C.addressof(buf), len(data), context_size, device, C.byref(self._h)))
        cfg = _lib.Config()
        check(self._lib.wick_cuda_model_config(self._h, C.byref(cfg)))
        kv = np.zeros(cfg.n_layers, np.uint32)
        check(self._lib.wick_cuda_model_kv_heads_per_layer(self._h, kv.ctypes.data, cfg.n_layers))
        self._config = ModelConfig(
            "lfm2", cfg.n_layers, cfg.hidden_size, cfg.intermediate_size, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size,
            cfg.max_seq_len, cfg.rope_theta, cfg.rms_norm_eps,
            tuple("Attention" if k else "GatedConv" for k in kv), cfg.conv_kernel_size, tuple(int(k) for k in kv))
        self.device = device
        return self

    # ---- lifetime -----------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value:
            self._lib.wick_cuda_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- trait Model ----------------------------------------------------------
    def config(self) -> ModelConfig:
        return self._config

    def forward(self, tokens: Sequence[int], pos: int, state: InferenceState) -> np.ndarray:
        """Model::forward (mod.rs:74): single token -> logits [vocab]."""
        assert len(tokens) == 1, "CUDA forward expects single token"
        logits = np.empty(self._config.vocab_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_forward(self._h, int(tokens[0]), int(pos), logits.ctypes.data))
        state.seq_len += 1
        return logits

    def forward_greedy(self, tokens: Sequence[int], pos: int, state: InferenceState) -> int:
        """Model::forward_greedy (mod.rs:274): argmax on the GPU, 4-byte readback."""
        assert len(tokens) == 1, "CUDA forward expects single token"
        out = C.c_uint32(0)
        with self._lock:
            check(self._lib.wick_cuda_forward_greedy(self._h, int(tokens[0]), int(pos), C.byref(out)))
        state.seq_len += 1
        return out.value

    def forward_prefill(self, tokens: Sequence[int], start_pos: int, state: InferenceState) -> np.ndarray:
        """Model::forward_prefill (mod.rs:79): logits of the last token; start_pos == 0 resets."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        assert t.size > 0, "forward_prefill requires at least one token"
        logits = np.empty(self._config.vocab_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_forward_prefill(self._h, t.ctypes.data, t.size, int(start_pos), logits.ctypes.data))
        state.seq_len = start_pos + t.size
        return logits

    # ── embedding-input methods (mod.rs:172-267; lfm2.rs:2291-2350, :2452-2500) ─────────────────
    def supports_embedding_input(self) -> bool:
        return True

    def forward_prefill_from_embeddings(self, embeddings, n_tokens: int, start_pos: int, state: InferenceState) -> np.ndarray:
        """Frames [n_tokens][hidden] row-major instead of token ids; logits of the last frame."""
        e = np.ascontiguousarray(embeddings, dtype=np.float32).reshape(-1)
        assert n_tokens > 0, "forward_prefill_from_embeddings requires at least one frame"
        assert e.size == n_tokens * self._config.hidden_size, \
            f"embeddings.len() ({e.size}) != n_tokens ({n_tokens}) * hidden_size ({self._config.hidden_size})"
        logits = np.empty(self._config.vocab_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_forward_prefill_from_embeddings(self._h, e.ctypes.data, n_tokens, int(start_pos),
                                                                      logits.ctypes.data))
        state.seq_len = start_pos + n_tokens
        return logits

    def forward_from_embedding(self, embedding, pos: int, state: InferenceState) -> np.ndarray:
        e = np.ascontiguousarray(embedding, dtype=np.float32).reshape(-1)
        assert e.size == self._config.hidden_size
        logits = np.empty(self._config.vocab_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_forward_from_embedding(self._h, e.ctypes.data, int(pos), logits.ctypes.data))
        state.seq_len += 1
        return logits

    def forward_hidden_from_embedding(self, embedding, pos: int, state: InferenceState) -> np.ndarray:
        e = np.ascontiguousarray(embedding, dtype=np.float32).reshape(-1)
        assert e.size == self._config.hidden_size
        hid = np.empty(self._config.hidden_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_forward_hidden_from_embedding(self._h, e.ctypes.data, int(pos), hid.ctypes.data))
        state.seq_len += 1
        return hid

    def forward_embedding(self, tokens: Sequence[int], pos: int, state: InferenceState) -> np.ndarray:
        """The output-normed hidden state of one token step, before the logit projection (mod.rs:172-184)."""
        assert len(tokens) == 1
        hid = np.empty(self._config.hidden_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_forward_embedding(self._h, int(tokens[0]), int(pos), hid.ctypes.data))
        state.seq_len += 1
        return hid

    def forward_prefill_chunked(self, tokens: Sequence[int], start_pos: int, state: InferenceState, ubatch: int,
                                cancel: Optional[threading.Event] = None) -> Tuple[int, Optional[np.ndarray]]:
        """Default trait method (mod.rs:111-140): ubatch-sized forward_prefill calls, cancel polled
        after each chunk, ubatch == 0 means one chunk."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        ub = max(t.size, 1) if ubatch == 0 else ubatch
        consumed, last = 0, None
        self.last_chunked_device_ms = 0.0   # GPU time of the chunks of this call (CUDA events on the library's stream)
        for c0 in range(0, t.size, ub):
            chunk = t[c0:c0 + ub]
            last = self.forward_prefill(chunk, start_pos + consumed, state)
            self.last_chunked_device_ms += self.last_elapsed_ms()
            consumed += chunk.size
            if cancel is not None and cancel.is_set() and consumed < t.size:
                break
        return consumed, last

    def generate_greedy(self, first_token: int, n_steps: int, state: InferenceState) -> np.ndarray:
        """The greedy loop of Session::generate (session.rs:1186-1257) run on the GPU."""
        out = np.empty(n_steps, np.uint32)
        with self._lock:
            check(self._lib.wick_cuda_generate_greedy(self._h, int(first_token), int(n_steps), out.ctypes.data))
        state.seq_len += n_steps
        return out

    def supports_kv_shift(self) -> bool:
        return True

    def shift_kv(self, state: InferenceState, n_keep: int, shift: int) -> None:
        """Model::shift_kv (mod.rs:158-170): drop KV cells [n_keep, n_keep + shift), re-rotate the moved K rows."""
        assert shift > 0, "shift must be > 0"
        with self._lock:
            check(self._lib.wick_cuda_shift_kv(self._h, int(n_keep), int(shift)))
        state.seq_len -= shift

    def turboquant_supported(self) -> bool:
        return False

    def gpu_memory_bytes(self) -> int:
        v = C.c_uint64(0)
        check(self._lib.wick_cuda_gpu_memory_bytes(self._h, C.byref(v)))
        return v.value

    def snapshot_state(self) -> bytes:
        """Model::snapshot_state (mod.rs:301)."""
        with self._lock:
            n = C.c_uint64(0)
            check(self._lib.wick_cuda_snapshot_size(self._h, C.byref(n)))
            buf = np.empty(n.value, np.uint8)
            check(self._lib.wick_cuda_snapshot(self._h, buf.ctypes.data, n.value))
        return buf.tobytes()

    def restore_state(self, snapshot: bytes, state: Optional[InferenceState] = None) -> None:
        """Model::restore_state (mod.rs:311): also sets the internal seq_len."""
        buf = np.frombuffer(snapshot, np.uint8)
        with self._lock:
            check(self._lib.wick_cuda_restore(self._h, buf.ctypes.data, buf.size))
        if state is not None:
            state.seq_len = self.seq_len

    # ---- extras -----------------------------------------------------------------
    def reset(self, state: Optional[InferenceState] = None) -> None:
        with self._lock:
            check(self._lib.wick_cuda_reset(self._h))
        if state is not None:
            state.seq_len = 0

    @property
    def seq_len(self) -> int:
        v = C.c_uint32(0)
        check(self._lib.wick_cuda_seq_len(self._h, C.byref(v)))
        return v.value

    def last_elapsed_ms(self) -> float:
        """Device time of the GPU work of the last forward* / generate call (CUDA events on the
        model's stream), cf. wick's GpuTimer (metal_lfm2.rs:3922-3984)."""
        v = C.c_float(0)
        check(self._lib.wick_cuda_last_elapsed_ms(self._h, C.byref(v)))
        return v.value

    def kernel_launches(self) -> int:
        v = C.c_uint64(0)
        check(self._lib.wick_cuda_kernel_launches(self._h, C.byref(v)))
        return v.value

    def decode_path(self) -> str:
        """'persistent' (one kernel runs whole decode steps) or 'graph' (captured per-kernel graph)."""
        v = C.c_int32(0)
        check(self._lib.wick_cuda_decode_path(self._h, C.byref(v)))
        return "persistent" if v.value else "graph"

    _PREFILL_MODES = {"exact": 0, "tensor": 1, "exact-cuda-cores": 2}

    def prefill_mode(self) -> str:
        """'exact' (default: bit-exact GEMM, on the tensor cores when the model's sizes allow),
        'tensor' (fused-chain tcgen05 GEMM, logits equal to f32 rounding per product) or
        'exact-cuda-cores' (the bit-exact CUDA-core GEMM)."""
        v = C.c_int32(0)
        check(self._lib.wick_cuda_prefill_mode(self._h, C.byref(v)))
        return {n: k for k, n in self._PREFILL_MODES.items()}[v.value]

    def set_prefill_mode(self, mode: str) -> None:
        if mode not in self._PREFILL_MODES:
            raise ValueError("prefill mode must be one of " + ", ".join(self._PREFILL_MODES))
        check(self._lib.wick_cuda_set_prefill_mode(self._h, self._PREFILL_MODES[mode]))

    def prefill_uses_tensor_cores(self) -> bool:
        v = C.c_int32(0)
        check(self._lib.wick_cuda_prefill_uses_tensor_cores(self._h, C.byref(v)))
        return bool(v.value)

    def set_decode_attention(self, mode: str) -> None:
        """'exact' (default) or 'splitk' (opt-in, not bit-exact): see wick_cuda_set_decode_attention."""
        check(self._lib.wick_cuda_set_decode_attention(self._h, {"exact": 0, "splitk": 1}[mode]))

    def profile_enable(self, on: bool = True) -> None:
        """Per-category device timers of forward_prefill (WICK_PROFILE in wick's GPU backends); clears the totals."""
        check(self._lib.wick_cuda_profile_enable(self._h, 1 if on else 0))

    def profile_read(self) -> dict:
        """Milliseconds per kernel category accumulated since profile_enable()."""
        n = 8
        ms = (C.c_double * n)()
        check(self._lib.wick_cuda_profile_read(self._h, ms, n))
        return {self._lib.wick_cuda_profile_category_name(i).decode(): float(ms[i]) for i in range(n)}

    def decode_profile(self):
        """Timeline of the last decode step of the persistent kernel: (kinds [n], ns [n, 4])."""
        n = C.c_uint32(0)
        check(self._lib.wick_cuda_decode_profile(self._h, None, None, 0, C.byref(n)))
        ns = np.zeros((n.value + 4, 4), np.uint64)
        kinds = np.zeros(n.value + 4, np.int32)
        check(self._lib.wick_cuda_decode_profile(self._h, ns.ctypes.data, kinds.ctypes.data, n.value + 4, C.byref(n)))
        self.last_profile_detail = ns[n.value:].reshape(-1)  # stamps of the phase named by WICK_CUDA_PROF_PHASE
        return kinds[:n.value], ns[:n.value]

    def read_kv(self, layer: int) -> Tuple[np.ndarray, np.ndarray]:
        kv_dim = self._config.kv_heads_per_layer[layer] * (self._config.hidden_size // self._config.n_heads)
        rows = self.seq_len
        k = np.empty((rows, kv_dim), np.float32)
        v = np.empty((rows, kv_dim), np.float32)
        check(self._lib.wick_cuda_read_kv(self._h, layer, k.ctypes.data, v.ctypes.data))
        return k, v

    def read_conv_state(self, layer: int) -> np.ndarray:
        s = np.empty((self._config.conv_kernel_size - 1, self._config.hidden_size), np.float32)
        check(self._lib.wick_cuda_read_conv_state(self._h, layer, s.ctypes.data))
        return s


    def forward_sample(self, tokens: Sequence[int], pos: int, state: InferenceState, temperature: float, top_k: int, top_p: float,
                       r: float) -> int:
        """Model::forward + Sampler::sample (sampler.rs:64-158) with the logits kept on the GPU; r is the caller's
        uniform draw in [0, 1)."""
        assert len(tokens) == 1, "CUDA forward expects single token"
        nxt = C.c_uint32(0)
        with self._lock:
            check(self._lib.wick_cuda_forward_sample(self._h, int(tokens[0]), int(pos), temperature, int(top_k), top_p, r, C.byref(nxt)))
        state.seq_len += 1
        return nxt.value

    # ---- many sequences on one model (extension; not part of trait Model) ------
    def seq_create(self) -> int:
        """A new sequence slot (own KV caches, conv buffers, length) on this model's weights."""
        sid = C.c_uint32(0)
        with self._lock:
            check(self._lib.wick_cuda_seq_create(self._h, C.byref(sid)))
        return sid.value

    def seq_destroy(self, seq_id: int) -> None:
        with self._lock:
            check(self._lib.wick_cuda_seq_destroy(self._h, int(seq_id)))

    def seq_length(self, seq_id: int) -> int:
        n = C.c_uint32(0)
        check(self._lib.wick_cuda_seq_length(self._h, int(seq_id), C.byref(n)))
        return n.value

    def seq_prefill(self, seq_id: int, tokens: Sequence[int], start_pos: int) -> np.ndarray:
        """forward_prefill on a slot: logits of the last position."""
        toks = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty(self._config.vocab_size, np.float32)
        with self._lock:
            check(self._lib.wick_cuda_seq_prefill(self._h, int(seq_id), toks.ctypes.data, len(toks), int(start_pos), logits.ctypes.data))
        return logits

    def decode_batch(self, tokens: Sequence[int], seq_ids: Sequence[int]) -> np.ndarray:
        """One greedy step for every listed slot in one pass over the weights: next token per row."""
        toks, ids = np.ascontiguousarray(tokens, np.uint32), np.ascontiguousarray(seq_ids, np.uint32)
        assert len(toks) == len(ids)
        out = np.empty(len(toks), np.uint32)
        with self._lock:
            check(self._lib.wick_cuda_decode_batch(self._h, toks.ctypes.data, ids.ctypes.data, len(toks), out.ctypes.data))
        return out

    def decode_batch_steps(self, first_tokens: Sequence[int], seq_ids: Sequence[int], n_steps: int) -> np.ndarray:
        """n_steps greedy steps for the listed slots, kept on the device: tokens [n_steps, rows]."""
        toks, ids = np.ascontiguousarray(first_tokens, np.uint32), np.ascontiguousarray(seq_ids, np.uint32)
        assert len(toks) == len(ids)
        out = np.empty((int(n_steps), len(toks)), np.uint32)
        with self._lock:
            check(self._lib.wick_cuda_decode_batch_steps(self._h, toks.ctypes.data, ids.ctypes.data, len(toks), int(n_steps), out.ctypes.data))
        return out

    def decode_batch_logits(self, tokens: Sequence[int], seq_ids: Sequence[int]) -> np.ndarray:
        """One step for every listed slot, returning logits [rows, vocab] (Model::forward for many sequences)."""
        toks, ids = np.ascontiguousarray(tokens, np.uint32), np.ascontiguousarray(seq_ids, np.uint32)
        assert len(toks) == len(ids)
        out = np.empty((len(toks), self._config.vocab_size), np.float32)
        with self._lock:
            check(self._lib.wick_cuda_decode_batch_logits(self._h, toks.ctypes.data, ids.ctypes.data, len(toks), out.ctypes.data))
        return out


def load_model_cuda(path: str, context_size: int = 4096, device: int = 0) -> CudaLfm2Model:
    """Counterpart of load_model_metal (model/mod.rs:386-403)."""
    return CudaLfm2Model(path, context_size, device)
