"""ctypes front end of the CPU oracle (oracle/wick_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.

The GGUF reader below is deliberately separate from the product's C++ parser so
that a parsing mistake cannot cancel out between the two sides of a parity test.
It follows the same rules as wick's loader (wick/src/gguf.rs:407-559: magic,
version 3 only, `general.alignment` default 32, absolute tensor offsets).
"""
from __future__ import annotations

import ctypes as C
import mmap
import os
import struct
import subprocess
from typing import Dict, List, Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libwick_oracle.so")

DT_Q4_0, DT_Q8_0, DT_Q6_K = 2, 8, 14
BLOCK_BYTES = {DT_Q4_0: 18, DT_Q8_0: 34}
QTYPE_ID = {"q4_0": DT_Q4_0, "q8_0": DT_Q8_0, "q6_k": DT_Q6_K}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "wick_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_f16_round.restype = C.c_float
        _lib.orc_f16_round.argtypes = [C.c_float]
        _lib.orc_argmax.restype = C.c_uint32
        _lib.orc_sample.restype = C.c_uint32
        _lib.orc_sample.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float]
        _lib.orc_model_create.restype = C.c_void_p
        _lib.orc_model_seq_len.restype = C.c_int
        _lib.orc_model_kv_rows.restype = C.c_int
        _lib.orc_model_shift_kv.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


def set_simd(on: bool) -> None:
    lib().orc_set_simd(int(on))


# ── kernels ─────────────────────────────────────────────────────────────────

def quantize_q8_0(x: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """x [..., k] f32 -> (scales [..., k/32] f32, quants [..., k] i8)."""
    x = _f32(x)
    k = x.shape[-1]
    n = x.size // k
    s = np.empty(x.shape[:-1] + (k // 32,), np.float32)
    q = np.empty(x.shape, np.int8)
    lib().orc_quantize_q8_0_rows(_p(x), C.c_int(n), C.c_int(k), _p(s), _p(q))
    return s, q


def gemv(dtype: int, a: np.ndarray, xs: np.ndarray, xq: np.ndarray, m: int, k: int) -> np.ndarray:
    a = np.ascontiguousarray(a, np.uint8)
    xs, xq = _f32(xs), np.ascontiguousarray(xq, np.int8)
    y = np.empty(m, np.float32)
    lib().orc_gemv(C.c_int(dtype), _p(a), _p(xs), _p(xq), _p(y), C.c_int(m), C.c_int(k))
    return y


def gemm(dtype: int, a: np.ndarray, bs: np.ndarray, bq: np.ndarray, m: int, n: int, k: int) -> np.ndarray:
    """Returns out [m, n] (row-major, the reference layout out[i*n+j])."""
    a = np.ascontiguousarray(a, np.uint8)
    bs, bq = _f32(bs), np.ascontiguousarray(bq, np.int8)
    out = np.empty((m, n), np.float32)
    lib().orc_gemm(C.c_int(dtype), _p(a), _p(bs), _p(bq), _p(out), C.c_int(m), C.c_int(n), C.c_int(k))
    return out


def block_sums(dtype: int, a: np.ndarray, xq: np.ndarray, m: int, k: int) -> Tuple[np.ndarray, np.ndarray]:
    a = np.ascontiguousarray(a, np.uint8)
    xq = np.ascontiguousarray(xq, np.int8)
    S = np.empty((m, k // 32), np.int32)
    P = np.empty((m, k // 32, 4), np.int32)
    lib().orc_block_sums(C.c_int(dtype), _p(a), _p(xq), C.c_int(m), C.c_int(k), _p(S), _p(P))
    return S, P


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    w = _f32(w)
    lib().orc_rmsnorm(_p(x), _p(w), C.c_int(x.size), C.c_float(eps))
    return x


def expf(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_expf(_p(x), _p(y), C.c_int(x.size))
    return y


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    g = _f32(gate).copy()
    u = _f32(up)
    lib().orc_silu_mul(_p(g), _p(u), C.c_int(g.size))
    return g


def softmax(x: np.ndarray) -> np.ndarray:
    x = _f32(x).copy()
    lib().orc_softmax(_p(x), C.c_int(x.size))
    return x


def rope(q: np.ndarray, k: np.ndarray, pos: int, n_heads: int, n_kv_heads: int, hd: int, base: float):
    q, k = _f32(q).copy(), _f32(k).copy()
    lib().orc_rope(_p(q), _p(k), C.c_int(pos), C.c_int(n_heads), C.c_int(n_kv_heads), C.c_int(hd), C.c_float(base))
    return q, k


def rope_table(n_pos: int, hd: int, base: float):
    c = np.empty((n_pos, hd // 2), np.float32)
    s = np.empty((n_pos, hd // 2), np.float32)
    lib().orc_rope_table(C.c_int(n_pos), C.c_int(hd), C.c_float(base), _p(c), _p(s))
    return c, s


def attention_naive(q, kc, vc, kv_dim, off, hd, scale, seq) -> np.ndarray:
    q, kc, vc = _f32(q), _f32(kc), _f32(vc)
    out = np.empty(hd, np.float32)
    lib().orc_attention_naive(_p(q), _p(kc), _p(vc), _p(out), C.c_int(kv_dim), C.c_int(off), C.c_int(hd),
                              C.c_float(scale), C.c_int(seq))
    return out


def attn_scores(q, kc, kv_dim, off, hd, scale, seq) -> np.ndarray:
    q, kc = _f32(q), _f32(kc)
    s = np.empty(seq, np.float32)
    lib().orc_attn_scores(_p(q), _p(kc), _p(s), C.c_int(kv_dim), C.c_int(off), C.c_int(hd), C.c_float(scale), C.c_int(seq))
    return s


def attn_values(scores, vc, kv_dim, off, hd, seq) -> np.ndarray:
    scores, vc = _f32(scores), _f32(vc)
    o = np.empty(hd, np.float32)
    lib().orc_attn_values(_p(scores), _p(vc), _p(o), C.c_int(kv_dim), C.c_int(off), C.c_int(hd), C.c_int(seq))
    return o


def flash_attention_gqa(q_mat, kc, vc, n_heads_start, group, n_queries, q_stride, kv_dim, kv_off, hd, scale, start_pos):
    q_mat, kc, vc = _f32(q_mat), _f32(kc), _f32(vc)
    out = np.empty((group, n_queries, hd), np.float32)
    lib().orc_flash_attention_gqa(_p(q_mat), _p(kc), _p(vc), _p(out), C.c_int(n_heads_start), C.c_int(group),
                                  C.c_int(n_queries), C.c_int(q_stride), C.c_int(kv_dim), C.c_int(kv_off),
                                  C.c_int(hd), C.c_float(scale), C.c_int(start_pos))
    return out


def argmax(x: np.ndarray) -> int:
    x = _f32(x)
    return int(lib().orc_argmax(_p(x), C.c_int(x.size)))


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, r: float) -> int:
    """Sampler::sample (sampler.rs:64-158) with the uniform draw r given by the caller."""
    x = _f32(logits)
    return int(lib().orc_sample(x.ctypes.data, C.c_int(x.size), C.c_float(temperature), C.c_int(top_k), C.c_float(top_p), C.c_float(r)))


def dequant_row(dtype: int, row: np.ndarray, k: int) -> np.ndarray:
    row = np.ascontiguousarray(row, np.uint8)
    out = np.empty(k, np.float32)
    lib().orc_dequant_row(C.c_int(dtype), _p(row), C.c_int(k), _p(out))
    return out


# ── GGUF reader (independent of the product's) ─────────────────────────────

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self.buf = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.meta: Dict[str, object] = {}
        self.meta_types: Dict[str, Tuple[int, Optional[int]]] = {}
        self.tensors: Dict[str, Tuple[Tuple[int, ...], int, int]] = {}  # name -> (ggml dims, type, abs offset)
        self._parse()

    def _parse(self) -> None:
        b = self.buf
        pos = 0

        def rd(fmt):
            nonlocal pos
            v = struct.unpack_from(fmt, b, pos)
            pos += struct.calcsize(fmt)
            return v[0]

        def rd_str():
            nonlocal pos
            n = rd("<Q")
            s = bytes(b[pos:pos + n]).decode("utf-8", "replace")
            pos += n
            return s

        def rd_val(t):
            if t in _SCALAR:
                return rd(_SCALAR[t]), None
            if t == 8:
                return rd_str(), None
            if t == 9:
                et = rd("<I")
                cnt = rd("<Q")
                return [rd_val(et)[0] for _ in range(cnt)], et
            raise ValueError(f"bad GGUF value type {t}")

        if len(b) < 24:
            raise ValueError("GGUF buffer too small")
        if rd("<I") != 0x46554747:
            raise ValueError("not a GGUF file")
        ver = rd("<I")
        if ver != 3:
            raise ValueError(f"unsupported GGUF version {ver}")
        n_t, n_kv = rd("<Q"), rd("<Q")
        for _ in range(n_kv):
            key = rd_str()
            t = rd("<I")
            v, et = rd_val(t)
            self.meta[key] = v
            self.meta_types[key] = (t, et)
        infos = []
        for _ in range(n_t):
            name = rd_str()
            nd = rd("<I")
            dims = tuple(rd("<Q") for _ in range(nd))
            tt = rd("<I")
            off = rd("<Q")
            infos.append((name, dims, tt, off))
        align = self.meta.get("general.alignment", 32) if self.meta_types.get("general.alignment", (None,))[0] == 4 else 32
        data0 = (pos + align - 1) // align * align
        for name, dims, tt, off in infos:
            self.tensors[name] = (dims, tt, data0 + off)

    def typed(self, key: str, t: int, et: Optional[int] = None):
        """Strict typed getter, like wick's get_u32 / get_f32 / get_i32_array."""
        if key not in self.meta or self.meta_types[key] != (t, et):
            return None
        return self.meta[key]

    def tensor_bytes(self, name: str) -> np.ndarray:
        dims, tt, off = self.tensors[name]
        n = int(np.prod(dims))
        if tt == 0:
            size = n * 4
        elif tt in BLOCK_BYTES:
            size = n // 32 * BLOCK_BYTES[tt]
        elif tt == DT_Q6_K:
            size = n // 256 * 210
        else:
            raise ValueError(f"tensor {name}: unsupported ggml type {tt}")
        return np.frombuffer(self.buf, dtype=np.uint8, count=size, offset=off)

    def f32(self, name: str) -> np.ndarray:
        dims, tt, _ = self.tensors[name]
        assert tt == 0, name
        return self.tensor_bytes(name).view(np.float32).copy()


# ── model ───────────────────────────────────────────────────────────────────

class _Weight(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("m", C.c_int32), ("k", C.c_int32)]


class _Layer(C.Structure):
    _fields_ = [("is_attn", C.c_int32), ("n_kv_heads", C.c_int32),
                ("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("conv_w", C.c_void_p),
                ("in_proj", _Weight), ("out_proj", _Weight), ("q", _Weight), ("k", _Weight), ("v", _Weight),
                ("o", _Weight), ("gate", _Weight), ("up", _Weight), ("down", _Weight)]


class _Desc(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32), ("n_heads", C.c_int32),
                ("vocab", C.c_int32), ("max_seq_len", C.c_int32), ("conv_kernel", C.c_int32),
                ("rope_theta", C.c_float), ("eps", C.c_float), ("output_norm", C.c_void_p), ("embd", _Weight),
                ("layers", C.POINTER(_Layer))]


class OracleModel:
    """wick's CPU `Lfm2Model` + one `InferenceState`, restated (lfm2.rs:97-338 for loading)."""

    def __init__(self, path: str, context_size: int = 4096):
        g = GgufFile(path)
        self.g = g
        if g.typed("general.architecture", 8) != "lfm2":
            raise ValueError("unsupported architecture")
        u32 = lambda k: g.typed("lfm2." + k, 4)
        self.n_layers = u32("block_count")
        self.hidden = u32("embedding_length")
        self.ffn = u32("feed_forward_length")
        self.n_heads = u32("attention.head_count")
        self.vocab = u32("vocab_size")
        for v, nme in ((self.n_layers, "block_count"), (self.hidden, "embedding_length"), (self.ffn, "feed_forward_length"),
                       (self.n_heads, "attention.head_count"), (self.vocab, "vocab_size")):
            if v is None:
                raise ValueError(f"missing lfm2.{nme}")
        ctx = u32("context_length")
        self.max_seq_len = min(context_size, ctx if ctx is not None else 128000)
        th = g.typed("lfm2.rope.freq_base", 6)
        self.rope_theta = th if th is not None else 1_000_000.0
        eps = g.typed("lfm2.attention.layer_norm_rms_epsilon", 6)
        self.eps = eps if eps is not None else 1e-5
        lc = u32("shortconv.l_cache")
        self.conv_kernel = lc if lc is not None else 3
        kvh = g.typed("lfm2.attention.head_count_kv", 9, 5)
        if kvh is None or len(kvh) < self.n_layers:
            raise ValueError("missing lfm2.attention.head_count_kv")
        self._keep: List[np.ndarray] = []

        def f32p(name):
            a = g.f32(name)
            self._keep.append(a)
            return a.ctypes.data

        def wref(name) -> _Weight:
            dims, tt, _ = g.tensors[name]
            if tt not in BLOCK_BYTES and not (tt == DT_Q6_K and name == "token_embd.weight"):
                raise ValueError(f"{name}: unsupported dtype {tt}")
            a = g.tensor_bytes(name)
            self._keep.append(a)
            return _Weight(a.ctypes.data, tt, dims[1] if len(dims) > 1 else 1, dims[0])

        layers = (_Layer * self.n_layers)()
        self.is_attn = []
        for i in range(self.n_layers):
            L = layers[i]
            p = f"blk.{i}."
            attn = (p + "attn_q.weight") in g.tensors
            self.is_attn.append(attn)
            L.is_attn = int(attn)
            L.attn_norm = f32p(p + "attn_norm.weight")
            L.ffn_norm = f32p(p + "ffn_norm.weight")
            L.gate, L.up, L.down = wref(p + "ffn_gate.weight"), wref(p + "ffn_up.weight"), wref(p + "ffn_down.weight")
            if attn:
                nkv = int(kvh[i])
                if nkv <= 0 or self.n_heads % nkv:
                    raise ValueError(f"layer {i}: bad n_kv_heads {nkv}")
                L.n_kv_heads = nkv
                L.q, L.k, L.v, L.o = (wref(p + f"attn_{n}.weight") for n in ("q", "k", "v", "output"))
                L.q_norm, L.k_norm = f32p(p + "attn_q_norm.weight"), f32p(p + "attn_k_norm.weight")
            else:
                L.n_kv_heads = 0
                L.in_proj, L.out_proj = wref(p + "shortconv.in_proj.weight"), wref(p + "shortconv.out_proj.weight")
                L.conv_w = f32p(p + "shortconv.conv.weight")
        self._layers = layers
        self.kv_heads = [int(layers[i].n_kv_heads) for i in range(self.n_layers)]
        d = _Desc(self.n_layers, self.hidden, self.ffn, self.n_heads, self.vocab, self.max_seq_len, self.conv_kernel,
                  self.rope_theta, self.eps, f32p("token_embd_norm.weight"), wref("token_embd.weight"), layers)
        self._desc = d
        self.h = C.c_void_p(lib().orc_model_create(C.byref(d)))

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        lib().orc_model_reset(self.h)

    @property
    def seq_len(self) -> int:
        return lib().orc_model_seq_len(self.h)

    def forward(self, token: int, want_hidden: bool = False):
        logits = np.empty(self.vocab, np.float32)
        hid = np.empty(self.hidden, np.float32) if want_hidden else None
        lib().orc_model_forward(self.h, C.c_uint32(int(token)), _p(logits), _p(hid) if want_hidden else None)
        return (logits, hid) if want_hidden else logits

    def forward_prefill(self, tokens, start_pos: int) -> np.ndarray:
        """One `Model::forward_prefill` call; start_pos == 0 starts a new sequence."""
        t = np.ascontiguousarray(tokens, np.uint32)
        assert t.size > 0
        if start_pos == 0:
            self.reset()
        logits = np.empty(self.vocab, np.float32)
        lib().orc_model_forward_prefill(self.h, _p(t), C.c_int(t.size), C.c_int(start_pos), _p(logits))
        return logits

    def shift_kv(self, n_keep: int, shift: int) -> None:
        """Model::shift_kv (lfm2.rs:2507-2516): n_keep context shift with RoPE re-rotation of the moved K rows."""
        if lib().orc_model_shift_kv(self.h, C.c_int(n_keep), C.c_int(shift)) != 0:
            raise ValueError(f"shift range out of bounds: n_keep={n_keep} + shift={shift} > seq_len={self.seq_len}")

    def forward_from_embedding(self, emb, want: str = "logits") -> np.ndarray:
        """forward_from_embedding (want="logits") / forward_hidden_from_embedding (want="hidden"), lfm2.rs:2295-2350."""
        e = np.ascontiguousarray(emb, np.float32)
        assert e.size == self.hidden
        logits = np.empty(self.vocab, np.float32) if want == "logits" else None
        hid = np.empty(self.hidden, np.float32) if want == "hidden" else None
        lib().orc_model_forward_from_embedding(self.h, _p(e), _p(logits) if logits is not None else None,
                                               _p(hid) if hid is not None else None)
        return logits if want == "logits" else hid

    def forward_embedding(self, token: int) -> np.ndarray:
        """forward_embedding (lfm2.rs:2326-2337): the output-normed hidden state of one token step."""
        return self.forward(token, want_hidden=True)[1]

    def forward_prefill_from_embeddings(self, emb, start_pos: int) -> np.ndarray:
        """forward_prefill_from_embeddings (lfm2.rs:2452-2500): frames [n][hidden] row-major."""
        e = np.ascontiguousarray(emb, np.float32)
        assert e.ndim == 2 and e.shape[1] == self.hidden and e.shape[0] > 0
        if start_pos == 0:
            self.reset()
        logits = np.empty(self.vocab, np.float32)
        lib().orc_model_forward_prefill_from_embeddings(self.h, _p(e), C.c_int(e.shape[0]), C.c_int(start_pos), _p(logits))
        return logits

    def forward_prefill_chunked(self, tokens, start_pos: int = 0, ubatch: int = 512) -> np.ndarray:
        """Default `forward_prefill_chunked` (model/mod.rs:111-140) without cancellation."""
        t = np.ascontiguousarray(tokens, np.uint32)
        ub = t.size if ubatch == 0 else ubatch
        logits = None
        for c0 in range(0, t.size, ub):
            logits = self.forward_prefill(t[c0:c0 + ub], start_pos + c0)
        return logits

    def generate_greedy(self, first_token: int, n_steps: int) -> np.ndarray:
        out = np.empty(n_steps, np.uint32)
        lib().orc_model_generate_greedy(self.h, C.c_uint32(int(first_token)), C.c_int(n_steps), _p(out))
        return out

    def kv(self, layer: int):
        rows = lib().orc_model_kv_rows(self.h, C.c_int(layer))
        kv_dim = self.kv_heads[layer] * self.head_dim
        k = np.empty((rows, kv_dim), np.float32)
        v = np.empty((rows, kv_dim), np.float32)
        if rows:
            lib().orc_model_get_kv(self.h, C.c_int(layer), _p(k), _p(v))
        return k, v

    def conv_state(self, layer: int) -> np.ndarray:
        s = np.empty((self.conv_kernel - 1, self.hidden), np.float32)
        lib().orc_model_get_conv_state(self.h, C.c_int(layer), _p(s))
        return s
