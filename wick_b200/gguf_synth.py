"""Seeded synthetic LFM2 / LFM2.5 GGUF files (numpy only).

wick's benchmarks run on public LFM2 checkpoints.  Those are not available
offline, so this module writes random-init models of the same architecture and
tensor shapes as GGUF v3 files that carry exactly the metadata keys and value
types wick's loader insists on (wick/src/model/lfm2.rs:105-148: UINT32 sizes,
FLOAT32 rope base / eps, an INT32 *array* for head_count_kv) and the tensor
names it resolves (lfm2.rs:188-285).  A minimal `tokenizer.ggml.tokens` array
is included because the engine refuses to load a file without one
(wick/src/tokenizer.rs:46-48).

The Q4_0 / Q8_0 quantisers restate ggml's reference row quantisers
(`quantize_row_q4_0_ref`, `quantize_row_q8_0_ref`): Q4_0 scale = (signed value
of largest magnitude) / -8, Q8_0 scale = amax / 127 with round-half-away.
"""
from __future__ import annotations

import dataclasses
import hashlib
import os
import struct
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747
GGUF_VERSION = 3
GGUF_ALIGNMENT = 32

# metadata value type ids (wick/src/gguf.rs:20-33)
T_UINT32, T_INT32, T_FLOAT32, T_STRING, T_ARRAY = 4, 5, 6, 8, 9
# tensor type ids (wick/src/gguf.rs:36-52)
GGML_F32, GGML_Q4_0, GGML_Q8_0 = 0, 2, 8

QK = 32  # elements per quantised block


@dataclasses.dataclass(frozen=True)
class Lfm2Spec:
    """Architecture of one synthetic model."""

    name: str
    hidden: int
    n_layers: int
    attn_layers: Tuple[int, ...]
    n_heads: int
    n_kv_heads: int
    ffn: int
    vocab: int
    context_length: int
    conv_kernel: int = 3
    rope_theta: float = 1_000_000.0
    rms_eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def quant_bytes(self, qtype: str) -> int:
        """Bytes of all quantised matmul weights (each read once per decoded token)."""
        bb = {"q4_0": 18, "q8_0": 34}[qtype]
        hs, f = self.hidden, self.ffn
        per_conv = 3 * hs * hs + hs * hs
        per_attn = hs * hs + 2 * self.kv_dim * hs + hs * hs
        ffn = 3 * hs * f
        n_attn = len(self.attn_layers)
        params = (self.n_layers - n_attn) * per_conv + n_attn * per_attn + self.n_layers * ffn
        params += self.vocab * hs
        return params // QK * bb

    def decode_bytes_per_token(self, qtype: str) -> int:
        """Algorithmic HBM bytes of one decode step: every quantised weight once (the tied
        vocabulary head included) plus the one embedding row that is looked up."""
        bb = {"q4_0": 18, "q8_0": 34}[qtype]
        return self.quant_bytes(qtype) + self.hidden // QK * bb


_LFM2_ATTN = (2, 5, 8, 10, 12, 14)

SPECS: Dict[str, Lfm2Spec] = {
    # 350M-class (LFM2-350M shapes)
    "lfm2-350m": Lfm2Spec("lfm2-350m", 1024, 16, _LFM2_ATTN, 16, 8, 4608, 65536, 8192),
    # 1.6B-class (LFM2.5-1.6B shapes)
    "lfm2.5-1.6b": Lfm2Spec("lfm2.5-1.6b", 2048, 16, _LFM2_ATTN, 32, 8, 6912, 65536, 8192),
    # small shapes for parity tests that a CPU reference finishes in seconds
    "tiny": Lfm2Spec("tiny", 256, 4, (1, 3), 4, 2, 512, 512, 1024),
    "tiny-wide": Lfm2Spec("tiny-wide", 512, 5, (2, 4), 8, 2, 1152, 1024, 2048),
    "tiny-hd128": Lfm2Spec("tiny-hd128", 512, 3, (1,), 4, 2, 768, 512, 1024),   # 128-wide heads
    "tiny-longctx": Lfm2Spec("tiny-longctx", 256, 4, (1, 3), 4, 2, 512, 512, 40000),  # contexts beyond 12K positions
}


# ── quantisers ──────────────────────────────────────────────────────────────

def _roundf(v: np.ndarray) -> np.ndarray:
    """C `roundf`: nearest, halves away from zero, evaluated without a +0.5 add."""
    a = np.abs(v)
    fl = np.floor(a)
    return np.copysign(fl + np.floor(np.float32(2.0) * (a - fl)), v)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., k] -> uint8 [..., k/32*18] of ggml Q4_0 blocks (f16 d, 16 nibble bytes)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    assert k % QK == 0
    blk = x.reshape(-1, QK)
    idx = np.abs(blk).argmax(axis=1)
    mx = blk[np.arange(blk.shape[0]), idx]
    d = mx / np.float32(-8.0)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1.0) / d).astype(np.float32)
    q = np.trunc(blk * inv[:, None] + np.float32(8.5)).astype(np.int32)
    q = np.clip(q, 0, 15).astype(np.uint8)
    out = np.empty((blk.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(*x.shape[:-1], k // QK * 18)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., k] -> uint8 [..., k/32*34] of ggml Q8_0 blocks (f16 d, 32 int8)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    assert k % QK == 0
    blk = x.reshape(-1, QK)
    d = np.abs(blk).max(axis=1) / np.float32(127.0)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1.0) / d).astype(np.float32)
    q = _roundf(blk * inv[:, None]).astype(np.int8)
    out = np.empty((blk.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(*x.shape[:-1], k // QK * 34)


def dequantize(raw: np.ndarray, qtype: str, k: int) -> np.ndarray:
    """Inverse of the quantisers above: raw block bytes -> f32 [..., k]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if qtype == "q4_0":
        b = raw.reshape(-1, 18)
        d = b[:, :2].copy().view(np.float16).astype(np.float32)
        lo = (b[:, 2:] & 0x0F).astype(np.int32) - 8
        hi = (b[:, 2:] >> 4).astype(np.int32) - 8
        v = np.concatenate([lo, hi], axis=1).astype(np.float32) * d
    elif qtype == "q8_0":
        b = raw.reshape(-1, 34)
        d = b[:, :2].copy().view(np.float16).astype(np.float32)
        v = b[:, 2:].view(np.int8).astype(np.float32) * d
    else:
        raise ValueError(qtype)
    return v.reshape(*raw.shape[:-1], k)


GGML_Q6_K = 14
QK_K = 256          # elements of a Q6_K super-block
Q6_K_BYTES = 210    # ql[128] + qh[64] + scales[16] (i8) + d (f16), wick/src/quant.rs:63-70


def quantize_q6_k(x: np.ndarray) -> np.ndarray:
    """f32 [..., k] -> uint8 [..., k/256*210] of Q6_K super-blocks.  The FORMAT is ggml's (decoded by
    quant.rs:380-413); the choice of scales is a plain max-abs fit per 16-element sub-block, not ggml's
    iterative search (any valid encoding exercises the same decode and dot-product code)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    assert k % QK_K == 0
    sb = x.reshape(-1, 16, 16)                                    # [super-block][sub-block][16]
    sub_scale = np.abs(sb).max(axis=2) / np.float32(31.0)         # element ~= q * sub_scale, q in [-32, 31]
    d = (sub_scale.max(axis=1) / np.float32(127.0)).astype(np.float16).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d[:, None] > 0, np.rint(sub_scale / d[:, None]), 0).astype(np.int32)
    sc = np.clip(sc, 0, 127).astype(np.int8)
    eff = d[:, None] * sc.astype(np.float32)                      # what the decoder multiplies by
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff[:, :, None] > 0, np.rint(sb / eff[:, :, None]), 0)
    q = (np.clip(q, -32, 31).astype(np.int32) + 32).astype(np.uint8).reshape(-1, 256)   # 0..63
    out = np.zeros((q.shape[0], Q6_K_BYTES), dtype=np.uint8)
    ql, qh = out[:, :128], out[:, 128:192]
    for n in range(2):                                            # two passes of 128 values (quant.rs:393-410)
        base = q[:, 128 * n:128 * (n + 1)]
        q1, q2, q3, q4 = base[:, 0:32], base[:, 32:64], base[:, 64:96], base[:, 96:128]
        ql[:, 64 * n:64 * n + 32] = (q1 & 0xF) | ((q3 & 0xF) << 4)
        ql[:, 64 * n + 32:64 * n + 64] = (q2 & 0xF) | ((q4 & 0xF) << 4)
        qh[:, 32 * n:32 * n + 32] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    return out.reshape(*x.shape[:-1], k // QK_K * Q6_K_BYTES)


def dequantize_q6_k(raw: np.ndarray, k: int) -> np.ndarray:
    """dequantize_q6_k_block (quant.rs:380-413) in numpy: d * scale * q, evaluated left to right in f32."""
    b = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, Q6_K_BYTES)
    ql, qh = b[:, :128].astype(np.int32), b[:, 128:192].astype(np.int32)
    sc = b[:, 192:208].copy().view(np.int8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32).reshape(-1)
    out = np.empty((b.shape[0], 256), dtype=np.float32)
    for n in range(2):
        l, h = ql[:, 64 * n:64 * n + 64], qh[:, 32 * n:32 * n + 32]
        q1 = ((l[:, :32] & 0xF) | ((h & 3) << 4)) - 32
        q2 = ((l[:, 32:] & 0xF) | (((h >> 2) & 3) << 4)) - 32
        q3 = ((l[:, :32] >> 4) | (((h >> 4) & 3) << 4)) - 32
        q4 = ((l[:, 32:] >> 4) | (((h >> 6) & 3) << 4)) - 32
        for j, qq in enumerate((q1, q2, q3, q4)):
            scale = np.repeat(sc[:, 8 * n + 2 * j:8 * n + 2 * j + 2], 16, axis=1)      # is = l / 16
            out[:, 128 * n + 32 * j:128 * n + 32 * j + 32] = (d[:, None] * scale) * qq.astype(np.float32)
    return out.reshape(*raw.shape[:-1], k)


QUANTIZERS = {"q4_0": (quantize_q4_0, GGML_Q4_0), "q8_0": (quantize_q8_0, GGML_Q8_0), "q6_k": (quantize_q6_k, GGML_Q6_K)}
BLOCK_GEOMETRY = {"q4_0": (QK, 18), "q8_0": (QK, 34), "q6_k": (QK_K, Q6_K_BYTES)}  # elements, bytes per block


# ── GGUF v3 writer ──────────────────────────────────────────────────────────

def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key.encode()) + struct.pack("<I", vtype) + payload


def kv_u32(key: str, v: int) -> bytes:
    return _kv(key, T_UINT32, struct.pack("<I", v))


def kv_f32(key: str, v: float) -> bytes:
    return _kv(key, T_FLOAT32, struct.pack("<f", v))


def kv_str(key: str, v: str) -> bytes:
    return _kv(key, T_STRING, _s(v.encode()))


def kv_i32_array(key: str, vals: Sequence[int]) -> bytes:
    body = struct.pack("<IQ", T_INT32, len(vals)) + struct.pack(f"<{len(vals)}i", *vals)
    return _kv(key, T_ARRAY, body)


def kv_str_array(key: str, vals: Iterable[str]) -> bytes:
    vals = list(vals)
    body = struct.pack("<IQ", T_STRING, len(vals)) + b"".join(_s(v.encode()) for v in vals)
    return _kv(key, T_ARRAY, body)


def _align(n: int, a: int = GGUF_ALIGNMENT) -> int:
    return (n + a - 1) // a * a


class GgufWriter:
    """Streams tensors to disk so a 1.6B-class file never sits in memory twice."""

    def __init__(self, path: str, kvs: List[bytes], tensor_plan: List[Tuple[str, Tuple[int, ...], int, int]]):
        # tensor_plan: (name, numpy shape (rows..., k), ggml type, nbytes)
        self.path = path
        self.plan = tensor_plan
        head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensor_plan), len(kvs)) + b"".join(kvs)
        infos = []
        off = 0
        self.offsets = []
        for name, shape, gtype, nbytes in tensor_plan:
            dims = tuple(reversed(shape))  # ggml order: innermost first
            infos.append(_s(name.encode()) + struct.pack("<I", len(dims))
                         + struct.pack(f"<{len(dims)}Q", *dims) + struct.pack("<IQ", gtype, off))
            self.offsets.append(off)
            off = _align(off + nbytes)
        head += b"".join(infos)
        self.data_start = _align(len(head))
        self.f = open(path, "wb")
        self.f.write(head)
        self.f.write(b"\0" * (self.data_start - len(head)))
        self.i = 0

    def write_tensor(self, name: str, raw: np.ndarray) -> None:
        pname, _, _, nbytes = self.plan[self.i]
        assert pname == name, (pname, name)
        raw = np.ascontiguousarray(raw)
        assert raw.nbytes == nbytes, (name, raw.nbytes, nbytes)
        assert self.f.tell() == self.data_start + self.offsets[self.i]
        self.f.write(raw.tobytes() if raw.nbytes < (1 << 20) else memoryview(raw).cast("B"))
        self.f.write(b"\0" * (_align(nbytes) - nbytes))
        self.i += 1

    def close(self) -> None:
        assert self.i == len(self.plan)
        self.f.close()


def _tensor_list(spec: Lfm2Spec) -> List[Tuple[str, Tuple[int, ...], str]]:
    """(name, numpy shape, kind) with kind in {'quant', 'norm', 'conv'}."""
    hs, f, kv = spec.hidden, spec.ffn, spec.kv_dim
    t: List[Tuple[str, Tuple[int, ...], str]] = [
        ("token_embd.weight", (spec.vocab, hs), "quant"),
        ("token_embd_norm.weight", (hs,), "norm"),
    ]
    for i in range(spec.n_layers):
        p = f"blk.{i}."
        t.append((p + "attn_norm.weight", (hs,), "norm"))
        if i in spec.attn_layers:
            t += [
                (p + "attn_q.weight", (hs, hs), "quant"),
                (p + "attn_k.weight", (kv, hs), "quant"),
                (p + "attn_v.weight", (kv, hs), "quant"),
                (p + "attn_output.weight", (hs, hs), "quant"),
                (p + "attn_q_norm.weight", (spec.head_dim,), "norm"),
                (p + "attn_k_norm.weight", (spec.head_dim,), "norm"),
            ]
        else:
            t += [
                (p + "shortconv.in_proj.weight", (3 * hs, hs), "quant"),
                (p + "shortconv.conv.weight", (hs, spec.conv_kernel), "conv"),
                (p + "shortconv.out_proj.weight", (hs, hs), "quant"),
            ]
        t += [
            (p + "ffn_norm.weight", (hs,), "norm"),
            (p + "ffn_gate.weight", (f, hs), "quant"),
            (p + "ffn_up.weight", (f, hs), "quant"),
            (p + "ffn_down.weight", (hs, f), "quant"),
        ]
    return t


def write_lfm2_gguf(path: str, spec: Lfm2Spec, qtype: str, seed: int = 0,
                    weight_std: float = 0.02, norm_jitter: float = 0.0, embd_qtype: Optional[str] = None) -> str:
    """Write a random-init model.  Matmul weights and `token_embd` ~ N(0, weight_std)
    in f32 then quantised per 32-element block; norm weights 1.0 (plus an optional
    uniform jitter used by tests so that a dropped norm weight is noticed); conv
    weights N(0, weight_std) kept in f32.  `embd_qtype` ("q6_k": what llama.cpp's Q4_0 files carry)
    overrides the type of `token_embd` only."""
    def qt(name):
        return embd_qtype if (embd_qtype and name == "token_embd.weight") else qtype

    tensors = _tensor_list(spec)
    plan = []
    for name, shape, kind in tensors:
        if kind == "quant":
            be, bb = BLOCK_GEOMETRY[qt(name)]
            plan.append((name, shape, QUANTIZERS[qt(name)][1], shape[0] * (shape[1] // be) * bb))
        else:
            plan.append((name, shape, GGML_F32, int(np.prod(shape)) * 4))
    kv_heads = [spec.n_kv_heads if i in spec.attn_layers else 0 for i in range(spec.n_layers)]
    kvs = [
        kv_str("general.architecture", "lfm2"),
        kv_str("general.name", f"synthetic-{spec.name}-{qtype}-seed{seed}"),
        kv_u32("general.alignment", GGUF_ALIGNMENT),
        kv_u32("lfm2.block_count", spec.n_layers),
        kv_u32("lfm2.embedding_length", spec.hidden),
        kv_u32("lfm2.feed_forward_length", spec.ffn),
        kv_u32("lfm2.attention.head_count", spec.n_heads),
        kv_i32_array("lfm2.attention.head_count_kv", kv_heads),
        kv_u32("lfm2.vocab_size", spec.vocab),
        kv_u32("lfm2.context_length", spec.context_length),
        kv_u32("lfm2.shortconv.l_cache", spec.conv_kernel),
        kv_f32("lfm2.rope.freq_base", spec.rope_theta),
        kv_f32("lfm2.attention.layer_norm_rms_epsilon", spec.rms_eps),
        kv_str("tokenizer.ggml.model", "gpt2"),
        kv_str_array("tokenizer.ggml.tokens", (f"<t{i}>" for i in range(spec.vocab))),
    ]
    rng = np.random.default_rng(seed)
    tmp = path + ".tmp"
    w = GgufWriter(tmp, kvs, plan)
    for name, shape, kind in tensors:
        if kind == "quant":
            rows, k = shape
            be, bb = BLOCK_GEOMETRY[qt(name)]
            quant_fn = QUANTIZERS[qt(name)][0]
            out = np.empty((rows, k // be * bb), dtype=np.uint8)
            step = max(1, (1 << 24) // k)  # ~64 MB of f32 per chunk
            for r0 in range(0, rows, step):
                r1 = min(rows, r0 + step)
                vals = rng.standard_normal((r1 - r0, k), dtype=np.float32) * np.float32(weight_std)
                out[r0:r1] = quant_fn(vals)
            w.write_tensor(name, out)
        elif kind == "norm":
            v = np.ones(shape, dtype=np.float32)
            if norm_jitter:
                v += rng.uniform(-norm_jitter, norm_jitter, size=shape).astype(np.float32)
            w.write_tensor(name, v)
        else:
            v = rng.standard_normal(shape, dtype=np.float32) * np.float32(weight_std)
            w.write_tensor(name, v)
    w.close()
    os.replace(tmp, path)
    return path


def cached_model(spec_name: str, qtype: str, seed: int = 0, cache_dir: Optional[str] = None,
                 **kw) -> str:
    """Path of the seeded model file, generating it on first use."""
    spec = SPECS[spec_name]
    cache_dir = cache_dir or os.environ.get("WICK_SYNTH_CACHE", "/tmp/wick_b200_models")
    os.makedirs(cache_dir, exist_ok=True)
    tag = hashlib.sha1(repr((dataclasses.astuple(spec), qtype, seed, sorted(kw.items()))).encode()).hexdigest()[:10]
    path = os.path.join(cache_dir, f"{spec.name}-{qtype}-s{seed}-{tag}.gguf")
    if not os.path.exists(path):
        write_lfm2_gguf(path, spec, qtype, seed, **kw)
    return path


def random_prompt(n: int, vocab: int, seed: int = 1) -> np.ndarray:
    """Uniform-random token ids, the prompt distribution the benchmark configs name."""
    return np.random.default_rng(seed).integers(0, vocab, size=n, dtype=np.uint32)
