"""Inputs and expected values of wick's own unit tests for the decode / prefill path,
re-created from the formulas in those tests (each helper cites its source inside the wick
repository).  They pin the CPU oracle (tests marked CPU) and are reused as inputs of the
CUDA parity tests.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def f16_bits(x: float) -> np.ndarray:
    return np.array([x], dtype=np.float32).astype(np.float16).view(np.uint8)


# ── wick/src/backend/simd.rs:1371-1419: the test-only quantisers (d = amax/7, not ggml's) ──
def build_q4_0_matrix(values: np.ndarray, m: int, k: int) -> np.ndarray:
    v = values.astype(F32).reshape(m, k // 32, 32)
    amax = np.abs(v).max(axis=2)
    d = (amax / F32(7.0)).astype(F32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, F32(1.0) / d, F32(0)).astype(F32)
    q = np.minimum((v * inv[..., None] + F32(8.5)).astype(F32).astype(np.uint8), 15)  # `as u8` truncates
    out = np.empty((m, k // 32, 18), np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, k // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(-1)


def build_q8_0_matrix(values: np.ndarray, m: int, k: int) -> np.ndarray:
    v = values.astype(F32).reshape(m, k // 32, 32)
    amax = np.abs(v).max(axis=2)
    d = (amax / F32(127.0)).astype(F32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, F32(1.0) / d, F32(0)).astype(F32)
    x = (v * inv[..., None]).astype(F32)
    r = np.copysign(np.floor(np.abs(x) + F32(0.5)), x)  # f32::round: half away from zero
    q = np.clip(r, -128, 127).astype(np.int8)
    out = np.empty((m, k // 32, 34), np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, k // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(-1)


# simd.rs:1448-1460: weights ((i*17+3)%29)*0.1-1.4, inputs ((i*13+j*7+5)%23)*0.2-2.3
def gemm_case(m: int, k: int, n: int):
    i = np.arange(m * k)
    weights = (((i * 17 + 3) % 29).astype(F32) * F32(0.1) - F32(1.4)).astype(F32)
    ii = np.arange(k)
    inputs = np.stack([(((ii * 13 + j * 7 + 5) % 23).astype(F32) * F32(0.2) - F32(2.3)).astype(F32) for j in range(n)])
    return weights, inputs


# simd.rs:1598-1623: n=1 single-column case
def gemm_single_column_case():
    m, k = 4, 32
    weights = ((np.arange(m * k) % 11).astype(F32) * F32(0.3) - F32(1.5)).astype(F32)
    inputs = ((np.arange(k) % 7).astype(F32) * F32(0.5) - F32(1.75)).astype(F32)[None, :]
    return m, k, weights, inputs


GEMM_SHAPES = [(8, 64, 7), (8, 64, 5), (8, 64, 8), (8, 64, 11), (8, 64, 16)]  # simd.rs:1442-1594


# ── wick/tests/metal_shaders_parity.rs:521-537: Q4_0 GEMV generator ─────────────────
METAL_GEMV_SHAPES = [(256, 1024), (1024, 1024), (2048, 1024), (1024, 2048)]


def metal_q4_0_gemv_case(m: int, k: int):
    nb = k // 32
    i = np.arange(m * nb)
    d = (F32(0.05) + np.sin((i.astype(F32) * F32(0.0017)).astype(F32)).astype(F32) * F32(0.02)).astype(F32)
    j = np.arange(16)
    qs = ((i[:, None] * 17 + j[None, :] * 53) & 0xFF).astype(np.uint8)
    raw = np.empty((m * nb, 18), np.uint8)
    raw[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    raw[:, 2:] = qs
    x = np.sin((np.arange(k).astype(F32) * F32(0.013)).astype(F32)).astype(F32)
    return raw.reshape(-1), x


# ── wick/tests/bench_perf.rs:866-891: Q8_0 GEMM known answer ────────────────────────
def q8_0_gemm_known_answer():
    m, k, n = 64, 32, 4
    raw = np.empty((m, 34), np.uint8)
    for row in range(m):
        raw[row, 0:2] = f16_bits(1.0 / (row + 1.0))
        raw[row, 2:] = (np.arange(32, dtype=np.int16) - 16).astype(np.int8).view(np.uint8)
    x = np.ones((n, k), F32)
    expected = np.array([[-16.0 / (row + 1.0) for row in range(m)] for _ in range(n)], F32)  # [n][m]
    return m, k, n, raw.reshape(-1), x, expected


# ── wick/tests/metal_shaders_parity.rs:143-155 / :290-345 / :348-400 / :710-733 ─────
def metal_rmsnorm_case():
    n = 2048
    i = np.arange(n).astype(F32)
    x = (np.sin((i * F32(0.031)).astype(F32)) * F32(2.0)).astype(F32)
    w = (F32(0.5) + np.cos((i * F32(0.017)).astype(F32)) * F32(0.5)).astype(F32)
    return x, w, 1e-5


def metal_rope_case():
    n_heads, n_kv, hd, pos, base = 4, 2, 64, 7, 10000.0
    q = np.sin((np.arange(n_heads * hd).astype(F32) * F32(0.011)).astype(F32)).astype(F32)
    k = np.cos((np.arange(n_kv * hd).astype(F32) * F32(0.017)).astype(F32)).astype(F32)

    def apply(buf, heads):
        buf = buf.astype(np.float64).copy()
        half = hd // 2
        for h in range(heads):
            for d in range(half):
                freq = 1.0 / (base ** (2.0 * d / hd))
                ang = pos * freq
                s, c = np.sin(ang), np.cos(ang)
                i0, i1 = h * hd + d, h * hd + d + half
                x0, x1 = buf[i0], buf[i1]
                buf[i0], buf[i1] = x0 * c - x1 * s, x0 * s + x1 * c
        return buf.astype(F32)

    return n_heads, n_kv, hd, pos, base, q, k, apply(q, n_heads), apply(k, n_kv)


def metal_attention_case():
    n_heads, n_kv, hd, seq = 4, 2, 32, 16
    kv_dim = n_kv * hd
    q = (np.sin((np.arange(n_heads * hd).astype(F32) * F32(0.013)).astype(F32)) * F32(0.3)).astype(F32)
    k = (np.cos((np.arange(seq * kv_dim).astype(F32) * F32(0.007)).astype(F32)) * F32(0.3)).astype(F32)
    v = (np.sin((np.arange(seq * kv_dim).astype(F32) * F32(0.019)).astype(F32)) * F32(0.3)).astype(F32)
    scale = 1.0 / np.sqrt(hd)
    group = n_heads // n_kv
    exp = np.zeros(n_heads * hd, np.float64)
    K = k.reshape(seq, kv_dim).astype(np.float64)
    V = v.reshape(seq, kv_dim).astype(np.float64)
    for h in range(n_heads):
        off = (h // group) * hd
        s = K[:, off:off + hd] @ q[h * hd:(h + 1) * hd].astype(np.float64) * scale
        p = np.exp(s - s.max())
        p /= p.sum()
        exp[h * hd:(h + 1) * hd] = p @ V[:, off:off + hd]
    return n_heads, n_kv, hd, seq, q, k, v, exp.astype(F32)


def metal_conv_case():
    hs, ks = 128, 3
    dc = ks - 1
    inp = np.sin((np.arange(hs).astype(F32) * F32(0.03)).astype(F32)).astype(F32)
    buf = np.cos((np.arange(dc * hs).astype(F32) * F32(0.05)).astype(F32)).astype(F32).reshape(dc, hs)
    w = np.sin((np.arange(hs * ks).astype(F32) * F32(0.011)).astype(F32)).astype(F32).reshape(hs, ks)
    exp = np.zeros(hs, F32)
    for ch in range(hs):
        s = F32(0)
        for kk in range(dc):
            s = F32(s + F32(buf[kk, ch] * w[ch, kk]))
        s = F32(s + F32(inp[ch] * w[ch, dc]))
        exp[ch] = s
    return hs, ks, inp, buf, w, exp


# ── wick/src/backend/cpu.rs:3011-3144: flash vs naive, LCG 0xCAFEBABE ───────────────
def flash_vs_naive_case():
    n_heads, n_kv, hd, n, start_pos = 4, 2, 64, 8, 4
    hs, kv_dim, total = n_heads * hd, n_kv * hd, start_pos + n
    seed = 0xCAFEBABE
    mask = (1 << 64) - 1

    def draw(count):
        nonlocal seed
        out = np.empty(count, F32)
        for i in range(count):
            seed = (seed * 6364136223846793005 + 1) & mask
            v = (seed >> 33) & 0xFFFFFFFF
            if v >= 1 << 31:
                v -= 1 << 32  # `as i32`
            out[i] = F32(F32(v) * F32(1e-9))
        return out

    q_mat = draw(hs * n).reshape(hs, n)            # [hs, n] stride-n
    k_cache = draw(total * kv_dim).reshape(total, kv_dim)
    v_cache = draw(total * kv_dim).reshape(total, kv_dim)
    return n_heads, n_kv, hd, n, start_pos, q_mat, k_cache, v_cache
