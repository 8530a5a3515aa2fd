"""Pins the CPU oracle against the known answers and self-consistency identities of wick's
own unit tests for this path (no GPU needed)."""
import numpy as np
import pytest

import refcases as rc

F32 = np.float32


def _quant_cols(orc, inputs):
    return orc.quantize_q8_0(inputs)


# wick/src/quant.rs:502-547: Q4_0 dequantisation closed forms
def test_q4_0_dequant_known_values(orc):
    blk = np.concatenate([rc.f16_bits(1.0), np.full(16, 0x88, np.uint8)])
    assert np.all(np.abs(orc.dequant_row(orc.DT_Q4_0, blk, 32)) < 1e-3)
    qs = (np.arange(16) | (15 << 4)).astype(np.uint8)
    out = orc.dequant_row(orc.DT_Q4_0, np.concatenate([rc.f16_bits(0.5), qs]), 32)
    assert np.allclose(out[:16], (np.arange(16) - 8.0) * 0.5, atol=1e-3)
    assert np.allclose(out[16:], 3.5, atol=1e-3)


# quant.rs:549-566, :721-741 and simd.rs:1288-1332: block dot == dequantise . y (tol 1e-3)
@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
def test_block_dot_matches_dequant(orc, dtype):
    y = ((np.arange(32) - 16.0) * 0.1).astype(F32)
    if dtype == "q4_0":
        qs = ((np.arange(16) % 13) | ((np.arange(16) % 7) << 4)).astype(np.uint8)
        blk = np.concatenate([rc.f16_bits(0.3), qs])
        dt = orc.DT_Q4_0
    else:
        q = (np.arange(32) * 3 - 48).astype(np.int8)
        blk = np.concatenate([rc.f16_bits(0.3), q.view(np.uint8)])
        dt = orc.DT_Q8_0
    deq = orc.dequant_row(dt, blk, 32)
    expected = float(np.dot(deq.astype(np.float64), y.astype(np.float64)))
    xs, xq = orc.quantize_q8_0(y)
    got = float(orc.gemv(dt, blk, xs, xq, 1, 32)[0])
    # the integer path also quantises y to 8 bits: allow that error on top of the 1e-3
    assert abs(got - expected) < 1e-3 + 0.02 * abs(expected)


# simd.rs:1440-1623: batched GEMM == sequential GEMV (documented bit-identical, blas_parity.rs:20-24)
@pytest.mark.parametrize("m,k,n", rc.GEMM_SHAPES)
@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
def test_gemm_matches_sequential_gemv(orc, dtype, m, k, n):
    w, x = rc.gemm_case(m, k, n)
    raw = rc.build_q4_0_matrix(w, m, k) if dtype == "q4_0" else rc.build_q8_0_matrix(w, m, k)
    dt = orc.QTYPE_ID[dtype]
    bs, bq = _quant_cols(orc, x)
    out = orc.gemm(dt, raw, bs, bq, m, n, k)
    for j in range(n):
        y = orc.gemv(dt, raw, bs[j], bq[j], m, k)
        assert np.array_equal(out[:, j], y)
    # and against the closed form dequant(W) . dequant(Q8(x)) within 1e-4 relative
    from wick_b200.gguf_synth import dequantize
    W = dequantize(raw.reshape(m, -1), dtype, k).astype(np.float64)
    Xq = (bq.reshape(n, k // 32, 32).astype(np.float64) * bs[..., None].astype(np.float64)).reshape(n, k)
    ref = W @ Xq.T
    assert np.allclose(out, ref, rtol=1e-4, atol=1e-4)


def test_gemm_single_column(orc):
    m, k, w, x = rc.gemm_single_column_case()
    raw = rc.build_q4_0_matrix(w, m, k)
    bs, bq = _quant_cols(orc, x)
    assert np.array_equal(orc.gemm(orc.DT_Q4_0, raw, bs, bq, m, 1, k)[:, 0], orc.gemv(orc.DT_Q4_0, raw, bs[0], bq[0], m, k))


# wick/tests/bench_perf.rs:866-891: Q8_0 GEMM, scale 1/(row+1), quants -16..15, inputs 1.0 -> -16/(row+1)
def test_q8_0_gemm_known_answer(orc):
    m, k, n, raw, x, expected = rc.q8_0_gemm_known_answer()
    bs, bq = _quant_cols(orc, x)
    out = orc.gemm(orc.DT_Q8_0, raw, bs, bq, m, n, k)  # [m, n]
    # inputs 1.0 quantise to 127 * (1/127 as f16): the f16 scale is the only inexact step
    assert np.allclose(out.T, expected, rtol=2e-3)


# wick/tests/metal_shaders_parity.rs:521-617: Q4_0 GEMV generator, tolerance max_abs 1e-2 or max_rel 1e-3
@pytest.mark.parametrize("m,k", rc.METAL_GEMV_SHAPES)
def test_q4_0_gemv_metal_generator(orc, m, k):
    raw, x = rc.metal_q4_0_gemv_case(m, k)
    from wick_b200.gguf_synth import dequantize
    xs, xq = orc.quantize_q8_0(x)
    y = orc.gemv(orc.DT_Q4_0, raw, xs, xq, m, k)
    W = dequantize(raw.reshape(m, -1), "q4_0", k).astype(np.float64)
    xd = (xq.reshape(-1, 32).astype(np.float64) * xs.reshape(-1, 1).astype(np.float64)).reshape(-1)
    ref_q = W @ xd
    d = np.abs(y - ref_q)
    assert d.max() < 1e-2 or (d / np.maximum(np.abs(ref_q), 1e-6)).max() < 1e-3
    # against the f32-activation product the Metal kernels compute: only the 8-bit activation error remains
    ref_f = W @ x.astype(np.float64)
    assert np.abs(y - ref_f).max() < 0.02 * np.abs(ref_f).max()


def test_avx2_path_is_bit_identical_to_scalar(orc):
    rng = np.random.default_rng(7)
    from wick_b200 import gguf_synth as gs
    for dtype, fn in (("q4_0", gs.quantize_q4_0), ("q8_0", gs.quantize_q8_0)):
        for m, k in ((5, 32), (9, 96), (33, 2048), (7, 6912)):
            raw = fn(rng.standard_normal((m, k), dtype=F32) * F32(0.02))
            xs, xq = orc.quantize_q8_0(rng.standard_normal(k, dtype=F32))
            orc.set_simd(True)
            a = orc.gemv(orc.QTYPE_ID[dtype], raw, xs, xq, m, k)
            orc.set_simd(False)
            b = orc.gemv(orc.QTYPE_ID[dtype], raw, xs, xq, m, k)
            orc.set_simd(True)
            assert np.array_equal(a, b)


def unfused_case():
    """One row, three Q8_0 blocks, built so that acc = fl(fl(p*d) + acc) and fma(p, d, acc) differ:
    block 0 leaves lane 0 at -4096; block 2 adds p = 4097 times d = (1 + 2^-10)^2.
    Separate rounding gives 9.005859375, a fused multiply-add 9.00586032867431640625."""
    k = 96
    w = np.zeros((3, 34), np.uint8)
    xq = np.zeros(k, np.int8)
    w[0, 0:2] = rc.f16_bits(1.0)
    q = np.zeros(32, np.int8); q[0:4] = 64; q[16:20] = 64
    w[0, 2:] = q.view(np.uint8)
    xq[0:4] = -8; xq[16:20] = -8                        # p = 8 * 64 * -8 = -4096
    w[2, 0:2] = rc.f16_bits(1.0 + 2.0 ** -10)
    q = np.zeros(32, np.int8); q[0] = 127; q[1] = 33
    w[2, 2:] = q.view(np.uint8)
    xq[64] = 32; xq[65] = 1                             # p = 127*32 + 33 = 4097
    xs = np.array([1.0, 1.0, 1.0 + 2.0 ** -10], F32)
    return w.reshape(-1), xs, xq, k, F32(9.005859375), F32(9.00586032867431640625)


def test_scale_accumulate_is_not_fused(orc):
    """vmlaq_n_f32 is multiply THEN add (simd.rs:387); Rust never contracts."""
    raw, xs, xq, k, unfused, fused = unfused_case()
    assert unfused != fused
    for simd in (True, False):
        orc.set_simd(simd)
        y = orc.gemv(orc.DT_Q8_0, raw, xs, xq, 1, k)
        assert y[0] == unfused, (simd, y[0])
    orc.set_simd(True)


# cpu.rs:2277-2315
def test_rmsnorm_known_values(orc):
    eps = 1e-5
    rms = np.sqrt(F32(7.5) + F32(eps))
    got = orc.rmsnorm([1, 2, 3, 4], [1, 1, 1, 1], eps)
    assert np.allclose(got, np.array([1, 2, 3, 4], F32) / rms, atol=1e-5)
    rms = np.sqrt(F32(4.0) + F32(eps))
    got = orc.rmsnorm([2, 2], [3, 0.5], eps)
    assert np.allclose(got, [2 / rms * 3, 2 / rms * 0.5], atol=1e-5)


# metal_shaders_parity.rs:143-174 (tol 1e-4)
def test_rmsnorm_metal_generator(orc):
    x, w, eps = rc.metal_rmsnorm_case()
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + eps) * w
    assert np.abs(orc.rmsnorm(x, w, eps) - ref).max() < 1e-4


# cpu.rs:2317-2347
def test_silu_known_values(orc):
    g = orc.silu_mul([0.0, 1.0, -1.0, 5.0], [1, 1, 1, 1])
    assert abs(g[0]) < 1e-5 and abs(g[1] - 0.7311) < 1e-3 and abs(g[2] + 0.2689) < 1e-3 and abs(g[3] - 4.9665) < 1e-3
    g2 = orc.silu_mul([0.0, 1.0, -1.0, 5.0], [2.0, 3.0, 0.5, 1.0])
    assert np.allclose(g2, g * np.array([2.0, 3.0, 0.5, 1.0], F32), atol=1e-6)


# cpu.rs:2373-2390, :2772-2780
def test_softmax_known_values(orc):
    s = orc.softmax([1.0, 2.0, 3.0])
    assert abs(s.sum() - 1) < 1e-5 and s[0] < s[1] < s[2]
    assert np.allclose(s, [0.0900, 0.2447, 0.6652], atol=1e-3)
    s = orc.softmax([1000.0, 1001.0, 1002.0])
    assert abs(s.sum() - 1) < 1e-5 and np.all(np.isfinite(s))


# cpu.rs:2750-2770
def test_ggml_expf(orc):
    xs = np.array([0.0, 1.0, -1.0, 2.0, -5.0, -10.0, -50.0, 80.0], F32)
    got = orc.expf(xs).astype(np.float64)
    exp = np.exp(xs.astype(np.float64))
    assert np.all(np.abs((got - exp) / exp) < 1e-5)
    hi, lo = orc.expf([100.0, -200.0])
    assert (np.isinf(hi) or hi > 1e30) and lo < 1e-30


# cpu.rs:2782-2809 and metal_shaders_parity.rs:290-345 (tol 1e-5)
def test_rope(orc):
    q, k = orc.rope([1, 2, 3, 4], [5, 6, 7, 8], 0, 1, 1, 4, 10000.0)
    assert np.allclose(q, [1, 2, 3, 4], atol=1e-5) and np.allclose(k, [5, 6, 7, 8], atol=1e-5)
    q, k = orc.rope([1, 0, 0, 0], [1, 0, 0, 0], 10, 1, 1, 4, 10000.0)
    assert abs(q[0] - 1.0) > 1e-3 or abs(q[2]) > 1e-3
    nh, nkv, hd, pos, base, q, k, qe, ke = rc.metal_rope_case()
    qg, kg = orc.rope(q, k, pos, nh, nkv, hd, base)
    assert np.abs(qg - qe).max() < 1e-5 and np.abs(kg - ke).max() < 1e-5


# metal_shaders_parity.rs:348-426 (tol 1e-4)
def test_attention_metal_generator(orc):
    nh, nkv, hd, seq, q, k, v, exp = rc.metal_attention_case()
    group = nh // nkv
    out = np.concatenate([orc.attention_naive(q[h * hd:(h + 1) * hd], k, v, nkv * hd, (h // group) * hd, hd,
                                              1.0 / np.sqrt(F32(hd)), seq) for h in range(nh)])
    assert np.abs(out - exp).max() < 1e-4


# cpu.rs:3011-3144: flash == naive within 1e-4
def test_flash_attention_matches_naive(orc):
    nh, nkv, hd, n, sp, q_mat, kc, vc = rc.flash_vs_naive_case()
    group, kv_dim = nh // nkv, nkv * hd
    scale = F32(1.0) / np.sqrt(F32(hd))
    for kv_h in range(nkv):
        fl = orc.flash_attention_gqa(q_mat, kc, vc, kv_h * group, group, n, n, kv_dim, kv_h * hd, hd, scale, sp)
        for g in range(group):
            h = kv_h * group + g
            for j in range(n):
                qh = np.ascontiguousarray(q_mat[h * hd:(h + 1) * hd, j])
                nv = orc.attention_naive(qh, kc, vc, kv_dim, kv_h * hd, hd, scale, sp + j + 1)
                assert np.abs(fl[g, j] - nv).max() < 1e-4


def test_attn_scores_seq_len_zero(orc):
    assert orc.attn_scores(np.zeros(64, F32), np.zeros(0, F32), 64, 0, 64, 0.125, 0).size == 0


# metal_shaders_parity.rs:710-752: rolling-state conv (checked through a one-layer state walk in
# test_host_logic; here the closed form itself)
def test_conv_closed_form_is_plain_f32(orc):
    hs, ks, inp, buf, w, exp = rc.metal_conv_case()
    ref = (buf[0] * w[:, 0]).astype(F32)
    ref = (ref + (buf[1] * w[:, 1]).astype(F32)).astype(F32)
    ref = (ref + (inp * w[:, 2]).astype(F32)).astype(F32)
    assert np.array_equal(ref, exp)


# wick/src/sampler.rs:8-19
def test_argmax_rule(orc):
    assert orc.argmax([1.0, 3.0, 2.0]) == 1
    assert orc.argmax([1.0, 3.0, 3.0, 0.0]) == 2          # last of equal maxima
    assert orc.argmax([np.nan, -1.0, np.nan]) == 1        # NaN never selected
    assert orc.argmax([-0.0, 0.0, -0.0]) == 1             # +0.0 ranks above -0.0
    assert orc.argmax([0.0, -0.0]) == 0
    assert orc.argmax([np.nan, np.nan]) == 1              # all NaN -> all -inf -> last
    assert orc.argmax([-np.inf, np.nan]) == 1


# simd.rs:255-323
def test_q8_0_activation_quantiser(orc):
    x = np.zeros(64, F32)
    x[32:] = np.linspace(-3, 3, 32, dtype=F32)
    s, q = orc.quantize_q8_0(x)
    assert s[0] == 0 and np.all(q[:32] == 0)                     # d == 0 -> id = 0
    d = F32(3.0) / F32(127.0)
    assert s[1] == np.float32(np.float16(d))                     # scale goes through f16
    inv = F32(1.0) / d
    assert np.array_equal(q[32:], np.rint(x[32:] * inv).astype(np.int8))  # ties to even
    # round-half-even, not half-away: 0.5 -> 0, 1.5 -> 2, 2.5 -> 2
    x = np.zeros(32, F32); x[0] = 127.0; x[1] = 0.5; x[2] = 1.5; x[3] = 2.5; x[4] = -2.5
    s, q = orc.quantize_q8_0(x)
    assert list(q[:5]) == [127, 0, 2, 2, -2]
