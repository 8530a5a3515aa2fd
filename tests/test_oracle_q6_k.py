"""CPU checks of the oracle's Q6_K restatement (block layout quant.rs:63-70, dequantisation quant.rs:380-413,
integer GEMV simd.rs:552-672) against an independent numpy decode, and of a model whose token_embd is Q6_K."""
import numpy as np

F32 = np.float32


def test_q6_k_dequant_matches_numpy(orc):
    from wick_b200 import gguf_synth as gs
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((5, 768)) * 0.03).astype(F32)
    raw = gs.quantize_q6_k(x)
    assert raw.shape == (5, 3 * 210)
    want = gs.dequantize_q6_k(raw, 768)
    assert np.abs(want - x).max() < 0.04 * np.abs(x).max()           # 6-bit quantiser round trip
    for r in range(5):
        got = orc.dequant_row(orc.DT_Q6_K, raw[r], 768)
        assert np.array_equal(got.view(np.uint32), want[r].view(np.uint32))


def test_q6_k_known_block(orc):
    """A hand-built super-block: every 6-bit value, scale and bit position can be told apart."""
    blk = np.zeros(210, np.uint8)
    q = (np.arange(256) * 7 + 3) % 64                                   # 0..63
    for n in range(2):
        b = q[128 * n:128 * n + 128]
        q1, q2, q3, q4 = b[0:32], b[32:64], b[64:96], b[96:128]
        blk[64 * n:64 * n + 32] = (q1 & 0xF) | ((q3 & 0xF) << 4)
        blk[64 * n + 32:64 * n + 64] = (q2 & 0xF) | ((q4 & 0xF) << 4)
        blk[128 + 32 * n:128 + 32 * n + 32] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    sc = (np.arange(16) - 5).astype(np.int8)
    blk[192:208] = sc.view(np.uint8)
    blk[208:210] = np.array([0.5], np.float16).view(np.uint8)
    got = orc.dequant_row(orc.DT_Q6_K, blk, 256)
    want = (F32(0.5) * sc[np.arange(256) // 16].astype(F32)) * (q.astype(F32) - 32)
    assert np.array_equal(got, want.astype(F32))
    # integer GEMV against a one-hot-ish activation: picks single weights back out
    x = np.zeros(256, F32)
    x[37] = 1.0
    xs, xq = orc.quantize_q8_0(x[None, :])
    y = orc.gemv(orc.DT_Q6_K, blk[None, :], xs[0], xq[0], 1, 256)
    assert np.isclose(y[0], want[37], rtol=1e-3)


def test_q6_k_gemv_close_to_float(orc):
    from wick_b200 import gguf_synth as gs
    rng = np.random.default_rng(2)
    m, k = 64, 1024
    w = (rng.standard_normal((m, k)) * 0.02).astype(F32)
    raw = gs.quantize_q6_k(w)
    x = rng.standard_normal(k).astype(F32)
    xs, xq = orc.quantize_q8_0(x[None, :])
    y = orc.gemv(orc.DT_Q6_K, raw, xs[0], xq[0], m, k)
    wd = gs.dequantize_q6_k(raw, k).astype(np.float64)
    xd = (xq[0].astype(np.float64).reshape(-1, 32) * xs[0][:, None]).reshape(-1)
    ref = wd @ xd
    assert np.abs(y - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max()) * 10


def test_model_with_q6_k_embedding(orc, model_dir):
    """token_embd in Q6_K (what llama.cpp's Q4_0 files carry): prefill == token-by-token, as for the other types."""
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir, embd_qtype="q6_k")
    a, b = orc.OracleModel(path, 64), orc.OracleModel(path, 64)
    toks = gs.random_prompt(20, gs.SPECS["tiny"].vocab, seed=5)
    lp = a.forward_prefill(toks, 0)
    for t in toks:
        ls = b.forward(int(t))
    assert np.array_equal(lp.view(np.uint32), ls.view(np.uint32))
    assert np.isfinite(lp).all() and np.abs(lp).max() > 0
