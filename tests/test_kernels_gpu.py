"""Parity of each CUDA operator with the CPU oracle, through the C ABI, on the same seeded
inputs.  Integer / index work and every f32 result are compared bit for bit unless a test
states a tolerance and why."""
import numpy as np
import pytest

import refcases as rc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.fixture(scope="module")
def ops(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from wick_b200 import ops
    return ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def bits(a):
    return np.ascontiguousarray(a, dtype=F32).view(np.uint32)


def assert_bit_equal(got, want, what=""):
    got, want = np.asarray(got, F32), np.asarray(want, F32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if not np.array_equal(bits(got), bits(want)):
        bad = np.flatnonzero(bits(got).ravel() != bits(want).ravel())
        i = bad[0]
        raise AssertionError(f"{what}: {bad.size}/{got.size} elements differ; first at {i}: "
                             f"got {got.ravel()[i]!r} want {want.ravel()[i]!r}; max abs diff {np.abs(got - want).max()}")


def rand_weights(rng, dtype, m, k, std=0.02):
    from wick_b200 import gguf_synth as gs
    fn = gs.QUANTIZERS[dtype][0]
    return fn(rng.standard_normal((m, k), dtype=F32) * F32(std)).reshape(-1)


# ── activation quantiser ──────────────────────────────────────────────────
@pytest.mark.parametrize("n,k", [(1, 32), (1, 2048), (3, 96), (17, 6912), (130, 1024)])
def test_quantize_q8_0(ops, orc, n, k):
    rng = np.random.default_rng(n * 1000 + k)
    x = rng.standard_normal((n, k), dtype=F32) * F32(rng.uniform(0.01, 30))
    x[0, :32] = 0                      # an all-zero block: d == 0
    x[-1, -32:] = 1e-30                # scale underflows f16
    if k >= 64:
        x[0, 32:64] = np.linspace(-2.5, 2.5, 32)   # exact halves after scaling
    s, q = ops.quantize_f32_to_q8_0(dev(x))
    so, qo = orc.quantize_q8_0(x)
    assert np.array_equal(host(q), qo)
    assert_bit_equal(host(s), so, "scales")


# ── GEMV ───────────────────────────────────────────────────────────────────────
GEMV_SHAPES = [(1, 32), (5, 64), (9, 96), (31, 160), (33, 1024), (256, 2048), (1024, 2048), (300, 6912), (2048, 4608)]


@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m,k", GEMV_SHAPES)
def test_gemv_bit_exact(ops, orc, dtype, m, k):
    rng = np.random.default_rng(m * 7 + k)
    raw = rand_weights(rng, dtype, m, k)
    x = rng.standard_normal(k, dtype=F32)
    xs, xq = orc.quantize_q8_0(x)
    w = ops.QuantWeight(orc.QTYPE_ID[dtype], raw, m, k)
    y = ops.gemv_q8(w, dev(xs), dev(xq))
    assert_bit_equal(host(y), orc.gemv(orc.QTYPE_ID[dtype], raw, xs, xq, m, k), f"gemv {dtype} {m}x{k}")
    # int32 block sums (the vdotq_s32 lanes added up) are exact
    S = ops.block_sums(w, dev(xq))
    So, _ = orc.block_sums(orc.QTYPE_ID[dtype], raw, xq, m, k)
    assert np.array_equal(host(S), So)


def test_gemv_unfused_scale_accumulate(ops, orc):
    from test_oracle_golden import unfused_case
    raw, xs, xq, k, unfused, fused = unfused_case()
    w = ops.QuantWeight(orc.DT_Q8_0, raw, 1, k)
    y = host(ops.gemv_q8(w, dev(xs), dev(xq)))
    assert y[0] == unfused and y[0] != fused


@pytest.mark.parametrize("m,k", rc.METAL_GEMV_SHAPES)
def test_gemv_metal_generator(ops, orc, m, k):
    """wick/tests/metal_shaders_parity.rs:521-617 inputs; its tolerance (1e-2 abs or 1e-3 rel)
    against the f64 product of the dequantised operands, and bit equality with the oracle."""
    from wick_b200.gguf_synth import dequantize
    raw, x = rc.metal_q4_0_gemv_case(m, k)
    xs, xq = orc.quantize_q8_0(x)
    w = ops.QuantWeight(orc.DT_Q4_0, raw, m, k)
    y = host(ops.gemv_q8(w, dev(xs), dev(xq)))
    assert_bit_equal(y, orc.gemv(orc.DT_Q4_0, raw, xs, xq, m, k))
    W = dequantize(raw.reshape(m, -1), "q4_0", k).astype(np.float64)
    xd = (xq.reshape(-1, 32).astype(np.float64) * xs.reshape(-1, 1)).reshape(-1)
    d = np.abs(y - W @ xd)
    assert d.max() < 1e-2 or (d / np.maximum(np.abs(W @ xd), 1e-6)).max() < 1e-3


# ── GEMM ───────────────────────────────────────────────────────────────────────
@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m,k,n", rc.GEMM_SHAPES + [(4, 32, 1)])
def test_gemm_reference_cases(ops, orc, dtype, m, k, n):
    """simd.rs:1440-1623: GEMM == sequential GEMV (here: bit-identical, and equal to the oracle)."""
    if (m, k, n) == (4, 32, 1):
        m, k, w_, x = rc.gemm_single_column_case()
    else:
        w_, x = rc.gemm_case(m, k, n)
    raw = rc.build_q4_0_matrix(w_, m, k) if dtype == "q4_0" else rc.build_q8_0_matrix(w_, m, k)
    dt = orc.QTYPE_ID[dtype]
    bs, bq = orc.quantize_q8_0(x)
    w = ops.QuantWeight(dt, raw, m, k)
    out = host(ops.gemm_q8(w, dev(bs), dev(bq)))          # [n, m]
    assert_bit_equal(out.T, orc.gemm(dt, raw, bs, bq, m, n, k), "gemm")
    for j in range(n):
        assert_bit_equal(out[j], host(ops.gemv_q8(w, dev(bs[j]), dev(bq[j]))), "gemm vs gemv")


def test_gemm_q8_0_known_answer(ops, orc):
    m, k, n, raw, x, expected = rc.q8_0_gemm_known_answer()
    bs, bq = orc.quantize_q8_0(x)
    w = ops.QuantWeight(orc.DT_Q8_0, raw, m, k)
    out = host(ops.gemm_q8(w, dev(bs), dev(bq)))
    assert np.allclose(out, expected, rtol=2e-3)
    assert_bit_equal(out.T, orc.gemm(orc.DT_Q8_0, raw, bs, bq, m, n, k))


@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m,k,n", [(33, 96, 1), (40, 2048, 8), (65, 1056, 33), (256, 2080, 130), (100, 6912, 17)])
def test_gemm_bit_exact_ragged(ops, orc, dtype, m, k, n):
    rng = np.random.default_rng(m + k + n)
    raw = rand_weights(rng, dtype, m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    bs, bq = orc.quantize_q8_0(x)
    w = ops.QuantWeight(orc.QTYPE_ID[dtype], raw, m, k)
    out = host(ops.gemm_q8(w, dev(bs), dev(bq)))
    assert_bit_equal(out.T, orc.gemm(orc.QTYPE_ID[dtype], raw, bs, bq, m, n, k), f"gemm {dtype} {m}x{k}x{n}")


@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("n", [1, 8, 128])
def test_matmul_sweep_shape(ops, orc, dtype, n):
    """The isolated quantised matmul sweep, m=6912 k=2048 (activation counts the oracle finishes in
    seconds): int32 block sums bit-exact, f32 outputs bit-exact (contract: relative 1e-5)."""
    m, k = 6912, 2048
    rng = np.random.default_rng(3)
    raw = rand_weights(rng, dtype, m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    bs, bq = orc.quantize_q8_0(x)
    w = ops.QuantWeight(orc.QTYPE_ID[dtype], raw, m, k)
    out = host(ops.gemm_q8(w, dev(bs), dev(bq)))
    ref = orc.gemm(orc.QTYPE_ID[dtype], raw, bs, bq, m, n, k).T
    assert np.abs(out - ref).max() <= 1e-5 * np.abs(ref).max()
    assert_bit_equal(out, ref)
    S = host(ops.block_sums(w, dev(bq[0])))
    assert np.array_equal(S, orc.block_sums(orc.QTYPE_ID[dtype], raw, bq[0], m, k)[0])


def test_gemm_linearity_large(ops, orc):
    """Size-independent property at the full sweep size (n = 4096): an integer GEMM row scales
    exactly with a power-of-two activation scale, and token order does not matter."""
    m, k, n = 512, 2048, 4096
    rng = np.random.default_rng(5)
    raw = rand_weights(rng, "q4_0", m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    w = ops.QuantWeight(orc.DT_Q4_0, raw, m, k)
    bs, bq = ops.quantize_f32_to_q8_0(dev(x))
    out = ops.gemm_q8(w, bs, bq)
    out2 = ops.gemm_q8(w, bs * 4.0, bq)
    assert torch.equal(out2, out * 4.0)
    perm = torch.randperm(n, device="cuda")
    assert torch.equal(ops.gemm_q8(w, bs[perm].contiguous(), bq[perm].contiguous()), out[perm])
    for j in (0, 1777, 4095):
        assert_bit_equal(host(out[j]), orc.gemv(orc.DT_Q4_0, raw, host(bs[j]), host(bq[j]), m, k))


# ── element-wise and norms ───────────────────────────────────────────────────────
def test_expf_bit_exact(ops, orc):
    x = np.concatenate([np.linspace(-110, 90, 20001, dtype=F32), np.array([0, -0.0, 88.37, 88.39, -103.9, -104.1, 127, -127], F32)])
    assert_bit_equal(host(ops.ggml_expf(dev(x))), orc.expf(x), "ggml_expf")


def test_silu_mul_bit_exact(ops, orc):
    rng = np.random.default_rng(2)
    g = (rng.standard_normal(6912 * 3, dtype=F32) * 4).astype(F32)
    u = rng.standard_normal(6912 * 3, dtype=F32)
    assert_bit_equal(host(ops.silu_mul_(dev(g), dev(u))), orc.silu_mul(g, u), "silu_mul")


@pytest.mark.parametrize("n,dim", [(1, 4), (1, 64), (3, 2048), (5, 1024), (2, 6912)])
def test_rmsnorm(ops, orc, n, dim):
    """f64 sum of squares is added in a different (fixed) order than the reference's serial loop;
    the sums agree to ~1e-15 relative, so the f32 results are expected bit-equal, and are required to
    be within 1 ulp."""
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((n, dim), dtype=F32) * 3
    w = rng.uniform(0.5, 1.5, dim).astype(F32)
    got = host(ops.rmsnorm_(dev(x), dev(w), 1e-5))
    ref = np.stack([orc.rmsnorm(x[i], w, 1e-5) for i in range(n)])
    ulp = np.abs(bits(got).astype(np.int64) - bits(ref).astype(np.int64))
    assert ulp.max() <= 1
    assert (ulp != 0).mean() < 1e-3


def test_rmsnorm_reference_cases(ops, orc):
    x, w, eps = rc.metal_rmsnorm_case()
    got = host(ops.rmsnorm_(dev(x[None, :]), dev(w), eps))[0]
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + eps) * w
    assert np.abs(got - ref).max() < 1e-4
    assert_bit_equal(got, orc.rmsnorm(x, w, eps))
    got = host(ops.rmsnorm_(dev(np.array([[1, 2, 3, 4]], F32)), dev(np.ones(4, F32)), 1e-5))[0]
    assert np.allclose(got, np.array([1, 2, 3, 4]) / np.sqrt(7.5 + 1e-5), atol=1e-5)


def test_rope_bit_exact(ops, orc):
    nh, nkv, hd, pos, base, q, k, qe, ke = rc.metal_rope_case()
    qg, kg = ops.rope_(dev(q), dev(k), pos, nh, nkv, hd, base)
    assert np.abs(host(qg) - qe).max() < 1e-5 and np.abs(host(kg) - ke).max() < 1e-5
    qo, ko = orc.rope(q, k, pos, nh, nkv, hd, base)
    assert_bit_equal(host(qg), qo, "rope q")
    assert_bit_equal(host(kg), ko, "rope k")
    rng = np.random.default_rng(0)
    for pos in (0, 1, 4095, 8191):
        q = rng.standard_normal(32 * 64, dtype=F32)
        k = rng.standard_normal(8 * 64, dtype=F32)
        qo, ko = orc.rope(q, k, pos, 32, 8, 64, 1e6)
        qg, kg = ops.rope_(dev(q), dev(k), pos, 32, 8, 64, 1e6)
        assert_bit_equal(host(qg), qo)
        assert_bit_equal(host(kg), ko)


def test_argmax_rule(ops, orc):
    cases = [[1.0, 3.0, 2.0], [1.0, 3.0, 3.0, 0.0], [np.nan, -1.0, np.nan], [-0.0, 0.0, -0.0], [0.0, -0.0],
             [np.nan, np.nan], [-np.inf, np.nan], [5.0]]
    for c in cases:
        assert int(host(ops.argmax(dev(np.array(c, F32))))[0]) == orc.argmax(c), c
    rng = np.random.default_rng(9)
    x = rng.standard_normal(65536, dtype=F32)
    x[[100, 40000, 65535]] = x.max() + 1           # three equal maxima: the last wins
    assert int(host(ops.argmax(dev(x)))[0]) == 65535 == orc.argmax(x)
    x[65535] = np.nan
    assert int(host(ops.argmax(dev(x)))[0]) == 40000 == orc.argmax(x)


# ── short conv ───────────────────────────────────────────────────────────────────
def _conv_ref(proj, w, state, ks):
    """forward_conv_block core in plain f32 steps (lfm2.rs:688-725), token by token."""
    n, hs = proj.shape[0], proj.shape[1] // 3
    dc = ks - 1
    st = state.copy()
    out = np.empty((n, hs), F32)
    for j in range(n):
        b, c, x = proj[j, :hs], proj[j, hs:2 * hs], proj[j, 2 * hs:]
        bx = (b * x).astype(F32)
        s = np.zeros(hs, F32)
        for kk in range(dc):
            s = (s + (st[kk] * w[:, kk]).astype(F32)).astype(F32)
        s = (s + (bx * w[:, dc]).astype(F32)).astype(F32)
        if dc > 0:
            st[:-1] = st[1:]
            st[-1] = bx
        out[j] = (c * s).astype(F32)
    return out, st


@pytest.mark.parametrize("n,hs,ks", [(1, 128, 3), (2, 64, 3), (1, 2048, 3), (7, 256, 3), (300, 1024, 3), (3, 64, 4), (1, 64, 2), (5, 32, 1)])
def test_shortconv_bit_exact(ops, n, hs, ks):
    rng = np.random.default_rng(n + hs)
    proj = rng.standard_normal((n, 3 * hs), dtype=F32)
    w = rng.standard_normal((hs, ks), dtype=F32)
    state = rng.standard_normal((max(ks - 1, 1), hs), dtype=F32)
    st = dev(state)
    out = ops.shortconv(dev(proj), dev(w), st, ks)
    ro, rs = _conv_ref(proj, w, state[: ks - 1], ks)
    assert_bit_equal(host(out), ro, "conv out")
    if ks > 1:
        assert_bit_equal(host(st)[: ks - 1], rs, "conv state")


def test_shortconv_reference_case(ops):
    """wick/tests/metal_shaders_parity.rs:710-752 with the gates set to one."""
    hs, ks, inp, buf, w, exp = rc.metal_conv_case()
    proj = np.concatenate([inp, np.ones(hs, F32), np.ones(hs, F32)])[None, :]   # b = input, c = 1, x = 1
    st = dev(buf)
    out = host(ops.shortconv(dev(proj), dev(w), st, ks))[0]
    assert np.abs(out - exp).max() < 1e-5
    assert_bit_equal(out, exp)
    assert_bit_equal(host(st), np.stack([buf[1], inp]))


def test_shortconv_chunking_invariance(ops):
    rng = np.random.default_rng(1)
    n, hs, ks = 50, 256, 3
    proj = rng.standard_normal((n, 3 * hs), dtype=F32)
    w = rng.standard_normal((hs, ks), dtype=F32)
    s1, s2 = dev(np.zeros((2, hs), F32)), dev(np.zeros((2, hs), F32))
    whole = ops.shortconv(dev(proj), dev(w), s1, ks)
    parts = torch.cat([ops.shortconv(dev(proj[a:b]), dev(w), s2, ks) for a, b in ((0, 1), (1, 2), (2, 33), (33, 50))])
    assert torch.equal(whole, parts) and torch.equal(s1, s2)


# ── attention ────────────────────────────────────────────────────────────────────
def _naive_ref(orc, q, kc, vc, n, start, nh, nkv, hd):
    out = np.empty((n, nh * hd), F32)
    scale = F32(1.0) / np.sqrt(F32(hd))
    for j in range(n):
        for h in range(nh):
            out[j, h * hd:(h + 1) * hd] = orc.attention_naive(q[j, h * hd:(h + 1) * hd], kc, vc, nkv * hd,
                                                              (h // (nh // nkv)) * hd, hd, scale, start + j + 1)
    return out


def test_attention_reference_case(ops, orc):
    nh, nkv, hd, seq, q, k, v, exp = rc.metal_attention_case()
    out = host(ops.attention_decode(dev(q), dev(k), dev(v), nh, nkv, hd, seq))
    assert np.abs(out - exp).max() < 1e-4
    assert_bit_equal(out, _naive_ref(orc, q[None, :], k, v, 1, seq - 1, nh, nkv, hd)[0])


@pytest.mark.parametrize("seq", [1, 2, 31, 32, 33, 127, 128, 129, 640, 1500])
def test_attention_decode_bit_exact(ops, orc, seq):
    nh, nkv, hd = 8, 2, 64
    rng = np.random.default_rng(seq)
    q = rng.standard_normal(nh * hd, dtype=F32)
    kc = rng.standard_normal((seq, nkv * hd), dtype=F32)
    vc = rng.standard_normal((seq, nkv * hd), dtype=F32)
    out = host(ops.attention_decode(dev(q), dev(kc), dev(vc), nh, nkv, hd, seq))
    assert_bit_equal(out, _naive_ref(orc, q[None, :], kc, vc, 1, seq - 1, nh, nkv, hd)[0], f"decode attention seq={seq}")


@pytest.mark.parametrize("n,start", [(1, 0), (7, 0), (17, 5), (33, 100), (130, 0)])
def test_attention_prefill_naive_bit_exact(ops, orc, n, start):
    nh, nkv, hd = 4, 2, 64
    rng = np.random.default_rng(n + start)
    q = rng.standard_normal((n, nh * hd), dtype=F32)
    kc = rng.standard_normal((start + n, nkv * hd), dtype=F32)
    vc = rng.standard_normal((start + n, nkv * hd), dtype=F32)
    out = host(ops.attention_prefill(dev(q), dev(kc), dev(vc), n, start, nh, nkv, hd, False))
    assert_bit_equal(out, _naive_ref(orc, q, kc, vc, n, start, nh, nkv, hd), "naive prefill attention")


def _flash_ref(orc, q, kc, vc, n, start, nh, nkv, hd):
    group, kv_dim = nh // nkv, nkv * hd
    q_mat = np.ascontiguousarray(q.T)      # [hs, n]
    out = np.empty((n, nh * hd), F32)
    for kv_h in range(nkv):
        fl = orc.flash_attention_gqa(q_mat, kc, vc, kv_h * group, group, n, n, kv_dim, kv_h * hd, hd,
                                     F32(1.0) / np.sqrt(F32(hd)), start)
        for g in range(group):
            h = kv_h * group + g
            out[:, h * hd:(h + 1) * hd] = fl[g]
    return out


@pytest.mark.parametrize("hd", [64, 32, 128])
@pytest.mark.parametrize("n,start,nh,nkv", [(8, 4, 4, 2), (1, 0, 4, 2), (31, 0, 8, 2), (64, 33, 4, 4), (100, 0, 6, 2), (257, 300, 8, 2),
                                            (300, 0, 8, 1), (513, 1027, 16, 4)])
def test_attention_flash_bit_exact(ops, orc, n, start, nh, nkv, hd):
    """Ragged query counts (not multiples of the 8 queries a warp owns), 1 to 8 query heads per KV head, start
    positions that are not multiples of the 32-key tile, all three head sizes."""
    rng = np.random.default_rng(n * 3 + start + hd)
    q = rng.standard_normal((n, nh * hd), dtype=F32)
    kc = rng.standard_normal((start + n, nkv * hd), dtype=F32)
    vc = rng.standard_normal((start + n, nkv * hd), dtype=F32)
    out = host(ops.attention_prefill(dev(q), dev(kc), dev(vc), n, start, nh, nkv, hd, True))
    assert_bit_equal(out, _flash_ref(orc, q, kc, vc, n, start, nh, nkv, hd), "flash attention")


def test_attention_flash_last_chunk_of_a_4096_prompt(ops, orc):
    """The 1.6B model's shape (32 query heads, 8 KV heads, head size 64) for the last 512-token chunk of a 4096-token
    prompt: every query attends 3585..4096 keys.  Also the case the profiler summaries of this kernel are taken on."""
    n, start, nh, nkv, hd = 512, 3584, 32, 8, 64
    rng = np.random.default_rng(4096)
    q = rng.standard_normal((n, nh * hd), dtype=F32)
    kc = rng.standard_normal((start + n, nkv * hd), dtype=F32)
    vc = rng.standard_normal((start + n, nkv * hd), dtype=F32)
    out = host(ops.attention_prefill(dev(q), dev(kc), dev(vc), n, start, nh, nkv, hd, True))
    assert_bit_equal(out, _flash_ref(orc, q, kc, vc, n, start, nh, nkv, hd), "flash attention, p4096 last chunk")


def test_attention_flash_reference_case(ops, orc):
    """cpu.rs:3011-3144 (LCG inputs): flash == naive within 1e-4, and each equals its oracle twin."""
    nh, nkv, hd, n, sp, q_mat, kc, vc = rc.flash_vs_naive_case()
    q = np.ascontiguousarray(q_mat.T)
    fl = host(ops.attention_prefill(dev(q), dev(kc), dev(vc), n, sp, nh, nkv, hd, True))
    nv = host(ops.attention_prefill(dev(q), dev(kc), dev(vc), n, sp, nh, nkv, hd, False))
    assert np.abs(fl - nv).max() < 1e-4
    assert_bit_equal(fl, _flash_ref(orc, q, kc, vc, n, sp, nh, nkv, hd))
    assert_bit_equal(nv, _naive_ref(orc, q, kc, vc, n, sp, nh, nkv, hd))


def test_attention_flash_rejects_unsupported_shapes(ops):
    from wick_b200._lib import WickCudaError
    z = torch.zeros((4, 16 * 96), dtype=torch.float32, device="cuda")
    with pytest.raises(WickCudaError):
        ops.attention_prefill(z, z, z, 4, 0, 16, 16, 96, True)      # head_dim 96
    z = torch.zeros((4, 16 * 64), dtype=torch.float32, device="cuda")
    with pytest.raises(WickCudaError):
        ops.attention_prefill(z, z[:, :64].contiguous(), z[:, :64].contiguous(), 4, 0, 16, 1, 64, True)   # 16 query heads per KV head


def test_attention_softmax_is_normalised_large(ops):
    """Property at full context (4096 queries): with V = 1 every output is the softmax mass, which
    must be 1 within f32 rounding of the f64 normaliser."""
    nh, nkv, hd, n = 8, 2, 64, 4096
    rng = np.random.default_rng(4)
    q = torch.from_numpy(rng.standard_normal((n, nh * hd), dtype=F32)).cuda()
    kc = torch.from_numpy(rng.standard_normal((n, nkv * hd), dtype=F32)).cuda()
    vc = torch.ones((n, nkv * hd), dtype=torch.float32, device="cuda")
    out = ops.attention_prefill(q, kc, vc, n, 0, nh, nkv, hd, True)
    assert float((out - 1).abs().max()) < 1e-4
