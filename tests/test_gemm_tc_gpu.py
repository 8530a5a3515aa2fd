"""Tensor-core (tcgen05 / TMEM / TMA) prefill GEMM through the C ABI against the CPU oracle.

Contract: the int32 block sums are bit-exact; the f32 outputs follow a different (fused, block-order)
accumulation than the NEON kernels and must agree within a relative 1e-5 of the output scale.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
F32 = np.float32


@pytest.fixture(scope="module")
def ops(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from wick_b200 import ops as o
    return o


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def rand_weights(rng, dtype, m, k, std=0.02):
    from wick_b200 import gguf_synth as gs
    w = (rng.standard_normal((m, k)) * std).astype(F32)
    return gs.quantize_q4_0(w) if dtype == "q4_0" else gs.quantize_q8_0(w)


def check_against_oracle(ops, orc, dtype, m, k, n, seed, oracle_tokens):
    rng = np.random.default_rng(seed)
    raw = rand_weights(rng, dtype, m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    bs, bq = orc.quantize_q8_0(x)
    dt = orc.QTYPE_ID[dtype]
    w = ops.QuantWeight(dt, raw, m, k)
    dbs, dbq = dev(bs), dev(bq)
    out, sums = ops.gemm_q8_tc(w, dbs, dbq, want_sums=True)
    out, sums = host(out), host(sums)
    exact = host(ops.gemm_q8(w, dbs, dbq))                      # bit-exact path, itself checked against the oracle
    scale = np.abs(exact).max()
    assert np.abs(out - exact).max() <= 1e-5 * scale, f"{dtype} {m}x{k}x{n}: {np.abs(out - exact).max()} vs scale {scale}"
    for j in oracle_tokens:
        S = orc.block_sums(dt, raw, bq[j], m, k)[0]
        assert np.array_equal(sums[j], S), f"block sums of token {j}"
        ref = orc.gemv(dt, raw, bs[j], bq[j], m, k)
        assert np.abs(out[j] - ref).max() <= 1e-5 * scale
    # the variant without the block-sum store is a different instantiation: same outputs, bit for bit
    out2 = host(ops.gemm_q8_tc(w, dbs, dbq))
    assert np.array_equal(out2.view(np.uint32), out.view(np.uint32))
    return out


@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m,k,n", [
    (128, 128, 16),      # one tile, one stage
    (128, 512, 64),      # every stage slot used once
    (256, 1152, 64),     # stage ring wraps (9 stages), two row tiles
    (384, 2048, 128),    # 128-token tiles, TMEM buffers reused 16 times
    (200, 256, 37),      # ragged rows and tokens (zero-padded tile rows, masked stores)
    (130, 384, 129),     # one token into the second token tile
    (64, 128, 1),        # single token, fewer rows than a tile
])
def test_gemm_tc_shapes(ops, orc, dtype, m, k, n):
    check_against_oracle(ops, orc, dtype, m, k, n, seed=m + k + n, oracle_tokens=sorted({0, n // 2, n - 1}))


@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("n", [8, 128, 2002])
def test_gemm_tc_matmul_sweep(ops, orc, dtype, n):
    """The isolated matmul sweep shape (m=6912, k=2048): more tiles than SMs, so CTAs loop over tiles."""
    check_against_oracle(ops, orc, dtype, 6912, 2048, n, seed=3, oracle_tokens=sorted({0, n - 1}))


@pytest.mark.parametrize("dtype", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m,k,n", [
    (128, 128, 16), (128, 512, 64), (256, 1152, 17), (384, 2048, 128), (200, 256, 37), (130, 384, 129), (64, 128, 1),
    (6912, 2048, 8), (6912, 2048, 128), (6912, 2048, 2002), (2048, 6912, 130),
])
def test_gemm_tc_exact_is_bit_exact(ops, orc, dtype, m, k, n):
    """The default prefill GEMM: tensor-core lane partials + the reference's eight chains.  Bit-equal to
    the CUDA-core kernel for every output, and to the oracle for sampled tokens."""
    rng = np.random.default_rng(m * 7 + k + n)
    raw = rand_weights(rng, dtype, m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    bs, bq = orc.quantize_q8_0(x)
    dt = orc.QTYPE_ID[dtype]
    w = ops.QuantWeight(dt, raw, m, k)
    dbs, dbq = dev(bs), dev(bq)
    out = host(ops.gemm_q8_tc_exact(w, dbs, dbq))
    exact = host(ops.gemm_q8(w, dbs, dbq))
    assert np.array_equal(out.view(np.uint32), exact.view(np.uint32)), \
        f"{dtype} {m}x{k}x{n}: {int((out.view(np.uint32) != exact.view(np.uint32)).sum())} outputs differ"
    for j in sorted({0, n // 2, n - 1}):
        ref = orc.gemv(dt, raw, bs[j], bq[j], m, k)
        assert np.array_equal(out[j].view(np.uint32), ref.view(np.uint32))


def test_gemm_tc_exact_full_size_properties(ops, orc):
    """n = 4096 (256 token tiles per row tile, CTAs loop over tiles): equals the CUDA-core kernel bit for
    bit, and sampled tokens equal the oracle."""
    m, k, n = 1024, 2048, 4096
    rng = np.random.default_rng(21)
    raw = rand_weights(rng, "q4_0", m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    w = ops.QuantWeight(orc.DT_Q4_0, raw, m, k)
    bs, bq = ops.quantize_f32_to_q8_0(dev(x))
    out = ops.gemm_q8_tc_exact(w, bs, bq)
    assert torch.equal(out, ops.gemm_q8(w, bs, bq))
    for j in (0, 1777, 4095):
        ref = orc.gemv(orc.DT_Q4_0, raw, host(bs[j]), host(bq[j]), m, k)
        assert np.array_equal(host(out[j]).view(np.uint32), ref.view(np.uint32))


def test_gemm_tc_extreme_values(ops, orc):
    """Largest possible block sums: all weights at -8 (Q4_0) against activations at +/-127."""
    m, k, n = 128, 256, 32
    from wick_b200 import gguf_synth as gs
    w = np.full((m, k), -8.0, F32)
    raw = gs.quantize_q4_0(w)
    x = np.where(np.arange(k) % 2 == 0, 127.0, -127.0).astype(F32)[None, :].repeat(n, 0)
    x[1] = 127.0
    bs, bq = orc.quantize_q8_0(x)
    wq = ops.QuantWeight(orc.DT_Q4_0, raw, m, k)
    out, sums = ops.gemm_q8_tc(wq, dev(bs), dev(bq), want_sums=True)
    S1 = orc.block_sums(orc.DT_Q4_0, raw, bq[1], m, k)[0]
    assert np.array_equal(host(sums)[1], S1)
    assert np.abs(S1).max() == 32 * 8 * 127
    exact = host(ops.gemm_q8(wq, dev(bs), dev(bq)))
    assert np.abs(host(out) - exact).max() <= 1e-5 * np.abs(exact).max()


def test_gemm_tc_exact_extreme_lane_partials(ops, orc):
    """The bit-exact kernel on the largest lane partials (8 * 8 * 127 = 8128 per NEON lane group and block) and on
    low-bit patterns next to them: hand-built integer operands that survive both quantisers unchanged."""
    from wick_b200 import gguf_synth as gs
    m, k, n = 128, 512, 48
    rng = np.random.default_rng(8128)
    # weights: integers of [-8, 7] times a power-of-two block scale; one -8 per block pins the scale
    wq = rng.choice(np.array([-8, -8, -8, -7, 7, 7, 6, -1, 1, 0]), size=(m, k))
    wq[:, ::32] = -8
    wq[:16] = -8                                   # rows of all -8
    wq[16:32] = np.where(np.arange(k) % 2 == 0, -8, 7)
    raw = gs.quantize_q4_0((wq * 0.0625).astype(F32))
    # activations: integers of [-127, 127] times a power-of-two scale; one +/-127 per block pins the scale
    xq = rng.choice(np.array([127, -127, 126, -126, 113, -113, 1, -1, 15, -16, 17, 0]), size=(n, k))
    xq[:, 5::32] = 127
    xq[0] = 127
    xq[1] = -127
    xq[2] = np.where(np.arange(k) % 2 == 0, 127, -127)
    xq[3] = np.where(np.arange(k) % 3 == 0, 127, 126)
    xq[3, 5::32] = 127
    x = (xq * 0.5).astype(F32)
    bs, bq = orc.quantize_q8_0(x)
    assert np.array_equal(bq.reshape(n, k).astype(np.int64), xq), "the test's activations must survive the quantiser"
    w = ops.QuantWeight(orc.DT_Q4_0, raw, m, k)
    S = orc.block_sums(orc.DT_Q4_0, raw, bq[0], m, k)[0]
    assert np.abs(S).max() == 32 * 8 * 127
    out = host(ops.gemm_q8_tc_exact(w, dev(bs), dev(bq)))
    exact = host(ops.gemm_q8(w, dev(bs), dev(bq)))
    assert np.array_equal(out.view(np.uint32), exact.view(np.uint32)), \
        f"{int((out.view(np.uint32) != exact.view(np.uint32)).sum())} outputs differ"
    for j in range(0, n, 7):
        ref = orc.gemv(orc.DT_Q4_0, raw, bs[j], bq[j], m, k)
        assert np.array_equal(out[j].view(np.uint32), ref.view(np.uint32))


def test_gemm_tc_properties_full_size(ops, orc):
    """Size-independent properties at n = 4096: power-of-two activation scales commute with the product
    bit for bit, tokens are independent of their position in the batch, and repeated runs are identical."""
    m, k, n = 2048, 2048, 4096
    rng = np.random.default_rng(11)
    raw = rand_weights(rng, "q4_0", m, k)
    x = rng.standard_normal((n, k), dtype=F32)
    w = ops.QuantWeight(orc.DT_Q4_0, raw, m, k)
    bs, bq = ops.quantize_f32_to_q8_0(dev(x))
    out = ops.gemm_q8_tc(w, bs, bq)
    assert torch.equal(ops.gemm_q8_tc(w, bs, bq), out)
    assert torch.equal(ops.gemm_q8_tc(w, bs * 4.0, bq), out * 4.0)
    perm = torch.randperm(n, device="cuda")
    assert torch.equal(ops.gemm_q8_tc(w, bs[perm].contiguous(), bq[perm].contiguous()), out[perm])
    exact = ops.gemm_q8(w, bs, bq)
    assert float((out - exact).abs().max()) <= 1e-5 * float(exact.abs().max())
    for j in (0, 2047, 4095):
        ref = orc.gemv(orc.DT_Q4_0, raw, host(bs[j]), host(bq[j]), m, k)
        assert np.abs(host(out[j]) - ref).max() <= 1e-5 * np.abs(ref).max()


def test_gemm_tc_rejects_unsupported_k(ops, orc):
    from wick_b200._lib import WickCudaError
    rng = np.random.default_rng(0)
    raw = rand_weights(rng, "q4_0", 64, 96)
    w = ops.QuantWeight(orc.DT_Q4_0, raw, 64, 96)
    x = rng.standard_normal((4, 96), dtype=F32)
    bs, bq = orc.quantize_q8_0(x)
    with pytest.raises(WickCudaError):
        ops.gemm_q8_tc(w, dev(bs), dev(bq))
