"""On-device Sampler::sample (wick_cuda_sample_logits / wick_cuda_forward_sample) through the C ABI against the oracle's
restatement of wick/src/sampler.rs:64-158, with the same uniform draw on both sides.  Integer result: the token must
be identical."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.fixture(scope="module")
def ops(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from wick_b200 import ops
    return ops


@pytest.mark.parametrize("n", [2, 33, 1000, 65536])
def test_sample_logits_matches_oracle(ops, orc, n):
    rng = np.random.default_rng(n)
    for case in range(40):
        logits = (rng.standard_normal(n) * rng.uniform(0.5, 8)).astype(F32)
        if case % 5 == 0:
            logits[rng.integers(0, n, size=min(n, 4))] = logits.max()            # ties at the top-k threshold / maximum
        if case % 9 == 0:
            logits[rng.integers(0, n, size=min(n, 3))] = -np.inf
        temperature = float(rng.choice([0.0, 0.2, 0.7, 1.0, 1.7]))
        top_k = int(rng.choice([0, 1, 2, 40, 200, 4096, n + 1]))
        top_p = float(rng.choice([0.05, 0.5, 0.9, 0.99, 1.0]))
        if top_p < 1.0 and (top_k == 0 or top_k > 4096 or top_k >= n) and n > 4096:
            top_p = 1.0                                                               # outside the on-device limit (own test below)
        r = float(F32(rng.random())) if case % 11 else 0.0
        got = ops.sample_logits(torch.from_numpy(logits).cuda(), temperature, top_k, top_p, r)
        want = orc.sample(logits, temperature, top_k, top_p, r)
        assert got == want, (n, case, temperature, top_k, top_p, r)


def test_sample_logits_reports_the_top_p_limit(ops):
    from wick_b200._lib import WickCudaError
    logits = torch.zeros(65536, dtype=torch.float32, device="cuda")
    with pytest.raises(WickCudaError):
        ops.sample_logits(logits, 0.7, 0, 0.9, 0.5)            # top-p over the whole vocabulary: host fallback
    assert ops.sample_logits(logits, 0.7, 0, 1.0, 0.0) == 0    # no top-p: any size works


def test_forward_sample_matches_oracle_on_a_model(cuda_lib, orc, model_dir):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import wick_b200.model as wick
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny-wide", "q4_0", 0, cache_dir=model_dir, norm_jitter=0.2, weight_std=0.05)
    cm, om = wick.CudaLfm2Model(path, 256), orc.OracleModel(path, 256)
    st = wick.InferenceState()
    toks = gs.random_prompt(20, cm.config().vocab_size, seed=3)
    cm.forward_prefill(toks, 0, st)
    om.forward_prefill(toks, 0)
    rng = np.random.default_rng(5)
    tok = 7
    for step in range(24):
        r = float(F32(rng.random()))
        temperature, top_k, top_p = [(0.7, 40, 0.9), (1.0, 0, 1.0), (0.3, 5, 0.5), (0.0, 40, 0.9)][step % 4]
        got = cm.forward_sample([tok], 20 + step, st, temperature, top_k, top_p, r)
        want = orc.sample(om.forward(tok), temperature, top_k, top_p, r)
        assert got == want, (step, temperature, top_k, top_p, r)
        tok = want
    assert st.seq_len == cm.seq_len == 44
