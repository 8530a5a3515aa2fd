"""forward_prefill on the tensor-core GEMM path against the CPU oracle, whole model, through the C ABI.

Contract for this path: logits within max-abs 1e-2 of the oracle and identical greedy tokens over the
first 64 decode steps (the integer block sums inside are bit-exact and tested per kernel).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.fixture(scope="module")
def wick(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import wick_b200.model as m
    return m


def _path(model_dir, spec, qtype):
    from wick_b200 import gguf_synth as gs
    return gs.cached_model(spec, qtype, 0, cache_dir=model_dir)


def _maxdiff(a, b):
    return float(np.abs(np.asarray(a, F32) - np.asarray(b, F32)).max())


@pytest.mark.parametrize("spec,qtype", [("tiny", "q4_0"), ("tiny", "q8_0"), ("tiny-wide", "q4_0"), ("tiny-wide", "q8_0")])
@pytest.mark.parametrize("n", [16, 100, 300])
def test_tensor_prefill_matches_oracle(wick, orc, model_dir, monkeypatch, spec, qtype, n):
    from wick_b200 import gguf_synth as gs
    monkeypatch.delenv("WICK_CUDA_PREFILL", raising=False)
    path = _path(model_dir, spec, qtype)
    m = wick.CudaLfm2Model(path, 512)
    assert m.prefill_mode() == "tensor"
    st = wick.InferenceState()
    toks = gs.random_prompt(n, m.config().vocab_size, seed=n)
    lg = m.forward_prefill(toks, 0, st)
    om = orc.OracleModel(path, 512)
    lo = om.forward_prefill(toks, 0)
    assert _maxdiff(lg, lo) <= 1e-2
    assert _maxdiff(lg, lo) <= 1e-4 * max(1.0, float(np.abs(lo).max()))      # in practice f32 rounding level
    first = orc.argmax(lo)
    assert int(np.argmax(lg)) == first
    want = om.generate_greedy(first, 64)
    got = m.generate_greedy(first, 64, st)
    assert list(got) == list(want)
    # state written by the tensor path: KV rows and conv buffers close to the oracle's
    for li, attn in enumerate(om.is_attn):
        if attn:
            k_o, v_o = om.kv(li)
            k_c, v_c = m.read_kv(li)
            assert _maxdiff(k_c, k_o) <= 1e-3 and _maxdiff(v_c, v_o) <= 1e-3
        else:
            assert _maxdiff(m.read_conv_state(li), om.conv_state(li)) <= 1e-3


def test_mode_switch_and_exact_agreement(wick, orc, model_dir, monkeypatch):
    """set_prefill_mode toggles the path on a live model; 'exact' reproduces the oracle bit for bit and
    'tensor' stays within tolerance of it; chunked tensor prefill equals one-shot tensor prefill."""
    from wick_b200 import gguf_synth as gs
    monkeypatch.delenv("WICK_CUDA_PREFILL", raising=False)
    path = _path(model_dir, "tiny-wide", "q4_0")
    m = wick.CudaLfm2Model(path, 1024)
    st = wick.InferenceState()
    toks = gs.random_prompt(600, m.config().vocab_size, seed=9)
    lt = m.forward_prefill(toks, 0, st)
    lt_chunked = m.forward_prefill_chunked(toks, 0, st, 256)
    m.set_prefill_mode("exact")
    assert m.prefill_mode() == "exact"
    le = m.forward_prefill(toks, 0, st)
    lo = orc.OracleModel(path, 1024).forward_prefill(toks, 0)
    assert np.array_equal(le.view(np.uint32), lo.view(np.uint32))
    assert _maxdiff(lt, lo) <= 1e-2
    assert _maxdiff(lt_chunked, lo) <= 1e-2
    m.set_prefill_mode("tensor")
    assert np.array_equal(m.forward_prefill(toks, 0, st), lt)          # deterministic
    with pytest.raises(ValueError):
        m.set_prefill_mode("fast")


def test_env_selects_exact(wick, model_dir, monkeypatch):
    monkeypatch.setenv("WICK_CUDA_PREFILL", "exact")
    m = wick.CudaLfm2Model(_path(model_dir, "tiny", "q4_0"), 64)
    assert m.prefill_mode() == "exact"


def test_350m_tensor_prefill_close_to_exact(wick, orc, model_dir, monkeypatch):
    """Benchmark-size model (350M-class, Q4_0), 512-token prompt: tensor and exact prefill agree within
    the logits tolerance and pick the same greedy continuation for 64 tokens."""
    from wick_b200 import gguf_synth as gs
    monkeypatch.delenv("WICK_CUDA_PREFILL", raising=False)
    path = _path(model_dir, "lfm2-350m", "q4_0")
    m = wick.CudaLfm2Model(path, 1024)
    st = wick.InferenceState()
    toks = gs.random_prompt(512, m.config().vocab_size, seed=4)
    lt = m.forward_prefill(toks, 0, st)
    gt = m.generate_greedy(int(np.argmax(lt)), 64, st)
    m.set_prefill_mode("exact")
    le = m.forward_prefill(toks, 0, st)
    ge = m.generate_greedy(int(np.argmax(le)), 64, st)
    assert _maxdiff(lt, le) <= 1e-2
    assert int(np.argmax(lt)) == int(np.argmax(le))
    assert list(gt) == list(ge)
