"""Model::shift_kv (n_keep context shift, kv_cache.rs:601-715) through the C ABI against the CPU oracle."""
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


def _same_state(cm, om):
    for li, attn in enumerate(om.is_attn):
        if attn:
            (kc, vc), (ko, vo) = cm.read_kv(li), om.kv(li)
            assert kc.shape == ko.shape
            assert np.array_equal(kc.view(np.uint32), ko.view(np.uint32)), f"K of layer {li}"
            assert np.array_equal(vc.view(np.uint32), vo.view(np.uint32)), f"V of layer {li}"
        else:
            assert np.array_equal(cm.read_conv_state(li), om.conv_state(li))


@pytest.mark.parametrize("spec,qtype", [("tiny", "q4_0"), ("tiny-wide", "q8_0")])
@pytest.mark.parametrize("n,n_keep,shift", [(40, 8, 16), (40, 0, 1), (64, 32, 32), (50, 4, 45)])
def test_shift_matches_oracle(wick, orc, model_dir, spec, qtype, n, n_keep, shift):
    """Prefill n tokens, shift, compare the caches bit for bit, then keep decoding: the logits of the
    following steps (which read the shifted, re-rotated K rows) stay bit-equal to the oracle."""
    from wick_b200 import gguf_synth as gs
    path = _path(model_dir, spec, qtype)
    cm, om = wick.CudaLfm2Model(path, 128), orc.OracleModel(path, 128)
    assert cm.supports_kv_shift()
    st = wick.InferenceState()
    toks = gs.random_prompt(n, cm.config().vocab_size, seed=n + shift)
    lg = cm.forward_prefill(toks, 0, st)
    lo = om.forward_prefill(toks, 0)
    assert np.array_equal(lg.view(np.uint32), lo.view(np.uint32))
    cm.shift_kv(st, n_keep, shift)
    om.shift_kv(n_keep, shift)
    assert st.seq_len == cm.seq_len == om.seq_len == n - shift
    _same_state(cm, om)
    tok = orc.argmax(lo)
    for _ in range(4):                                   # single steps through the persistent kernel
        a, b = cm.forward([tok], st.seq_len, st), om.forward(tok)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        tok = orc.argmax(b)
    more = gs.random_prompt(20, cm.config().vocab_size, seed=1)      # and a prefill chunk after the shift
    assert np.array_equal(cm.forward_prefill(more, st.seq_len, st).view(np.uint32), om.forward_prefill(more, om.seq_len).view(np.uint32))
    _same_state(cm, om)


def test_shift_all_retained_dropped_and_errors(wick, orc, model_dir):
    """n_keep + shift == seq_len leaves nothing to move (metal_lfm2.rs:2498-2508); out-of-range arguments are
    error codes, and the state is untouched by a rejected call."""
    from wick_b200 import gguf_synth as gs
    from wick_b200._lib import WickCudaError
    path = _path(model_dir, "tiny", "q4_0")
    cm, om = wick.CudaLfm2Model(path, 64), orc.OracleModel(path, 64)
    st = wick.InferenceState()
    toks = gs.random_prompt(30, cm.config().vocab_size, seed=6)
    cm.forward_prefill(toks, 0, st)
    om.forward_prefill(toks, 0)
    with pytest.raises(WickCudaError):
        cm.shift_kv(st, 20, 11)
    assert cm.seq_len == 30
    cm.shift_kv(st, 10, 20)
    om.shift_kv(10, 20)
    assert cm.seq_len == om.seq_len == 10
    _same_state(cm, om)
    a, b = cm.forward([7], st.seq_len, st), om.forward(7)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_shift_long_context_350m(wick, orc, model_dir):
    """Benchmark-size model: fill most of a 1024-token context, shift half of it away keeping 32, decode on."""
    from wick_b200 import gguf_synth as gs
    path = _path(model_dir, "lfm2-350m", "q4_0")
    cm, om = wick.CudaLfm2Model(path, 1024), orc.OracleModel(path, 1024)
    st = wick.InferenceState()
    toks = gs.random_prompt(200, cm.config().vocab_size, seed=8)
    lg, lo = cm.forward_prefill(toks, 0, st), om.forward_prefill(toks, 0)
    assert np.array_equal(lg.view(np.uint32), lo.view(np.uint32))
    cm.shift_kv(st, 32, 100)
    om.shift_kv(32, 100)
    _same_state(cm, om)
    first = orc.argmax(lo)
    assert list(cm.generate_greedy(first, 12, st)) == list(om.generate_greedy(first, 12))
