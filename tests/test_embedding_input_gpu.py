"""Embedding-input methods of the Model trait (mod.rs:172-267) through the C ABI against the CPU oracle."""
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


def bits(a):
    return np.ascontiguousarray(a, F32).view(np.uint32)


@pytest.mark.parametrize("spec,qtype", [("tiny", "q4_0"), ("tiny-wide", "q8_0")])
def test_single_frame_methods_bit_exact(wick, orc, model_dir, spec, qtype):
    """A few token steps, then frames fed as embeddings: logits, hidden rows and the state they leave
    behind equal the oracle bit for bit; token steps and embedding steps can be mixed freely."""
    path = _path(model_dir, spec, qtype)
    cm, om = wick.CudaLfm2Model(path, 128), orc.OracleModel(path, 128)
    assert cm.supports_embedding_input()
    st = wick.InferenceState()
    rng = np.random.default_rng(5)
    hs = cm.config().hidden_size
    for t in (3, 77):
        assert np.array_equal(bits(cm.forward([t], st.seq_len, st)), bits(om.forward(t)))
    for i in range(3):
        e = (rng.standard_normal(hs) * 0.05).astype(F32)
        assert np.array_equal(bits(cm.forward_from_embedding(e, 999, st)), bits(om.forward_from_embedding(e)))   # pos is ignored
    e = (rng.standard_normal(hs) * 0.05).astype(F32)
    assert np.array_equal(bits(cm.forward_hidden_from_embedding(e, 0, st)), bits(om.forward_from_embedding(e, want="hidden")))
    assert np.array_equal(bits(cm.forward_embedding([11], 0, st)), bits(om.forward_embedding(11)))
    assert st.seq_len == om.seq_len == 7 and cm.seq_len == 7
    # the next token step sees the same state
    assert np.array_equal(bits(cm.forward([5], st.seq_len, st)), bits(om.forward(5)))
    for li, attn in enumerate(om.is_attn):
        if attn:
            (kc, vc), (ko, vo) = cm.read_kv(li), om.kv(li)
            assert np.array_equal(kc, ko) and np.array_equal(vc, vo)
        else:
            assert np.array_equal(cm.read_conv_state(li), om.conv_state(li))


@pytest.mark.parametrize("spec,qtype,n", [("tiny", "q4_0", 5), ("tiny-wide", "q4_0", 40), ("tiny-wide", "q8_0", 300)])
def test_prefill_from_embeddings_bit_exact(wick, orc, model_dir, spec, qtype, n):
    """n frames in one call (naive and flash attention paths, CUDA-core and tensor-core GEMMs), then a
    continuation chunk at start_pos = n, then greedy decode."""
    path = _path(model_dir, spec, qtype)
    cm, om = wick.CudaLfm2Model(path, 512), orc.OracleModel(path, 512)
    st = wick.InferenceState()
    rng = np.random.default_rng(n)
    hs = cm.config().hidden_size
    emb = (rng.standard_normal((n, hs)) * 0.05).astype(F32)
    lg = cm.forward_prefill_from_embeddings(emb, n, 0, st)
    lo = om.forward_prefill_from_embeddings(emb, 0)
    assert np.array_equal(bits(lg), bits(lo))
    more = (rng.standard_normal((20, hs)) * 0.05).astype(F32)
    assert np.array_equal(bits(cm.forward_prefill_from_embeddings(more, 20, n, st)), bits(om.forward_prefill_from_embeddings(more, n)))
    first = orc.argmax(lo)
    assert list(cm.generate_greedy(first, 16, st)) == list(om.generate_greedy(first, 16))


def test_frames_equal_token_rows(wick, model_dir):
    """Feeding the dequantised embedding rows of a prompt as frames is the same computation as feeding
    its token ids."""
    from wick_b200 import gguf_synth as gs
    from oracle import oracle as orc
    path = _path(model_dir, "tiny-wide", "q4_0")
    cm = wick.CudaLfm2Model(path, 256)
    st = wick.InferenceState()
    toks = gs.random_prompt(48, cm.config().vocab_size, seed=3)
    want = cm.forward_prefill(toks, 0, st)
    g = orc.GgufFile(path)
    dims, tt, _ = g.tensors["token_embd.weight"]
    k = int(dims[0])
    raw = g.tensor_bytes("token_embd.weight").reshape(int(dims[1]), -1)        # one row of blocks per token id
    rows = np.stack([orc.dequant_row(tt, raw[int(t)], k) for t in toks])
    got = cm.forward_prefill_from_embeddings(rows, len(toks), 0, st)
    assert np.array_equal(bits(got), bits(want))


def test_argument_checks(wick, model_dir):
    cm = wick.CudaLfm2Model(_path(model_dir, "tiny", "q4_0"), 32)
    st = wick.InferenceState()
    hs = cm.config().hidden_size
    with pytest.raises(AssertionError):
        cm.forward_prefill_from_embeddings(np.zeros(hs * 2 + 1, F32), 2, 0, st)
    with pytest.raises(AssertionError):
        cm.forward_prefill_from_embeddings(np.zeros(0, F32), 0, 0, st)
    from wick_b200._lib import WickCudaError
    with pytest.raises(WickCudaError):                      # context overflow is an error code, not a crash
        cm.forward_prefill_from_embeddings(np.zeros((33, hs), F32), 33, 0, st)
