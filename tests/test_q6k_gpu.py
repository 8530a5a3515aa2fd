"""Models whose token_embd is stored as Q6_K (llama.cpp's Q4_0 files): embedding rows and the vocabulary
mat-vec through the C ABI against the CPU oracle, bit for bit."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wick(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import wick_b200.model as m
    return m


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("spec,qtype", [("tiny", "q4_0"), ("tiny-wide", "q4_0"), ("tiny-wide", "q8_0")])
def test_q6k_embedding_model_bit_exact(wick, orc, model_dir, spec, qtype):
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model(spec, qtype, 0, cache_dir=model_dir, embd_qtype="q6_k")
    cm, om = wick.CudaLfm2Model(path, 512), orc.OracleModel(path, 512)
    assert cm.decode_path() == "persistent"        # layers in the persistent kernel, Q6_K logits as a kernel of its own
    st = wick.InferenceState()
    vocab = cm.config().vocab_size
    # single steps: embedding row lookup + logits mat-vec every step
    for t in (0, 1, vocab - 1, 17):
        assert np.array_equal(bits(cm.forward([t], st.seq_len, st)), bits(om.forward(t)))
    # hidden state of a token step (embedding row in, no logits)
    assert np.array_equal(bits(cm.forward_embedding([5], 0, st)), bits(om.forward_embedding(5)))
    # prefill (naive and flash attention lengths), then greedy decode on the device
    for n in (40, 300):
        toks = gs.random_prompt(n, vocab, seed=n)
        lg, lo = cm.forward_prefill(toks, 0, st), om.forward_prefill(toks, 0)
        assert np.array_equal(bits(lg), bits(lo))
        first = orc.argmax(lo)
        assert int(cm.forward_greedy([first], st.seq_len, st)) == int(om.generate_greedy(first, 1)[0])
        nxt = orc.argmax(om.forward(7))
        cm.forward([7], st.seq_len, st)
        assert list(cm.generate_greedy(nxt, 24, st)) == list(om.generate_greedy(nxt, 24))


def test_q6k_350m_vocab_head(wick, orc, model_dir):
    """Benchmark-size vocabulary (65536 x 1024 in Q6_K): 2048 CTAs of the logits kernel, four super-blocks per row."""
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("lfm2-350m", "q4_0", 0, cache_dir=model_dir, embd_qtype="q6_k")
    cm, om = wick.CudaLfm2Model(path, 256), orc.OracleModel(path, 256)
    st = wick.InferenceState()
    toks = gs.random_prompt(24, cm.config().vocab_size, seed=2)
    lg, lo = cm.forward_prefill(toks, 0, st), om.forward_prefill(toks, 0)
    assert np.array_equal(bits(lg), bits(lo))
    first = orc.argmax(lo)
    assert list(cm.generate_greedy(first, 8, st)) == list(om.generate_greedy(first, 8))


def test_q6k_only_for_token_embd(wick, model_dir, tmp_path):
    """Q6_K is accepted for token_embd only; a layer matrix in Q6_K is an unsupported-dtype load error."""
    from wick_b200 import gguf_synth as gs
    from wick_b200._lib import WickCudaError
    good = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir, embd_qtype="q6_k")
    data = bytearray(open(good, "rb").read())
    # flip the ggml type of blk.0.ffn_gate.weight (Q4_0 = 2) to Q6_K (14) in the tensor directory
    name = b"blk.0.ffn_gate.weight"
    i = data.index(name) + len(name)
    n_dims = int.from_bytes(data[i:i + 4], "little")
    type_off = i + 4 + 8 * n_dims
    assert int.from_bytes(data[type_off:type_off + 4], "little") == 2
    data[type_off:type_off + 4] = (14).to_bytes(4, "little")
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(bytes(data))
    with pytest.raises(WickCudaError) as e:
        wick.CudaLfm2Model(str(bad), 64)
    assert "Q4_0 and Q8_0" in str(e.value) or "type" in str(e.value)
