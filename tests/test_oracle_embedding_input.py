"""CPU checks of the oracle's embedding-input entry points (lfm2.rs:2291-2350, :2452-2500): feeding the
dequantised embedding row of a token is the same computation as feeding the token id."""
import numpy as np


def _rows(orc, path, toks):
    g = orc.GgufFile(path)
    dims, tt, _ = g.tensors["token_embd.weight"]
    raw = g.tensor_bytes("token_embd.weight").reshape(int(dims[1]), -1)
    return np.stack([orc.dequant_row(tt, raw[int(t)], int(dims[0])) for t in toks])


def test_frame_steps_equal_token_steps(orc, model_dir):
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir)
    a, b = orc.OracleModel(path, 64), orc.OracleModel(path, 64)
    toks = gs.random_prompt(6, gs.SPECS["tiny"].vocab, seed=2)
    rows = _rows(orc, path, toks)
    for t, r in zip(toks, rows):
        la, ha = a.forward(int(t), want_hidden=True)
        lb = b.forward_from_embedding(r)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    hb = b.forward_from_embedding(rows[0], want="hidden")
    ha = a.forward_embedding(int(toks[0]))
    assert np.array_equal(ha.view(np.uint32), hb.view(np.uint32))
    assert a.seq_len == b.seq_len == 7


def test_prefill_frames_equal_prefill_tokens(orc, model_dir):
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny-wide", "q8_0", 0, cache_dir=model_dir)
    a, b = orc.OracleModel(path, 128), orc.OracleModel(path, 128)
    toks = gs.random_prompt(40, gs.SPECS["tiny-wide"].vocab, seed=4)
    la = a.forward_prefill(toks, 0)
    lb = b.forward_prefill_from_embeddings(_rows(orc, path, toks), 0)
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    assert list(a.generate_greedy(orc.argmax(la), 8)) == list(b.generate_greedy(orc.argmax(lb), 8))
