"""Opt-in split-K decode attention against the exact kernel and the CPU oracle: agreement within rounding (the runs'
partial sums are combined in a different order), never bit-exactness; and the multi-sequence step with it switched on
stays within the logits tolerance of the contract (max-abs 1e-2 on these models)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.mark.parametrize("seq,nh,nkv,hd", [(1, 4, 2, 64), (255, 4, 2, 64), (256, 8, 2, 64), (257, 8, 8, 32), (1000, 16, 4, 64), (4100, 32, 8, 64), (700, 4, 2, 128)])
def test_splitk_matches_exact_within_rounding(cuda_lib, orc, seq, nh, nkv, hd):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from wick_b200 import ops
    rng = np.random.default_rng(seq + nh)
    q = rng.standard_normal(nh * hd, dtype=F32)
    kc = rng.standard_normal((seq, nkv * hd), dtype=F32)
    vc = rng.standard_normal((seq, nkv * hd), dtype=F32)
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (q, kc, vc))
    exact = ops.attention_decode(dq, dk, dv, nh, nkv, hd, seq).cpu().numpy()
    split = ops.attention_decode_splitk(dq, dk, dv, nh, nkv, hd, seq).cpu().numpy()
    scale = float(np.abs(exact).max())
    assert float(np.abs(split - exact).max()) <= 2e-6 * max(scale, 1.0), float(np.abs(split - exact).max())
    if seq <= 256:      # a single run: the same arithmetic as the exact kernel up to the final division
        assert float(np.abs(split - exact).max()) <= 3e-7 * max(scale, 1.0)


def test_batched_decode_with_splitk_stays_within_tolerance(cuda_lib, orc, model_dir):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import wick_b200.model as wick
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny-wide", "q4_0", 0, cache_dir=model_dir, norm_jitter=0.2, weight_std=0.05)
    cm = wick.CudaLfm2Model(path, 1024)
    cm.set_decode_attention("splitk")
    vocab = cm.config().vocab_size
    ids, oracles, nxt = [], [], []
    for i, L in enumerate([600, 300, 5]):
        om = orc.OracleModel(path, 1024)
        toks = gs.random_prompt(L, vocab, seed=60 + i)
        sid = cm.seq_create()
        lo = om.forward_prefill(toks, 0)
        assert np.array_equal(cm.seq_prefill(sid, toks, 0), lo)          # prefill is unaffected by the switch
        ids.append(sid)
        oracles.append(om)
        nxt.append(orc.argmax(lo))
    worst = 0.0
    for step in range(4):
        lg = cm.decode_batch_logits(nxt, ids)
        for i, om in enumerate(oracles):
            lo = om.forward(int(nxt[i]))
            worst = max(worst, float(np.abs(lg[i] - lo).max()))
            nxt[i] = orc.argmax(lo)
    assert worst <= 1e-2, worst
    cm.set_decode_attention("exact")          # the switch goes both ways; fresh sequences are bit-exact again
    om = orc.OracleModel(path, 1024)
    toks = gs.random_prompt(40, vocab, seed=70)
    sid = cm.seq_create()
    first = orc.argmax(om.forward_prefill(toks, 0))
    cm.seq_prefill(sid, toks, 0)
    assert np.array_equal(cm.decode_batch_logits([first], [sid])[0], om.forward(first))
