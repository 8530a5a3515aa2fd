"""Multi-sequence decode (wick_cuda_seq_* / wick_cuda_decode_batch) through the C ABI against the CPU oracle.

wick decodes one sequence per model; the batched step serves many sequences from one pass over the weights and
must give every sequence exactly what it would get alone: logits bit-equal to the oracle's run of that sequence,
greedy tokens identical, whatever else shares the batch, and the model's own sequence undisturbed.
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


def bits(a):
    return np.ascontiguousarray(a, F32).view(np.uint32)


def _path(model_dir, spec, qtype, **kw):
    from wick_b200 import gguf_synth as gs
    return gs.cached_model(spec, qtype, 0, cache_dir=model_dir, **kw)


@pytest.mark.parametrize("spec,qtype,n_seq", [("tiny", "q4_0", 5), ("tiny-wide", "q8_0", 3), ("tiny-wide", "q4_0", 20)])
def test_batched_decode_matches_oracle_per_sequence(wick, orc, model_dir, spec, qtype, n_seq):
    """Ragged prompts (1 .. 300 tokens, so both prefill attention paths and both GEMM paths, n < 16 and n >= 16 rows,
    are used), then interleaved batched steps: logits and tokens of every row equal the oracle's."""
    from wick_b200 import gguf_synth as gs
    path = _path(model_dir, spec, qtype, norm_jitter=0.2, weight_std=0.05)
    cm = wick.CudaLfm2Model(path, 512)
    vocab = cm.config().vocab_size
    rng = np.random.default_rng(7)
    lens = [1, 300, 17, 64, 2] + [int(x) for x in rng.integers(1, 120, size=max(0, n_seq - 5))]
    lens = lens[:n_seq]
    oracles, ids, nxt = [], [], []
    for i, L in enumerate(lens):
        om = orc.OracleModel(path, 512)
        toks = gs.random_prompt(L, vocab, seed=100 + i)
        sid = cm.seq_create()
        lg, lo = cm.seq_prefill(sid, toks, 0), om.forward_prefill(toks, 0)
        assert np.array_equal(bits(lg), bits(lo)), f"prefill of sequence {i}"
        assert cm.seq_length(sid) == L
        oracles.append(om)
        ids.append(sid)
        nxt.append(orc.argmax(lo))
    # one step returning logits
    lg = cm.decode_batch_logits(nxt, ids)
    for i, om in enumerate(oracles):
        lo = om.forward(int(nxt[i]))
        assert np.array_equal(bits(lg[i]), bits(lo)), f"batched logits of sequence {i}"
        nxt[i] = orc.argmax(lo)
    # greedy steps, one call per step
    for step in range(6):
        got = cm.decode_batch(nxt, ids)
        for i, om in enumerate(oracles):
            want = om.generate_greedy(int(nxt[i]), 1)[0]
            assert int(got[i]) == int(want), f"step {step} sequence {i}"
            nxt[i] = int(want)
    # a sub-batch in another order, several steps on the device
    sub = list(range(n_seq))[::-1][: max(1, n_seq // 2)]
    out = cm.decode_batch_steps([nxt[i] for i in sub], [ids[i] for i in sub], 5)
    for col, i in enumerate(sub):
        want = oracles[i].generate_greedy(int(nxt[i]), 5)
        assert list(out[:, col]) == list(want), f"device-loop tokens of sequence {i}"
        assert cm.seq_length(ids[i]) == lens[i] + 1 + 6 + 5


def test_slots_leave_the_models_own_sequence_alone(wick, orc, model_dir):
    from wick_b200 import gguf_synth as gs
    from wick_b200._lib import WickCudaError
    path = _path(model_dir, "tiny-wide", "q4_0", norm_jitter=0.2, weight_std=0.05)
    cm, om = wick.CudaLfm2Model(path, 256), orc.OracleModel(path, 256)
    vocab = cm.config().vocab_size
    st = wick.InferenceState()
    toks = gs.random_prompt(40, vocab, seed=5)
    first = orc.argmax(om.forward_prefill(toks, 0))
    cm.forward_prefill(toks, 0, st)
    a, b = cm.seq_create(), cm.seq_create()
    cm.seq_prefill(a, gs.random_prompt(70, vocab, seed=6), 0)
    cm.seq_prefill(b, gs.random_prompt(9, vocab, seed=7), 0)
    cm.decode_batch([1, 2], [a, b])
    # the model's own sequence continues as if nothing had happened (persistent decode kernel reads its own state)
    assert list(cm.generate_greedy(first, 12, st)) == list(om.generate_greedy(first, 12))
    # misuse
    with pytest.raises(WickCudaError):
        cm.decode_batch([1, 2], [a, a])            # a slot twice in one batch
    with pytest.raises(WickCudaError):
        cm.decode_batch([1], [99])                 # no such slot
    with pytest.raises(WickCudaError):
        cm.decode_batch([vocab], [a])              # token out of range
    cm.seq_destroy(b)
    with pytest.raises(WickCudaError):
        cm.decode_batch([1], [b])
    c = cm.seq_create()                            # recycles b's buffers, starting from an empty sequence
    assert c == b and cm.seq_length(c) == 0
    o2 = orc.OracleModel(path, 256)
    p = gs.random_prompt(5, vocab, seed=8)
    assert np.array_equal(bits(cm.seq_prefill(c, p, 0)), bits(o2.forward_prefill(p, 0)))


def test_batched_decode_context_full(wick, model_dir):
    from wick_b200 import gguf_synth as gs
    from wick_b200._lib import WickCudaError
    path = _path(model_dir, "tiny", "q4_0")
    cm = wick.CudaLfm2Model(path, 16)
    s = cm.seq_create()
    cm.seq_prefill(s, gs.random_prompt(15, cm.config().vocab_size), 0)
    cm.decode_batch([3], [s])
    with pytest.raises(WickCudaError) as e:
        cm.decode_batch([3], [s])
    assert e.value.code == -5


def test_batched_decode_1p6b_q4_0_eight_sequences(wick, orc, model_dir):
    """The serving configuration's model (1.6B-class Q4_0): 8 interleaved sequences with 16..200-token prompts,
    24 batched greedy steps on the device: every sequence's tokens equal the oracle's run of that sequence."""
    from wick_b200 import gguf_synth as gs
    path = _path(model_dir, "lfm2.5-1.6b", "q4_0")
    cm = wick.CudaLfm2Model(path, 1024)
    vocab = cm.config().vocab_size
    om = orc.OracleModel(path, 1024)
    lens = [16, 200, 33, 128, 64, 17, 90, 150]
    ids, firsts, prompts = [], [], []
    for i, L in enumerate(lens):
        toks = gs.random_prompt(L, vocab, seed=40 + i)
        sid = cm.seq_create()
        lg = cm.seq_prefill(sid, toks, 0)
        ids.append(sid)
        prompts.append(toks)
        firsts.append(int(np.argmax(lg)))
    out = cm.decode_batch_steps(firsts, ids, 24)
    for i in (0, 1, 5, 7):          # the oracle is one model instance: sequences are replayed one after another
        lo = om.forward_prefill(prompts[i], 0)
        assert orc.argmax(lo) == firsts[i]
        assert list(out[:, i]) == list(om.generate_greedy(firsts[i], 24)), f"sequence {i}"
