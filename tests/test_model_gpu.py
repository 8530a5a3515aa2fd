"""Whole-model parity of the CUDA backend with the CPU oracle on identical seeded GGUF files and
prompts, through the C ABI (via the Model-trait mirror).  Small models are compared bit for bit;
the benchmark-size models are checked through size-independent properties."""
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


@pytest.fixture(autouse=True)
def exact_prefill(monkeypatch):
    """This file checks the bit-exact paths; the tensor-core prefill has its own tests."""
    monkeypatch.setenv("WICK_CUDA_PREFILL", "exact")


def _model_path(model_dir, spec, qtype, seed=0, **kw):
    from wick_b200 import gguf_synth as gs
    return gs.cached_model(spec, qtype, seed, cache_dir=model_dir, **kw)


def _diff(a, b):
    return float(np.abs(np.asarray(a, F32) - np.asarray(b, F32)).max())


def assert_logits_equal(got, want, what):
    if not np.array_equal(got.view(np.uint32), want.view(np.uint32)):
        nbad = int((got.view(np.uint32) != want.view(np.uint32)).sum())
        raise AssertionError(f"{what}: {nbad}/{got.size} logits differ, max abs diff {_diff(got, want)}")


CASES = [("tiny", "q4_0"), ("tiny", "q8_0"), ("tiny-wide", "q4_0"), ("tiny-wide", "q8_0")]


@pytest.mark.parametrize("spec,qtype", CASES)
def test_decode_logits_bit_exact(wick, orc, model_dir, spec, qtype):
    """Model::forward token by token from an empty sequence."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, spec, qtype, norm_jitter=0.2, weight_std=0.05)
    cm = wick.CudaLfm2Model(path, 256)
    om = orc.OracleModel(path, 256)
    st = wick.InferenceState()
    toks = gs.random_prompt(24, cm.config().vocab_size, seed=3)
    for i, t in enumerate(toks):
        lg = cm.forward([int(t)], i, st)
        lo = om.forward(int(t))
        assert_logits_equal(lg, lo, f"{spec}/{qtype} decode step {i}")
    assert st.seq_len == cm.seq_len == om.seq_len == 24
    for li, kvh in enumerate(cm.config().kv_heads_per_layer):
        if kvh:
            k, v = cm.read_kv(li)
            ko, vo = om.kv(li)
            assert np.array_equal(k, ko) and np.array_equal(v, vo), f"kv cache layer {li}"
        else:
            assert np.array_equal(cm.read_conv_state(li), om.conv_state(li)), f"conv state layer {li}"


@pytest.mark.parametrize("spec,qtype", CASES)
@pytest.mark.parametrize("n", [1, 2, 31, 130])
def test_prefill_naive_path_bit_exact(wick, orc, model_dir, spec, qtype, n):
    """forward_prefill with n < 256 (per-token attention), then greedy decode."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, spec, qtype, norm_jitter=0.2, weight_std=0.05)
    cm = wick.CudaLfm2Model(path, 512)
    om = orc.OracleModel(path, 512)
    st = wick.InferenceState()
    toks = gs.random_prompt(n, cm.config().vocab_size, seed=n)
    lg = cm.forward_prefill(toks, 0, st)
    lo = om.forward_prefill(toks, 0)
    assert_logits_equal(lg, lo, f"prefill n={n}")
    first = orc.argmax(lo)
    want = om.generate_greedy(first, 20)
    tok, got = first, []
    for i in range(20):
        tok = cm.forward_greedy([tok], n + i, st)
        got.append(tok)
    assert list(want) == got
    assert st.seq_len == n + 20


@pytest.mark.parametrize("spec,qtype", [("tiny", "q4_0"), ("tiny-wide", "q8_0")])
def test_prefill_flash_path_and_chunking_bit_exact(wick, orc, model_dir, spec, qtype):
    """A 700-token prompt the way Session::append_tokens feeds it (ubatch 512: one 512-token chunk on
    the tiled-attention path, one 188-token chunk on the per-token path), then a whole-prompt call."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, spec, qtype, norm_jitter=0.2, weight_std=0.05)
    cm = wick.CudaLfm2Model(path, 1024)
    om = orc.OracleModel(path, 1024)
    st = wick.InferenceState()
    toks = gs.random_prompt(700, cm.config().vocab_size, seed=8)
    consumed, lg = cm.forward_prefill_chunked(toks, 0, st, 512)
    lo = om.forward_prefill_chunked(toks, 0, 512)
    assert consumed == 700 and st.seq_len == 700
    assert_logits_equal(lg, lo, "chunked prefill")
    for li, kvh in enumerate(cm.config().kv_heads_per_layer):
        if kvh:
            k, v = cm.read_kv(li)
            ko, vo = om.kv(li)
            assert np.array_equal(k, ko) and np.array_equal(v, vo)
    # device-resident greedy loop == per-token calls == oracle
    first = orc.argmax(lo)
    want = om.generate_greedy(first, 32)
    got = cm.generate_greedy(first, 32, st)
    assert list(want) == list(got) and st.seq_len == 732
    # one 700-token call: every token on the tiled path
    lg2 = cm.forward_prefill(toks, 0, st)
    lo2 = om.forward_prefill(toks, 0)
    assert_logits_equal(lg2, lo2, "single-call prefill")
    assert st.seq_len == 700


def test_generate_matches_forward_greedy(wick, model_dir):
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-wide", "q4_0", norm_jitter=0.2, weight_std=0.05)
    a, b = wick.CudaLfm2Model(path, 256), wick.CudaLfm2Model(path, 256)
    sa, sb = wick.InferenceState(), wick.InferenceState()
    toks = gs.random_prompt(40, a.config().vocab_size)
    la, lb = a.forward_prefill(toks, 0, sa), b.forward_prefill(toks, 0, sb)
    assert np.array_equal(la, lb)
    first = int(np.argmax(la))
    ga = a.generate_greedy(first, 64, sa)
    tok, gb = first, []
    for i in range(64):
        tok = b.forward_greedy([tok], 40 + i, sb)
        gb.append(tok)
    assert list(ga) == gb


def test_trait_semantics(wick, orc, model_dir):
    from wick_b200 import gguf_synth as gs
    from wick_b200._lib import WickCudaError
    path = _model_path(model_dir, "tiny", "q4_0")
    m = wick.CudaLfm2Model(path, 48)
    cfg = m.config()
    spec = gs.SPECS["tiny"]
    assert cfg.max_seq_len == 48 and cfg.n_layers == spec.n_layers and cfg.hidden_size == spec.hidden
    assert cfg.block_types == tuple("Attention" if i in spec.attn_layers else "GatedConv" for i in range(spec.n_layers))
    assert cfg.kv_heads_per_layer == tuple(spec.n_kv_heads if i in spec.attn_layers else 0 for i in range(spec.n_layers))
    assert m.gpu_memory_bytes() > 0 and m.supports_kv_shift() and m.supports_embedding_input()
    st = wick.InferenceState()
    toks = gs.random_prompt(40, cfg.vocab_size)
    with pytest.raises(WickCudaError) as e:                     # out-of-range token
        m.forward_prefill([cfg.vocab_size], 0, st)
    assert e.value.code == -1
    with pytest.raises(AssertionError):                         # empty prompt asserts, like wick
        m.forward_prefill([], 0, st)
    m.forward_prefill(toks, 0, st)
    with pytest.raises(WickCudaError) as e:                     # wrong position
        m.forward([1], 7, st)
    assert e.value.code == -1
    with pytest.raises(WickCudaError) as e:                     # context overflow on prefill
        m.forward_prefill(toks[:9], 40, st)
    assert e.value.code == -5
    for i in range(8):
        m.forward_greedy([1], 40 + i, st)
    assert st.seq_len == 48
    with pytest.raises(WickCudaError) as e:                     # context full on decode
        m.forward_greedy([1], 48, st)
    assert e.value.code == -5
    # start_pos == 0 starts a new sequence: same logits as a fresh model
    l1 = m.forward_prefill(toks, 0, st)
    l2 = wick.CudaLfm2Model(path, 48).forward_prefill(toks, 0, wick.InferenceState())
    assert np.array_equal(l1, l2) and st.seq_len == 40
    # context_size is capped by the file's context_length
    assert wick.CudaLfm2Model(path, 1 << 20).config().max_seq_len == spec.context_length


def test_snapshot_restore_roundtrip(wick, model_dir):
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-wide", "q8_0")
    m = wick.CudaLfm2Model(path, 256)
    st = wick.InferenceState()
    toks = gs.random_prompt(90, m.config().vocab_size, seed=2)
    m.forward_prefill(toks[:60], 0, st)
    snap = m.snapshot_state()
    want = m.forward_prefill(toks[60:], 60, st)
    m.forward_prefill(toks[:5], 0, st)                          # clobber the state
    m.restore_state(snap, st)
    assert st.seq_len == 60
    assert np.array_equal(m.forward_prefill(toks[60:], 60, st), want)
    other = wick.CudaLfm2Model(path, 256)                       # restore into another instance
    st2 = wick.InferenceState()
    other.restore_state(snap, st2)
    assert np.array_equal(other.forward_prefill(toks[60:], 60, st2), want)
    with pytest.raises(Exception):
        other.restore_state(snap[:-4])


def test_from_bytes_equals_from_file(wick, model_dir):
    path = _model_path(model_dir, "tiny", "q8_0")
    a = wick.CudaLfm2Model(path, 64)
    b = wick.CudaLfm2Model.from_bytes(open(path, "rb").read(), 64)
    la = a.forward([5], 0, wick.InferenceState())
    lb = b.forward([5], 0, wick.InferenceState())
    assert np.array_equal(la, lb)


@pytest.mark.parametrize("qtype", ["q4_0"])
def test_350m_prefill_equals_sequential_decode(wick, orc, model_dir, qtype):
    """Size-independent identity at benchmark size (350M-class): a prefill shorter than 256 tokens is
    bit-identical to feeding the tokens one by one (wick/tests/blas_parity.rs:20-24), and the first
    decode steps agree with the oracle (logits within 1e-2 by contract; here bit-equal)."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "lfm2-350m", qtype)
    m = wick.CudaLfm2Model(path, 512)
    st = wick.InferenceState()
    toks = gs.random_prompt(48, m.config().vocab_size)
    lp = m.forward_prefill(toks, 0, st)
    m.reset(st)
    for i, t in enumerate(toks):
        ls = m.forward([int(t)], i, st)
    assert np.array_equal(lp, ls)
    om = orc.OracleModel(path, 512)
    lo = om.forward_prefill(toks, 0)
    assert _diff(lp, lo) <= 1e-2
    assert_logits_equal(lp, lo, "350M prefill")
    first = orc.argmax(lo)
    want = om.generate_greedy(first, 8)
    got = m.generate_greedy(first, 8, st)
    assert list(want) == list(got)


def test_persistent_and_graph_decode_agree(wick, orc, model_dir, monkeypatch):
    """The persistent decode kernel and the captured per-kernel graph are two schedules of the same
    arithmetic: identical logits, KV rows and greedy tokens (and both equal the oracle)."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-wide", "q4_0", norm_jitter=0.2, weight_std=0.05)
    a = wick.CudaLfm2Model(path, 256)
    monkeypatch.setenv("WICK_CUDA_DECODE", "graph")
    b = wick.CudaLfm2Model(path, 256)
    monkeypatch.delenv("WICK_CUDA_DECODE")
    assert a.decode_path() == "persistent" and b.decode_path() == "graph"
    om = orc.OracleModel(path, 256)
    sa, sb = wick.InferenceState(), wick.InferenceState()
    toks = gs.random_prompt(20, a.config().vocab_size, seed=4)
    for i, t in enumerate(toks):
        la, lb, lo = a.forward([int(t)], i, sa), b.forward([int(t)], i, sb), om.forward(int(t))
        assert_logits_equal(la, lo, f"persistent step {i}")
        assert_logits_equal(lb, lo, f"graph step {i}")
    ga, gb = a.generate_greedy(7, 40, sa), b.generate_greedy(7, 40, sb)
    assert list(ga) == list(gb) == list(om.generate_greedy(7, 40))
    for li, kvh in enumerate(a.config().kv_heads_per_layer):
        if kvh:
            assert all(np.array_equal(x, y) for x, y in zip(a.read_kv(li), b.read_kv(li)))
        else:
            assert np.array_equal(a.read_conv_state(li), b.read_conv_state(li))


def test_bounded_waits_report_timeout(wick, model_dir):
    """Failure detection without a GPU fault: a grid-wide wait whose condition never comes true runs
    out after a bounded number of polls, the call reports TIMEOUT, and the context stays usable."""
    import ctypes as C
    from wick_b200 import gguf_synth as gs
    from wick_b200._lib import WickCudaError, check
    path = _model_path(model_dir, "tiny", "q4_0")
    m = wick.CudaLfm2Model(path, 64)
    if m.decode_path() != "persistent":
        pytest.skip("graph decode has no device-side waits")
    st = wick.InferenceState()
    toks = gs.random_prompt(8, m.config().vocab_size)
    want = m.forward_prefill(toks, 0, st)
    t1 = m.forward_greedy([3], 8, st)
    check(m._lib.wick_cuda_debug_skew_barrier(m._h, C.c_int64(5)))      # wait for arrivals nobody makes
    with pytest.raises(WickCudaError) as e:
        m.generate_greedy(3, 2, st)
    assert e.value.code == -6
    # the same handle works again after a reset
    st = wick.InferenceState()
    assert np.array_equal(m.forward_prefill(toks, 0, st), want)
    assert m.forward_greedy([3], 8, st) == t1


def test_split_scores_long_context_decode(wick, orc, model_dir, monkeypatch):
    """From 768 cached tokens on, decode computes the cached keys' scores in a phase of its own (keys split over
    all CTAs).  Same bits as the in-phase loop (switched back on by WICK_CUDA_NO_SPLIT_SCORES) and as the oracle,
    across the switch-over point and for the device-resident loop."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-wide", "q4_0")
    toks = gs.random_prompt(760, gs.SPECS["tiny-wide"].vocab, seed=12)
    a = wick.CudaLfm2Model(path, 2048)
    sa = wick.InferenceState()
    la = a.forward_prefill(toks, 0, sa)
    om = orc.OracleModel(path, 2048)
    lo = om.forward_prefill(toks, 0)
    assert_logits_equal(la, lo, "prefill")
    tok = orc.argmax(lo)
    for i in range(20):                      # positions 760..779: the list switches at 768
        x, y = a.forward([tok], sa.seq_len, sa), om.forward(tok)
        assert_logits_equal(x, y, f"step {i}")
        tok = orc.argmax(y)
    dev = a.generate_greedy(tok, 40, sa)
    assert list(dev) == list(om.generate_greedy(tok, 40))
    monkeypatch.setenv("WICK_CUDA_NO_SPLIT_SCORES", "1")
    b = wick.CudaLfm2Model(path, 2048)
    sb = wick.InferenceState()
    more = gs.random_prompt(900, gs.SPECS["tiny-wide"].vocab, seed=13)
    lb = b.forward_prefill(more, 0, sb)
    monkeypatch.delenv("WICK_CUDA_NO_SPLIT_SCORES")
    la2 = a.forward_prefill(more, 0, sa)
    assert_logits_equal(la2, lb, "prefill again")
    first = int(np.argmax(lb))
    monkeypatch.setenv("WICK_CUDA_NO_SPLIT_SCORES", "1")
    gb = b.generate_greedy(first, 32, sb)
    monkeypatch.delenv("WICK_CUDA_NO_SPLIT_SCORES")
    ga = a.generate_greedy(first, 32, sa)
    assert list(ga) == list(gb)


@pytest.mark.parametrize("spec,qtype", [("tiny", "q4_0"), ("tiny-wide", "q8_0")])
def test_flagged_hidden_handover_matches_barrier_path(wick, orc, model_dir, monkeypatch, spec, qtype):
    """RMSNorm phases take the hidden row from flagged 64-bit words instead of waiting at a grid barrier.  A model
    created with WICK_CUDA_NO_FLAGGED_HIDDEN keeps the barriers: both must give the oracle's bits, step by step and
    in the device-resident loop (many steps per launch, so phase ids run on across steps and launches)."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, spec, qtype)
    toks = gs.random_prompt(24, gs.SPECS[spec].vocab, seed=31)
    a = wick.CudaLfm2Model(path, 512)
    monkeypatch.setenv("WICK_CUDA_NO_FLAGGED_HIDDEN", "1")
    b = wick.CudaLfm2Model(path, 512)
    monkeypatch.delenv("WICK_CUDA_NO_FLAGGED_HIDDEN")
    om = orc.OracleModel(path, 512)
    sa, sb = wick.InferenceState(), wick.InferenceState()
    la, lb, lo = a.forward_prefill(toks, 0, sa), b.forward_prefill(toks, 0, sb), om.forward_prefill(toks, 0)
    assert_logits_equal(la, lo, "prefill")
    assert_logits_equal(lb, lo, "prefill (barriers)")
    tok = orc.argmax(lo)
    for i in range(6):
        y = om.forward(tok)
        assert_logits_equal(a.forward([tok], sa.seq_len, sa), y, f"step {i}")
        assert_logits_equal(b.forward([tok], sb.seq_len, sb), y, f"step {i} (barriers)")
        tok = orc.argmax(y)
    want = list(om.generate_greedy(tok, 100))
    assert list(a.generate_greedy(tok, 100, sa)) == want
    assert list(b.generate_greedy(tok, 100, sb)) == want
    # the persistent kernel is what ran (a fallback to the per-kernel graph would not exercise the hand-over)
    assert a.decode_path() == "persistent" and b.decode_path() == "persistent"


def test_head_dim_128_prefill_and_decode(wick, orc, model_dir):
    """128-wide heads: a 300-token prompt (tiled attention path, n >= 256), a continuation chunk and decode steps,
    all bit-equal to the oracle."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-hd128", "q4_0", norm_jitter=0.2, weight_std=0.05)
    cm, om = wick.CudaLfm2Model(path, 1024), orc.OracleModel(path, 1024)
    st = wick.InferenceState()
    toks = gs.random_prompt(300 + 260, cm.config().vocab_size, seed=9)
    assert_logits_equal(cm.forward_prefill(toks[:300], 0, st), om.forward_prefill(toks[:300], 0), "hd128 prefill 300")
    assert_logits_equal(cm.forward_prefill(toks[300:], 300, st), om.forward_prefill(toks[300:], 300), "hd128 continuation 260")
    first = 5
    assert list(cm.generate_greedy(first, 12, st)) == list(om.generate_greedy(first, 12))


def test_two_models_with_different_long_contexts(wick, orc, model_dir):
    """The per-token attention kernel's opt-in shared-memory limit belongs to the kernel on a device, not to a model:
    a second model with a shorter (but still > 48 KB of scores) context must not lower it under the first."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-longctx", "q4_0")
    m1 = wick.CudaLfm2Model(path, 32768)
    m2 = wick.CudaLfm2Model(path, 16384)
    st1, st2 = wick.InferenceState(), wick.InferenceState()
    toks = gs.random_prompt(40, m1.config().vocab_size, seed=2)
    om = orc.OracleModel(path, 32768)
    want = om.forward_prefill(toks, 0)
    assert_logits_equal(m2.forward_prefill(toks, 0, st2), want, "second model")
    assert_logits_equal(m1.forward_prefill(toks, 0, st1), want, "first model, after the second one was created and used")


def test_prefill_category_timers(wick, model_dir):
    """The per-category device timers change nothing in the results and account for the time of a prefill call."""
    from wick_b200 import gguf_synth as gs
    path = _model_path(model_dir, "tiny-wide", "q4_0")
    m = wick.CudaLfm2Model(path, 1024)
    st = wick.InferenceState()
    toks = gs.random_prompt(600, m.config().vocab_size, seed=5)
    plain = m.forward_prefill(toks, 0, st)
    m.profile_enable(True)
    timed = m.forward_prefill(toks, 0, st)
    total_ms = m.last_elapsed_ms()
    prof = m.profile_read()
    m.profile_enable(False)
    assert np.array_equal(plain, timed)
    assert set(prof) == {"embedding", "rmsnorm+quantise", "gemm", "short-conv", "qk-norm+rope+kv-append", "attention",
                         "activation+quantise", "output-norm+logits"}
    assert all(v >= 0 for v in prof.values()) and prof["gemm"] > 0 and prof["attention"] > 0
    assert 0.5 * total_ms <= sum(prof.values()) <= 1.05 * total_ms, (prof, total_ms)
    assert all(v == 0 for v in m.profile_read().values())        # disabling clears the totals
