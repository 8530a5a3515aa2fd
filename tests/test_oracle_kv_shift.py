"""CPU checks of the oracle's shift_kv restatement (kv_cache.rs:601-715) against the properties the
reference's own tests use (kv_cache.rs shift tests): V rows slide unchanged, kept rows are untouched, and a
K row re-rotated by R(-shift) equals, to rounding, the row freshly rotated for its new position."""
import numpy as np


def test_shift_properties(orc, model_dir):
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir)
    om = orc.OracleModel(path, 64)
    toks = gs.random_prompt(24, gs.SPECS["tiny"].vocab, seed=3)
    om.forward_prefill(toks, 0)
    li = [i for i, a in enumerate(om.is_attn) if a][0]
    k0, v0 = om.kv(li)
    conv0 = [om.conv_state(i) for i, a in enumerate(om.is_attn) if not a]
    n_keep, shift = 5, 7
    om.shift_kv(n_keep, shift)
    assert om.seq_len == 24 - shift
    k1, v1 = om.kv(li)
    assert k1.shape[0] == 24 - shift
    assert np.array_equal(v1[:n_keep], v0[:n_keep]) and np.array_equal(v1[n_keep:], v0[n_keep + shift:])
    assert np.array_equal(k1[:n_keep], k0[:n_keep])
    # rotation preserves the norm of every (i, i + hd/2) pair and is not the identity
    hd = om.head_dim
    half = hd // 2
    moved_old = k0[n_keep + shift:].reshape(-1, hd)
    moved_new = k1[n_keep:].reshape(-1, hd)
    r_old = moved_old[:, :half] ** 2 + moved_old[:, half:] ** 2
    r_new = moved_new[:, :half] ** 2 + moved_new[:, half:] ** 2
    assert np.allclose(r_old, r_new, rtol=1e-5, atol=1e-9)
    assert not np.allclose(moved_old, moved_new)
    # conv buffers are left alone
    for c_old, i in zip(conv0, [i for i, a in enumerate(om.is_attn) if not a]):
        assert np.array_equal(c_old, om.conv_state(i))
    # composing two shifts == one shift of the sum, to rounding (rotations add)
    a, b = orc.OracleModel(path, 64), orc.OracleModel(path, 64)
    a.forward_prefill(toks, 0)
    b.forward_prefill(toks, 0)
    a.shift_kv(4, 3)
    a.shift_kv(4, 2)
    b.shift_kv(4, 5)
    ka, _ = a.kv(li)
    kb, _ = b.kv(li)
    assert np.allclose(ka, kb, rtol=1e-4, atol=1e-6)
    import pytest
    with pytest.raises(ValueError):
        b.shift_kv(10, 100)
