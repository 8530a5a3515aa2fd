"""The synthetic GGUF writer against ggml's own Python package (format, metadata types, quantisers)."""
import numpy as np
import pytest

from wick_b200 import gguf_synth as gs

gguf = pytest.importorskip("gguf")


@pytest.mark.parametrize("name,T", [("q4_0", "Q4_0"), ("q8_0", "Q8_0")])
def test_quantisers_match_ggml(name, T):
    from gguf import quants, GGMLQuantizationType
    rng = np.random.default_rng(11)
    x = rng.standard_normal((37, 256), dtype=np.float32) * np.float32(0.02)
    x[3, :32] = 0
    x[4, 5] = 1e4
    fn = gs.QUANTIZERS[name][0]
    assert np.array_equal(fn(x), quants.quantize(x, getattr(GGMLQuantizationType, T)))
    assert np.array_equal(gs.dequantize(fn(x), name, 256), quants.dequantize(fn(x), getattr(GGMLQuantizationType, T)))


@pytest.mark.parametrize("qtype", ["q4_0", "q8_0"])
def test_file_is_readable_by_ggml_reader(model_dir, qtype):
    path = gs.cached_model("tiny", qtype, 0, cache_dir=model_dir)
    r = gguf.GGUFReader(path)
    spec = gs.SPECS["tiny"]
    f = r.fields
    # value types wick's loader insists on (lfm2.rs:105-148)
    for key in ("block_count", "embedding_length", "feed_forward_length", "attention.head_count", "vocab_size",
                "context_length", "shortconv.l_cache"):
        assert f["lfm2." + key].types == [gguf.GGUFValueType.UINT32], key
    assert f["lfm2.rope.freq_base"].types == [gguf.GGUFValueType.FLOAT32]
    assert f["lfm2.attention.layer_norm_rms_epsilon"].types == [gguf.GGUFValueType.FLOAT32]
    kv = f["lfm2.attention.head_count_kv"]
    assert kv.types == [gguf.GGUFValueType.ARRAY, gguf.GGUFValueType.INT32]
    assert [int(kv.parts[i][0]) for i in kv.data] == [spec.n_kv_heads if i in spec.attn_layers else 0 for i in range(spec.n_layers)]
    assert len(f["tokenizer.ggml.tokens"].data) == spec.vocab
    names = {t.name: t for t in r.tensors}
    assert "token_embd.weight" in names and "token_embd_norm.weight" in names and "output.weight" not in names
    t = names["blk.0.shortconv.in_proj.weight"]
    assert list(t.shape) == [spec.hidden, 3 * spec.hidden]          # GGUF dims [k, m]
    assert list(names["blk.0.shortconv.conv.weight"].shape) == [spec.conv_kernel, spec.hidden]
    assert "blk.1.attn_q.weight" in names and "blk.1.attn_q_norm.weight" in names


def test_same_seed_same_bytes(tmp_path):
    a = gs.write_lfm2_gguf(str(tmp_path / "a.gguf"), gs.SPECS["tiny"], "q4_0", seed=5)
    b = gs.write_lfm2_gguf(str(tmp_path / "b.gguf"), gs.SPECS["tiny"], "q4_0", seed=5)
    c = gs.write_lfm2_gguf(str(tmp_path / "c.gguf"), gs.SPECS["tiny"], "q4_0", seed=6)
    assert open(a, "rb").read() == open(b, "rb").read() != open(c, "rb").read()


def test_weight_byte_counts_match_the_roofline_numerators():
    # bytes of quantised matmul weights read once per decoded token + the one embedding row looked up
    a, b = gs.SPECS["lfm2-350m"], gs.SPECS["lfm2.5-1.6b"]
    assert a.decode_bytes_per_token("q4_0") == 199_361_088
    assert a.decode_bytes_per_token("q8_0") == 376_570_944
    assert b.decode_bytes_per_token("q4_0") == 587_465_856
    assert b.decode_bytes_per_token("q8_0") == 1_109_657_728
