"""Host-side logic of the tensor-parallel variant (no GPU): the partition arithmetic, slicing of quantised block rows,
the winner merge of the split vocabulary head, and a world-size-2 gloo run in which the shards' partial products,
all-reduced, reproduce the unsplit product."""
import os
import socket

import numpy as np
import pytest

from wick_b200 import gguf_synth as gs
from wick_b200 import tensor_parallel as tp

F32 = np.float32


def plan(world, rank, hidden=2048, ffn=6912, nh=32, nkv=8, vocab=65536):
    return tp.TpPlan(hidden, ffn, nh, nkv, hidden // nh, vocab, world, rank)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_tile_every_matrix_exactly(world):
    """1.6B-class shapes: every rank's ranges are whole 32-element blocks and together cover each axis once."""
    for getter, total in (("q_rows", 2048), ("kv_rows", 512), ("ffn_rows", 6912), ("vocab_rows", 65536), ("channels", 2048),
                          ("o_cols", 2048), ("out_proj_cols", 2048), ("down_cols", 6912)):
        covered = []
        for r in range(world):
            a, b = getattr(plan(world, r), getter)()
            assert a % 32 == 0 and b % 32 == 0 and b > a
            covered.append((a, b))
        assert covered[0][0] == 0 and covered[-1][1] == total
        assert all(covered[i][1] == covered[i + 1][0] for i in range(world - 1))
    p = plan(world, world - 1)
    thirds = p.in_proj_row_ranges()
    c0, c1 = p.channels()
    assert thirds == [(c0, c1), (2048 + c0, 2048 + c1), (4096 + c0, 4096 + c1)]


def test_impossible_splits_are_refused():
    with pytest.raises(ValueError):
        plan(3, 0)                                   # 32 heads / 3
    plan(8, 0, ffn=4608, hidden=1024, nh=16)         # the 350M-class shapes do split 8 ways
    with pytest.raises(ValueError):
        plan(16, 0)
    with pytest.raises(ValueError):
        plan(2, 2)
    with pytest.raises(ValueError):
        tp.TpPlan(2048, 6912 + 32, 32, 8, 64, 65536, 8, 0)   # ffn shard would cut a 32-element block


@pytest.mark.parametrize("qtype,dt", [("q4_0", tp.DT_Q4_0), ("q8_0", tp.DT_Q8_0)])
def test_block_row_slicing_matches_dequantised_slices(qtype, dt):
    rng = np.random.default_rng(0)
    m, k = 24, 256
    w = rng.standard_normal((m, k)).astype(F32) * F32(0.05)
    raw = gs.QUANTIZERS[qtype][0](w).reshape(m, -1)
    full = tp.dequantize_rows(raw, dt)
    assert full.shape == (m, k) and np.abs(full - w).max() < 0.05
    assert np.array_equal(tp.dequantize_rows(tp.slice_k(raw, dt, 64, 192), dt), full[:, 64:192])
    assert np.array_equal(tp.dequantize_rows(tp.slice_rows(raw, [(2, 5), (10, 12)]), dt), np.concatenate([full[2:5], full[10:12]]))


def test_merge_argmax_follows_cpu_argmax():
    # largest value wins; among equal values the LAST index; NaN never wins (sampler.rs:8-19)
    assert tp.merge_argmax(np.array([1.0, 3.0, 2.0], F32), np.array([5, 70, 130])) == 70
    assert tp.merge_argmax(np.array([3.0, 3.0, 2.0], F32), np.array([5, 70, 130])) == 70
    assert tp.merge_argmax(np.array([np.nan, -1.0], F32), np.array([5, 70])) == 70


def test_rope_table_iterates_theta_in_f32():
    cos, sin = tp.rope_tables(5, 8, 1e6)
    scale = F32(np.power(F32(1e6), F32(-2.0) / F32(8)))
    theta = F32(3.0)
    for i in range(4):
        assert abs(float(cos[3, i]) - float(np.cos(theta))) < 1e-6 and abs(float(sin[3, i]) - float(np.sin(theta))) < 1e-6
        theta = F32(theta * scale)
    assert np.all(cos[0] == 1.0) and np.all(sin[0] == 0.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(1)                      # same draws on every rank: replicated weights and input
        hs, ffn, nh, nkv, vocab = 128, 192, 4, 2, 256
        p = tp.TpPlan(hs, ffn, nh, nkv, hs // nh, vocab, world, rank)
        x = rng.standard_normal(hs).astype(F32)
        w_up = tp.dequantize_rows(gs.quantize_q4_0(rng.standard_normal((ffn, hs)).astype(F32) * F32(0.05)).reshape(ffn, -1), tp.DT_Q4_0)
        down_raw = gs.quantize_q4_0(rng.standard_normal((hs, ffn)).astype(F32) * F32(0.05)).reshape(hs, -1)
        w_down = tp.dequantize_rows(down_raw, tp.DT_Q4_0)
        # column split then row split, as in the FFN: act shard -> partial of the hidden row -> all-reduce
        r0, r1 = p.ffn_rows()
        act = w_up[r0:r1] @ x
        k0, k1 = p.down_cols()
        assert (k0, k1) == (r0, r1)
        part = tp.dequantize_rows(tp.slice_k(down_raw, tp.DT_Q4_0, k0, k1), tp.DT_Q4_0) @ act
        t = torch.from_numpy(part.astype(np.float64))
        dist.all_reduce(t)
        want = w_down.astype(np.float64) @ (w_up.astype(np.float64) @ x.astype(np.float64))
        err = float(np.abs(t.numpy() - want).max())
        # the vocabulary head: per-rank winners merged
        logits = rng.standard_normal(vocab).astype(F32)
        v0, v1 = p.vocab_rows()
        local = int(np.argmax(logits[v0:v1]))
        pair = torch.tensor([float(logits[v0 + local]), float(v0 + local)], dtype=torch.float64)
        parts = [torch.empty_like(pair) for _ in range(world)]
        dist.all_gather(parts, pair)
        host = torch.stack(parts).numpy()
        q.put((rank, err, tp.merge_argmax(host[:, 0].astype(F32), host[:, 1].astype(np.int64)), int(np.argmax(logits))))
    finally:
        dist.destroy_process_group()


def test_world_size_2_partials_all_reduce_to_the_unsplit_product():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=120) for _ in procs]
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    for rank, err, merged, want in res:
        assert err < 1e-4, (rank, err)
        assert merged == want
