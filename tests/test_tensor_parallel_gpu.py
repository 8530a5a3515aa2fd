"""Tensor-parallel LFM2 (wick_b200/tensor_parallel.py) on GPUs against the CPU oracle.

World size 1 runs on any GPU box and checks the operator pipeline the variant is built from; world size 2 needs two
GPUs (skipped otherwise) and exercises the split, the NCCL all-reduce of prefill and the one-shot peer-memory
all-reduce of decode.  Parity is by tolerance: the shards' partial sums are added in rank order, which is not the
single-device accumulation order, and the RoPE table comes from numpy instead of the C library.
"""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
F32 = np.float32
REL_TOL = 2e-2      # of the largest |logit|: a last-bit change of an activation can move a Q8_0 quant one step


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, path, fused, q):
    import torch
    import torch.distributed as dist
    from wick_b200 import gguf_synth as gs
    from wick_b200 import tensor_parallel as tp
    from oracle import oracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl" if world > 1 else "gloo", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank) if world > 1 else None)
    try:
        m = tp.TpLfm2Model(path, 512, rank, world, rank, fused_allreduce=fused)
        om = orc.OracleModel(path, 512)
        toks = gs.random_prompt(300, m.vocab, seed=11)
        out = {}
        lg, lo = m.forward_prefill(toks[:270], 0), om.forward_prefill(toks[:270], 0)          # tiled-attention chunk
        out["prefill"] = float(np.abs(lg - lo).max() / np.abs(lo).max())
        lg, lo = m.forward_prefill(toks[270:], 270), om.forward_prefill(toks[270:], 270)      # continuation, per-token attention
        out["continuation"] = float(np.abs(lg - lo).max() / np.abs(lo).max())
        worst, same = 0.0, 0
        tok = orc.argmax(lo)
        for _ in range(8):
            lg, lo = m.forward(tok), om.forward(tok)
            worst = max(worst, float(np.abs(lg - lo).max() / np.abs(lo).max()))
            tok = orc.argmax(lo)
        out["decode"] = worst
        want = om.generate_greedy(tok, 16)
        got, t = [], tok
        for _ in range(16):
            t = m.forward_greedy(t)
            got.append(t)
        m.check_status()
        out["tokens_equal"] = int(sum(int(a) == int(b) for a, b in zip(got, want)))
        out["first_mismatch_free"] = int(got[0]) == int(want[0])
        q.put((rank, out, [int(x) for x in got]))
        m.close()
    finally:
        dist.destroy_process_group()


def _run(world, path, fused):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, path, fused, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return sorted(res)


def _check(res):
    tokens = res[0][2]
    for rank, out, got in res:
        assert out["prefill"] <= REL_TOL and out["continuation"] <= REL_TOL and out["decode"] <= REL_TOL, (rank, out)
        assert got == tokens, "ranks must compute identical tokens"
    return res[0][1]


@pytest.fixture(scope="module")
def tiny_wide(cuda_lib, orc, model_dir):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from wick_b200 import gguf_synth as gs
    return gs.cached_model("tiny-wide", "q4_0", 0, cache_dir=model_dir, norm_jitter=0.2, weight_std=0.05)


def test_world_1_pipeline_matches_oracle(tiny_wide):
    out = _check(_run(1, tiny_wide, False))
    assert out["tokens_equal"] == 16        # nothing is reordered with one rank; only the RoPE table's origin differs


@pytest.mark.parametrize("fused", [True, False])
def test_world_2_matches_oracle_within_tolerance(tiny_wide, fused):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _check(_run(2, tiny_wide, fused))
    assert out["first_mismatch_free"]
