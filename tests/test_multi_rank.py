"""world_size-2 (and 3) gloo runs of the multi-GPU host logic on CPU.

The path shards by sequence with no data-path collective, so what needs covering is that
(1) every sequence is decoded by exactly one rank, (2) a sequence's tokens do not depend on the
rank it lands on, and (3) the whole-job figures are tokens summed over ranks over the slowest
rank's time.  The CPU oracle stands in for the decoder here (tests only).
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from wick_b200 import sharding  # noqa: E402

N_SEQ = 5
PROMPT = 12
DECODE = 6


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _decode_sequences(model_path, indices):
    from oracle import oracle as orc
    from wick_b200 import gguf_synth as gs
    om = orc.OracleModel(model_path, 256)
    vocab = gs.SPECS["tiny"].vocab
    outs = []
    for i in indices:
        om.reset()
        toks = gs.random_prompt(PROMPT, vocab, seed=sharding.prompt_seed(1, i))
        first = orc.argmax(om.forward_prefill(toks, 0))
        outs.append([first] + [int(t) for t in om.generate_greedy(first, DECODE)])
    return outs


def _worker(rank, world, port, model_path, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sharding.shard_sequences(N_SEQ, world, rank)
        outs = _decode_sequences(model_path, mine)
        local_tokens = sum(len(o) for o in outs)
        local_seconds = 1.0 + 0.25 * rank            # made-up per-rank device times
        tot = sharding.job_totals(local_tokens, local_seconds)
        streams = sharding.gather_token_streams(outs, mine, N_SEQ)
        dist.barrier()
        q.put((rank, mine, tot.tokens, tot.seconds, tot.per_rank_tokens, streams))
    finally:
        dist.destroy_process_group()


def test_shard_sequences_partition():
    for world in (1, 2, 3, 4, 8):
        for n in (0, 1, 5, 8, 17):
            seen = []
            for r in range(world):
                seen += sharding.shard_sequences(n, world, r)
            assert sorted(seen) == list(range(n))
            sizes = [len(sharding.shard_sequences(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_sequences(4, 2, 2)


def test_job_totals_single_process():
    t = sharding.job_totals(256, 0.5)
    assert t.tokens == 256 and t.seconds == 0.5 and t.tokens_per_second == 512.0


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_decode_matches_single_rank(world, orc, model_dir):
    from wick_b200 import gguf_synth as gs
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=str(model_dir))
    single = _decode_sequences(path, list(range(N_SEQ)))

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, path, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0

    per_rank_expected = [len(sharding.shard_sequences(N_SEQ, world, r)) * (DECODE + 1) for r in range(world)]
    for rank, mine, tokens, seconds, per_rank, streams in results:
        assert mine == list(range(rank, N_SEQ, world))
        assert tokens == N_SEQ * (DECODE + 1)
        assert per_rank == per_rank_expected
        assert seconds == pytest.approx(1.0 + 0.25 * (world - 1))      # the slowest rank's time
        assert streams == single                                        # bit-identical tokens per sequence
    assert len({tuple(map(tuple, r[5])) for r in results}) == 1
    assert np.asarray(single).shape == (N_SEQ, DECODE + 1)
