#!/usr/bin/env python
"""Benchmark of the CUDA LFM2 backend on wick's headline metric.

Workload (one "step"): the `wick bench` decode protocol on a seeded random-init
LFM2.5-1.6B-class Q4_0 model, batch 1: a 128-token uniform-random prompt is prefilled
(not timed, as in wick: decode tok/s excludes the prefill, wick-cli/src/main.rs:2655-2676),
then 128 greedy decode tokens are generated (tg128, positions 128..255) and timed.

  value   decode tok/s with the loop resident on the GPU (wick_cuda_generate_greedy: the
          argmax of step i feeds step i+1 on the device), timed with CUDA events on the
          library's own stream.
  e2e     the same 128 tokens through the reference-facing call a wick Session makes,
          one wick_cuda_forward_greedy per token: the token id goes host->device from
          pinned memory and the chosen id comes back device->host every step; host wall clock.
  roofline  algorithmic weight bytes per token / device time per token, against the measured
          HBM copy bandwidth (MEASURED_PEAKS.json, else a fallback constant).

`--impl reference` times the CPU oracle (the restatement of wick's own CPU path; wick is Rust and
cannot be built here) on the host cores for the same workload, on a bounded sample.

With N > 1 (torchrun) every rank decodes its own independent sequence on its own GPU: sequences
are the unit of sharding, there is no data-path collective ("weak" scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

PROMPT_TOKENS = 128
DECODE_TOKENS = 128
PREFILL_REPEATS = 5     # side measurements of prefill: p50 over this many repeats after one warm call
# serving side line: independent sequences per GPU, each with its own prompt, decoded together in batched steps
SERVE_SEQUENCES, SERVE_PROMPT, SERVE_DECODE = 64, 512, 256
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per decoded token from an ncu capture of the decode
# kernels, keyed by (model, qtype); None until captured.
NCU_TRAFFIC_BYTES_PER_TOKEN = {("lfm2.5-1.6b", "q4_0"): 588.7e6}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks + throttle reasons every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append((time.time(), ln.strip()))

    def stop(self, t0: float, t1: float):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for ts, ln in self.lines:
            if ts < t0 - 0.1 or ts > t1 + 0.3:
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_file(args, rank: int, world: int):
    """Seeded synthetic model; rank 0 writes it, the others wait for the file."""
    from wick_b200 import gguf_synth as gs
    spec = gs.SPECS[args.model]
    if rank == 0:
        return gs.cached_model(args.model, args.qtype, 0), spec
    cache_dir = os.environ.get("WICK_SYNTH_CACHE", "/tmp/wick_b200_models")
    deadline = time.time() + 600
    while time.time() < deadline:
        if os.path.isdir(cache_dir):
            hits = [f for f in os.listdir(cache_dir) if f.startswith(f"{spec.name}-{args.qtype}-s0-") and f.endswith(".gguf")]
            if hits:
                return os.path.join(cache_dir, hits[0]), spec
        time.sleep(1.0)
    raise RuntimeError("timed out waiting for rank 0 to write the model file")


def cpu_baseline(path: str, spec, sample_tokens: int, warm: int = 2):
    """The CPU oracle on this host's cores: 128-token prefill (not timed) then `sample_tokens`
    greedy decode tokens (timed)."""
    from wick_b200 import gguf_synth as gs
    from oracle import oracle as orc
    orc.build()
    orc.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    om = orc.OracleModel(path, 4096)
    toks = gs.random_prompt(PROMPT_TOKENS, spec.vocab, seed=1)
    lg = om.forward_prefill(toks, 0)
    first = orc.argmax(lg)
    out = om.generate_greedy(first, warm)
    t0 = time.perf_counter()
    om.generate_greedy(int(out[-1]), sample_tokens)
    dt = time.perf_counter() - t0
    return sample_tokens / dt, orc.num_threads()


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    from wick_b200 import gguf_synth as gs
    from oracle import oracle as orc
    orc.build()
    # all host threads this process may use (torchrun exports OMP_NUM_THREADS=1 for its workers)
    orc.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    path, spec = model_file(args, 0, 1)
    om = orc.OracleModel(path, 4096)
    toks = gs.random_prompt(PROMPT_TOKENS, spec.vocab, seed=1)
    tok = orc.argmax(om.forward_prefill(toks, 0))
    per_step = 8  # decode tokens per step: a bounded sample of the tg128 run
    for _ in range(args.warmup):
        tok = int(om.generate_greedy(tok, per_step)[-1])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        if om.seq_len + per_step > 4000:
            tok = orc.argmax(om.forward_prefill(toks, 0))
        tok = int(om.generate_greedy(tok, per_step)[-1])
    dt = time.perf_counter() - t0
    val = args.steps * per_step / dt
    cores = orc.num_threads()
    sample = f"{PROMPT_TOKENS}-token prefill (untimed), then {per_step} greedy decode tokens per step"
    line = {
        "impl": "reference", "metric": "decode tok/s bs=1 (tg128)", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(args, spec),
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def gemm_flop_per_token(spec) -> float:
    """2 * (parameters of the per-layer matrices): the multiply-adds one prompt token costs in the GEMMs."""
    return 2.0 * sum(
        (3 * spec.hidden * spec.ffn) + ((spec.hidden * spec.hidden * 2 + 2 * spec.hidden * spec.kv_dim) if i in spec.attn_layers
                                        else 4 * spec.hidden * spec.hidden)
        for i in range(spec.n_layers))


def int8_peak_tflops():
    """int8 dense tensor peak used as the prefill roofline: 2 x the measured sustained bf16 figure (the
    file holds no int8 measurement; int8 is twice bf16 on this part)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return 2.0 * float(json.load(f)["bf16_tflops_sustained"]), "2 x bf16_tflops_sustained (measured)"
    except Exception:
        return 2.0 * 1400.0, "2 x 1400 (fallback)"


def run_prefill_only(args, m, st, spec, gs):
    """Profiling aid (single GPU): each step is one prompt of --prompt-tokens through
    forward_prefill_chunked in --prefill-mode; prints a JSON line of its own, not the headline metric."""
    m.set_prefill_mode(args.prefill_mode)
    n = args.prompt_tokens
    toks = gs.random_prompt(n, spec.vocab, seed=7)
    for _ in range(args.warmup):
        m.forward_prefill_chunked(toks, 0, st, args.ubatch)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        m.forward_prefill_chunked(toks, 0, st, args.ubatch)
    dt = (time.perf_counter() - t0) / args.steps
    peak, src = int8_peak_tflops()
    tf = n / dt * gemm_flop_per_token(spec) / 1e12
    print(json.dumps({
        "metric": f"prefill tok/s @{n}", "value": n / dt, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"{spec.name} {args.qtype.upper()} prefill of {n} tokens, ubatch {args.ubatch}, mode {args.prefill_mode}"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                     "peak_source": src, "note": "GEMM flops of the whole prefill over its wall time (attention and the small kernels included in the time)"},
    }))


def serving_side_line(m, spec, args, gs, hbm_peak):
    """Batched multi-sequence decode on one GPU: SERVE_SEQUENCES independent sequences, each prefilled with its own
    SERVE_PROMPT-token uniform-random prompt, then SERVE_DECODE greedy steps in which every step reads the weights
    once for all sequences (wick_cuda_decode_batch_steps).  Not the headline metric; reported with its own roofline
    (weight bytes once per step over the device time of a step)."""
    ids, firsts = [], []
    t0 = time.perf_counter()
    for i in range(SERVE_SEQUENCES):
        sid = m.seq_create()
        toks = gs.random_prompt(SERVE_PROMPT, spec.vocab, seed=1000 + i)
        firsts.append(int(np.argmax(m.seq_prefill(sid, toks, 0))))
        ids.append(sid)
    prefill_s = time.perf_counter() - t0
    warm = m.decode_batch_steps(firsts, ids, 4)
    t0 = time.perf_counter()
    out = m.decode_batch_steps(warm[-1], ids, SERVE_DECODE - 4)
    wall = time.perf_counter() - t0
    dev = m.last_elapsed_ms() * 1e-3
    steps = SERVE_DECODE - 4
    # the same through one call per step (tokens host -> device, choices device -> host every step)
    tok = out[-1]
    n_e2e = 32
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        if m.seq_length(ids[0]) + 1 >= args.context:
            break
        tok = m.decode_batch(tok, ids)
    e2e = time.perf_counter() - t0
    for sid in ids:
        m.seq_destroy(sid)
    bpt = spec.decode_bytes_per_token(args.qtype)
    return {
        "workload": f"{SERVE_SEQUENCES} sequences x ({SERVE_PROMPT}-token prompt + {SERVE_DECODE} greedy tokens), one batched step per token",
        "decode_tok_s_device": SERVE_SEQUENCES * steps / dev, "decode_tok_s_wall": SERVE_SEQUENCES * steps / wall,
        "decode_tok_s_per_step_calls": SERVE_SEQUENCES * n_e2e / e2e,
        "ms_per_step": dev / steps * 1e3,
        "prefill_tok_s_wall": SERVE_SEQUENCES * SERVE_PROMPT / prefill_s,
        "roofline": {"bound": "hbm", "achieved": bpt / (dev / steps) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                     "frac": bpt / (dev / steps) / 1e9 / hbm_peak,
                     "note": "weight bytes once per batched step; at 64 rows the step is bound by the exact GEMM's epilogue, not by HBM"},
    }


def workload_config(args, spec):
    return {
        "workload": f"{spec.name} {args.qtype.upper()} bs=1: {PROMPT_TOKENS}-token uniform-random prompt prefill (untimed), "
                    f"then tg{DECODE_TOKENS} greedy decode (timed)",
        "weights": "random init N(0,0.02) seed 0, quantised per 32-element block; synthetic stand-in for the public checkpoint",
        "l2": f"inputs larger than L2: {spec.decode_bytes_per_token(args.qtype) / 1e6:.0f} MB of weights are streamed per token (L2 126 MB)",
        "context": args.context,
    }


def main():
    global PROMPT_TOKENS, DECODE_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--model", default="lfm2.5-1.6b")
    ap.add_argument("--qtype", default="q4_0", choices=["q4_0", "q8_0"])
    ap.add_argument("--prompt-tokens", type=int, default=PROMPT_TOKENS, help="profiling aid; the metric is quoted at 128")
    ap.add_argument("--decode-tokens", type=int, default=DECODE_TOKENS, help="profiling aid; the metric is quoted at 128")
    ap.add_argument("--no-extra", action="store_true", help="skip the prefill / tg512 side measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default="decode", choices=["decode", "prefill"],
                    help="profiling aid: 'prefill' times forward_prefill_chunked of --prompt-tokens instead of the headline decode")
    ap.add_argument("--prefill-mode", default="exact", choices=["exact", "tensor", "exact-cuda-cores"])
    ap.add_argument("--context", type=int, default=4096, help="context size the model is created with (prompt + decode tokens must fit)")
    ap.add_argument("--ubatch", type=int, default=512, help="prefill chunk of --only prefill (0 = one call); wick's default is 512")
    args = ap.parse_args()
    PROMPT_TOKENS, DECODE_TOKENS = args.prompt_tokens, args.decode_tokens
    args.warmup = max(args.warmup, 3) if args.impl == "cuda" and args.only == "decode" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from wick_b200 import gguf_synth as gs
    from wick_b200 import sharding
    from wick_b200.model import CudaLfm2Model, InferenceState

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA backend has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    path, spec = model_file(args, rank, world)
    barrier()
    m = CudaLfm2Model(path, args.context, device=local_rank)
    st = InferenceState()
    # one independent sequence per rank (round-robin over `world` sequences), no data-path collective
    seq_index = sharding.shard_sequences(world, world, rank)[0]
    prompt = gs.random_prompt(PROMPT_TOKENS, spec.vocab, seed=sharding.prompt_seed(1, seq_index))

    if args.only == "prefill":
        run_prefill_only(args, m, st, spec, gs)
        return

    counters = {"decode_launches": 0}

    def one_step(e2e: bool):
        """Returns (decode seconds, tokens)."""
        logits = m.forward_prefill(prompt, 0, st)
        first = int(np.argmax(logits))
        if not e2e:
            before = m.kernel_launches()
            m.generate_greedy(first, DECODE_TOKENS, st)
            counters["decode_launches"] += m.kernel_launches() - before
            return m.last_elapsed_ms() * 1e-3
        tok = first
        t0 = time.perf_counter()
        for i in range(DECODE_TOKENS):
            tok = m.forward_greedy([tok], PROMPT_TOKENS + i, st)
        return time.perf_counter() - t0

    for _ in range(args.warmup):
        one_step(False)
    one_step(True)

    counters["decode_launches"] = 0
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    barrier()
    t_wall0 = time.time()
    dev_s = 0.0
    for _ in range(args.steps):
        dev_s += one_step(False)
    barrier()
    # e2e leg
    barrier()
    e2e_s = 0.0
    for _ in range(args.steps):
        e2e_s += one_step(True)
    barrier()
    t_wall2 = time.time()
    clocks = sampler.stop(t_wall0, t_wall2)

    local_tokens = args.steps * DECODE_TOKENS
    tot = sharding.job_totals(local_tokens, dev_s)          # tokens summed, device time max over ranks
    tot_e2e = sharding.job_totals(local_tokens, e2e_s)
    dev_s, e2e_s, tokens = tot.seconds, tot_e2e.seconds, tot.tokens
    value = tot.tokens_per_second
    e2e = tot_e2e.tokens_per_second
    ms_per_token = dev_s / (args.steps * DECODE_TOKENS) * 1e3

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    bpt = spec.decode_bytes_per_token(args.qtype)
    achieved = bpt / (ms_per_token * 1e-3) / 1e9
    # kernels per decoded token: the decode graph's node count
    per_token_kernels = None
    try:
        a = m.kernel_launches()
        m.forward_prefill(prompt, 0, st)
        b = m.kernel_launches()
        m.generate_greedy(1, 1, st)
        per_token_kernels = m.kernel_launches() - b
        prefill_kernels = b - a
    except Exception:
        prefill_kernels = 0
    line = {
        "metric": "decode tok/s bs=1 (tg128)", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": workload_config(args, spec),
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 * DECODE_TOKENS, "d2h_bytes_per_step": 4 * DECODE_TOKENS},
        # launches of this library's kernels inside the device-timed region on rank 0: the persistent decode
        # kernel runs a whole generate call (all --decode-tokens steps) per launch
        "gpu_launches": int(counters["decode_launches"]),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_TOKEN.get((args.model, args.qtype)), "peak_source": peak_kind,
                     "kernel": "k_decode_mega (persistent: one launch = DECODE_TOKENS decode steps); figures are per decode step",
                     "algorithmic_bytes_per_step": bpt, "launches_per_generate_call": per_token_kernels},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        sample_tokens = 32
        cpu_tps, cores = cpu_baseline(path, spec, sample_tokens)
        line["cpu_baseline"] = {"value": cpu_tps, "unit": "tok/s", "cores": cores, "kind": "port",
                                "sample": f"{PROMPT_TOKENS}-token prefill (untimed) + {sample_tokens} greedy decode tokens of the same model and prompt"}
    if world == 1 and not args.no_extra:
        # side measurements (not the headline): prefill in both GEMM modes, and decode at tg512
        extra = {}
        flop_tok = gemm_flop_per_token(spec)
        tensor_peak, peak_src = int8_peak_tflops()
        for mode in ("exact", "tensor", "exact-cuda-cores"):
            try:
                m.set_prefill_mode(mode)
            except Exception as e:                      # tensor mode needs sizes that are multiples of 128
                extra[f"prefill_{mode}"] = f"unavailable: {e}"
                continue
            for n, ub in ((128, 512), (1024, 512), (4096, 512), (4096, 0)):
                toks = gs.random_prompt(n, spec.vocab, seed=7)
                m.forward_prefill_chunked(toks, 0, st, ub)          # warm
                wall, dev = [], []
                for _ in range(PREFILL_REPEATS):
                    t0 = time.perf_counter()
                    m.forward_prefill_chunked(toks, 0, st, ub)      # Session::append_tokens; ubatch 512 is wick's default
                    wall.append(time.perf_counter() - t0)
                    dev.append(m.last_chunked_device_ms * 1e-3)
                tps = n / statistics.median(wall)                   # p50 of the host wall clock of the whole call (wick bench's clock)
                key = f"prefill_{mode}_p{n}" + ("_one_call" if ub == 0 else "") + "_tok_s"
                extra[key] = tps
                extra[key.replace("_tok_s", "_device_tok_s")] = n / statistics.median(dev)   # p50, CUDA events around each chunk
                if n == 4096 and mode != "exact-cuda-cores":
                    extra[key.replace("_tok_s", "_gemm_frac_of_int8_peak")] = tps * flop_tok / 1e12 / tensor_peak
        m.set_prefill_mode("exact")
        # where a 4096-token exact prefill (ubatch 512) spends its device time, by kernel category
        toks = gs.random_prompt(4096, spec.vocab, seed=7)
        m.profile_enable(True)
        m.forward_prefill_chunked(toks, 0, st, 512)
        cats = m.profile_read()
        m.profile_enable(False)
        tot_ms = sum(cats.values()) or 1.0
        extra["prefill_exact_p4096_device_ms_by_category"] = {k: round(v, 3) for k, v in cats.items()}
        extra["prefill_exact_p4096_attention_share"] = cats.get("attention", 0.0) / tot_ms
        extra["int8_peak_tflops_used"] = tensor_peak
        extra["int8_peak_source"] = peak_src
        extra["gemm_gflop_per_token"] = flop_tok / 1e9
        logits = m.forward_prefill(prompt, 0, st)
        m.generate_greedy(int(np.argmax(logits)), 512, st)
        extra["decode_tg512_tok_s"] = 512 / (m.last_elapsed_ms() * 1e-3)
        extra["prefill_repeats"] = PREFILL_REPEATS
        try:
            extra["serving"] = serving_side_line(m, spec, args, gs, peak)
        except Exception as e:                              # e.g. not enough device memory for the sequence slots
            extra["serving"] = f"unavailable: {e}"
        extra["prefill_paths"] = {"exact": "default: bit-exact GEMM on tcgen05 (lane partials in tensor memory, eight unfused chains) + exact-order attention",
                                  "tensor": "tcgen05 int8 GEMM (exact block sums, one fused f32 chain) + exact-order attention",
                                  "exact-cuda-cores": "bit-exact CUDA-core integer GEMM + exact-order attention"}
        line["extra"] = extra
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
