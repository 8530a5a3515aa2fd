"""Tensor-parallel variant of the LFM2 forward pass over the GPUs of one node (one process per GPU).

wick itself runs one sequence on one device; this module is the optional 2 / 4 / 8-way split of the 1.6B-class model
that the serving configuration names.  The split follows the structure of `run_layers` (wick/src/model/lfm2.rs:1020-1124):

  column split (rows of the weight): attention Q / K / V by head, FFN gate / up by row, short-conv in_proj by channel
      (the depthwise conv and both gates are per channel, so a channel shard needs no exchange, lfm2.rs:688-725);
  row split (along K, at multiples of 32 so that Q8_0 activation blocks stay whole): attention output, short-conv
      out_proj, FFN down; each leaves a partial sum of the hidden row on every rank -> one all-reduce, two per layer;
  vocabulary head: rows split, the logits shards are gathered (greedy: a max over per-rank (value, index) pairs).

Decode (one row, 8 KB messages) uses the library's one-shot all-reduce over peer memory fused with the residual add,
RMSNorm and Q8_0 quantiser that follow it (wick_cuda_tp_allreduce_add_rmsnorm_quant); prefill chunks use NCCL
(`torch.distributed.all_reduce`).  torch is the allocator and the process-group plumbing; all arithmetic runs in the
library's kernels through the operator entry points of the C ABI.

Parity: the all-reduce adds the K-shards' partial sums in rank order, which is not the single-device accumulation
order, so results agree with wick's CPU path within a tolerance (logits ~1e-2 relative after 16 layers of Q8_0
re-quantisation), not bit for bit; every rank computes identical bits, so the replicas never diverge.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import List, Optional, Sequence, Tuple

import numpy as np

DT_Q4_0, DT_Q8_0 = 2, 8
BLOCK_BYTES = {DT_Q4_0: 18, DT_Q8_0: 34}


# ── partition arithmetic (no GPU needed) ────────────────────────────────────

@dataclasses.dataclass(frozen=True)
class TpPlan:
    """Which slice of every matrix rank `rank` of `world` owns."""
    hidden: int
    ffn: int
    n_heads: int
    n_kv_heads: int      # of the attention layers (equal across layers in LFM2 files)
    head_dim: int
    vocab: int
    world: int
    rank: int

    def __post_init__(self):
        T = self.world
        if not (1 <= T <= 8 and 0 <= self.rank < T):
            raise ValueError("world must be 1..8 and rank < world")
        bad = []
        if self.n_heads % T or (self.n_kv_heads and self.n_kv_heads % T):
            bad.append(f"heads {self.n_heads}/{self.n_kv_heads}")
        if self.hidden % (32 * T):
            bad.append(f"hidden {self.hidden}")
        if self.ffn % (32 * T):
            bad.append(f"ffn {self.ffn}")
        if self.vocab % T:
            bad.append(f"vocab {self.vocab}")
        if (self.n_heads // T) * self.head_dim % 32:
            bad.append("heads per rank x head_dim")
        if bad:
            raise ValueError(f"cannot split {', '.join(bad)} {T} ways (row-split shards must be whole 32-element blocks)")

    # column splits: row ranges [lo, hi) of the weight
    def _share(self, n: int) -> Tuple[int, int]:
        per = n // self.world
        return self.rank * per, (self.rank + 1) * per

    def channels(self) -> Tuple[int, int]:
        return self._share(self.hidden)

    def q_heads(self) -> Tuple[int, int]:
        return self._share(self.n_heads)

    def kv_heads(self) -> Tuple[int, int]:
        return self._share(self.n_kv_heads)

    def q_rows(self) -> Tuple[int, int]:
        a, b = self.q_heads()
        return a * self.head_dim, b * self.head_dim

    def kv_rows(self) -> Tuple[int, int]:
        a, b = self.kv_heads()
        return a * self.head_dim, b * self.head_dim

    def ffn_rows(self) -> Tuple[int, int]:
        return self._share(self.ffn)

    def vocab_rows(self) -> Tuple[int, int]:
        return self._share(self.vocab)

    def in_proj_row_ranges(self) -> List[Tuple[int, int]]:
        """The (b, c, x) thirds of the short-conv in_proj, this rank's channels of each."""
        c0, c1 = self.channels()
        return [(t * self.hidden + c0, t * self.hidden + c1) for t in range(3)]

    # row splits: K ranges [lo, hi) (multiples of 32)
    def o_cols(self) -> Tuple[int, int]:
        return self.q_rows()            # the attention output concatenates the heads

    def out_proj_cols(self) -> Tuple[int, int]:
        return self.channels()

    def down_cols(self) -> Tuple[int, int]:
        return self.ffn_rows()


def slice_rows(raw: np.ndarray, ranges: Sequence[Tuple[int, int]]) -> np.ndarray:
    """raw [m, row_bytes] block rows -> the rows of `ranges`, concatenated."""
    return np.ascontiguousarray(np.concatenate([raw[a:b] for a, b in ranges], axis=0))


def slice_k(raw: np.ndarray, dtype: int, k0: int, k1: int) -> np.ndarray:
    """raw [m, (k/32) * block_bytes] block rows -> blocks k0/32 .. k1/32 of every row."""
    assert k0 % 32 == 0 and k1 % 32 == 0
    bb = BLOCK_BYTES[dtype]
    return np.ascontiguousarray(raw[:, (k0 // 32) * bb:(k1 // 32) * bb])


def dequantize_rows(raw: np.ndarray, dtype: int) -> np.ndarray:
    """Block rows -> f32 [m, k] (quant.rs:78-105, :154-177): value = f32(int) * f32(f16 scale)."""
    m = raw.shape[0]
    bb = BLOCK_BYTES[dtype]
    blocks = raw.reshape(m, -1, bb)
    d = blocks[:, :, :2].copy().view(np.float16).astype(np.float32)            # [m, nb, 1]
    if dtype == DT_Q4_0:
        qs = blocks[:, :, 2:]
        lo = (qs & 0x0F).astype(np.int32) - 8
        hi = (qs >> 4).astype(np.int32) - 8
        v = np.concatenate([lo, hi], axis=2)
    else:
        v = blocks[:, :, 2:].copy().view(np.int8).astype(np.int32)
    return (v.astype(np.float32) * d).reshape(m, -1)


def rope_tables(n_pos: int, head_dim: int, base: float) -> Tuple[np.ndarray, np.ndarray]:
    """cos / sin of every (position, pair) in wick's iteration order (cpu.rs:2145-2158): theta starts at the position
    as f32 and is multiplied by base^(-2/hd) pair by pair, all in f32."""
    half = head_dim // 2
    scale = np.float32(np.power(np.float32(base), np.float32(-2.0) / np.float32(head_dim)))
    theta = np.arange(n_pos, dtype=np.float32)
    cos = np.empty((n_pos, half), np.float32)
    sin = np.empty((n_pos, half), np.float32)
    for i in range(half):
        cos[:, i] = np.cos(theta)
        sin[:, i] = np.sin(theta)
        theta = (theta * scale).astype(np.float32)
    return cos, sin


def merge_argmax(values: np.ndarray, indices: np.ndarray) -> int:
    """cpu_argmax over per-rank winners (sampler.rs:8-19): largest value, the last index among equals; NaN never wins."""
    v = np.where(np.isnan(values), -np.inf, values).astype(np.float32)
    best = np.flatnonzero(v == v.max())
    return int(indices[best].max())


# ── the model ───────────────────────────────────────────────────────────────

class TpLfm2Model:
    """One rank of a tensor-parallel LFM2 model.  Every rank must make the same calls in the same order."""

    def __init__(self, path: str, context_size: int, rank: int, world: int, device: int, group=None, fused_allreduce: bool = True):
        import torch
        import torch.distributed as dist
        from gguf import GGUFReader
        from . import _lib, ops
        self.torch, self.dist, self.ops = torch, dist, ops
        self._lib = _lib.load()
        self.rank, self.world, self.group = rank, world, group
        self.dev = torch.device("cuda", device)
        torch.cuda.set_device(self.dev)
        rd = GGUFReader(path)
        f = rd.fields

        def u32(key, default=None):
            return int(f[key].contents()) if key in f else default

        def f32(key, default):
            return float(f[key].contents()) if key in f else default

        self.n_layers = u32("lfm2.block_count")
        self.hs = u32("lfm2.embedding_length")
        self.ffn = u32("lfm2.feed_forward_length")
        self.n_heads = u32("lfm2.attention.head_count")
        self.vocab = u32("lfm2.vocab_size")
        self.max_seq = min(context_size, u32("lfm2.context_length", 128000))
        self.theta = f32("lfm2.rope.freq_base", 1e6)
        self.eps = f32("lfm2.attention.layer_norm_rms_epsilon", 1e-5)
        self.ks = u32("lfm2.shortconv.l_cache", 3)
        kvh = [int(x) for x in f["lfm2.attention.head_count_kv"].contents()]
        self.hd = self.hs // self.n_heads
        tensors = {t.name: t for t in rd.tensors}
        self.is_attn = [f"blk.{i}.attn_q.weight" in tensors for i in range(self.n_layers)]
        n_kv = max([k for k, a in zip(kvh, self.is_attn) if a] or [0])
        self.plan = TpPlan(self.hs, self.ffn, self.n_heads, n_kv, self.hd, self.vocab, world, rank)
        P = self.plan

        def raw(name):
            t = tensors[name]
            dt = int(t.tensor_type)
            if dt not in BLOCK_BYTES:
                raise ValueError(f"{name}: ggml type {dt} is not supported by the tensor-parallel path (Q4_0 / Q8_0 only)")
            return np.asarray(t.data), dt

        def weight(arr, dt, k):
            return ops.QuantWeight(dt, arr.reshape(-1), arr.shape[0], k)

        def vec(name, sl=None):
            a = np.asarray(tensors[name].data, dtype=np.float32)
            if sl is not None:
                a = a[sl[0]:sl[1]]
            return torch.from_numpy(np.ascontiguousarray(a)).to(self.dev)

        self.embd_raw, self.embd_dt = raw("token_embd.weight")          # host: rows are dequantised one by one
        v0, v1 = P.vocab_rows()
        self.w_vocab = weight(slice_rows(self.embd_raw, [(v0, v1)]), self.embd_dt, self.hs)
        self.output_norm = vec("token_embd_norm.weight")
        self.layers = []
        dc = self.ks - 1
        c0, c1 = P.channels()
        for i in range(self.n_layers):
            p = f"blk.{i}."
            L = {"attn_norm": vec(p + "attn_norm.weight"), "ffn_norm": vec(p + "ffn_norm.weight")}
            g, dt = raw(p + "ffn_gate.weight")
            L["gate"] = weight(slice_rows(g, [P.ffn_rows()]), dt, self.hs)
            u, dt = raw(p + "ffn_up.weight")
            L["up"] = weight(slice_rows(u, [P.ffn_rows()]), dt, self.hs)
            d, dt = raw(p + "ffn_down.weight")
            k0, k1 = P.down_cols()
            L["down"] = weight(slice_k(d, dt, k0, k1), dt, k1 - k0)
            if self.is_attn[i]:
                q, dt = raw(p + "attn_q.weight")
                L["q"] = weight(slice_rows(q, [P.q_rows()]), dt, self.hs)
                k, dt = raw(p + "attn_k.weight")
                L["k"] = weight(slice_rows(k, [P.kv_rows()]), dt, self.hs)
                v, dt = raw(p + "attn_v.weight")
                L["v"] = weight(slice_rows(v, [P.kv_rows()]), dt, self.hs)
                o, dt = raw(p + "attn_output.weight")
                k0, k1 = P.o_cols()
                L["o"] = weight(slice_k(o, dt, k0, k1), dt, k1 - k0)
                L["q_norm"], L["k_norm"] = vec(p + "attn_q_norm.weight"), vec(p + "attn_k_norm.weight")
                kvd = (P.kv_heads()[1] - P.kv_heads()[0]) * self.hd
                L["k_cache"] = torch.zeros((self.max_seq, kvd), dtype=torch.float32, device=self.dev)
                L["v_cache"] = torch.zeros((self.max_seq, kvd), dtype=torch.float32, device=self.dev)
            else:
                ip, dt = raw(p + "shortconv.in_proj.weight")
                L["in_proj"] = weight(slice_rows(ip, P.in_proj_row_ranges()), dt, self.hs)
                op, dt = raw(p + "shortconv.out_proj.weight")
                k0, k1 = P.out_proj_cols()
                L["out_proj"] = weight(slice_k(op, dt, k0, k1), dt, k1 - k0)
                L["conv_w"] = vec(p + "shortconv.conv.weight", (c0, c1)).reshape(-1).contiguous()
                L["conv_state"] = torch.zeros((max(dc, 1), c1 - c0), dtype=torch.float32, device=self.dev)
            self.layers.append(L)
        cos, sin = rope_tables(self.max_seq, self.hd, self.theta)
        self.rope_cos = torch.from_numpy(cos).to(self.dev)
        self.rope_sin = torch.from_numpy(sin).to(self.dev)
        self.nh_local = P.q_heads()[1] - P.q_heads()[0]
        self.nkv_local = P.kv_heads()[1] - P.kv_heads()[0] if n_kv else 0
        self.seq_len = 0
        self.hidden = torch.zeros(self.hs, dtype=torch.float32, device=self.dev)
        self.q8s = torch.zeros(max(self.hs, self.ffn) // 32, dtype=torch.float32, device=self.dev)
        self.q8q = torch.zeros(max(self.hs, self.ffn), dtype=torch.int8, device=self.dev)
        # fused one-shot all-reduce over peer memory (decode)
        self.comm = None
        self.fused = bool(fused_allreduce) and world > 1
        if self.fused:
            from ._lib import check
            self.comm = C.c_void_p()
            check(self._lib.wick_cuda_tp_comm_create(world, rank, self.hs, C.byref(self.comm)), self._tp_err)
            handle = (C.c_uint8 * 64)()
            check(self._lib.wick_cuda_tp_comm_export(self.comm, handle), self._tp_err)
            gathered: List[Optional[bytes]] = [None] * world
            dist.all_gather_object(gathered, bytes(handle), group=group)
            blob = (C.c_uint8 * (64 * world)).from_buffer_copy(b"".join(gathered))
            check(self._lib.wick_cuda_tp_comm_connect(self.comm, blob), self._tp_err)
            dist.barrier(group=group)

    def _tp_err(self) -> str:
        return self._lib.wick_cuda_tp_last_error().decode()

    def close(self):
        if getattr(self, "comm", None) is not None and self.comm.value:
            self.dist.barrier(group=self.group)   # nobody may still be reading this rank's buffer
            self._lib.wick_cuda_tp_comm_destroy(self.comm)
            self.comm = None

    # ---- helpers ----------------------------------------------------------------
    def _stream(self) -> int:
        return self.torch.cuda.current_stream().cuda_stream

    def _embed(self, tokens: Sequence[int]):
        rows = dequantize_rows(np.stack([self.embd_raw[int(t)] for t in tokens]), self.embd_dt)
        return self.torch.from_numpy(rows).to(self.dev)

    def _norm_quant(self, x, w):
        xn = self.ops.rmsnorm_(x.clone(), w, self.eps)
        return self.ops.quantize_f32_to_q8_0(xn)

    def _allreduce(self, t):
        if self.world > 1:
            self.dist.all_reduce(t, group=self.group)
        return t

    def reset(self):
        self.seq_len = 0
        for L in self.layers:
            if "conv_state" in L:
                L["conv_state"].zero_()

    # ---- prefill: batched kernels, NCCL all-reduce -------------------------------
    def forward_prefill(self, tokens: Sequence[int], start_pos: int) -> np.ndarray:
        """Model::forward_prefill for the whole group: logits [vocab] of the last position (same on every rank)."""
        torch, ops = self.torch, self.ops
        n = len(tokens)
        assert n > 0 and (start_pos == 0 or start_pos == self.seq_len) and start_pos + n <= self.max_seq
        if start_pos == 0:
            self.reset()
        hidden = self._embed(tokens)                       # [n, hs], replicated
        flash = n >= 256                                   # FLASH_ATTN_THRESHOLD, lfm2.rs:1646-1647
        for L, attn in zip(self.layers, self.is_attn):
            xs, xq = self._norm_quant(hidden, L["attn_norm"])
            if attn:
                q, k, v = ops.gemm_q8(L["q"], xs, xq), ops.gemm_q8(L["k"], xs, xq), ops.gemm_q8(L["v"], xs, xq)
                ops.qknorm_rope_kv_(q, k, v, L["q_norm"], L["k_norm"], self.eps, self.rope_cos, self.rope_sin, L["k_cache"], L["v_cache"],
                                    start_pos, self.nh_local, self.nkv_local, self.hd)
                a = ops.attention_prefill(q, L["k_cache"], L["v_cache"], n, start_pos, self.nh_local, self.nkv_local, self.hd, flash)
                s2, q2 = ops.quantize_f32_to_q8_0(a)
                part = ops.gemm_q8(L["o"], s2, q2)
            else:
                proj = ops.gemm_q8(L["in_proj"], xs, xq)
                y = ops.shortconv(proj, L["conv_w"], L["conv_state"], self.ks)
                s2, q2 = ops.quantize_f32_to_q8_0(y)
                part = ops.gemm_q8(L["out_proj"], s2, q2)
            hidden = hidden + self._allreduce(part)
            xs, xq = self._norm_quant(hidden, L["ffn_norm"])
            g, u = ops.gemm_q8(L["gate"], xs, xq), ops.gemm_q8(L["up"], xs, xq)
            ops.silu_mul_(g, u)
            s2, q2 = ops.quantize_f32_to_q8_0(g)
            hidden = hidden + self._allreduce(ops.gemm_q8(L["down"], s2, q2))
        self.seq_len = start_pos + n
        xs, xq = self._norm_quant(hidden[n - 1].contiguous(), self.output_norm)
        return self._gather_logits(ops.gemv_q8(self.w_vocab, xs.reshape(-1), xq.reshape(-1)))

    def _gather_logits(self, shard) -> np.ndarray:
        if self.world == 1:
            return shard.cpu().numpy()
        parts = [self.torch.empty_like(shard) for _ in range(self.world)]
        self.dist.all_gather(parts, shard, group=self.group)
        return self.torch.cat(parts).cpu().numpy()

    # ---- decode: one row, fused peer-memory all-reduce ---------------------------
    def _partial_ptr(self) -> int:
        p = C.c_void_p()
        self._lib.wick_cuda_tp_partial_buffer(self.comm, C.byref(p))
        return p.value

    def _rowsplit_reduce_norm_quant(self, w, s2, q2, norm_w):
        """hidden += all-reduce(w . x); returns the Q8_0 quantisation of RMSNorm(hidden) with norm_w."""
        from ._lib import check
        ops, lib = self.ops, self._lib
        if self.fused:
            check(lib.wick_cuda_gemv_q8(w._h, s2.data_ptr(), q2.data_ptr(), self._partial_ptr(), self._stream()))
            check(lib.wick_cuda_tp_allreduce_add_rmsnorm_quant(self.comm, self.hidden.data_ptr(), norm_w.data_ptr(), self.eps, self.hs,
                                                               self.q8s.data_ptr(), self.q8q.data_ptr(), None, self._stream()), self._tp_err)
            return self.q8s[: self.hs // 32], self.q8q[: self.hs]
        part = ops.gemv_q8(w, s2, q2)
        self.hidden += self._allreduce(part)
        xs, xq = self._norm_quant(self.hidden, norm_w)
        return xs.reshape(-1), xq.reshape(-1)

    def _decode_layers(self, token: int):
        torch, ops = self.torch, self.ops
        pos = self.seq_len
        assert pos < self.max_seq
        self.hidden.copy_(self._embed([token])[0])
        xs, xq = self._norm_quant(self.hidden, self.layers[0]["attn_norm"])
        xs, xq = xs.reshape(-1), xq.reshape(-1)
        for i, (L, attn) in enumerate(zip(self.layers, self.is_attn)):
            if attn:
                q, k, v = ops.gemv_q8(L["q"], xs, xq), ops.gemv_q8(L["k"], xs, xq), ops.gemv_q8(L["v"], xs, xq)
                q, k, v = q.reshape(1, -1), k.reshape(1, -1), v.reshape(1, -1)
                ops.qknorm_rope_kv_(q, k, v, L["q_norm"], L["k_norm"], self.eps, self.rope_cos, self.rope_sin, L["k_cache"], L["v_cache"],
                                    pos, self.nh_local, self.nkv_local, self.hd)
                a = ops.attention_prefill(q, L["k_cache"], L["v_cache"], 1, pos, self.nh_local, self.nkv_local, self.hd, False)
                s2, q2 = ops.quantize_f32_to_q8_0(a.reshape(-1))
                w = L["o"]
            else:
                proj = ops.gemv_q8(L["in_proj"], xs, xq).reshape(1, -1)
                y = ops.shortconv(proj, L["conv_w"], L["conv_state"], self.ks)
                s2, q2 = ops.quantize_f32_to_q8_0(y.reshape(-1))
                w = L["out_proj"]
            xs, xq = self._rowsplit_reduce_norm_quant(w, s2.reshape(-1), q2.reshape(-1), L["ffn_norm"])
            g, u = ops.gemv_q8(L["gate"], xs, xq), ops.gemv_q8(L["up"], xs, xq)
            ops.silu_mul_(g, u)
            s2, q2 = ops.quantize_f32_to_q8_0(g)
            nxt = self.layers[i + 1]["attn_norm"] if i + 1 < self.n_layers else self.output_norm
            xs, xq = self._rowsplit_reduce_norm_quant(L["down"], s2.reshape(-1), q2.reshape(-1), nxt)
        self.seq_len = pos + 1
        return ops.gemv_q8(self.w_vocab, xs, xq)           # this rank's logits shard

    def forward(self, token: int) -> np.ndarray:
        """Model::forward for the group: logits [vocab] (same on every rank)."""
        return self._gather_logits(self._decode_layers(token))

    def forward_greedy(self, token: int) -> int:
        """Model::forward_greedy: every rank finds the winner of its vocabulary shard, the winners are merged."""
        shard = self._decode_layers(token)
        idx = self.ops.argmax(shard)
        v0 = self.plan.vocab_rows()[0]
        pair = self.torch.stack([shard[idx.long()].reshape(()), (idx.reshape(()) + v0).to(self.torch.float32)])
        if self.world == 1:
            return int(pair[1].item())
        parts = [self.torch.empty_like(pair) for _ in range(self.world)]
        self.dist.all_gather(parts, pair, group=self.group)
        host = self.torch.stack(parts).cpu().numpy()
        return merge_argmax(host[:, 0], host[:, 1].astype(np.int64))

    def check_status(self):
        """Synchronise and raise if a peer never arrived at an all-reduce (bounded device-side wait)."""
        if self.comm is not None:
            from ._lib import check
            mask = C.c_uint32(0)
            check(self._lib.wick_cuda_tp_status(self.comm, self._stream(), C.byref(mask)), self._tp_err)


# ── measurement entry point (run under torchrun, one process per GPU) ───────

def _bench_main():
    """`python -m torch.distributed.run --nproc-per-node T -m wick_b200.tensor_parallel [--model ...]`: decode tok/s of
    the T-way split with the fused peer-memory all-reduce and with NCCL, and the time of one all-reduce of each kind."""
    import argparse
    import json
    import os
    import time

    import torch
    import torch.distributed as dist

    from . import gguf_synth as gs
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="lfm2.5-1.6b")
    ap.add_argument("--qtype", default="q4_0")
    ap.add_argument("--prompt-tokens", type=int, default=128)
    ap.add_argument("--decode-tokens", type=int, default=64)
    ap.add_argument("--context", type=int, default=1024)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl" if world > 1 else "gloo", device_id=torch.device("cuda", local) if world > 1 else None)
    if rank == 0:
        path = gs.cached_model(args.model, args.qtype, 0)
    dist.barrier()
    path = gs.cached_model(args.model, args.qtype, 0)
    spec = gs.SPECS[args.model]
    prompt = gs.random_prompt(args.prompt_tokens, spec.vocab, seed=1)
    out = {"metric": "decode tok/s bs=1, tensor parallel", "n_gpus": world, "unit": "tok/s",
           "config": {"workload": f"{spec.name} {args.qtype.upper()} bs=1 split {world} ways: {args.prompt_tokens}-token prompt (untimed), "
                                  f"then {args.decode_tokens} greedy tokens, one forward_greedy call per token"}}
    for name, fused in (("fused_peer_allreduce", True), ("nccl_allreduce", False)):
        m = TpLfm2Model(path, args.context, rank, world, local, fused_allreduce=fused)
        tok = int(np.argmax(m.forward_prefill(prompt, 0)))
        for _ in range(4):
            tok = m.forward_greedy(tok)
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.decode_tokens):
            tok = m.forward_greedy(tok)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device="cuda")
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        out[name + "_tok_s"] = args.decode_tokens / float(dt.item())
        # one all-reduce of a hidden row, alone: the fused kernel (with residual add, norm and quantiser) or NCCL
        reps = 200
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            buf = torch.zeros(m.hs, dtype=torch.float32, device="cuda")
            dist.barrier()
            ev0.record()
            for _ in range(reps):
                if fused:
                    m._lib.wick_cuda_tp_allreduce_add_rmsnorm_quant(m.comm, m.hidden.data_ptr(), m.output_norm.data_ptr(), m.eps, m.hs,
                                                                    m.q8s.data_ptr(), m.q8q.data_ptr(), None, m._stream())
                else:
                    dist.all_reduce(buf)
            ev1.record()
            torch.cuda.synchronize()
            m.check_status()
            out[name + "_us_per_allreduce"] = ev0.elapsed_time(ev1) * 1e3 / reps
            out[name + "_allreduce_us_per_token"] = out[name + "_us_per_allreduce"] * 2 * m.n_layers
        m.close()
        del m
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    _bench_main()
