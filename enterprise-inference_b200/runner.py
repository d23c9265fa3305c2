"""Device state of one TP rank and one scheduler step through the C-ABI.

Mirrors the worker/model-runner of the image the chart deploys (one worker process per TP rank,
/root/reference/core/helm-charts/vllm/xeon-values.yaml:78-79; [V22] vllm/v1/worker/*model_runner*):
it owns the weights, the paged KV cache and the step inputs, and runs `execute_model` — here
`b200_decode_step_host` — once per scheduler iteration.  torch allocates; CUDA computes.
"""
from __future__ import annotations

import os

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _abi
from .config import ModelConfig, rope_cos_sin


@dataclass
class StepBatch:
    """Step inputs.  One entry per token row; block_tables one row per sequence."""
    ids: List[int] = field(default_factory=list)
    positions: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)
    ctx_lens: List[int] = field(default_factory=list)
    row_to_seq: List[int] = field(default_factory=list)
    logit_rows: List[int] = field(default_factory=list)
    block_tables: List[Sequence[int]] = field(default_factory=list)
    # models with per-sequence state (recurrent layers, convolution tails): the state slot of every sequence of the step
    seq_slots: List[int] = field(default_factory=list)

    @property
    def n_tokens(self):
        return len(self.ids)

    @property
    def max_ctx(self):
        c = self.ctx_lens
        return int(c.max()) if isinstance(c, np.ndarray) else max(c)


class ModelRunner:
    def __init__(self, cfg: ModelConfig, device: Optional[torch.device] = None, *, max_tokens: int = 2048,
                 max_model_len: int = 8192, block_size: int = 128, n_blocks: Optional[int] = None,
                 kv_cache_gib: Optional[float] = None, tp_rank: int = 0, tp_world: int = 1,
                 graphs: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("ModelRunner needs a CUDA device (B200, sm_100a); there is no CPU path")
        self.lib = _abi.lib()
        self.cfg = cfg
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        if not self.lib.b200_device_ok():
            raise RuntimeError("the current CUDA device is not compute capability 10.x (B200)")
        self.block_size = block_size
        self.max_tokens = max_tokens
        self.max_model_len = max_model_len
        self.max_blocks_per_seq = (max_model_len + block_size - 1) // block_size
        self.tp_rank, self.tp_world = tp_rank, tp_world
        self.hq = cfg.n_q_heads // tp_world
        self.hkv = cfg.n_kv_heads // tp_world
        self.inter = cfg.intermediate // tp_world
        self.vocab_local = cfg.vocab // tp_world
        self.stream = torch.cuda.Stream(device=self.device)

        mc = _abi.ModelCfg(hidden=cfg.hidden, n_layers=cfg.n_layers, n_q_heads=cfg.n_q_heads,
                           n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, intermediate=cfg.intermediate,
                           vocab=cfg.vocab, qkv_bias=int(cfg.qkv_bias), rms_eps=cfg.rms_eps,
                           block_size=block_size, max_tokens=max_tokens,
                           max_blocks_per_seq=self.max_blocks_per_seq, tp_rank=tp_rank, tp_world=tp_world)
        h = C.c_void_p()
        _abi.check(self.lib.b200_ctx_create(C.byref(mc), C.byref(h)))
        self.ctx = h
        _abi.check(self.lib.b200_ctx_set_graphs(self.ctx, int(graphs)))

        # KV cache [L][n_blocks][hkv][block][128] bf16, zero-filled (a masked tail never reads NaNs)
        per_block = cfg.n_layers * self.hkv * block_size * cfg.head_dim * 2 * 2
        if n_blocks is None:
            if kv_cache_gib is None:
                free, _ = torch.cuda.mem_get_info(self.device)
                kv_cache_gib = max(free / 2 ** 30 * 0.5, 0.25)
            n_blocks = max(int(kv_cache_gib * 2 ** 30) // per_block, 2)
        self.n_blocks = n_blocks
        shape = (cfg.n_layers, n_blocks, self.hkv, block_size, cfg.head_dim)
        self.k_cache = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        self.v_cache = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        _abi.check(self.lib.b200_set_kv_cache(self.ctx, self.k_cache.data_ptr(), self.v_cache.data_ptr(), n_blocks))
        self.cos_sin = rope_cos_sin(cfg, max(max_model_len, 16)).to(self.device)
        _abi.check(self.lib.b200_set_rope_cache(self.ctx, self.cos_sin.data_ptr(), self.cos_sin.shape[0]))

        self._alloc_host_buffers()

    def _alloc_host_buffers(self, max_logit_rows: int = 512):
        max_tokens = self.max_tokens
        self._weights: List[torch.Tensor] = []   # keeps the borrowed device tensors alive
        meta_ints = 7 * max_tokens + max_tokens * self.max_blocks_per_seq
        # two pinned (metadata, tokens) pairs: step_async alternates them, so the host can pack step n+1 while the
        # copies of step n are still in flight; the synchronous calls use pair 0
        self._h_meta2 = [torch.empty(meta_ints, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._h_out2 = [torch.empty(max(max_tokens, 1), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._done2 = [torch.cuda.Event() for _ in range(2)]
        self._flip = 0
        self._h_meta, self._h_out = self._h_meta2[0], self._h_out2[0]
        self._h_meta_np = self._h_meta.numpy()
        self._h_out_np = self._h_out.numpy()
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.max_logit_rows = min(max_tokens, max_logit_rows)
        self._h_sample = torch.zeros(self.max_logit_rows * 32, dtype=torch.uint8).pin_memory()
        self._h_sample_np = self._h_sample.numpy()
        self._h_lp_tok = torch.zeros(self.max_logit_rows, dtype=torch.int32).pin_memory()
        self._h_lp_out = torch.zeros(self.max_logit_rows * (1 + 2 * 32), dtype=torch.float32).pin_memory()

    # ---- weights ---------------------------------------------------------------------------
    def _set(self, layer: int, kind: int, t: torch.Tensor):
        t = t.to(device=self.device, dtype=torch.bfloat16).contiguous()
        self._weights.append(t)
        rows, cols = (t.shape[0], t.shape[1]) if t.dim() == 2 else (t.shape[0], 1)
        _abi.check(self.lib.b200_set_weight(self.ctx, layer, kind, t.data_ptr(), rows, cols))

    def load_weights(self, w: Dict[str, torch.Tensor]):
        """HF-named tensors, fused and sharded for this TP rank by weights.shard_weights."""
        from .weights import shard_weights
        for layer, kind, t in shard_weights(w, self.cfg, self.tp_rank, self.tp_world):
            self._set(layer, kind, t)

    def init_random_weights(self, seed: int = 1234, std: float = 0.02):
        """Random-init N(0, std^2) weights generated on the device (benchmarks; no checkpoint
        is reachable without network).  Norm weights are 1."""
        c = self.cfg
        g = torch.Generator(device=self.device)
        g.manual_seed(seed + 7919 * self.tp_rank)

        def rnd(*shape):
            t = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            t.normal_(0.0, std, generator=g)
            return t

        ones = torch.ones(c.hidden, dtype=torch.bfloat16, device=self.device)
        ge = torch.Generator(device=self.device)
        ge.manual_seed(seed)  # the embedding is replicated: same bytes on every rank
        emb = torch.empty((c.vocab, c.hidden), dtype=torch.bfloat16, device=self.device)
        emb.normal_(0.0, std, generator=ge)
        self._set(0, _abi.W_EMBED, emb)
        qkv_rows = (self.hq + 2 * self.hkv) * c.head_dim
        for l in range(c.n_layers):
            self._set(l, _abi.W_LN1, ones)
            self._set(l, _abi.W_QKV, rnd(qkv_rows, c.hidden))
            if c.qkv_bias:
                self._set(l, _abi.W_QKV_BIAS, rnd(qkv_rows))
            self._set(l, _abi.W_O, rnd(c.hidden, self.hq * c.head_dim))
            self._set(l, _abi.W_LN2, ones)
            self._set(l, _abi.W_GATE_UP_INTERLEAVED if self.inter % 64 == 0 else _abi.W_GATE_UP,
                      rnd(2 * self.inter, c.hidden))
            self._set(l, _abi.W_DOWN, rnd(c.hidden, self.inter))
        self._set(0, _abi.W_FINAL_NORM, ones)
        self._set(0, _abi.W_LM_HEAD, rnd(self.vocab_local, c.hidden))

    # ---- TP --------------------------------------------------------------------------------
    def init_tp(self, group=None, peer_allreduce: bool = None):
        """Create the ctx's NCCL communicator; the 128-byte id travels over torch.distributed."""
        if self.tp_world == 1:
            return
        import os
        import torch.distributed as dist
        if peer_allreduce is None:
            peer_allreduce = os.environ.get("B200_PEER_ALLREDUCE", "1") != "0"
        buf = (C.c_char * 128)()
        if self.tp_rank == 0:
            _abi.check(self.lib.b200_nccl_unique_id(buf))
        obj = [bytes(buf)]
        dist.broadcast_object_list(obj, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        idb = (C.c_char * 128).from_buffer_copy(obj[0])
        _abi.check(self.lib.b200_nccl_init(self.ctx, idb))
        if peer_allreduce:
            # exchange the CUDA-IPC handles of the all-reduce buffers: from here on the per-layer
            # all-reduces are one peer-memory kernel per rank instead of NCCL
            h = (C.c_char * 64)()
            _abi.check(self.lib.b200_tp_ipc_export(self.ctx, h))
            handles = [None] * self.tp_world
            dist.all_gather_object(handles, bytes(h), group=group)
            allh = (C.c_char * (64 * self.tp_world)).from_buffer_copy(b"".join(handles))
            _abi.check(self.lib.b200_tp_ipc_import(self.ctx, allh, self.tp_world))
            dist.barrier(group=group)

    # ---- one step ---------------------------------------------------------------------------
    def pack(self, b: StepBatch, into: Optional[np.ndarray] = None):
        """Write the dense packed int32 buffer b200_decode_step_host expects into pinned memory."""
        T, R, S = b.n_tokens, len(b.logit_rows), len(b.block_tables)
        tables = b.block_tables
        bt_stride = tables.shape[1] if isinstance(tables, np.ndarray) else max(max(len(r) for r in tables), 1)
        a = self._h_meta_np if into is None else into
        a[0:T] = b.ids
        a[T:2 * T] = b.positions
        a[2 * T:3 * T] = b.slots
        a[3 * T:4 * T] = b.ctx_lens
        a[4 * T:5 * T] = b.row_to_seq
        a[5 * T:5 * T + R] = b.logit_rows
        o = 5 * T + R
        bt = a[o:o + S * bt_stride].reshape(S, bt_stride)
        if isinstance(tables, np.ndarray):
            bt[:] = tables
        else:
            bt.fill(0)
            for i, row in enumerate(tables):
                bt[i, :len(row)] = row
        n = o + S * bt_stride
        if getattr(self, "n_state_slots", 0) > 0:
            if len(b.seq_slots) != S:
                raise ValueError(f"step of {S} sequences names {len(b.seq_slots)} state slots")
            a[n:n + S] = b.seq_slots
            n += S
        return T, R, S, bt_stride, n

    def step(self, b: StepBatch, sync: bool = True) -> np.ndarray:
        """Host-buffer step (the serving path and bench.py's e2e): pinned H2D, step, D2H."""
        T, R, S, bt_stride, n_ints = self.pack(b)
        return self.step_packed(T, R, S, bt_stride, b.max_ctx, n_ints, sync)

    def step_packed(self, T: int, R: int, S: int, bt_stride: int, max_ctx: int, n_ints: int, sync: bool = True) -> np.ndarray:
        """The step over whatever is in the pinned packed buffer (filled by pack(), or by a broadcast
        from rank 0 on a tensor-parallel worker)."""
        _abi.check(self.lib.b200_decode_step_host(self.ctx, self._h_meta.data_ptr(), T, S, bt_stride, max_ctx, R,
                                                  self._h_out.data_ptr(), self.stream.cuda_stream))
        self.h2d_bytes_last, self.d2h_bytes_last = n_ints * 4, R * 4
        if sync:
            self.stream.synchronize()
        return self._h_out_np[:R]

    def step_async(self, b: StepBatch) -> int:
        """Enqueue a host-buffer step and return at once; step_result(handle) waits for its tokens.  At most two steps
        may be outstanding.  Ids of -(j+1) in `b` mean "the token of logit row j of the step enqueued just before"."""
        k = self._flip
        self._flip ^= 1
        T, R, S, bt_stride, n_ints = self.pack(b, self._h_meta2[k].numpy())
        _abi.check(self.lib.b200_decode_step_host(self.ctx, self._h_meta2[k].data_ptr(), T, S, bt_stride, b.max_ctx, R,
                                                  self._h_out2[k].data_ptr(), self.stream.cuda_stream))
        self._done2[k].record(self.stream)
        self.h2d_bytes_last, self.d2h_bytes_last = n_ints * 4, R * 4
        return k | (R << 1)

    def step_result(self, handle: int) -> np.ndarray:
        k, R = handle & 1, handle >> 1
        self._done2[k].synchronize()
        return self._h_out2[k].numpy()[:R]

    def step_device(self, ids, positions, slots, block_table, ctx_lens, max_ctx, *, row_to_seq=None,
                    logit_rows=None, out_tokens=None, out_logits=None, stream=None):
        """Device-pointer step (inputs already resident in HBM): bench.py's `value`, and tests."""
        T = ids.numel()
        R = logit_rows.numel() if logit_rows is not None else T
        if out_tokens is None:
            out_tokens = torch.empty(R, dtype=torch.int32, device=self.device)
        s = (stream or self.stream).cuda_stream
        _abi.check(self.lib.b200_decode_step(
            self.ctx, ids.data_ptr(), positions.data_ptr(), slots.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), _abi.ptr(row_to_seq), ctx_lens.data_ptr(), T, int(max_ctx),
            _abi.ptr(logit_rows), R, out_tokens.data_ptr(), _abi.ptr(out_logits), s))
        return out_tokens

    def pack_sampling(self, temperature, top_k, top_p, seeds, draws, min_p=None) -> int:
        """Per-row sampling parameters of the last step's logit rows into the pinned buffer
        (layout of b200_ctx_sample_last); returns the row count."""
        n = len(temperature)
        if not 0 < n <= self.max_logit_rows:
            raise ValueError(f"sample_last: {n} rows outside (0, {self.max_logit_rows}]")
        a = self._h_sample_np
        a[0:4 * n].view(np.float32)[:] = temperature
        a[4 * n:8 * n].view(np.int32)[:] = top_k
        a[8 * n:12 * n].view(np.float32)[:] = top_p
        a[12 * n:16 * n].view(np.float32)[:] = 0.0 if min_p is None else min_p
        a[16 * n:24 * n].view(np.uint64)[:] = np.asarray(seeds, dtype=np.uint64)
        a[24 * n:32 * n].view(np.uint64)[:] = np.asarray(draws, dtype=np.uint64)
        return n

    def sample_packed(self, n: int, sync: bool = True) -> np.ndarray:
        _abi.check(self.lib.b200_ctx_sample_last(self.ctx, n, self._h_sample.data_ptr(), self._h_out.data_ptr(),
                                                 self.stream.cuda_stream))
        if sync:
            self.stream.synchronize()
        return self._h_out_np[:n]

    def sample_last(self, temperature, top_k, top_p, seeds, draws, sync: bool = True, min_p=None) -> np.ndarray:
        """Tokens for the logit rows of the LAST step under per-row (temperature, top_k, top_p, seed, draw);
        temperature 0 rows return the step's greedy token.  The greedy hot path never calls this."""
        return self.sample_packed(self.pack_sampling(temperature, top_k, top_p, seeds, draws, min_p), sync)

    ADJUST_MAX_WORDS = 4 << 20    # b200_ctx_adjust_last's buffer (16 MiB)

    def pack_adjust(self, rows) -> tuple:
        """rows: one entry per logit row of the last step, None (untouched) or a dict(prompt, output, rep, freq, pres,
        bias={token: value}).  Writes the packed buffer of b200_ctx_adjust_last into pinned memory (allocated on first
        use); returns (n_rows, n_entries).  One entry per distinct token of a row's prompt, output and bias table."""
        n = len(rows)
        if not 0 < n <= self.max_logit_rows:
            raise ValueError(f"adjust_last: {n} rows outside (0, {self.max_logit_rows}]")
        if getattr(self, "_h_adjust", None) is None:
            self._h_adjust = torch.zeros(self.ADJUST_MAX_WORDS, dtype=torch.int32)
            if torch.cuda.is_available():
                self._h_adjust = self._h_adjust.pin_memory()
            self._h_adjust_np = self._h_adjust.numpy()
        ids, counts, seen, bias, offsets = [], [], [], [], [0]
        params = np.empty(3 * n, dtype=np.float32)
        for i, r in enumerate(rows):
            if r is None:
                params[3 * i:3 * i + 3] = (1.0, 0.0, 0.0)
                offsets.append(offsets[-1])
                continue
            params[3 * i:3 * i + 3] = (r["rep"], r["freq"], r["pres"])
            out_t, out_c = np.unique(np.asarray(r["output"], dtype=np.int64), return_counts=True)
            hist = np.union1d(np.asarray(r["prompt"], dtype=np.int64), out_t)
            b = r.get("bias") or {}
            toks = np.union1d(hist, np.fromiter(b.keys(), dtype=np.int64, count=len(b))) if b else hist
            c = np.zeros(len(toks), dtype=np.int32)
            c[np.searchsorted(toks, out_t)] = out_c
            bb = np.zeros(len(toks), dtype=np.float32)
            if b:
                bb[np.searchsorted(toks, np.fromiter(b.keys(), dtype=np.int64, count=len(b)))] = np.fromiter(b.values(), dtype=np.float32, count=len(b))
            ids.append(toks.astype(np.int32))
            counts.append(c)
            seen.append(np.isin(toks, hist).astype(np.int32))
            bias.append(bb)
            offsets.append(offsets[-1] + len(toks))
        E = offsets[-1]
        words = 3 * n + n + 1 + 4 * E
        if words > self.ADJUST_MAX_WORDS:
            raise ValueError(f"adjust_last: {E} (row, token) entries exceed the step's buffer")
        a = self._h_adjust_np
        a[:3 * n].view(np.float32)[:] = params
        a[3 * n:4 * n + 1] = offsets
        o = 4 * n + 1
        if E:
            a[o:o + E] = np.concatenate(ids)
            a[o + E:o + 2 * E] = np.concatenate(counts)
            a[o + 2 * E:o + 3 * E] = np.concatenate(seen)
            a[o + 3 * E:o + 4 * E].view(np.float32)[:] = np.concatenate(bias)
        return n, E

    def adjust_packed(self, n: int, n_entries: int):
        _abi.check(self.lib.b200_ctx_adjust_last(self.ctx, n, self._h_adjust.data_ptr(), n_entries, self.stream.cuda_stream))

    def adjust_last(self, rows):
        """logit_bias / penalties on the logit rows of the LAST step, in place, before sample_last (see pack_adjust)."""
        self.adjust_packed(*self.pack_adjust(rows))

    def logprobs_last(self, token_ids, n_top: int = 0):
        """Log-probabilities (log softmax of the raw logits) of `token_ids` under the LAST step's logit rows, plus
        the n_top most likely tokens per row: (logprob[n], top_ids[n, n_top], top_logprobs[n, n_top])."""
        n = len(token_ids)
        if not 0 < n <= self.max_logit_rows or not 0 <= n_top <= 32:
            raise ValueError(f"logprobs_last: {n} rows / n_top {n_top} out of range")
        self._h_lp_tok.numpy()[:n] = token_ids
        _abi.check(self.lib.b200_ctx_logprobs_last(self.ctx, n, self._h_lp_tok.data_ptr(), n_top, self._h_lp_out.data_ptr(),
                                                   self.stream.cuda_stream))
        self.stream.synchronize()
        out = self._h_lp_out.numpy()
        lp = out[:n].copy()
        ids = out[n:n + n * n_top].view(np.int32).reshape(n, n_top).copy()
        tlp = out[n + n * n_top:n + 2 * n * n_top].reshape(n, n_top).copy()
        return lp, ids, tlp

    def logits_last(self, n_rows: int) -> np.ndarray:
        """The logit rows of the LAST step as fp32 [n_rows, vocab] (a copy).  A ctx in 32-bit mode returns its unrounded logits."""
        if not 0 < n_rows <= self.max_logit_rows:
            raise ValueError(f"logits_last: {n_rows} rows outside (0, {self.max_logit_rows}]")
        V = self.cfg.vocab
        if getattr(self, "_h_logits", None) is None or self._h_logits.numel() < n_rows * V:
            self._h_logits = torch.empty(max(n_rows, 64) * V, dtype=torch.float32).pin_memory()
        _abi.check(self.lib.b200_ctx_logits_last_f32(self.ctx, n_rows, self._h_logits.data_ptr(), self.stream.cuda_stream))
        self.stream.synchronize()
        return self._h_logits.numpy()[:n_rows * V].reshape(n_rows, V).copy()

    def last_step_launches(self) -> int:
        return int(self.lib.b200_ctx_last_step_launches(self.ctx))

    def set_graphs(self, on: bool):
        _abi.check(self.lib.b200_ctx_set_graphs(self.ctx, int(on)))

    def close(self):
        if getattr(self, "ctx", None):
            torch.cuda.synchronize(self.device)
            self.lib.b200_ctx_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class StackRunner(ModelRunner):
    """Device state of a model described layer by layer (config.is_stack_config): same step, sampling and read-back calls as
    ModelRunner (they are the ctx's), its own construction: per-layer descriptors, per-layer paged caches (head sizes differ
    by layer), fp32 cos|sin tables shared between layers of equal rotation.  dtype "float32" runs activations, caches and
    matrix products in true fp32."""

    def __init__(self, cfg, device: Optional[torch.device] = None, *, max_tokens: int = 2048, max_model_len: int = 8192,
                 block_size: int = 64, n_blocks: Optional[int] = None, kv_cache_gib: Optional[float] = None,
                 graphs: bool = True, dtype: str = "bfloat16", max_logit_rows: int = 512, tp_rank: int = 0, tp_world: int = 1,
                 n_state_slots: int = 257):
        if not torch.cuda.is_available():
            raise RuntimeError("StackRunner needs a CUDA device (B200, sm_100a); there is no CPU path")
        if tp_world != 1:
            raise ValueError("layer-list models run on one GPU (tensor_parallel_size 1)")
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype {dtype!r}: bfloat16 or float32")
        self.lib = _abi.lib()
        self.cfg = cfg
        self.f32 = dtype == "float32"
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        if not self.lib.b200_device_ok():
            raise RuntimeError("the current CUDA device is not compute capability 10.x (B200)")
        self.block_size, self.max_tokens, self.max_model_len = block_size, max_tokens, max_model_len
        self.max_blocks_per_seq = (max_model_len + block_size - 1) // block_size
        self.tp_rank, self.tp_world = 0, 1
        self.vocab_local = cfg.vocab
        self.stream = torch.cuda.Stream(device=self.device)

        # rotation tables, one per distinct specification
        self._tables: List[torch.Tensor] = []
        keys: Dict[tuple, int] = {}

        def table_of(spec) -> int:
            if spec is None:
                return -1
            k = spec.key()
            if k not in keys:
                if len(self._tables) >= 16:
                    raise ValueError("more than 16 distinct rotation tables")
                keys[k] = len(self._tables)
                self._tables.append(spec.table(max(max_model_len, 16)).to(self.device))
            return keys[k]

        from .config import AttentionSpec, ChannelDeltaSpec, DupolornConfig, FutidraConfig, HeadDeltaSpec, MLSTMSpec, RudolixConfig, StateSpaceSpec
        self.parallel = isinstance(cfg, DupolornConfig)
        self.postnorm = isinstance(cfg, FutidraConfig)
        self.hyper = isinstance(cfg, RudolixConfig)
        # dense feed-forwards of the post-norm form in bf16: gate activation and product in the gate|up linear's epilogue
        self.fuse_gate_up = self.postnorm and not self.f32 and os.environ.get("B200_STACK_FUSE_GATE_UP", "1") != "0"
        stateful = (self.parallel or self.postnorm or self.hyper) and cfg.needs_state
        self.n_state_slots = int(n_state_slots) if stateful else 0
        if stateful and self.n_state_slots <= 0:
            raise ValueError("this model keeps per-sequence state: n_state_slots must be positive")
        layers = (_abi.StackLayer * cfg.n_layers)()
        for i, L in enumerate(cfg.layers):
            a, f = L.mixer, L.mlp
            if self.hyper:
                if isinstance(a, AttentionSpec):
                    flags = (0 if a.qk_norm else _abi.MIXF_NO_QK_NORM) | (_abi.MIXF_ROT_HALF if a.rot_half else 0) | \
                            (_abi.MIXF_SINK if a.sink else 0) | (_abi.MIXF_SINK_ONE if a.sink_one else 0)
                    d = dict(mixer=_abi.MIXER_ATTENTION, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim,
                             rot_dims=a.rot.dims if a.rot else 0, rot_table=table_of(a.rot), vrot_table=-1, scale=a.scale,
                             mixer_flags=flags, window=a.window)
                elif isinstance(a, HeadDeltaSpec):
                    d = dict(mixer=_abi.MIXER_DELTA, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, rot_table=-1, vrot_table=-1,
                             conv_taps=a.conv, mixer_flags=_abi.MIXF_HEAD_DECAY)
                else:
                    d = dict(mixer=_abi.MIXER_SSD, heads=a.heads, kv_heads=a.groups, dim=a.state, vdim=a.vdim, rot_table=-1, vrot_table=-1,
                             conv_taps=a.conv, norm_groups=a.norm_groups)
                if f is not None and f.kind == "dense":
                    d.update(mlp=_abi.MLP_DENSE, ff=f.ff, act=_abi.ACTS[f.act], ungated=int(not f.gated), act_limit=f.limit)
                elif f is not None:
                    d.update(mlp=_abi.MLP_MOE, experts=f.experts, top=f.top, groups=1, keep=1, ff=f.ff, act=_abi.ACTS[f.act],
                             ungated=int(not f.gated), act_limit=f.limit, route_chosen=int(f.router == "chosen_softmax"))
                layers[i] = _abi.StackLayer(**d)
                continue
            if self.postnorm:
                if isinstance(a, AttentionSpec):
                    flags = (_abi.MIXF_HEAD_NORM if a.head_norm else 0) | (_abi.MIXF_VALUE_IS_KEY if a.value_is_key else 0) | \
                            (_abi.MIXF_SINK_ONE if a.sink_one else 0)
                    d = dict(mixer=_abi.MIXER_ATTENTION, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim,
                             rot_dims=a.rot.dims if a.rot else 0, rot_table=table_of(a.rot), vrot_table=-1, scale=a.scale,
                             mixer_flags=flags, window=a.window)
                elif isinstance(a, ChannelDeltaSpec):
                    d = dict(mixer=_abi.MIXER_DELTA, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, rot_table=-1, vrot_table=-1,
                             conv_taps=a.conv, decay_rank=a.decay_rank, gate_rank=a.gate_rank)
                else:
                    d = dict(mixer=_abi.MIXER_LATENT, heads=a.heads, kv_heads=1, dim=a.dim, vdim=a.vdim, rot_table=-1, vrot_table=-1,
                             scale=a.scale, kv_rank=a.kv_rank, q_rank=a.q_rank, window=a.window,
                             mixer_flags=_abi.MIXF_HEAD_GATE if a.head_gate else 0, kv_share=0 if a.kv_from is None else a.kv_from + 1)
                if f is not None:
                    d.update(mlp=_abi.MLP_DENSE, ff=f.ff, act=_abi.ACTS[f.act])
                layers[i] = _abi.StackLayer(**d)
                continue
            if not self.parallel:
                layers[i] = _abi.StackLayer(
                    mixer=_abi.MIXER_ATTENTION, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim,
                    rot_dims=a.rot.dims if a.rot else 0, rot_table=table_of(a.rot), vrot_table=table_of(a.value_rot), scale=a.scale,
                    mlp=_abi.MLP_MOE if f else _abi.MLP_NONE, experts=f.experts if f else 0, top=f.top if f else 0,
                    groups=f.groups if f else 0, keep=f.keep if f else 0, ff=f.ff if f else 0)
                continue
            if isinstance(a, MLSTMSpec):
                d = dict(mixer=_abi.MIXER_MLSTM, heads=a.heads, kv_heads=a.heads, dim=a.dim, vdim=a.vdim, rot_table=-1, vrot_table=-1,
                         gate_cap=a.gate_cap)
            else:
                d = dict(mixer=_abi.MIXER_LATENT, heads=a.heads, kv_heads=1, dim=a.dim, vdim=a.vdim, rot_dims=a.rot.dims if a.rot else 0,
                         rot_table=table_of(a.rot), vrot_table=-1, scale=a.scale, kv_rank=a.kv_rank, rot_dim=a.rot_dim,
                         mixer_flags=(_abi.MIXF_SINK if a.sink else 0) | (_abi.MIXF_GATE if a.gate else 0))
            if f is not None and f.kind == "dense":
                d.update(mlp=_abi.MLP_DENSE, ff=f.ff, act=_abi.ACTS[f.act])
            elif f is not None:
                d.update(mlp=_abi.MLP_MOE, experts=f.experts, top=f.top, groups=1, keep=1, ff=f.ff, act=_abi.ACTS[f.act], ungated=1,
                         sigmoid_scores=1, weight_input=1, shared_ff=f.shared_ff)
            layers[i] = _abi.StackLayer(**d)
        sc = _abi.StackCfg(width=cfg.width, vocab=cfg.vocab, n_layers=cfg.n_layers, embed_scale=cfg.embed_scale,
                           norm_eps=cfg.norm_eps, f32=int(self.f32), block_size=block_size, max_tokens=max_tokens,
                           max_blocks_per_seq=self.max_blocks_per_seq, max_logit_rows=min(max_logit_rows, max_tokens))
        if self.parallel:
            sc.form, sc.canon_taps, sc.depth_avg = _abi.FORM_PARALLEL, cfg.canon_taps, int(cfg.depth_avg)
            sc.bigram_buckets, sc.bigram_mul_prev, sc.bigram_mul_cur = cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur
            sc.logit_softcap, sc.n_state_slots = cfg.logit_softcap, self.n_state_slots
        if self.postnorm:
            sc.form, sc.residual_alpha, sc.n_state_slots = _abi.FORM_POSTNORM, cfg.postln_alpha, self.n_state_slots
        if self.hyper:
            sc.form, sc.canon_taps, sc.n_state_slots = _abi.FORM_HYPER, cfg.canon_taps, self.n_state_slots
            sc.streams, sc.residual_mult = cfg.streams, cfg.residual_mult
        h = C.c_void_p()
        _abi.check(self.lib.b200_stack_create(C.byref(sc), layers, C.byref(h)))
        self.ctx = h
        _abi.check(self.lib.b200_ctx_set_graphs(self.ctx, int(graphs)))
        for i, t in enumerate(self._tables):
            _abi.check(self.lib.b200_stack_set_rot_table(self.ctx, i, t.data_ptr(), t.shape[0], t.shape[2]))

        # paged caches, one pair per layer: [n_blocks][kv_heads][block][row widths the ctx names], zero-filled
        self.cache_dims = []
        for i in range(len(cfg.layers)):
            kd, vd = C.c_int32(), C.c_int32()
            _abi.check(self.lib.b200_stack_cache_dims(self.ctx, i, C.byref(kd), C.byref(vd)))
            self.cache_dims.append((kd.value, vd.value))
        kvh = [getattr(L.mixer, "kv_heads", 1) for L in cfg.layers]
        per_block = max(sum(h * (kd + vd) for h, (kd, vd) in zip(kvh, self.cache_dims)) * (4 if self.f32 else 2) * block_size, 1)
        if n_blocks is None:
            if kv_cache_gib is None:
                free, _ = torch.cuda.mem_get_info(self.device)
                kv_cache_gib = max(free / 2 ** 30 * 0.5, 0.25)
            n_blocks = max(int(kv_cache_gib * 2 ** 30) // per_block, 2)
        self.n_blocks = n_blocks
        cdt = torch.float32 if self.f32 else torch.bfloat16
        self.k_cache, self.v_cache = [], []
        for i, L in enumerate(cfg.layers):
            kd, vd = self.cache_dims[i]
            k = torch.zeros((n_blocks, kvh[i], block_size, kd), dtype=cdt, device=self.device) if kd else None
            v = torch.zeros((n_blocks, kvh[i], block_size, vd), dtype=cdt, device=self.device) if vd else None
            self.k_cache.append(k)
            self.v_cache.append(v)
            if k is not None:
                _abi.check(self.lib.b200_stack_set_kv_cache(self.ctx, i, k.data_ptr(), _abi.ptr(v), n_blocks))
        # per-sequence state slots (previous token, convolution tails, recurrent state): the scheduler hands a slot to every
        # running sequence; a sequence that starts at position 0 ignores what the slot held
        self.state = None
        if self.n_state_slots > 0:
            self.state_bytes = int(self.lib.b200_stack_state_bytes(self.ctx))
            self.state = torch.zeros(self.n_state_slots * self.state_bytes, dtype=torch.uint8, device=self.device)
            _abi.check(self.lib.b200_stack_set_state(self.ctx, self.state.data_ptr()))
        self._alloc_host_buffers(max_logit_rows)
        self._tap = None

    def _set(self, layer: int, kind: int, t: torch.Tensor):
        dt = torch.float32 if kind in _abi.SW_F32 else torch.bfloat16
        t = t.to(device=self.device, dtype=dt)
        if kind == _abi.SW_MLP_GATE_UP and self.fuse_gate_up and (t.shape[0] // 2) % 64 == 0 and t.shape[1] % 8 == 0:
            # the tcgen05 linear activates and multiplies in its epilogue over slabs of 64 gate rows + the 64 matching up rows
            from .weights import interleave_gate_up
            ff = t.shape[0] // 2
            t, kind = interleave_gate_up(t[:ff], t[ff:]), _abi.SW_MLP_GATE_UP_INTERLEAVED
        t = t.contiguous()
        self._weights.append(t)
        rows, cols = (t.shape[0], t.shape[1]) if t.dim() == 2 else (t.shape[0], 1)
        _abi.check(self.lib.b200_stack_set_weight(self.ctx, layer, kind, t.data_ptr(), rows, cols))

    def load_weights(self, w: Dict[str, torch.Tensor]):
        from .weights import STACK_WEIGHT_MAPS
        for layer, kind, t in STACK_WEIGHT_MAPS[self.cfg.architecture](w, self.cfg):
            self._set(layer, kind, t)

    def _init_random_parallel(self, seed: int, std: float):
        from .config import MLSTMSpec
        c, A = self.cfg, _abi
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)

        def rnd(*shape, sd=std):
            t = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            t.normal_(0.0, sd, generator=g)
            return t

        one = torch.ones(1, device=self.device)
        self._set(0, A.SW_EMBED, rnd(c.vocab, c.width, sd=1.0))
        if c.bigram_buckets > 0:
            self._set(0, A.SW_BIGRAM, rnd(c.bigram_buckets + 1, c.width, sd=1.0))
        self._set(0, A.SW_FINAL_NORM, one)
        self._set(0, A.SW_HEAD, rnd(c.vocab, c.width))
        for i, L in enumerate(c.layers):
            a, f = L.mixer, L.mlp
            self._set(i, A.SW_NORM_MIX_PRE, one)
            if f is not None:
                self._set(i, A.SW_NORM_MLP_PRE, one)
            if c.canon_taps >= 1:
                self._set(i, A.SW_CANON, rnd(c.width, c.canon_taps, sd=0.2).float())
            if c.depth_avg:
                d = torch.full((i + 2,), 0.1 / (i + 1), device=self.device)
                d[-1] = 0.9
                self._set(i, A.SW_DEPTH_AVG, d)
            if isinstance(a, MLSTMSpec):
                self._set(i, A.SW_QKV, rnd(2 * a.heads * a.dim + 2 * a.heads * a.vdim, c.width))
                self._set(i, A.SW_GATES, rnd(2 * a.heads, c.width))
                self._set(i, A.SW_GATES_BIAS, torch.cat([torch.zeros(a.heads), torch.full((a.heads,), 3.0)]).to(self.device))
                self._set(i, A.SW_HEAD_NORM, torch.ones(a.heads * a.vdim, device=self.device))
            else:
                self._set(i, A.SW_QKV, rnd(a.heads * (a.dim + a.rot_dim) + a.kv_rank + a.rot_dim + (a.heads * a.vdim if a.gate else 0), c.width))
                self._set(i, A.SW_K_NORM, torch.ones(a.kv_rank, device=self.device))
                self._set(i, A.SW_UK_T, rnd(a.heads * a.kv_rank, a.dim, sd=a.kv_rank ** -0.5))
                self._set(i, A.SW_UV, rnd(a.heads * a.vdim, a.kv_rank, sd=a.kv_rank ** -0.5))
                if a.sink:
                    self._set(i, A.SW_SINK, torch.zeros(a.heads, device=self.device))
            self._set(i, A.SW_O, rnd(c.width, a.heads * a.vdim))
            if f is None:
                continue
            if f.kind == "dense":
                self._set(i, A.SW_MLP_GATE_UP, rnd(2 * f.ff, c.width))
                self._set(i, A.SW_MLP_DOWN, rnd(c.width, f.ff))
            else:
                self._set(i, A.SW_ROUTER, rnd(f.experts, c.width))
                self._set(i, A.SW_EXPERT_GATE_UP, rnd(f.experts * f.ff, c.width))
                self._set(i, A.SW_EXPERT_DOWN, rnd(f.experts * c.width, f.ff))
                if f.shared_ff > 0:
                    self._set(i, A.SW_SHARED_UP, rnd(f.shared_ff, c.width))
                    self._set(i, A.SW_SHARED_DOWN, rnd(c.width, f.shared_ff))

    def _init_random_postnorm(self, seed: int, std: float):
        from .config import AttentionSpec, ChannelDeltaSpec
        from .weights import delta_fused_offsets
        c, A = self.cfg, _abi
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)

        def rnd(*shape, sd=std):
            t = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            t.normal_(0.0, sd, generator=g)
            return t

        ones, zeros = torch.ones(c.width, device=self.device), torch.zeros(c.width, device=self.device)
        emb = rnd(c.vocab, c.width, sd=1.0)
        self._set(0, A.SW_EMBED, emb)
        self._set(0, A.SW_HEAD, emb)
        self._set(0, A.SW_FINAL_NORM, ones)
        self._set(0, A.SW_FINAL_NORM_BIAS, zeros)
        for i, L in enumerate(c.layers):
            a, f = L.mixer, L.mlp
            self._set(i, A.SW_NORM_MIX_POST, ones)
            self._set(i, A.SW_NORM_MIX_POST_BIAS, zeros)
            if isinstance(a, AttentionSpec):
                self._set(i, A.SW_QKV, rnd((a.heads + a.kv_heads) * a.dim, c.width))
                self._set(i, A.SW_Q_NORM, torch.ones(a.dim, device=self.device))
                self._set(i, A.SW_K_NORM, torch.ones(a.dim, device=self.device))
            elif isinstance(a, ChannelDeltaSpec):
                rows, off = delta_fused_offsets(a)
                fused = rnd(rows, c.width)
                for lo, n in zip(off, (a.kv_heads * a.dim, a.kv_heads * a.dim, a.heads * a.vdim, a.decay_rank, a.gate_rank, a.heads)):
                    fused[lo + n:(off[off.index(lo) + 1] if lo != off[-1] else rows)] = 0
                self._set(i, A.SW_QKV, fused)
                self._set(i, A.SW_CONV, rnd(2 * a.kv_heads * a.dim + a.heads * a.vdim, a.conv, sd=0.5).float())
                self._set(i, A.SW_DECAY_UP, rnd(a.heads * a.dim, a.decay_rank))
                self._set(i, A.SW_DECAY_BIAS, torch.zeros(a.heads * a.dim, device=self.device))
                self._set(i, A.SW_DECAY_LOG, torch.zeros(a.heads, device=self.device))
                self._set(i, A.SW_GATE_UP, rnd(a.heads * a.vdim, a.gate_rank))
                self._set(i, A.SW_HEAD_NORM, torch.ones(a.heads * a.vdim, device=self.device))
            else:
                own = a.kv_from is None
                self._set(i, A.SW_QKV, rnd(a.q_rank + (a.kv_rank if own else 0) + a.heads, c.width))
                self._set(i, A.SW_Q_LATENT_NORM, torch.ones(a.q_rank, device=self.device))
                self._set(i, A.SW_UQ, rnd(a.heads * a.dim, a.q_rank, sd=a.q_rank ** -0.5))
                if own:
                    self._set(i, A.SW_K_NORM, torch.ones(a.kv_rank, device=self.device))
                self._set(i, A.SW_UK_T, rnd(a.heads * a.kv_rank, a.dim, sd=a.kv_rank ** -0.5))
                self._set(i, A.SW_UV, rnd(a.heads * a.vdim, a.kv_rank, sd=a.kv_rank ** -0.5))
            self._set(i, A.SW_O, rnd(c.width, a.heads * a.vdim))
            if f is not None:
                self._set(i, A.SW_NORM_MLP_POST, ones)
                self._set(i, A.SW_NORM_MLP_POST_BIAS, zeros)
                self._set(i, A.SW_MLP_GATE_UP, rnd(2 * f.ff, c.width))
                self._set(i, A.SW_MLP_DOWN, rnd(c.width, f.ff))

    def _init_random_hyper(self, seed: int, std: float):
        from .config import AttentionSpec, HeadDeltaSpec
        c, A = self.cfg, _abi
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)

        def rnd(*shape, sd=std):
            t = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            t.normal_(0.0, sd, generator=g)
            return t

        ones, zeros = torch.ones(c.width, device=self.device), torch.zeros(c.width, device=self.device)
        n = c.streams
        # every stream is read and written with equal weight; the streams keep themselves
        hc = torch.cat([torch.full((n,), 1.0 / n), torch.ones(n), torch.eye(n).reshape(-1)]).to(self.device)
        emb = rnd(c.vocab, c.width, sd=1.0)
        self._set(0, A.SW_EMBED, emb)
        self._set(0, A.SW_HEAD, emb)
        self._set(0, A.SW_FINAL_NORM, ones)
        self._set(0, A.SW_FINAL_NORM_BIAS, zeros)
        for i, L in enumerate(c.layers):
            a, f = L.mixer, L.mlp
            self._set(i, A.SW_NORM_MIX_PRE, ones)
            self._set(i, A.SW_NORM_MIX_PRE_BIAS, zeros)
            self._set(i, A.SW_SCALE_MIX, ones)
            self._set(i, A.SW_HC_MIX, hc)
            if c.canon_taps >= 1:
                self._set(i, A.SW_CANON, rnd(c.width, c.canon_taps, sd=0.2).float())
            self._set(i, A.SW_QKV, rnd(c.mixer_rows(a), c.width))
            if isinstance(a, AttentionSpec):
                if a.sink:
                    self._set(i, A.SW_SINK, torch.zeros(a.heads, device=self.device))
            elif isinstance(a, HeadDeltaSpec):
                self._set(i, A.SW_CONV, rnd(2 * a.kv_heads * a.dim + a.heads * a.vdim, a.conv, sd=0.5).float())
                self._set(i, A.SW_DECAY_BIAS, torch.zeros(a.heads, device=self.device))
                self._set(i, A.SW_DECAY_LOG, torch.zeros(a.heads, device=self.device))
                self._set(i, A.SW_HEAD_NORM, torch.ones(a.heads * a.vdim, device=self.device))
            else:
                ch = a.heads * a.vdim + 2 * a.groups * a.state
                self._set(i, A.SW_CONV, rnd(ch, a.conv, sd=0.5).float())
                self._set(i, A.SW_CONV_BIAS, torch.zeros(ch, device=self.device))
                self._set(i, A.SW_DECAY_BIAS, torch.zeros(a.heads, device=self.device))
                self._set(i, A.SW_DECAY_LOG, torch.zeros(a.heads, device=self.device))
                self._set(i, A.SW_SKIP, torch.ones(a.heads, device=self.device))
                self._set(i, A.SW_HEAD_NORM, torch.ones(a.heads * a.vdim, device=self.device))
            self._set(i, A.SW_O, rnd(c.width, a.heads * a.vdim))
            if f is None:
                continue
            self._set(i, A.SW_NORM_MLP_PRE, ones)
            self._set(i, A.SW_NORM_MLP_PRE_BIAS, zeros)
            self._set(i, A.SW_SCALE_MLP, ones)
            self._set(i, A.SW_HC_MLP, hc)
            if c.canon_taps >= 1:
                self._set(i, A.SW_CANON_MLP, rnd(c.width, c.canon_taps, sd=0.2).float())
            if f.kind == "dense":
                self._set(i, A.SW_MLP_GATE_UP, rnd((2 if f.gated else 1) * f.ff, c.width))
                self._set(i, A.SW_MLP_DOWN, rnd(c.width, f.ff))
                if f.act == "polynorm":
                    self._set(i, A.SW_MLP_ACT, torch.tensor([1.0, 0.5, 0.25, 0.0], device=self.device))
            else:
                self._set(i, A.SW_ROUTER, rnd(f.experts, c.width))
                self._set(i, A.SW_ROUTER_BIAS, torch.zeros(f.experts, device=self.device))
                self._set(i, A.SW_EXPERT_GATE_UP, rnd(f.experts * (2 if f.gated else 1) * f.ff, c.width))
                self._set(i, A.SW_EXPERT_DOWN, rnd(f.experts * c.width, f.ff))

    def set_step_slots(self, seq_slots: Optional[torch.Tensor]):
        """Device-pointer steps (step_device) of a model with state slots: int32 device tensor, one slot per sequence of the step."""
        self._step_slots = seq_slots
        _abi.check(self.lib.b200_stack_set_step_slots(self.ctx, _abi.ptr(seq_slots), 0 if seq_slots is None else seq_slots.numel()))

    def init_random_weights(self, seed: int = 1234, std: float = 0.02):
        """Random-init weights generated on the device (benchmarks).  Norm weights are 1, the router bias 0."""
        if self.parallel:
            return self._init_random_parallel(seed, std)
        if self.postnorm:
            return self._init_random_postnorm(seed, std)
        if self.hyper:
            return self._init_random_hyper(seed, std)
        c, A = self.cfg, _abi
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)

        def rnd(*shape, sd=std):
            t = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            t.normal_(0.0, sd, generator=g)
            return t

        ones = torch.ones(c.width, dtype=torch.float32, device=self.device)
        self._set(0, A.SW_EMBED, rnd(c.vocab, c.width, sd=1.0))
        self._set(0, A.SW_FINAL_NORM, ones)
        self._set(0, A.SW_HEAD, rnd(c.vocab, c.width))
        for i, L in enumerate(c.layers):
            a, f = L.mixer, L.mlp
            for kind in (A.SW_NORM_MIX_PRE, A.SW_NORM_MIX_POST):
                self._set(i, kind, ones)
            self._set(i, A.SW_QKV, rnd(a.heads * a.dim + a.kv_heads * (a.dim + a.vdim), c.width))
            self._set(i, A.SW_Q_NORM, torch.ones(a.heads * a.dim, device=self.device))
            self._set(i, A.SW_K_NORM, torch.ones(a.kv_heads * a.dim, device=self.device))
            self._set(i, A.SW_O, rnd(c.width, a.heads * a.vdim))
            if f:
                for kind in (A.SW_NORM_MLP_PRE, A.SW_NORM_MLP_POST):
                    self._set(i, kind, ones)
                self._set(i, A.SW_ROUTER, rnd(f.experts, c.width))
                self._set(i, A.SW_EXPERT_GATE_UP, rnd(f.experts * 2 * f.ff, c.width))
                self._set(i, A.SW_EXPERT_DOWN, rnd(f.experts * c.width, f.ff))

    def init_tp(self, group=None, peer_allreduce: bool = None):
        return

    def set_stream_tap(self, on: bool) -> Optional[torch.Tensor]:
        """Parity tests: after every step, [n_layers][max_tokens rows used][width] fp32 residual streams (graph replay off)."""
        if on:
            self._tap = torch.zeros(self.cfg.n_layers * self.max_tokens * self.cfg.width, dtype=torch.float32, device=self.device)
            _abi.check(self.lib.b200_stack_set_stream_tap(self.ctx, self._tap.data_ptr()))
        else:
            _abi.check(self.lib.b200_stack_set_stream_tap(self.ctx, None))
            self._tap = None
        return self._tap


def make_runner(cfg, **kw):
    """The runner class follows the configuration class (config.load_model_config picks that by config.json)."""
    from .config import is_stack_config
    if is_stack_config(cfg):
        kw.pop("tp_rank", None), kw.pop("tp_world", None)
        return StackRunner(cfg, **kw)
    kw.pop("dtype", None), kw.pop("max_logit_rows", None), kw.pop("n_state_slots", None)
    return ModelRunner(cfg, **kw)
