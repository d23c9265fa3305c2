"""Host-side weight plumbing: HF names -> fused, per-rank shards (pure torch, no CUDA needed).

Packing follows [V22] vllm/model_executor/models/llama.py:437-444 (q|k|v -> qkv_proj, gate|up ->
gate_up_proj); sharding is Megatron-style as in SURVEY.md §8e: QKV and gate_up column-parallel (by
head / by intermediate feature), O and down row-parallel, lm_head vocab-parallel, embedding and norms
replicated.  Weights come from the HF cache the chart mounts at /data
(/root/reference/core/helm-charts/vllm/templates/configmap.yaml:18-21).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from .config import ModelConfig

# kinds of include/b200_decode.h (b200_weight_kind)
EMBED, LN1, QKV, QKV_BIAS, O, LN2, GATE_UP, DOWN, FINAL_NORM, LM_HEAD, GATE_UP_INTERLEAVED = range(11)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I,h],[I,h] -> [2I,h] in 128-row slabs: 64 gate rows then the 64 matching up rows."""
    I, h = gate.shape
    return torch.stack([gate.reshape(I // 64, 64, h), up.reshape(I // 64, 64, h)], dim=1).reshape(2 * I, h)


def shard_weights(w: Dict[str, torch.Tensor], cfg: ModelConfig, rank: int = 0, world: int = 1
                  ) -> Iterator[Tuple[int, int, torch.Tensor]]:
    """Yield (layer, kind, tensor) for one TP rank, in the order the runner uploads them."""
    d = cfg.head_dim
    hq, hkv = cfg.n_q_heads // world, cfg.n_kv_heads // world
    inter, vloc = cfg.intermediate // world, cfg.vocab // world
    if cfg.n_q_heads % world or cfg.n_kv_heads % world or cfg.intermediate % world or cfg.vocab % world:
        raise ValueError(f"model does not divide over tensor_parallel_size={world}")
    qs = slice(rank * hq * d, (rank + 1) * hq * d)
    ks = slice(rank * hkv * d, (rank + 1) * hkv * d)
    is_ = slice(rank * inter, (rank + 1) * inter)
    vs = slice(rank * vloc, (rank + 1) * vloc)
    yield 0, EMBED, w["model.embed_tokens.weight"]
    for l in range(cfg.n_layers):
        p = f"model.layers.{l}."
        yield l, LN1, w[p + "input_layernorm.weight"]
        yield l, QKV, torch.cat([w[p + "self_attn.q_proj.weight"][qs], w[p + "self_attn.k_proj.weight"][ks],
                                 w[p + "self_attn.v_proj.weight"][ks]], 0)
        if cfg.qkv_bias:
            yield l, QKV_BIAS, torch.cat([w[p + "self_attn.q_proj.bias"][qs], w[p + "self_attn.k_proj.bias"][ks],
                                          w[p + "self_attn.v_proj.bias"][ks]], 0)
        yield l, O, w[p + "self_attn.o_proj.weight"][:, qs]
        yield l, LN2, w[p + "post_attention_layernorm.weight"]
        gate, up = w[p + "mlp.gate_proj.weight"][is_], w[p + "mlp.up_proj.weight"][is_]
        if inter % 64 == 0:
            yield l, GATE_UP_INTERLEAVED, interleave_gate_up(gate, up)
        else:
            yield l, GATE_UP, torch.cat([gate, up], 0)
        yield l, DOWN, w[p + "mlp.down_proj.weight"][:, is_]
    yield 0, FINAL_NORM, w["model.norm.weight"]
    yield 0, LM_HEAD, w.get("lm_head.weight", w["model.embed_tokens.weight"])[vs]


def load_safetensors_dir(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of an HF checkpoint directory (model.safetensors or sharded + index)."""
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted({os.path.join(path, v) for v in json.load(f)["weight_map"].values()})
    out = {}
    for fn in files:
        with safe_open(fn, framework="pt", device="cpu") as f:
            for k in f.keys():
                out[k] = f.get_tensor(k)
    return out


def resolve_hf_snapshot(model_id: str, hf_home: str = None) -> str:
    """Path of a cached snapshot of `model_id` under HF_HOME (no network access is attempted)."""
    if os.path.isdir(model_id):
        return model_id
    hf_home = hf_home or os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface"))
    base = os.path.join(hf_home, "hub", "models--" + model_id.replace("/", "--"), "snapshots")
    snaps = sorted(glob.glob(os.path.join(base, "*")))
    if not snaps:
        raise FileNotFoundError(f"{model_id} is not in the HF cache at {hf_home} (HF_HOME); the server does not download")
    return snaps[-1]


def bopilorn_weights(w: Dict[str, torch.Tensor], cfg) -> Iterator[Tuple[int, int, torch.Tensor]]:
    """(layer, b200_stack_weight kind, tensor) of a Bopilorn checkpoint: `embed`, `head`, `final.norm`, and per layer i
    `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.q|k|v|o`, `l<i>.mix.q.norm|k.norm`, `l<i>.mlp.router|correction`,
    `l<i>.mlp.e<j>.gate|up|down`.  q|k|v are fused row-wise, the experts stacked ([E][2 ff][width] gate rows then up rows,
    [E][width][ff]); vectors are handed over in fp32."""
    from . import _abi as A
    yield 0, A.SW_EMBED, w["embed"]
    yield 0, A.SW_FINAL_NORM, w["final.norm"]
    yield 0, A.SW_HEAD, w["head"]
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        yield i, A.SW_NORM_MIX_PRE, w[p + "norm1"]
        yield i, A.SW_NORM_MIX_POST, w[p + "norm1b"]
        yield i, A.SW_QKV, torch.cat([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"]], 0)
        yield i, A.SW_Q_NORM, w[p + "mix.q.norm"]
        yield i, A.SW_K_NORM, w[p + "mix.k.norm"]
        yield i, A.SW_O, w[p + "mix.o"]
        if L.mlp is None:
            continue
        yield i, A.SW_NORM_MLP_PRE, w[p + "norm2"]
        yield i, A.SW_NORM_MLP_POST, w[p + "norm2b"]
        yield i, A.SW_ROUTER, w[p + "mlp.router"]
        if p + "mlp.correction" in w:
            yield i, A.SW_ROUTER_BIAS, w[p + "mlp.correction"]
        E = L.mlp.experts
        yield i, A.SW_EXPERT_GATE_UP, torch.cat([torch.cat([w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"]], 0) for e in range(E)], 0)
        yield i, A.SW_EXPERT_DOWN, torch.cat([w[f"{p}mlp.e{e}.down"] for e in range(E)], 0)


def dupolorn_weights(w: Dict[str, torch.Tensor], cfg) -> Iterator[Tuple[int, int, torch.Tensor]]:
    """(layer, b200_stack_weight kind, tensor) of a Dupolorn checkpoint: `embed`, `bigram`, `head`, `final.norm`, and per layer i
    `l<i>.norm1|norm2` (one number each), `l<i>.canon1` [width, taps], `l<i>.dwa` [i + 2], the mixer `l<i>.mix.*` and the
    feed-forward `l<i>.mlp.*`.  The projections that read the mixer's input are fused row-wise (latent: q | dkv | g; mLSTM:
    q | k | v | g, and i | f as the gate rows); a head's key expansion is handed over transposed ([heads][kv_rank][dim]); experts are
    stacked [E][ff][width] and [E][width][ff]; vectors and scalars go over in fp32."""
    from . import _abi as A
    from .config import MLSTMSpec
    yield 0, A.SW_EMBED, w["embed"]
    if cfg.bigram_buckets > 0:
        yield 0, A.SW_BIGRAM, w["bigram"]
    yield 0, A.SW_FINAL_NORM, w["final.norm"].reshape(1)
    yield 0, A.SW_HEAD, w["head"]
    for i, L in enumerate(cfg.layers):
        p, a, f = f"l{i}.", L.mixer, L.mlp
        yield i, A.SW_NORM_MIX_PRE, w[p + "norm1"].reshape(1)
        if f is not None:
            yield i, A.SW_NORM_MLP_PRE, w[p + "norm2"].reshape(1)
        if cfg.canon_taps >= 1:
            yield i, A.SW_CANON, w[p + "canon1"]
        if cfg.depth_avg:
            yield i, A.SW_DEPTH_AVG, w[p + "dwa"]
        if isinstance(a, MLSTMSpec):
            yield i, A.SW_QKV, torch.cat([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"]], 0)
            yield i, A.SW_GATES, torch.cat([w[p + "mix.i"], w[p + "mix.f"]], 0)
            yield i, A.SW_GATES_BIAS, torch.cat([w[p + "mix.i.b"], w[p + "mix.f.b"]], 0)
            yield i, A.SW_HEAD_NORM, w[p + "mix.norm"]
        else:
            yield i, A.SW_QKV, torch.cat([w[p + "mix.q"], w[p + "mix.dkv"]] + ([w[p + "mix.g"]] if a.gate else []), 0)
            yield i, A.SW_K_NORM, w[p + "mix.dkv.norm"]
            yield i, A.SW_UK_T, w[p + "mix.uk"].reshape(a.heads, a.dim, a.kv_rank).transpose(1, 2).reshape(a.heads * a.kv_rank, a.dim)
            yield i, A.SW_UV, w[p + "mix.uv"]
            if a.sink:
                yield i, A.SW_SINK, w[p + "mix.sink"]
        yield i, A.SW_O, w[p + "mix.o"]
        if f is None:
            continue
        if f.kind == "dense":
            yield i, A.SW_MLP_GATE_UP, torch.cat([w[p + "mlp.gate"], w[p + "mlp.up"]], 0)
            yield i, A.SW_MLP_DOWN, w[p + "mlp.down"]
        else:
            yield i, A.SW_ROUTER, w[p + "mlp.router"]
            yield i, A.SW_EXPERT_GATE_UP, torch.cat([w[f"{p}mlp.e{e}.up"] for e in range(f.experts)], 0)
            yield i, A.SW_EXPERT_DOWN, torch.cat([w[f"{p}mlp.e{e}.down"] for e in range(f.experts)], 0)
            if f.shared_ff > 0:
                yield i, A.SW_SHARED_UP, w[p + "mlp.shared.up"]
                yield i, A.SW_SHARED_DOWN, w[p + "mlp.shared.down"]


def delta_fused_offsets(a) -> Tuple[int, list]:
    """(rows, [q, k, v, a1, g1, b offsets]) of the delta mixer's fused projection: the three small groups start at multiples of 8
    rows and the total is a multiple of 8 (the rows between are zeros), as b200_delta_fused_rows lays them out."""
    up8 = lambda v: (v + 7) // 8 * 8
    o = [0, a.kv_heads * a.dim, 2 * a.kv_heads * a.dim]
    o.append(up8(o[2] + a.heads * a.vdim))
    o.append(up8(o[3] + a.decay_rank))
    o.append(up8(o[4] + a.gate_rank))
    return up8(o[5] + a.heads), o


def futidra_weights(w: Dict[str, torch.Tensor], cfg) -> Iterator[Tuple[int, int, torch.Tensor]]:
    """(layer, b200_stack_weight kind, tensor) of a Futidra checkpoint: `embed` (also the output projection), `final.norm[.b]`, per
    layer i `l<i>.norm1[.b]`, `l<i>.norm2[.b]`, the mixer `l<i>.mix.*` and the feed-forward `l<i>.mlp.gate|up|down`.  Projections
    of the mixer's input are fused row-wise: attention q | k; latent dq | dkv | g (no dkv where the layer reads another layer's
    latents); delta q | k | v | a1 | g1 | b with zero rows so that a1, g1 and b start at multiples of 8.  A latent head's key
    expansion goes over transposed ([heads][kv_rank][dim]); the delta mixer's head norm weight is repeated for every head; the
    three convolution kernels are stacked; vectors go over in fp32."""
    from . import _abi as A
    from .config import AttentionSpec, ChannelDeltaSpec
    yield 0, A.SW_EMBED, w["embed"]
    yield 0, A.SW_HEAD, w["embed"]
    yield 0, A.SW_FINAL_NORM, w["final.norm"]
    yield 0, A.SW_FINAL_NORM_BIAS, w["final.norm.b"]
    for i, L in enumerate(cfg.layers):
        p, a, f = f"l{i}.", L.mixer, L.mlp
        yield i, A.SW_NORM_MIX_POST, w[p + "norm1"]
        yield i, A.SW_NORM_MIX_POST_BIAS, w[p + "norm1.b"]
        if isinstance(a, AttentionSpec):
            yield i, A.SW_QKV, torch.cat([w[p + "mix.q"], w[p + "mix.k"]], 0)
            yield i, A.SW_Q_NORM, w[p + "mix.q.norm"]
            yield i, A.SW_K_NORM, w[p + "mix.k.norm"]
        elif isinstance(a, ChannelDeltaSpec):
            rows, o = delta_fused_offsets(a)
            fused = torch.zeros((rows, cfg.width), dtype=w[p + "mix.q"].dtype)
            for off, name in zip(o, ("q", "k", "v", "a1", "g1", "b")):
                t = w[p + "mix." + name]
                fused[off:off + t.shape[0]] = t
            yield i, A.SW_QKV, fused
            yield i, A.SW_CONV, torch.cat([w[p + "mix.q.conv"], w[p + "mix.k.conv"], w[p + "mix.v.conv"]], 0)
            yield i, A.SW_DECAY_UP, w[p + "mix.a2"]
            yield i, A.SW_DECAY_BIAS, w[p + "mix.dt_bias"]
            yield i, A.SW_DECAY_LOG, w[p + "mix.A_log"]
            yield i, A.SW_GATE_UP, w[p + "mix.g2"]
            yield i, A.SW_HEAD_NORM, w[p + "mix.norm"].repeat(a.heads)
        else:
            own = a.kv_from is None
            yield i, A.SW_QKV, torch.cat([w[p + "mix.dq"]] + ([w[p + "mix.dkv"]] if own else []) + [w[p + "mix.g"]], 0)
            yield i, A.SW_Q_LATENT_NORM, w[p + "mix.dq.norm"]
            yield i, A.SW_UQ, w[p + "mix.uq"]
            if own:
                yield i, A.SW_K_NORM, w[p + "mix.dkv.norm"]
            yield i, A.SW_UK_T, w[p + "mix.uk"].reshape(a.heads, a.dim, a.kv_rank).transpose(1, 2).reshape(a.heads * a.kv_rank, a.dim)
            yield i, A.SW_UV, w[p + "mix.uv"]
        yield i, A.SW_O, w[p + "mix.o"]
        if f is not None:
            yield i, A.SW_NORM_MLP_POST, w[p + "norm2"]
            yield i, A.SW_NORM_MLP_POST_BIAS, w[p + "norm2.b"]
            yield i, A.SW_MLP_GATE_UP, torch.cat([w[p + "mlp.gate"], w[p + "mlp.up"]], 0)
            yield i, A.SW_MLP_DOWN, w[p + "mlp.down"]


def rudolix_weights(w: Dict[str, torch.Tensor], cfg) -> Iterator[Tuple[int, int, torch.Tensor]]:
    """(layer, b200_stack_weight kind, tensor) of a Rudolix checkpoint: `embed` (also the output projection), `final.norm[.b]`, per
    layer i the pre-norms `l<i>.norm1[.b]`, `l<i>.norm2[.b]`, the per-channel result scales `l<i>.ls1|ls2`, the stream coefficients
    `l<i>.hc1|hc2.in|out|mix` (packed in | out | mix), the input convolutions `l<i>.canon1|canon2`, the mixer `l<i>.mix.*` and the
    feed-forward `l<i>.mlp.*`.  Projections of the mixer's input are fused row-wise: attention q | k | v; delta q | k | v | g | b | a;
    the state-space mixer's `in` is one tensor already (z | x | B | C | dt).  The delta mixer's read-out weight is repeated for every
    head, its three convolution kernels are stacked; an expert's gate and up rows are stacked per expert; vectors go over in fp32."""
    from . import _abi as A
    from .config import AttentionSpec, HeadDeltaSpec
    yield 0, A.SW_EMBED, w["embed"]
    yield 0, A.SW_HEAD, w["embed"]
    yield 0, A.SW_FINAL_NORM, w["final.norm"]
    yield 0, A.SW_FINAL_NORM_BIAS, w["final.norm.b"]
    taps = cfg.canon_taps

    def hc(prefix):
        return torch.cat([w[prefix + ".in"].reshape(-1).float(), w[prefix + ".out"].reshape(-1).float(), w[prefix + ".mix"].reshape(-1).float()])

    for i, L in enumerate(cfg.layers):
        p, a, f = f"l{i}.", L.mixer, L.mlp
        yield i, A.SW_NORM_MIX_PRE, w[p + "norm1"]
        yield i, A.SW_NORM_MIX_PRE_BIAS, w[p + "norm1.b"]
        yield i, A.SW_SCALE_MIX, w[p + "ls1"]
        yield i, A.SW_HC_MIX, hc(p + "hc1")
        if taps >= 1:
            yield i, A.SW_CANON, w[p + "canon1"]
        if isinstance(a, AttentionSpec):
            yield i, A.SW_QKV, torch.cat([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"]], 0)
            yield i, A.SW_SINK, w[p + "mix.sink"]
        elif isinstance(a, HeadDeltaSpec):
            yield i, A.SW_QKV, torch.cat([w[p + "mix." + n] for n in ("q", "k", "v", "g", "b", "a")], 0)
            yield i, A.SW_CONV, torch.cat([w[p + "mix.q.conv"], w[p + "mix.k.conv"], w[p + "mix.v.conv"]], 0)
            yield i, A.SW_DECAY_BIAS, w[p + "mix.dt_bias"]
            yield i, A.SW_DECAY_LOG, w[p + "mix.A_log"]
            yield i, A.SW_HEAD_NORM, w[p + "mix.norm"].repeat(a.heads)
        else:
            yield i, A.SW_QKV, w[p + "mix.in"]
            yield i, A.SW_CONV, w[p + "mix.conv"]
            yield i, A.SW_CONV_BIAS, w[p + "mix.conv.b"]
            yield i, A.SW_DECAY_BIAS, w[p + "mix.dt_bias"]
            yield i, A.SW_DECAY_LOG, w[p + "mix.A_log"]
            yield i, A.SW_SKIP, w[p + "mix.D"]
            yield i, A.SW_HEAD_NORM, w[p + "mix.norm"]
        yield i, A.SW_O, w[p + "mix.o"]
        if f is None:
            continue
        yield i, A.SW_NORM_MLP_PRE, w[p + "norm2"]
        yield i, A.SW_NORM_MLP_PRE_BIAS, w[p + "norm2.b"]
        yield i, A.SW_SCALE_MLP, w[p + "ls2"]
        yield i, A.SW_HC_MLP, hc(p + "hc2")
        if taps >= 1:
            yield i, A.SW_CANON_MLP, w[p + "canon2"]
        if f.kind == "dense":
            yield i, A.SW_MLP_GATE_UP, w[p + "mlp.up"]
            yield i, A.SW_MLP_DOWN, w[p + "mlp.down"]
            yield i, A.SW_MLP_ACT, w[p + "mlp.act"]
        else:
            yield i, A.SW_ROUTER, w[p + "mlp.router"]
            yield i, A.SW_ROUTER_BIAS, w[p + "mlp.router.b"]
            yield i, A.SW_EXPERT_GATE_UP, torch.cat([t for e in range(f.experts) for t in (w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"])], 0)
            yield i, A.SW_EXPERT_DOWN, torch.cat([w[f"{p}mlp.e{e}.down"] for e in range(f.experts)], 0)


STACK_WEIGHT_MAPS = {"Bopilorn": bopilorn_weights, "Dupolorn": dupolorn_weights, "Futidra": futidra_weights, "Rudolix": rudolix_weights}
