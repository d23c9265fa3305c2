"""Model shapes (SURVEY.md §8 shape table) and the RoPE cache, product side.

The reference names models only by HF id (/root/reference/core/helm-charts/vllm/xeon-values.yaml:61,124;
gaudi-values.yaml:165); the shapes are the public HF configs of those ids.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class ModelConfig:
    name: str = "tiny"
    hidden: int = 512
    n_layers: int = 2
    n_q_heads: int = 4
    n_kv_heads: int = 1
    head_dim: int = 128
    intermediate: int = 1024
    vocab: int = 1024
    qkv_bias: bool = False
    rope_theta: float = 500000.0
    rope_llama3: bool = True
    rms_eps: float = 1e-5
    max_pos: int = 32768
    # llama3 rope scaling (config.json rope_scaling): Llama-3.1 = 8 / 1 / 4 / 8192, Llama-3.2 uses factor 32
    rope_factor: float = 8.0
    rope_low_freq: float = 1.0
    rope_high_freq: float = 4.0
    rope_orig_max_pos: int = 8192

    def to_dict(self):
        return asdict(self)

    @property
    def q_size(self):
        return self.n_q_heads * self.head_dim

    @property
    def kv_size(self):
        return self.n_kv_heads * self.head_dim

    def decode_params(self) -> int:
        h, L, I, V = self.hidden, self.n_layers, self.intermediate, self.vocab
        return L * (h * (self.q_size + 2 * self.kv_size) + self.q_size * h + 3 * h * I) + V * h

    def weight_bytes(self) -> int:
        return 2 * self.decode_params()

    def kv_bytes_per_token(self) -> int:
        return 2 * self.n_kv_heads * self.head_dim * 2 * self.n_layers


MODELS: Dict[str, ModelConfig] = {
    "tiny": ModelConfig(),
    # ONE rank's share of Llama-3.1-70B at tensor-parallel 8 as a model of its own (8 of 64 q heads, 1 of 8 kv heads, 1/8 of
    # the MLP and of the vocabulary, full hidden size): the kernels of a TP8 step minus its collectives, for single-GPU
    # profiling (ncu must not wrap a multi-rank command)
    "llama-3.1-70b-tp8-shard": ModelConfig(name="llama-3.1-70b-tp8-shard", hidden=8192, n_layers=80, n_q_heads=8, n_kv_heads=1,
                                           intermediate=3584, vocab=16032, max_pos=131072),
    # the 70B head ratio (G = 8) over 8 kv heads on a small body: shards over 2, 4 and 8 tensor-parallel ranks
    "tiny-g8x8": ModelConfig(name="tiny-g8x8", hidden=1024, n_layers=2, n_q_heads=64, n_kv_heads=8, intermediate=4096,
                             vocab=4096),
    "meta-llama/Llama-3.1-8B-Instruct": ModelConfig(
        name="meta-llama/Llama-3.1-8B-Instruct", hidden=4096, n_layers=32, n_q_heads=32, n_kv_heads=8,
        intermediate=14336, vocab=128256, max_pos=131072),
    "deepseek-ai/DeepSeek-R1-Distill-Qwen-32B": ModelConfig(
        name="deepseek-ai/DeepSeek-R1-Distill-Qwen-32B", hidden=5120, n_layers=64, n_q_heads=40, n_kv_heads=8,
        intermediate=27648, vocab=152064, qkv_bias=True, rope_theta=1e6, rope_llama3=False, max_pos=131072),
    "meta-llama/Llama-3.1-70B-Instruct": ModelConfig(
        name="meta-llama/Llama-3.1-70B-Instruct", hidden=8192, n_layers=80, n_q_heads=64, n_kv_heads=8,
        intermediate=28672, vocab=128256, max_pos=131072),
}
ALIASES = {"llama-3.1-8b": "meta-llama/Llama-3.1-8B-Instruct",
           "qwen2-32b": "deepseek-ai/DeepSeek-R1-Distill-Qwen-32B",
           "llama-3.1-70b": "meta-llama/Llama-3.1-70B-Instruct"}


def get_config(name: str) -> ModelConfig:
    return MODELS[ALIASES.get(name, name)]


def from_hf_config(path: str) -> ModelConfig:
    """Read an HF config.json (the /data HF_HOME cache of the chart, templates/configmap.yaml:18-21)."""
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    rs = c.get("rope_scaling") or c.get("rope_parameters") or {}
    # what the kernels implement, and nothing else: a config outside it must fail here, not produce wrong logits
    mt = c.get("model_type", "llama")
    if mt not in ("llama", "qwen2"):
        raise ValueError(f"unsupported model_type {mt!r} (llama and qwen2 decoder stacks only)")
    rope_type = rs.get("rope_type", rs.get("type")) or "default"
    if rope_type not in ("default", "llama3"):
        raise ValueError(f"unsupported rope scaling type {rope_type!r} (plain and llama3 RoPE only)")
    if c.get("use_sliding_window") and c.get("sliding_window"):
        raise ValueError("sliding-window attention is not supported")
    head_dim = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]
    if head_dim != 128:
        raise ValueError(f"head_dim {head_dim} is not supported (the attention kernels are built for 128)")
    extra = {}
    if rope_type == "llama3":
        extra = dict(rope_factor=float(rs.get("factor", 8.0)), rope_low_freq=float(rs.get("low_freq_factor", 1.0)),
                     rope_high_freq=float(rs.get("high_freq_factor", 4.0)),
                     rope_orig_max_pos=int(rs.get("original_max_position_embeddings", 8192)))
    return ModelConfig(**extra, 
        name=c.get("_name_or_path", path), hidden=c["hidden_size"], n_layers=c["num_hidden_layers"],
        n_q_heads=c["num_attention_heads"], n_kv_heads=c.get("num_key_value_heads", c["num_attention_heads"]),
        head_dim=head_dim,
        intermediate=c["intermediate_size"], vocab=c["vocab_size"],
        qkv_bias=bool(c.get("attention_bias", False)) or c.get("model_type") == "qwen2",
        rope_theta=float(c.get("rope_theta", rs.get("rope_theta", 10000.0))),
        rope_llama3=(rope_type == "llama3"),
        rms_eps=float(c.get("rms_norm_eps", 1e-5)), max_pos=int(c.get("max_position_embeddings", 8192)))


def rope_cos_sin(cfg: ModelConfig, max_pos: Optional[int] = None) -> torch.Tensor:
    """[max_pos, head_dim] bf16 cache, cos | sin, computed on the CPU in fp32 then rounded
    (stored-bf16 is a rounding point: [V22] rotary_embedding/base.py:58-63; llama3 scaling
    llama3_rope.py:33-54)."""
    d = cfg.head_dim
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    if cfg.rope_llama3:
        factor, low, high, orig = cfg.rope_factor, cfg.rope_low_freq, cfg.rope_high_freq, cfg.rope_orig_max_pos
        wavelen = 2 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        mid = (1 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, mid))
    t = torch.arange(max_pos or cfg.max_pos, dtype=torch.float32)
    fr = torch.outer(t, inv)
    return torch.cat((fr.cos(), fr.sin()), dim=-1).to(torch.bfloat16)


# ---- models described layer by layer ------------------------------------------------------------------------------------
# The chart's model list is Llama / Qwen2 only; designs whose layers carry their own sizes and mechanisms are read from the
# layer list of their config.json into the descriptors of include/b200_decode.h (b200_stack_layer).

@dataclass
class RotarySpec:
    """Rotation of the leading `dims` dimensions of a head in the interleaved pair layout (2i, 2i+1), pair i turning by
    position * f_i with f_i = base^(-2i/dims).  With YaRN scaling (factor, original, fast, slow) the frequencies are
    blended between f_i and f_i / factor by a linear ramp over the pair index and cos/sin are multiplied by
    0.1 ln(factor) + 1.  kind "bands" scales by wavelength instead: with l = 2 pi / f_i, pairs with l < original / fast keep
    f_i, pairs with l > original / slow get f_i / factor, and those between are blended linearly in original / l; cos/sin keep
    their magnitude."""
    base: float
    dims: int
    factor: float = 1.0
    original: int = 0
    fast: float = 0.0
    slow: float = 0.0
    scaled: bool = False
    kind: str = "yarn"

    def key(self) -> tuple:
        return (self.base, self.dims, self.factor, self.original, self.fast, self.slow, self.scaled, self.kind)

    def frequencies(self) -> Tuple[torch.Tensor, float]:
        """(f[dims/2] float64, magnitude factor)."""
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = torch.tensor(self.base, dtype=torch.float64) ** (-2.0 * i / self.dims)
        if not self.scaled:
            return f, 1.0
        if self.kind == "bands":
            lam = 2.0 * math.pi / f
            blend = (self.original / lam - self.slow) / (self.fast - self.slow)
            mid = (1.0 - blend) * f / self.factor + blend * f
            out = torch.where(lam < self.original / self.fast, f, torch.where(lam > self.original / self.slow, f / self.factor, mid))
            return out, 1.0

        def pair_of(turns: float) -> float:   # the (fractional) pair index whose wavelength makes `turns` turns over `original` positions
            return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo = max(math.floor(pair_of(self.fast)), 0)
        hi = min(math.ceil(pair_of(self.slow)), self.dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp), 0.1 * math.log(self.factor) + 1.0

    def table(self, n_pos: int) -> torch.Tensor:
        """[n_pos][2][dims/2] fp32: cos row and sin row of every position (angles in float64, rounded once)."""
        f, mag = self.frequencies()
        a = torch.arange(n_pos, dtype=torch.float64)[:, None] * f[None, :]
        return torch.stack((a.cos() * mag, a.sin() * mag), dim=1).to(torch.float32).contiguous()


@dataclass
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotarySpec] = None       # q/k rotation (None: none)
    value_rot: Optional[RotarySpec] = None  # values rotate by their position, outputs turn back by the query's (None: off)
    window: int = 0                        # positions a query sees, its own included (0: all)
    head_norm: bool = False                # q/k RMS norm per head with one weight of `dim` entries (else over the whole projection)
    value_is_key: bool = False             # no value projection: a value is the key projection before norm and rotation
    sink_one: bool = False                 # one more unit in the softmax denominator
    qk_norm: bool = True                   # False: plain q/k/v projections, no norm of q and k at all
    rot_half: bool = False                 # rotated dimension i pairs with i + rot.dims / 2 (else 2i with 2i + 1)
    sink: bool = False                     # a learned per-head term exp(sink) in the softmax denominator


@dataclass
class MoESpec:
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1


@dataclass
class StackLayerSpec:
    mixer: object                     # AttentionSpec | LatentAttentionSpec | ChannelDeltaSpec | HeadDeltaSpec | StateSpaceSpec
    mlp: Optional[object] = None      # MoESpec | FeedForwardSpec


@dataclass
class BopilornConfig:
    """Bopilorn: decoder-only; every layer is [layer norm, attention, layer norm] + [layer norm, routed experts, layer norm]
    over an fp32 residual stream.  Attention: grouped-query, RMS norm of q and of k over the whole projection, partial
    interleaved rotary with YaRN scaling, unit-RMS values rotated by their position with the output turned back, a score
    scale of its own.  Experts: softmax router with a choice bias, group-limited top-k, unrenormalised weights."""
    name: str = "bopilorn"
    width: int = 256
    vocab: int = 1024
    embed_scale: float = 1.0
    norm_eps: float = 1e-5
    layers: List[StackLayerSpec] = field(default_factory=list)
    architecture: str = "Bopilorn"

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def to_dict(self):
        return asdict(self)

    def decode_params(self) -> int:
        """Weights one decode row touches (chosen experts only)."""
        n = self.vocab * self.width
        for L in self.layers:
            a = L.mixer
            n += self.width * (a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)) + a.heads * a.vdim * self.width
            if L.mlp:
                n += L.mlp.experts * self.width + L.mlp.top * 3 * L.mlp.ff * self.width
        return n

    def weight_bytes(self) -> int:
        n = 2 * self.vocab * self.width
        for L in self.layers:
            a = L.mixer
            n += self.width * (a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)) + a.heads * a.vdim * self.width
            if L.mlp:
                n += L.mlp.experts * (self.width + 3 * L.mlp.ff * self.width)
        return 2 * n

    def kv_bytes_per_token(self, f32: bool = False) -> int:
        return sum(L.mixer.kv_heads * (L.mixer.dim + L.mixer.vdim) for L in self.layers) * (4 if f32 else 2)

    @staticmethod
    def from_dict(c: dict, name: str = "bopilorn") -> "BopilornConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            if l.get("type") != "attention":
                raise ValueError(f"layer {i}: unsupported mixer type {l.get('type')!r} (this design has 'attention')")
            m = l["mixer"]
            rot = vrot = None
            r = m.get("rot")
            if r:
                sc = r.get("scaling") or None
                rot = RotarySpec(base=float(r["base"]), dims=int(r["dims"]))
                if sc:
                    rot = RotarySpec(base=float(r["base"]), dims=int(r["dims"]), factor=float(sc["factor"]),
                                     original=int(sc["original"]), fast=float(sc["fast"]), slow=float(sc["slow"]), scaled=True)
                vrot = RotarySpec(base=float(r["base"]), dims=int(m["vdim"]))   # values: every pair, never scaled
                if rot.dims == 0:
                    rot = None
            att = AttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), rot=rot, value_rot=vrot)
            mlp = None
            f = l.get("mlp")
            if f:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unsupported feed-forward kind {f.get('kind')!r}")
                ro, g = f["router"], (f["router"].get("groups") or {})
                mlp = MoESpec(experts=int(ro["experts"]), top=int(ro["top"]), ff=int(f["expert"]["ff"]),
                              groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))))
            layers.append(StackLayerSpec(mixer=att, mlp=mlp))
        return BopilornConfig(name=name, width=int(c["width"]), vocab=int(c["vocab"]),
                              embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                              norm_eps=float((c.get("norm") or {}).get("eps", 1e-5)), layers=layers)


# ---- Dupolorn ---------------------------------------------------------------------------------------------------------------
@dataclass
class LatentAttentionSpec:
    """Attention over one cached latent vector per token: per head `dim` plain and `rot_dim` rotated query/key dimensions, the
    rotated key part shared by all heads, keys and values expanded from the latent of `kv_rank` dimensions.  sink: a learned
    per-head term in the softmax denominator; gate: sigmoid output gate read from the mixer's input."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[RotarySpec] = None
    sink: bool = False
    gate: bool = False
    kind: str = "latent"
    q_rank: int = 0                        # > 0: queries pass a normed latent of this size
    window: int = 0                        # positions a query sees, its own included (0: all)
    head_gate: bool = False                # one sigmoid gate per head (instead of one per output)
    kv_from: Optional[int] = None          # the layer whose cached latent rows this layer reads (None: its own)


@dataclass
class MLSTMSpec:
    """Matrix-memory recurrence: `heads` heads of key size `dim` and value size `vdim`; the log gates are capped by
    cap * tanh(z / cap)."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float
    kind: str = "mlstm"


@dataclass
class FeedForwardSpec:
    """kind "dense": down(act(gate h) * (up h)).  kind "moe": `experts` ungated experts down(act(up h)) of which a token uses
    `top`, chosen by sigmoid scores that scale the expert's input; `shared_ff` > 0 adds one expert every token uses."""
    kind: str
    ff: int
    act: str = "gelu_tanh"
    experts: int = 0
    top: int = 0
    shared_ff: int = 0
    gated: Optional[bool] = None           # None: the design's default shape (dense gated, experts ungated)
    limit: float = 0.0                     # act "swiglu_clamp": min(gate, limit) * sigmoid(1.702 gate) * (clamp(up, +-limit) + 1)
    router: str = ""                       # "chosen_softmax": bias inside the logits, weights = softmax over the chosen logits


@dataclass
class ParallelLayerSpec:
    mixer: object                     # LatentAttentionSpec | MLSTMSpec
    mlp: Optional[FeedForwardSpec] = None


@dataclass
class DupolornConfig:
    """Dupolorn: decoder-only, layers in the parallel form x += mixer(conv(norm1 x)) + ff(norm2 x) with one-number RMS norms, a
    causal per-channel input convolution, a depth-weighted average over all layer results, a hashed bigram embedding and
    capped logits.  Mixers: latent attention (plain, or with sink and output gate) and mLSTM."""
    name: str = "dupolorn"
    width: int = 256
    vocab: int = 1024
    embed_scale: float = 1.0
    norm_eps: float = 1e-6
    canon_taps: int = 0
    bigram_buckets: int = 0
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    logit_softcap: float = 0.0
    depth_avg: bool = True
    layers: List[ParallelLayerSpec] = field(default_factory=list)
    architecture: str = "Dupolorn"

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @property
    def needs_state(self) -> bool:
        return self.canon_taps > 1 or self.bigram_buckets > 0 or any(isinstance(L.mixer, MLSTMSpec) for L in self.layers)

    def to_dict(self):
        return asdict(self)

    def _layer_params(self, L: ParallelLayerSpec, active_only: bool) -> int:
        W, a, n = self.width, L.mixer, 0
        if isinstance(a, MLSTMSpec):
            n += W * (2 * a.heads * a.dim + 2 * a.heads * a.vdim + 2 * a.heads) + a.heads * a.vdim * W
        else:
            n += W * (a.heads * (a.dim + a.rot_dim) + a.kv_rank + a.rot_dim + (a.heads * a.vdim if a.gate else 0))
            n += a.heads * a.kv_rank * (a.dim + a.vdim) + a.heads * a.vdim * W
        f = L.mlp
        if f and f.kind == "dense":
            n += 3 * f.ff * W
        elif f:
            n += f.experts * W + (f.top if active_only else f.experts) * 2 * f.ff * W + 2 * f.shared_ff * W
        return n

    def decode_params(self) -> int:
        """Weights one decode row touches (chosen experts only)."""
        return self.vocab * self.width + sum(self._layer_params(L, True) for L in self.layers)

    def weight_bytes(self) -> int:
        return 2 * (2 * self.vocab * self.width + (self.bigram_buckets + 1) * self.width * (1 if self.bigram_buckets else 0)
                    + sum(self._layer_params(L, False) for L in self.layers))

    def kv_bytes_per_token(self, f32: bool = False) -> int:
        return sum(L.mixer.kv_rank + L.mixer.rot_dim for L in self.layers if isinstance(L.mixer, LatentAttentionSpec)) * (4 if f32 else 2)

    @staticmethod
    def from_dict(c: dict, name: str = "dupolorn") -> "DupolornConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            kind, m = l.get("type"), l["mixer"]
            if kind in ("latent_attention", "latent_attention_2"):
                rot = None
                r = m.get("rot")
                if r and int(r["dims"]) > 0 and int(m.get("rot_dim", 0)) > 0:
                    rot = RotarySpec(base=float(r["base"]), dims=int(r["dims"]))
                    if rot.dims > int(m["rot_dim"]) or rot.dims % 2:
                        raise ValueError(f"layer {i}: {rot.dims} rotated dimensions in a part of {m['rot_dim']}")
                second = kind == "latent_attention_2"
                mixer = LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m.get("rot_dim", 0)), vdim=int(m["vdim"]),
                                            kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot=rot, sink=second, gate=second)
            elif kind == "mlstm":
                mixer = MLSTMSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), gate_cap=float(m["gate_cap"]))
            else:
                raise ValueError(f"layer {i}: unsupported mixer type {kind!r} (this design has latent_attention, latent_attention_2, mlstm)")
            mlp = None
            f = l.get("mlp")
            if f:
                if f.get("kind") == "dense":
                    mlp = FeedForwardSpec(kind="dense", ff=int(f["ff"]), act="gelu_tanh")
                elif f.get("kind") == "moe":
                    sh = f.get("shared") or {}
                    mlp = FeedForwardSpec(kind="moe", ff=int(f["expert"]["ff"]), act="relu2", experts=int(f["router"]["experts"]),
                                          top=int(f["router"]["top"]), shared_ff=int(sh.get("ff", 0)))
                else:
                    raise ValueError(f"layer {i}: unsupported feed-forward kind {f.get('kind')!r}")
            layers.append(ParallelLayerSpec(mixer=mixer, mlp=mlp))
        emb = c.get("embedding") or {}
        bg = emb.get("bigram") or {}
        return DupolornConfig(name=name, width=int(c["width"]), vocab=int(c["vocab"]), embed_scale=float(emb.get("scale", 1.0)),
                              norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)), canon_taps=int((c.get("canon") or {}).get("taps", 0)),
                              bigram_buckets=int(bg.get("buckets", 0)), bigram_mul_prev=int(bg.get("mul_prev", 0)),
                              bigram_mul_cur=int(bg.get("mul_cur", 0)), logit_softcap=float(c.get("logit_softcap") or 0.0), layers=layers)


# ---- Futidra ----------------------------------------------------------------------------------------------------------------
@dataclass
class ChannelDeltaSpec:
    """Delta-rule recurrence with one decay per head and key channel: q/k in `kv_heads` heads of `dim`, values in `heads` heads of
    `vdim`, a causal convolution of `conv` taps on q, k and v, two-step projections of inner sizes `decay_rank` / `gate_rank` for
    the decays and the output gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int
    kind: str = "delta"


@dataclass
class FutidraConfig:
    """Futidra: decoder-only, norm after the sum: x = LN(alpha x + mixer(x)), x = LN(alpha x + ff(x)) with layer norms that have
    weight and bias.  Mixers: windowed grouped-query attention whose values are its keys (per-head q/k norms, partial pair
    rotation with band-scaled frequencies, one more unit in the softmax denominator); windowed latent attention without positions
    (query latent, per-head output gate, optionally reading another layer's cached latents); the channel-decay delta rule.
    Dense relu-gated feed-forwards; the output projection is the embedding table."""
    name: str = "futidra"
    width: int = 256
    vocab: int = 1024
    norm_eps: float = 1e-6
    postln_alpha: float = 1.0
    layers: List[StackLayerSpec] = field(default_factory=list)
    architecture: str = "Futidra"
    embed_scale: float = 1.0

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @property
    def needs_state(self) -> bool:
        return any(isinstance(L.mixer, ChannelDeltaSpec) for L in self.layers)

    def to_dict(self):
        return asdict(self)

    def _layer_params(self, L) -> int:
        W, a = self.width, L.mixer
        if isinstance(a, ChannelDeltaSpec):
            n = W * (2 * a.kv_heads * a.dim + a.heads * a.vdim + a.heads + a.decay_rank + a.gate_rank)
            n += a.heads * a.dim * a.decay_rank + a.heads * a.vdim * a.gate_rank + a.heads * a.vdim * W
        elif isinstance(a, LatentAttentionSpec):
            n = W * (a.q_rank + (0 if a.kv_from is not None else a.kv_rank) + a.heads) + a.heads * a.dim * a.q_rank
            n += a.heads * a.kv_rank * (a.dim + a.vdim) + a.heads * a.vdim * W
        else:
            n = W * (a.heads + a.kv_heads) * a.dim + a.heads * a.vdim * W
        if L.mlp is not None:
            n += 3 * L.mlp.ff * W
        return n

    def decode_params(self) -> int:
        return self.vocab * self.width + sum(self._layer_params(L) for L in self.layers)

    def weight_bytes(self) -> int:
        return 2 * self.decode_params()

    def kv_bytes_per_token(self, f32: bool = False) -> int:
        n = 0
        for L in self.layers:
            a = L.mixer
            if isinstance(a, AttentionSpec):
                n += a.kv_heads * (a.dim + a.vdim)
            elif isinstance(a, LatentAttentionSpec) and a.kv_from is None:
                n += a.kv_rank
        return n * (4 if f32 else 2)

    @staticmethod
    def from_dict(c: dict, name: str = "futidra", shapes: Optional[Dict[str, list]] = None) -> "FutidraConfig":
        """`shapes` (tensor name -> shape, from the checkpoint) gives the sizes config.json does not name: the inner sizes of the
        delta mixer's two-step projections."""
        layers = []
        for i, l in enumerate(c["layers"]):
            kind, m = l.get("type"), l["mixer"]
            window = int((m.get("mask") or {}).get("size", 0))
            if kind == "attention":
                rot = None
                r = m.get("rot")
                if r and int(r["dims"]) > 0:
                    sc = r.get("scaling") or None
                    if sc:
                        rot = RotarySpec(base=float(r["base"]), dims=int(r["dims"]), factor=float(sc["factor"]), original=int(sc["original"]),
                                         fast=float(sc["high"]), slow=float(sc["low"]), scaled=True, kind="bands")
                    else:
                        rot = RotarySpec(base=float(r["base"]), dims=int(r["dims"]))
                    if rot.dims % 2 or rot.dims > int(m["dim"]):
                        raise ValueError(f"layer {i}: {rot.dims} rotated dimensions in heads of {m['dim']}")
                mixer = AttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                      vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), rot=rot, window=window, head_norm=True,
                                      value_is_key=True, sink_one=True)
                if mixer.vdim > mixer.dim:
                    raise ValueError(f"layer {i}: values of {mixer.vdim} dimensions cannot be keys of {mixer.dim}")
            elif kind == "latent_attention":
                src = m.get("kv_from")
                mixer = LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=0, vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                            scale=float(m["scale"]), q_rank=int(m["q_rank"]), window=window, head_gate=True,
                                            kv_from=None if src is None else int(src))
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    if not (0 <= j < i) or not isinstance(layers[j].mixer, LatentAttentionSpec) or layers[j].mixer.kv_from is not None \
                            or layers[j].mixer.kv_rank != mixer.kv_rank:
                        raise ValueError(f"layer {i}: kv_from {j} is not an earlier latent layer with a latent of its own of size {mixer.kv_rank}")
            elif kind == "channel_delta":
                ranks = []
                for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if shapes is not None and tensor in shapes:
                        ranks.append(int(shapes[tensor][0]))
                    elif key in m:
                        ranks.append(int(m[key]))
                    else:
                        raise ValueError(f"layer {i}: the size of {tensor} is needed (checkpoint shapes or mixer[{key!r}])")
                mixer = ChannelDeltaSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                         conv=int(m.get("conv", 1)), decay_rank=ranks[0], gate_rank=ranks[1])
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} q/k heads")
            else:
                raise ValueError(f"layer {i}: unsupported mixer type {kind!r} (this design has attention, latent_attention, channel_delta)")
            mlp = None
            f = l.get("mlp")
            if f:
                if f.get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: unsupported feed-forward kind {f.get('kind')!r}")
                mlp = FeedForwardSpec(kind="dense", ff=int(f["ff"]), act="relu")
            layers.append(StackLayerSpec(mixer=mixer, mlp=mlp))
        return FutidraConfig(name=name, width=int(c["width"]), vocab=int(c["vocab"]), norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)),
                             postln_alpha=float(c.get("postln_alpha", 1.0)), layers=layers)


# ---- Rudolix ----------------------------------------------------------------------------------------------------------------
@dataclass
class HeadDeltaSpec:
    """Delta-rule recurrence with ONE decay per head: q/k in `kv_heads` heads of `dim`, values in `heads` heads of `vdim`, a causal
    convolution of `conv` taps and silu on q, k and v, beta and the decay from single projections, read-out times a weight shared by
    the heads and silu of a gate projection."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    kind: str = "head_delta"


@dataclass
class StateSpaceSpec:
    """State-space recurrence (scalar decay per head): `heads` heads of `vdim` channels, `groups` shared B / C vectors of `state`
    entries, a causal convolution of `conv` taps with bias over x | B | C, the gated output normalised in `norm_groups` parts."""
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int
    kind: str = "ssd"


@dataclass
class RudolixConfig:
    """Rudolix: decoder-only, pre-norm sublayers over `streams` copies of the residual (hyper-connections): a sublayer reads a
    weighted sum of the streams through a layer norm with weight and bias and a causal per-channel input convolution, and its result,
    scaled per channel and by `residual_mult`, is dealt back to every stream while the streams are mixed by a matrix.  Mixers:
    grouped-query attention with half-layout partial rotation and a learned sink, the gated delta rule with one decay per head, the
    Mamba-2 state-space recurrence.  Feed-forwards: ungated dense with a polynomial of unit-RMS powers, or routed experts (softmax over
    the chosen logits, clamped gated experts).  The output projection is the embedding table."""
    name: str = "rudolix"
    width: int = 256
    vocab: int = 1024
    embed_scale: float = 1.0
    norm_eps: float = 1e-6
    canon_taps: int = 0
    streams: int = 1
    residual_mult: float = 1.0
    layers: List[StackLayerSpec] = field(default_factory=list)
    architecture: str = "Rudolix"

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @property
    def needs_state(self) -> bool:
        return self.canon_taps > 1 or any(isinstance(L.mixer, (HeadDeltaSpec, StateSpaceSpec)) for L in self.layers)

    def to_dict(self):
        return asdict(self)

    def mixer_rows(self, a) -> int:
        """Rows of the fused projection of a mixer's input."""
        if isinstance(a, HeadDeltaSpec):
            return 2 * a.kv_heads * a.dim + 2 * a.heads * a.vdim + 2 * a.heads
        if isinstance(a, StateSpaceSpec):
            return 2 * a.heads * a.vdim + 2 * a.groups * a.state + a.heads
        return a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)

    def _layer_params(self, L, active_only: bool) -> int:
        W, a = self.width, L.mixer
        n = W * self.mixer_rows(a) + a.heads * a.vdim * W
        f = L.mlp
        if f is not None and f.kind == "dense":
            n += 2 * f.ff * W
        elif f is not None:
            n += f.experts * W + (f.top if active_only else f.experts) * 3 * f.ff * W
        return n

    def decode_params(self) -> int:
        """Weights one decode row touches (chosen experts only)."""
        return self.vocab * self.width + sum(self._layer_params(L, True) for L in self.layers)

    def weight_bytes(self) -> int:
        return 2 * (self.vocab * self.width + sum(self._layer_params(L, False) for L in self.layers))

    def kv_bytes_per_token(self, f32: bool = False) -> int:
        return sum(L.mixer.kv_heads * (L.mixer.dim + L.mixer.vdim) for L in self.layers if isinstance(L.mixer, AttentionSpec)) * (4 if f32 else 2)

    @staticmethod
    def from_dict(c: dict, name: str = "rudolix") -> "RudolixConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            kind, m = l.get("type"), l["mixer"]
            if kind == "attention":
                rot = None
                r = m.get("rot")
                if r and int(r.get("dims", 0)) > 0:
                    rot = RotarySpec(base=float(r["base"]), dims=int(r["dims"]))
                    if rot.dims % 2 or rot.dims > int(m["dim"]):
                        raise ValueError(f"layer {i}: {rot.dims} rotated dimensions in heads of {m['dim']}")
                mixer = AttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                      vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), rot=rot, qk_norm=False, rot_half=True, sink=True)
            elif kind == "delta":
                mixer = HeadDeltaSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                      conv=int(m.get("conv", 1)))
            elif kind == "mamba2":
                mixer = StateSpaceSpec(heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]), groups=int(m.get("groups", 1)),
                                       norm_groups=int(m.get("norm_groups", 1)), conv=int(m.get("conv", 1)))
                if mixer.heads % mixer.groups or (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ValueError(f"layer {i}: {mixer.heads} heads of {mixer.vdim} over {mixer.groups} groups and {mixer.norm_groups} norm parts")
            else:
                raise ValueError(f"layer {i}: unsupported mixer type {kind!r} (this design has attention, delta, mamba2)")
            if not isinstance(mixer, StateSpaceSpec) and mixer.heads % mixer.kv_heads:
                raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key heads")
            mlp = None
            f = l.get("mlp")
            if f:
                if f.get("kind") == "dense":
                    mlp = FeedForwardSpec(kind="dense", ff=int(f["ff"]), act="polynorm", gated=False)
                elif f.get("kind") == "moe":
                    mlp = FeedForwardSpec(kind="moe", ff=int(f["expert"]["ff"]), act="swiglu_clamp", experts=int(f["router"]["experts"]),
                                          top=int(f["router"]["top"]), gated=True, limit=float(f["expert"]["limit"]), router="chosen_softmax")
                    if not 0 < mlp.top <= mlp.experts:
                        raise ValueError(f"layer {i}: top {mlp.top} of {mlp.experts} experts")
                else:
                    raise ValueError(f"layer {i}: unsupported feed-forward kind {f.get('kind')!r}")
            layers.append(StackLayerSpec(mixer=mixer, mlp=mlp))
        streams = int(c.get("streams", 1))
        if not 1 <= streams <= 8:
            raise ValueError(f"{streams} residual streams (1 to 8 are served)")
        return RudolixConfig(name=name, width=int(c["width"]), vocab=int(c["vocab"]), embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                             norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)), canon_taps=int((c.get("canon") or {}).get("taps", 0)),
                             streams=streams, residual_mult=float(c.get("residual_mult", 1.0)), layers=layers)


def checkpoint_shapes(path: str) -> Dict[str, list]:
    """Tensor name -> shape of every *.safetensors file under `path`, from the files' headers alone (8-byte little-endian
    length, then that many bytes of JSON)."""
    import glob
    import struct
    out: Dict[str, list] = {}
    for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with open(fn, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            head = json.loads(f.read(n))
        for k, v in head.items():
            if k != "__metadata__":
                out[k] = list(v["shape"])
    return out


# config.json "architecture" -> reader.  HF-style configs (model_type) go through from_hf_config.
ARCHITECTURES = {"Bopilorn": BopilornConfig.from_dict, "Dupolorn": DupolornConfig.from_dict, "Futidra": FutidraConfig.from_dict,
                 "Rudolix": RudolixConfig.from_dict}
NEEDS_SHAPES = {"Futidra"}   # readers that take the checkpoint's tensor shapes for sizes config.json does not name


def load_model_config(path: str):
    """The model class is chosen by config.json: an `architecture` of the registry above, else an HF decoder config."""
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    arch = c.get("architecture")
    if arch is not None:
        if arch not in ARCHITECTURES:
            raise ValueError(f"unsupported architecture {arch!r} (known: {sorted(ARCHITECTURES)})")
        if arch in NEEDS_SHAPES:
            return ARCHITECTURES[arch](c, name=c.get("_name_or_path", path), shapes=checkpoint_shapes(path))
        return ARCHITECTURES[arch](c, name=c.get("_name_or_path", path))
    return from_hf_config(path)


def is_stack_config(cfg) -> bool:
    return hasattr(cfg, "layers") and not isinstance(cfg, ModelConfig)
