"""Futidra in plain float64 torch, one function per mechanism, for the tests.  Nothing here is shared with the package:
the configuration dictionary is read directly and every step is written token by token or as a dense matrix, slowly.

Notation: T tokens, W width, H query heads, G key/value heads, d key size, e value size, r latent size.
A weight M is stored [out, in] and applied as x @ M.T.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i/n) for the n/2 pairs, then the three-band wavelength rule when `scaling` is given."""
    n = int(rot["dims"])
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / n) for i in range(n // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = f.clone()
    for i in range(n // 2):
        lam = 2.0 * math.pi / float(f[i])
        if lam < orig / high:
            continue
        if lam > orig / low:
            out[i] = f[i] / factor
        else:
            s = (orig / lam - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, d]; neighbours (2i, 2i+1) of the leading 2 * len(freqs) dimensions turn by pos * freqs[i]."""
    n = 2 * freqs.numel()
    a = pos.to(F64)[:, None, None] * freqs[None, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def window_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: row i sees column j iff 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def windowed_softmax(scores: torch.Tensor, mask: torch.Tensor, extra_one: bool) -> torch.Tensor:
    """Row-wise weights exp(s_j) / (sum exp(s_j) [+ 1]) over the visible columns."""
    s = scores.masked_fill(~mask, float("-inf"))
    m = s.max(-1, keepdim=True).values
    if extra_one:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if extra_one:
        den = den + torch.exp(-m)
    return e / den


def attention_mixer(h, p: Dict[str, torch.Tensor], m: dict, eps: float):
    """Grouped-query attention whose values are the raw key projections; per-head RMS norm of q and k, partial pair rotation,
    sliding window, one extra unit in the softmax denominator."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ p["q"].T).reshape(T, H, d)
    kraw = (h @ p["k"].T).reshape(T, G, d)
    v = kraw[..., :e]
    q = rms_norm(q, p["q.norm"], eps)
    k = rms_norm(kraw, p["k.norm"], eps)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        fr = rotary_frequencies(rot)
        pos = torch.arange(T)
        q, k = rotate_pairs(q, pos, fr), rotate_pairs(k, pos, fr)
    mask = window_mask(T, int(m["mask"]["size"]))
    out = torch.zeros(T, H, e, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        out[:, hh] = windowed_softmax(s, mask, True) @ v[:, g]
    return out.reshape(T, H * e) @ p["o"].T


def latent_of(h, p, eps):
    return rms_norm(h @ p["dkv"].T, p["dkv.norm"], eps)


def latent_mixer(h, p, m: dict, eps: float, c: torch.Tensor):
    """Attention without positions over keys and values expanded from the latent rows c [T, r] (this layer's or another's);
    queries through a normed latent of their own; per-head sigmoid gate read from h."""
    T = h.shape[0]
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).reshape(T, H, d)
    k = (c @ p["uk"].T).reshape(T, H, d)
    v = (c @ p["uv"].T).reshape(T, H, e)
    gate = torch.sigmoid(h @ p["g"].T)          # [T, H]
    mask = window_mask(T, int(m["mask"]["size"]))
    out = torch.zeros(T, H, e, dtype=F64)
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh].T) * float(m["scale"])
        out[:, hh] = (windowed_softmax(s, mask, False) @ v[:, hh]) * gate[:, hh:hh + 1]
    return out.reshape(T, H * e) @ p["o"].T


def causal_conv_silu(x, w):
    """x [T, C], w [C, taps] (last column = current token), zeros before the start; then silu."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j][None, :]
    return y * torch.sigmoid(y)


def channel_delta_mixer(h, p, m: dict, eps: float, state: Optional[dict] = None):
    """Delta rule with one decay per head and key channel.  `state` (optional, updated in place): {"S": [H, d, e],
    "tail": [taps - 1, channels of q | k | v]} so that a sequence can be fed in portions."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    taps = int(m["conv"])
    raw = torch.cat([h @ p["q"].T, h @ p["k"].T, h @ p["v"].T], -1)
    wc = torch.cat([p["q.conv"], p["k.conv"], p["v.conv"]], 0)
    if state is not None and "tail" in state:
        full = torch.cat([state["tail"], raw], 0)
    else:
        full = torch.cat([torch.zeros(taps - 1, raw.shape[1], dtype=F64), raw], 0)
    conv = torch.zeros_like(raw)
    for j in range(taps):
        conv = conv + full[j:j + T] * wc[:, j][None, :]
    conv = conv * torch.sigmoid(conv)
    if state is not None:
        state["tail"] = full[full.shape[0] - (taps - 1):].clone()
    q = conv[:, :G * d].reshape(T, G, d)
    k = conv[:, G * d:2 * G * d].reshape(T, G, d)
    v = conv[:, 2 * G * d:].reshape(T, H, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                   # [T, H]
    z = (h @ p["a1"].T) @ p["a2"].T + p["dt_bias"]
    decay = torch.exp(-torch.exp(p["A_log"])[None, :, None] * torch.nn.functional.softplus(z).reshape(T, H, d))
    S = state["S"] if state is not None and "S" in state else torch.zeros(H, d, e, dtype=F64)
    o = torch.zeros(T, H, e, dtype=F64)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            Sh = S[hh] * decay[t, hh][:, None]
            u = beta[t, hh] * (v[t, hh] - Sh.T @ k[t, g])
            Sh = Sh + torch.outer(k[t, g], u)
            S[hh] = Sh
            o[t, hh] = Sh.T @ q[t, g]
    if state is not None:
        state["S"] = S
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * p["norm"]
    gate = torch.sigmoid((h @ p["g1"].T) @ p["g2"].T).reshape(T, H, e)
    return (o * gate).reshape(T, H * e) @ p["o"].T


def dense_ff(h, p):
    return (torch.relu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in w.items() if k.startswith(prefix)}


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int]):
    """(logits [T, vocab], streams [layers, T, W]) of one whole sequence."""
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    E = w["embed"].to(F64)
    x = E[torch.tensor(tokens, dtype=torch.long)]
    latents: Dict[int, torch.Tensor] = {}
    streams = []
    for i, L in enumerate(cfg["layers"]):
        m, kind = L["mixer"], L["type"]
        p = sub(w, f"l{i}.mix.")
        if kind == "attention":
            y = attention_mixer(x, p, m, eps)
        elif kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(x, p, eps)
                src = i
            y = latent_mixer(x, p, m, eps, latents[int(src)])
        elif kind == "channel_delta":
            y = channel_delta_mixer(x, p, m, eps)
        else:
            raise ValueError(kind)
        x = layer_norm(alpha * x + y, w[f"l{i}.norm1"].to(F64), w[f"l{i}.norm1.b"].to(F64), eps)
        if L.get("mlp"):
            y = dense_ff(x, sub(w, f"l{i}.mlp."))
            x = layer_norm(alpha * x + y, w[f"l{i}.norm2"].to(F64), w[f"l{i}.norm2.b"].to(F64), eps)
        streams.append(x.clone())
    xf = layer_norm(x, w["final.norm"].to(F64), w["final.norm.b"].to(F64), eps)
    return xf @ E.T, torch.stack(streams)


def generate(cfg: dict, w, prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        lg, _ = forward(cfg, w, toks)
        out.append(int(torch.argmax(lg[-1])))
        toks.append(out[-1])
    return out
