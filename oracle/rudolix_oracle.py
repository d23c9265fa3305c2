"""Float64 restatement of the Rudolix design, one function per mechanism, for the tests.  Shares no code with the package.

A model is a dict `cfg` in the layout of the design's config.json and a dict `w` of tensors under the checkpoint's names.
Notation: T tokens of ONE sequence, rows are time steps; W width; every function takes and returns float64 tensors.

    streams X_1..X_n = E[id] * scale
    sublayer q of layer i:  u = sum_s a_q[s] X_s;  h = LN(u);  h = h + conv(h);  y = ls_q * sublayer(h)
                            X_t <- sum_s M_q[s, t] X_s + m * b_q[t] * y          (all streams from the old ones)
    logits = E LN_f(sum_s X_s)
"""
import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(h, w, bias=None, history=None):
    """out[t, c] = sum_j w[c, j] h[t - K + 1 + j, c] (+ bias[c]); rows before the sequence are zeros, or `history` ([K-1, C],
    oldest first) when the sequence is continued.  The last tap is the current row's."""
    T, C = h.shape
    K = w.shape[1]
    past = torch.zeros((K - 1, C), dtype=F64) if history is None else history
    full = torch.cat([past, h], 0)
    out = torch.zeros((T, C), dtype=F64)
    for j in range(K):
        out += full[j:j + T] * w[:, j]
    if bias is not None:
        out = out + bias
    return out


def rotate_half(x, pos, dims, base):
    """x [T, heads, dim]: entries i and i + dims/2 (i < dims/2) turn by pos * base^(-2i/dims); the rest pass."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor(base, dtype=F64) ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    ang = pos.to(F64)[:, None] * f[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def sink_attention(q, k, v, scale, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; the denominator of head h also holds exp(sink[h])."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    mask = torch.tril(torch.ones((T, T), dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h])
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def attention_mixer(h, w, p, m, pos):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    r = m.get("rot") or {}
    q = rotate_half(q, pos, int(r.get("dims", 0)), float(r.get("base", 10000.0)))
    k = rotate_half(k, pos, int(r.get("dims", 0)), float(r.get("base", 10000.0)))
    o = sink_attention(q, k, v, float(m["scale"]), w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def delta_rule(q, k, v, beta, g, S=None):
    """Per head: S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q.  q, k [T, H, d]; v [T, H, dv]; beta, g [T, H]."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros((H, d, dv), dtype=F64) if S is None else S.clone()
    o = torch.zeros((T, H, dv), dtype=F64)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def delta_mixer(h, w, p, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o, _ = delta_rule(q, k, v, beta, g)
    o = unit_rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def ssd_scan(x, B, C, dt, a_log, D, S=None):
    """Per head: S = exp(-exp(a_log) dt) S + dt B x^T (S is [N, dv]); y = S^T C + D x.  x [T, H, dv]; B, C [T, H, N]; dt [T, H]."""
    T, H, dv = x.shape
    N = B.shape[2]
    S = torch.zeros((H, N, dv), dtype=F64) if S is None else S.clone()
    y = torch.zeros((T, H, dv), dtype=F64)
    for t in range(T):
        S = S * torch.exp(-torch.exp(a_log) * dt[t])[:, None, None] + torch.einsum("hn,hv->hnv", B[t] * dt[t][:, None], x[t])
        y[t] = torch.einsum("hnv,hn->hv", S, C[t]) + D[:, None] * x[t]
    return y, S


def mamba2_mixer(h, w, p, m, eps):
    H, dv, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    T = h.shape[0]
    inner = H * dv
    z_all = h @ w[p + "in"].T
    z, xbc, dt = z_all[:, :inner], z_all[:, inner:2 * inner + 2 * G * N], z_all[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, 1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, 1)
    dt = softplus(dt + w[p + "dt_bias"])
    y, _ = ssd_scan(x, B, C, dt, w[p + "A_log"], w[p + "D"])
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def poly_norm(z, coef, eps):
    return coef[0] * unit_rms(z, eps) + coef[1] * unit_rms(z * z, eps) + coef[2] * unit_rms(z * z * z, eps) + coef[3]


def dense_ff(h, w, p, eps):
    return poly_norm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def route(h, w_router, bias, top):
    """Indices [T, top] of the largest logits (ties: lowest index) and the softmax over those logits alone."""
    z = h @ w_router.T + bias
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), -1)


def expert(h, wg, wu, wd, limit):
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def moe_ff(h, w, p, f):
    ids, wt = route(h, w[p + "router"], w[p + "router.b"], int(f["router"]["top"]))
    out = torch.zeros((h.shape[0], w[p + "e0.down"].shape[0]), dtype=F64)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += wt[t, j] * expert(h[t:t + 1], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], float(f["expert"]["limit"]))[0]
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], streams_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence run as a whole; `streams_out` receives the sum of the streams after every layer."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps, m, n = float(cfg["norm"]["eps"]), float(cfg["residual_mult"]), int(cfg["streams"])
    T = len(ids)
    pos = torch.arange(T)
    x0 = w["embed"][torch.tensor(ids)] * float(cfg["embedding"]["scale"])
    X = [x0.clone() for _ in range(n)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and not L.get("mlp"):
                continue
            u = sum(w[f"{p}hc{q}.in"][s] * X[s] for s in range(n))
            h = layer_norm(u, w[f"{p}norm{q}"], w[f"{p}norm{q}.b"], eps)
            h = h + causal_conv(h, w[f"{p}canon{q}"])
            if q == 1:
                kind = L["type"]
                if kind == "attention":
                    y = attention_mixer(h, w, p + "mix.", L["mixer"], pos)
                elif kind == "delta":
                    y = delta_mixer(h, w, p + "mix.", L["mixer"], eps)
                elif kind == "mamba2":
                    y = mamba2_mixer(h, w, p + "mix.", L["mixer"], eps)
                else:
                    raise ValueError(kind)
            else:
                f = L["mlp"]
                y = dense_ff(h, w, p + "mlp.", eps) if f["kind"] == "dense" else moe_ff(h, w, p + "mlp.", f)
            y = y * w[f"{p}ls{q}"]
            mix, out = w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"]
            X = [sum(mix[s, t] * X[s] for s in range(n)) + m * out[t] * y for t in range(n)]
        if streams_out is not None:
            streams_out.append(sum(X))
    xf = layer_norm(sum(X), w["final.norm"], w["final.norm.b"], eps)
    return xf @ w["embed"].T


def greedy(cfg, w, prompt: List[int], n_new: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]
