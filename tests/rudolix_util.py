"""Small Rudolix configurations with random weights for the tests: a config.json-shaped dict and bf16-exact weights under the
checkpoint's tensor names.  The engine helpers (replay, rel_rms, write_checkpoint, make_engine) are those of stack_util."""
import torch

from conftest import pkg
from stack_util import bf16_exact


def attention(heads=4, kv_heads=2, dim=24, vdim=20, rot_dims=16, base=5000.0, scale=0.3, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=20, vdim=12, conv=3, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def mamba2(heads=4, vdim=12, state=20, groups=2, norm_groups=2, conv=3, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv},
            "mlp": mlp}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, limit=1.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def make_cfg(width=72, vocab=130, layers=None, eps=1e-5, streams=2, mult=0.5, taps=3, scale=4.0):
    if layers is None:
        layers = [mamba2(mlp=dense()), attention(mlp=moe()), delta(), mamba2(heads=2, vdim=28, state=36, groups=1, norm_groups=1, conv=4, mlp=moe(5, 3, 16, 0.7)),
                  delta(heads=2, kv_heads=2, dim=36, vdim=40, conv=4, mlp=dense(48)), attention(heads=3, kv_heads=3, dim=16, vdim=16, rot_dims=16)]
    return {"architecture": "Rudolix", "canon": {"taps": taps}, "embedding": {"scale": scale}, "norm": {"eps": eps}, "residual_mult": mult,
            "streams": streams, "vocab": vocab, "width": width, "layers": layers}


def make_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    W, V, n, taps = cfg["width"], cfg["vocab"], cfg["streams"], cfg["canon"]["taps"]

    def mat(o, i, s=None):
        return bf16_exact(torch.randn(o, i, generator=g) * (s if s is not None else i ** -0.5))

    def vec(k, mean=1.0, jitter=0.1):
        return bf16_exact(mean + jitter * torch.randn(k, generator=g))

    w = {"embed": mat(V, W, 0.3), "final.norm": vec(W), "final.norm.b": vec(W, 0.0, 0.2)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        for q in ("1", "2") if L["mlp"] else ("1",):
            w[p + "norm" + q], w[p + "norm" + q + ".b"] = vec(W), vec(W, 0.0, 0.2)
            w[p + "ls" + q] = vec(W, 0.8, 0.3)
            w[p + f"hc{q}.in"], w[p + f"hc{q}.out"] = vec(n, 1.0 / n, 0.3), vec(n, 1.0, 0.4)
            w[p + f"hc{q}.mix"] = bf16_exact(torch.eye(n) + 0.2 * torch.randn(n, n, generator=g))
            w[p + "canon" + q] = mat(W, taps, 0.4)
        H, e = m["heads"], m["vdim"]
        if L["type"] == "attention":
            G, d = m["kv_heads"], m["dim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, W), mat(G * d, W), mat(G * e, W)
            w[p + "mix.sink"] = vec(H, 0.5, 1.0)
        elif L["type"] == "delta":
            G, d, k = m["kv_heads"], m["dim"], m["conv"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(G * d, W), mat(G * d, W), mat(H * e, W)
            for n_, ch in (("q", G * d), ("k", G * d), ("v", H * e)):
                w[p + f"mix.{n_}.conv"] = mat(ch, k, 0.6)
            w[p + "mix.b"], w[p + "mix.a"] = mat(H, W, 2.0 * W ** -0.5), mat(H, W, 2.0 * W ** -0.5)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"] = vec(H, -0.5, 0.8), vec(H, -1.0, 1.0)
            w[p + "mix.norm"], w[p + "mix.g"] = vec(e, 1.0, 0.3), mat(H * e, W)
        else:
            N, G, k = m["state"], m["groups"], m["conv"]
            ch = H * e + 2 * G * N
            w[p + "mix.in"] = mat(2 * H * e + 2 * G * N + H, W)
            w[p + "mix.conv"], w[p + "mix.conv.b"] = mat(ch, k, 0.6), vec(ch, 0.0, 0.3)
            w[p + "mix.dt_bias"], w[p + "mix.A_log"], w[p + "mix.D"] = vec(H, -1.0, 1.0), vec(H, -0.5, 0.8), vec(H, 1.0, 0.5)
            w[p + "mix.norm"] = vec(H * e, 1.0, 0.3)
        w[p + "mix.o"] = mat(W, H * e)
        f = L["mlp"]
        if f and f["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(f["ff"], W), mat(W, f["ff"])
            w[p + "mlp.act"] = bf16_exact(torch.tensor([0.9, 0.4, -0.3, 0.1]) + 0.1 * torch.randn(4, generator=g))
        elif f:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = mat(E, W, 3.0 * W ** -0.5)      # spread-out logits: few near-ties
            w[p + "mlp.router.b"] = vec(E, 0.0, 0.5)
            for x in range(E):
                w[f"{p}mlp.e{x}.gate"], w[f"{p}mlp.e{x}.up"], w[f"{p}mlp.e{x}.down"] = mat(ff, W, 2.0 * W ** -0.5), mat(ff, W, 2.0 * W ** -0.5), mat(W, ff)
    return w


def product_config(cfg):
    return pkg("config").RudolixConfig.from_dict(cfg, name="test")


def make_runner(cfg, w, dtype="float32", **kw):
    kw.setdefault("max_tokens", 512)
    kw.setdefault("max_model_len", 1024)
    kw.setdefault("block_size", 16)
    kw.setdefault("n_blocks", 80)
    kw.setdefault("max_logit_rows", 512)
    kw.setdefault("n_state_slots", 5)
    r = pkg("runner").make_runner(product_config(cfg), dtype=dtype, **kw)
    r.load_weights({k: v.clone() for k, v in w.items()})
    return r
