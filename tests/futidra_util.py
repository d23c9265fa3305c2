"""Small Futidra configurations with random weights for the tests: a config.json-shaped dict and bf16-exact weights under the
checkpoint's tensor names.  The engine helpers (replay, rel_rms, write_checkpoint, make_engine) are those of stack_util."""
import torch

from conftest import pkg
from stack_util import bf16_exact


def attention(heads=4, kv_heads=2, dim=24, vdim=None, window=9, rot_dims=16, base=3000.0, scale=0.3,
              scaling=dict(factor=4.0, low=1.0, high=3.0, original=40), mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim, "scale": scale, "mask": {"size": window}}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads=3, dim=20, vdim=12, kv_rank=28, q_rank=36, window=11, scale=0.25, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=20, vdim=12, conv=3, a_rank=10, g_rank=6, mlp=None):
    """a_rank / g_rank are not part of config.json: they size the weights, and the product reads them from the tensor shapes."""
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp, "_ranks": (a_rank, g_rank)}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def make_cfg(width=72, vocab=130, layers=None, eps=1e-5, alpha=2.5):
    if layers is None:
        layers = [latent(mlp=dense()), delta(), attention(mlp=dense(40)), latent(kv_from=0, heads=2, dim=16, vdim=20, q_rank=24, window=30),
                  delta(heads=2, kv_heads=2, dim=36, vdim=40, conv=4, mlp=dense(48)), attention(heads=3, kv_heads=3, dim=16, window=64, rot_dims=16, scaling=None)]
    return {"architecture": "Futidra", "norm": {"eps": eps}, "postln_alpha": alpha, "vocab": vocab, "width": width, "layers": layers}


def public_cfg(cfg):
    """The dict as a config.json would hold it (without the test-only rank hints)."""
    return {**cfg, "layers": [{k: v for k, v in L.items() if k != "_ranks"} for L in cfg["layers"]]}


def make_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=None):
        return bf16_exact(torch.randn(o, i, generator=g) * (s if s is not None else i ** -0.5))

    def vec(n, mean=1.0, jitter=0.1):
        return bf16_exact(mean + jitter * torch.randn(n, generator=g))

    w = {"embed": mat(V, W, 1.0), "final.norm": vec(W), "final.norm.b": vec(W, 0.0, 0.2)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        w[p + "norm1"], w[p + "norm1.b"] = vec(W), vec(W, 0.0, 0.2)
        if L["mlp"]:
            ff = L["mlp"]["ff"]
            w[p + "norm2"], w[p + "norm2.b"] = vec(W), vec(W, 0.0, 0.2)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W), mat(ff, W), mat(W, ff)
        H, d, e = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m["kv_heads"]
            w[p + "mix.q"], w[p + "mix.k"] = mat(H * d, W), mat(G * d, W)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(d, 1.0, 0.3), vec(d, 1.0, 0.3)
        elif L["type"] == "latent_attention":
            r, qr = m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(qr, W), vec(qr, 1.0, 0.3), mat(H * d, qr, 2.0 * qr ** -0.5)
            if m.get("kv_from") is None:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(r, W), vec(r, 1.0, 0.3)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * d, r, 2.0 * r ** -0.5), mat(H * e, r)
            w[p + "mix.g"] = mat(H, W, 2.0 * W ** -0.5)
        else:
            G, taps = m["kv_heads"], m["conv"]
            ra, rg = L["_ranks"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(G * d, W), mat(G * d, W), mat(H * e, W)
            for n_, ch in (("q", G * d), ("k", G * d), ("v", H * e)):
                w[p + f"mix.{n_}.conv"] = mat(ch, taps, 0.6)
            w[p + "mix.b"], w[p + "mix.A_log"] = mat(H, W, 2.0 * W ** -0.5), vec(H, -0.5, 0.8)
            w[p + "mix.norm"] = vec(e, 1.0, 0.3)
            w[p + "mix.a1"], w[p + "mix.a2"], w[p + "mix.dt_bias"] = mat(ra, W), mat(H * d, ra, 1.5 * ra ** -0.5), vec(H * d, -1.0, 1.0)
            w[p + "mix.g1"], w[p + "mix.g2"] = mat(rg, W), mat(H * e, rg, 1.5 * rg ** -0.5)
        w[p + "mix.o"] = mat(W, H * e)
    return w


def product_config(cfg, w):
    return pkg("config").FutidraConfig.from_dict(public_cfg(cfg), name="test", shapes={k: list(v.shape) for k, v in w.items()})


def make_runner(cfg, w, dtype="float32", **kw):
    kw.setdefault("max_tokens", 512)
    kw.setdefault("max_model_len", 1024)
    kw.setdefault("block_size", 16)
    kw.setdefault("n_blocks", 80)
    kw.setdefault("max_logit_rows", 512)
    kw.setdefault("n_state_slots", 5)
    r = pkg("runner").make_runner(product_config(cfg, w), dtype=dtype, **kw)
    r.load_weights({k: v.clone() for k, v in w.items()})
    return r
