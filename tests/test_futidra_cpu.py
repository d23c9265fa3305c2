"""Futidra without a GPU: the registry and every part of the configuration, the weight mapping (fusions, padding rows, the
transposed key expansion), the band-scaled rotation table against the oracle's frequencies, and the oracle's own invariants
(windows, the extra unit of the denominator, values that are keys, shared latents, state carried across portions)."""
import json
import os

import pytest
import torch

import futidra_util as F
import stack_util as U
from conftest import pkg
from oracle import futidra_oracle as O


def test_registry_reads_the_layer_list_and_takes_ranks_from_the_checkpoint(tmp_path):
    cfg = F.make_cfg()
    w = F.make_weights(cfg, 1)
    path = str(tmp_path / "ckpt")
    U.write_checkpoint(path, F.public_cfg(cfg), w)
    C = pkg("config")
    pc = C.load_model_config(path)
    assert type(pc).__name__ == "FutidraConfig" and C.is_stack_config(pc) and pc.needs_state
    assert pc.width == 72 and pc.vocab == 130 and pc.postln_alpha == 2.5 and pc.norm_eps == 1e-5 and pc.n_layers == 6
    a, b, c, d = pc.layers[0].mixer, pc.layers[1].mixer, pc.layers[2].mixer, pc.layers[3].mixer
    assert (a.heads, a.dim, a.vdim, a.kv_rank, a.q_rank, a.window, a.kv_from, a.head_gate) == (3, 20, 12, 28, 36, 11, None, True)
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.conv, b.decay_rank, b.gate_rank) == (4, 2, 20, 12, 3, 10, 6)
    assert (c.heads, c.kv_heads, c.dim, c.vdim, c.window) == (4, 2, 24, 24, 9) and c.head_norm and c.value_is_key and c.sink_one
    assert c.rot.kind == "bands" and (c.rot.dims, c.rot.factor, c.rot.original, c.rot.fast, c.rot.slow) == (16, 4.0, 40, 3.0, 1.0)
    assert d.kv_from == 0 and d.window == 30
    assert pc.layers[1].mlp is None and pc.layers[0].mlp.ff == 56 and pc.layers[0].mlp.act == "relu"
    assert pc.layers[5].mixer.rot.scaled is False
    assert pc.kv_bytes_per_token() == 2 * (28 + 2 * 48 + 3 * 32)


def test_configuration_errors():
    C = pkg("config")
    cfg = F.make_cfg(layers=[F.latent(kv_from=0)])
    with pytest.raises(ValueError):
        C.FutidraConfig.from_dict(F.public_cfg(cfg))
    cfg = F.make_cfg(layers=[F.latent(), F.latent(kv_from=0, kv_rank=12)])
    with pytest.raises(ValueError):
        C.FutidraConfig.from_dict(F.public_cfg(cfg))
    cfg = F.make_cfg(layers=[F.delta()])
    with pytest.raises(ValueError):      # the ranks are in no config.json: without shapes the reader cannot size the layer
        C.FutidraConfig.from_dict(F.public_cfg(cfg))
    cfg = F.make_cfg(layers=[{"type": "mlstm", "mixer": {}, "mlp": None}])
    with pytest.raises(ValueError):
        C.FutidraConfig.from_dict(cfg)


def test_band_scaled_table_matches_the_oracles_frequencies():
    C = pkg("config")
    for sc in (None, dict(factor=4.0, low=1.0, high=3.0, original=40), dict(factor=16.0, low=0.5, high=8.0, original=300)):
        rot = {"base": 777.0, "dims": 12}
        spec = C.RotarySpec(base=777.0, dims=12)
        if sc:
            rot["scaling"] = sc
            spec = C.RotarySpec(base=777.0, dims=12, factor=sc["factor"], original=sc["original"], fast=sc["high"], slow=sc["low"], scaled=True,
                                kind="bands")
        f = O.rotary_frequencies(rot)
        t = spec.table(50).double()
        pos = torch.arange(50, dtype=torch.float64)[:, None]
        assert torch.allclose(t[:, 0], torch.cos(pos * f), atol=1e-6) and torch.allclose(t[:, 1], torch.sin(pos * f), atol=1e-6)
    # all three bands occur in the second case
    f0 = O.rotary_frequencies({"base": 777.0, "dims": 12})
    f1 = O.rotary_frequencies({"base": 777.0, "dims": 12, "scaling": dict(factor=4.0, low=1.0, high=3.0, original=40)})
    ratio = (f1 / f0).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-12 and any(0.25 < r < 1.0 for r in ratio)


def test_weight_mapping_fuses_pads_and_transposes():
    A = pkg("_abi")
    cfg = F.make_cfg()
    w = F.make_weights(cfg, 2)
    pc = F.product_config(cfg, w)
    items = {}
    for layer, kind, t in pkg("weights").futidra_weights(w, pc):
        items[(layer, kind)] = t
    assert items[(0, A.SW_HEAD)] is items[(0, A.SW_EMBED)]
    # latent with its own latent: dq | dkv | g
    q = items[(0, A.SW_QKV)]
    assert q.shape == (36 + 28 + 3, 72) and torch.equal(q[36:64], w["l0.mix.dkv"]) and torch.equal(q[64:], w["l0.mix.g"])
    uk = items[(0, A.SW_UK_T)].reshape(3, 28, 20)
    assert torch.equal(uk[1], w["l0.mix.uk"][20:40].T)
    # latent reading layer 0's latents: no dkv rows, no latent norm
    assert items[(3, A.SW_QKV)].shape == (24 + 2, 72) and (3, A.SW_K_NORM) not in items
    # delta: q | k | v | a1 | g1 | b with a1, g1, b at multiples of 8 and zero rows between
    rows, off = pkg("weights").delta_fused_offsets(pc.layers[1].mixer)
    assert off == [0, 40, 80, 128, 144, 152] and rows == 160
    fz = items[(1, A.SW_QKV)]
    assert fz.shape == (160, 72) and torch.equal(fz[128:138], w["l1.mix.a1"]) and torch.equal(fz[152:156], w["l1.mix.b"])
    assert float(fz[138:144].abs().sum()) == 0.0 and float(fz[150:152].abs().sum()) == 0.0 and float(fz[156:].abs().sum()) == 0.0
    assert torch.equal(items[(1, A.SW_CONV)][40:80], w["l1.mix.k.conv"])
    assert torch.equal(items[(1, A.SW_HEAD_NORM)], w["l1.mix.norm"].repeat(4))
    assert items[(2, A.SW_QKV)].shape == ((4 + 2) * 24, 72) and items[(2, A.SW_Q_NORM)].shape == (24,)
    assert (1, A.SW_NORM_MLP_POST) not in items and (0, A.SW_MLP_GATE_UP) in items


# ---- the oracle's own invariants ------------------------------------------------------------------------------------------------
def _dbl(w):
    return {k: v.double() for k, v in w.items()}


def test_oracle_window_and_the_extra_unit():
    g = torch.Generator().manual_seed(3)
    s = torch.randn(12, 12, generator=g).double()
    m = O.window_mask(12, 4)
    assert m[7].tolist() == [False] * 4 + [True] * 4 + [False] * 4 and m[1].tolist() == [True, True] + [False] * 10
    p0, p1 = O.windowed_softmax(s, m, False), O.windowed_softmax(s, m, True)
    assert torch.allclose(p0.sum(-1), torch.ones(12, dtype=torch.float64))
    e = torch.exp(s).masked_fill(~m, 0.0)
    assert torch.allclose(p1, e / (1.0 + e.sum(-1, keepdim=True)))
    assert float(p1.sum(-1).max()) < 1.0


def test_oracle_attention_sees_exactly_its_window_and_values_are_raw_keys():
    cfg = F.make_cfg(layers=[F.attention(window=5, heads=2, kv_heads=1, dim=8, rot_dims=4)])
    w = _dbl(F.make_weights(cfg, 5))
    p, m = O.sub(w, "l0.mix."), cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(1)
    h = torch.randn(20, 72, generator=g).double()
    base = O.attention_mixer(h, p, m, 1e-5)
    h2 = h.clone()
    h2[10] += 1.0                    # position 10 is seen by 10 .. 14 only
    moved = (O.attention_mixer(h2, p, m, 1e-5) - base).abs().sum(-1) > 1e-9
    assert moved.tolist() == [False] * 10 + [True] * 5 + [False] * 5
    # a single token: weight e^s / (1 + e^s) on its own raw key projection
    one = O.attention_mixer(h[:1], p, m, 1e-5)
    kraw = h[:1] @ p["k"].T
    q = O.rms_norm((h[:1] @ p["q"].T).reshape(1, 2, 8), p["q.norm"], 1e-5)
    k = O.rms_norm(kraw.reshape(1, 1, 8), p["k.norm"], 1e-5)
    sc = (q[0] * k[0]).sum(-1) * m["scale"]          # position 0: no rotation
    wgt = torch.exp(sc) / (1.0 + torch.exp(sc))
    want = (wgt[:, None] * kraw.reshape(1, 8)).reshape(1, 16) @ p["o"].T
    assert torch.allclose(one, want, atol=1e-12)


def test_oracle_shared_latents_and_portions_of_the_recurrence():
    cfg = F.make_cfg()
    w = F.make_weights(cfg, 7)
    ids = torch.randint(0, 130, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    full, streams = O.forward(F.public_cfg(cfg), w, ids)
    short, _ = O.forward(F.public_cfg(cfg), w, ids[:25])
    assert torch.allclose(full[:25], short, atol=1e-9)        # causal
    assert streams.shape == (6, 40, 72)
    # the recurrence fed in portions, its state and convolution tail carried, equals the whole sequence
    p, m = O.sub(_dbl(w), "l1.mix."), cfg["layers"][1]["mixer"]
    h = torch.randn(30, 72, generator=torch.Generator().manual_seed(4)).double()
    whole = O.channel_delta_mixer(h, p, m, 1e-5)
    st, parts = {}, []
    for lo, n in ((0, 1), (1, 2), (3, 1), (4, 9), (13, 17)):
        parts.append(O.channel_delta_mixer(h[lo:lo + n], p, m, 1e-5, state=st))
    assert torch.allclose(torch.cat(parts), whole, atol=1e-10)


def test_oracle_convolution_taps_and_start():
    x = torch.arange(1.0, 9.0, dtype=torch.float64).reshape(4, 2)
    w = torch.tensor([[0.5, -1.0, 2.0], [0.0, 0.0, 1.0]], dtype=torch.float64)        # last column: the current token
    y = O.causal_conv_silu(x, w)
    pre = torch.tensor([[2.0 * 1, 2.0], [2.0 * 3 - 1.0 * 1, 4.0], [2.0 * 5 - 3.0 + 0.5 * 1, 6.0], [2.0 * 7 - 5.0 + 0.5 * 3, 8.0]], dtype=torch.float64)
    assert torch.allclose(y, pre * torch.sigmoid(pre))
