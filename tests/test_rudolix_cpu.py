"""Rudolix without a GPU: the registry and every part of the configuration, the weight mapping (fusions, packed stream
coefficients, stacked experts), and the oracle's own invariants (causality, recurrences carried across portions, the sink's
share, rotation by distance, the router's weights, the clamp, streams that collapse to a plain residual)."""
import math

import pytest
import torch

import rudolix_util as R
import stack_util as U
from conftest import pkg
from oracle import rudolix_oracle as O


def test_registry_reads_the_layer_list(tmp_path):
    cfg = R.make_cfg()
    w = R.make_weights(cfg, 1)
    path = str(tmp_path / "ckpt")
    U.write_checkpoint(path, cfg, w)
    C = pkg("config")
    pc = C.load_model_config(path)
    assert type(pc).__name__ == "RudolixConfig" and C.is_stack_config(pc) and pc.needs_state
    assert (pc.width, pc.vocab, pc.streams, pc.residual_mult, pc.canon_taps, pc.embed_scale, pc.norm_eps, pc.n_layers) == (72, 130, 2, 0.5, 3, 4.0, 1e-5, 6)
    a, b, c = pc.layers[0].mixer, pc.layers[1].mixer, pc.layers[2].mixer
    assert (a.heads, a.vdim, a.state, a.groups, a.norm_groups, a.conv) == (4, 12, 20, 2, 2, 3)
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.scale) == (4, 2, 24, 20, 0.3) and b.rot_half and b.sink and not b.qk_norm
    assert (b.rot.dims, b.rot.base, b.rot.scaled) == (16, 5000.0, False)
    assert (c.heads, c.kv_heads, c.dim, c.vdim, c.conv) == (4, 2, 20, 12, 3)
    f0, f1 = pc.layers[0].mlp, pc.layers[1].mlp
    assert (f0.kind, f0.ff, f0.act, f0.gated) == ("dense", 56, "polynorm", False)
    assert (f1.kind, f1.experts, f1.top, f1.ff, f1.act, f1.limit, f1.router, f1.gated) == ("moe", 6, 2, 24, "swiglu_clamp", 1.0, "chosen_softmax", True)
    assert pc.layers[2].mlp is None
    assert pc.mixer_rows(a) == 2 * 48 + 2 * 40 + 4 and pc.mixer_rows(c) == 2 * 40 + 2 * 48 + 8 and pc.mixer_rows(b) == 96 + 48 + 40
    assert pc.kv_bytes_per_token() == 2 * (2 * 44 + 3 * 32)


def test_configuration_errors_and_defaults():
    C = pkg("config")
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(layers=[{"type": "mlstm", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(layers=[R.attention(heads=3, kv_heads=2)]))
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(layers=[R.attention(rot_dims=26)]))
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(layers=[R.mamba2(heads=3, groups=2)]))
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(layers=[R.delta(mlp=R.moe(experts=2, top=3))]))
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(layers=[R.delta(mlp={"kind": "glu", "ff": 8})]))
    with pytest.raises(ValueError):
        C.RudolixConfig.from_dict(R.make_cfg(streams=9))
    pc = C.RudolixConfig.from_dict(R.make_cfg(layers=[R.attention(rot_dims=0)], streams=1, taps=1))
    assert pc.layers[0].mixer.rot is None and not pc.needs_state and pc.streams == 1
    assert C.RudolixConfig.from_dict(R.make_cfg(layers=[R.attention()], taps=2)).needs_state


def test_weight_mapping_fuses_packs_and_stacks():
    A = pkg("_abi")
    cfg = R.make_cfg()
    w = R.make_weights(cfg, 2)
    pc = R.product_config(cfg)
    items = {}
    for layer, kind, t in pkg("weights").rudolix_weights(w, pc):
        assert (layer, kind) not in items
        items[(layer, kind)] = t
    assert items[(0, A.SW_HEAD)] is items[(0, A.SW_EMBED)]
    q = items[(1, A.SW_QKV)]
    assert q.shape == (96 + 48 + 40, 72) and torch.equal(q[:96], w["l1.mix.q"]) and torch.equal(q[96:144], w["l1.mix.k"]) and torch.equal(q[144:], w["l1.mix.v"])
    d = items[(2, A.SW_QKV)]
    assert d.shape[0] == pc.mixer_rows(pc.layers[2].mixer)
    at = 0
    for n in ("q", "k", "v", "g", "b", "a"):
        t = w["l2.mix." + n]
        assert torch.equal(d[at:at + t.shape[0]], t), n
        at += t.shape[0]
    assert torch.equal(items[(2, A.SW_HEAD_NORM)], w["l2.mix.norm"].repeat(4)) and items[(2, A.SW_CONV)].shape == (2 * 40 + 48, 3)
    assert items[(0, A.SW_QKV)] is w["l0.mix.in"] and items[(0, A.SW_HEAD_NORM)].shape == (48,) and items[(0, A.SW_SKIP)].shape == (4,)
    hc = items[(1, A.SW_HC_MLP)]
    assert hc.shape == (2 + 2 + 4,) and torch.equal(hc[:2], w["l1.hc2.in"]) and torch.equal(hc[2:4], w["l1.hc2.out"])
    assert torch.equal(hc[4:].view(2, 2), w["l1.hc2.mix"])
    gu = items[(1, A.SW_EXPERT_GATE_UP)]
    assert gu.shape == (6 * 48, 72) and torch.equal(gu[48:72], w["l1.mlp.e1.gate"]) and torch.equal(gu[72:96], w["l1.mlp.e1.up"])
    assert items[(1, A.SW_EXPERT_DOWN)].shape == (6 * 72, 24) and items[(1, A.SW_ROUTER_BIAS)].shape == (6,)
    assert items[(0, A.SW_MLP_GATE_UP)].shape == (56, 72) and items[(0, A.SW_MLP_ACT)].shape == (4,)
    assert (2, A.SW_NORM_MLP_PRE) not in items and (2, A.SW_CANON_MLP) not in items and (0, A.SW_CANON_MLP) in items
    assert all(k in A.SW_F32 for k in (A.SW_HC_MIX, A.SW_SCALE_MLP, A.SW_CONV_BIAS, A.SW_SKIP, A.SW_MLP_ACT, A.SW_NORM_MIX_PRE_BIAS))


def test_a_logit_row_does_not_depend_on_what_follows():
    cfg = R.make_cfg()
    w = R.make_weights(cfg, 3)
    ids = torch.randint(0, cfg["vocab"], (30,), generator=torch.Generator().manual_seed(1)).tolist()
    full = O.forward(cfg, w, ids)
    assert torch.allclose(O.forward(cfg, w, ids[:17]), full[:17], atol=1e-10)


def test_recurrences_carried_across_portions_equal_the_whole():
    g = torch.Generator().manual_seed(4)
    T, H, d, dv = 23, 3, 5, 4
    q, k = torch.randn(T, H, d, generator=g, dtype=torch.float64), torch.randn(T, H, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    beta, dec = torch.rand(T, H, generator=g, dtype=torch.float64), torch.rand(T, H, generator=g, dtype=torch.float64)
    whole, _ = O.delta_rule(q, k, v, beta, dec)
    a, S = O.delta_rule(q[:9], k[:9], v[:9], beta[:9], dec[:9])
    b, _ = O.delta_rule(q[9:], k[9:], v[9:], beta[9:], dec[9:], S)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)
    dt = torch.rand(T, H, generator=g, dtype=torch.float64)
    a_log, D = torch.randn(H, generator=g, dtype=torch.float64), torch.randn(H, generator=g, dtype=torch.float64)
    whole, _ = O.ssd_scan(v, k, q, dt, a_log, D)
    a, S = O.ssd_scan(v[:9], k[:9], q[:9], dt[:9], a_log, D)
    b, _ = O.ssd_scan(v[9:], k[9:], q[9:], dt[9:], a_log, D, S)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)
    # the delta rule without decay, with beta 1 and orthonormal keys, reads back exactly what was written
    keys = torch.linalg.qr(torch.randn(d, d, generator=g, dtype=torch.float64)).Q[:4].unsqueeze(1)
    vals = torch.randn(4, 1, dv, generator=g, dtype=torch.float64)
    _, S = O.delta_rule(keys, keys, vals, torch.ones(4, 1, dtype=torch.float64), torch.ones(4, 1, dtype=torch.float64))
    assert torch.allclose(torch.einsum("hdv,thd->thv", S, keys), vals, atol=1e-12)
    h = torch.randn(T, 6, generator=g, dtype=torch.float64)
    cw = torch.randn(6, 4, generator=g, dtype=torch.float64)
    assert torch.allclose(torch.cat([O.causal_conv(h[:5], cw), O.causal_conv(h[5:], cw, history=h[2:5])]), O.causal_conv(h, cw), atol=1e-12)
    assert torch.allclose(O.causal_conv(h, cw)[0], h[0] * cw[:, 3])          # the last tap is the current token's


def test_the_sink_takes_its_share_and_rotation_depends_on_distance():
    g = torch.Generator().manual_seed(5)
    q, k, v = torch.randn(1, 2, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 6, generator=g, dtype=torch.float64)
    sink = torch.tensor([0.7, -2.0], dtype=torch.float64)
    out = O.sink_attention(q, k, v, 0.4, sink)
    for h in range(2):
        s = float((q[0, h] @ k[0, 0]) * 0.4)
        assert torch.allclose(out[0, h], v[0, 0] * math.exp(s) / (math.exp(s) + math.exp(float(sink[h]))), atol=1e-12)
    x, y = torch.randn(1, 1, 12, generator=g, dtype=torch.float64), torch.randn(1, 1, 12, generator=g, dtype=torch.float64)
    dots = [float((O.rotate_half(x, torch.tensor([p + 5]), 8, 100.0) * O.rotate_half(y, torch.tensor([p]), 8, 100.0)).sum()) for p in (0, 3, 400)]
    assert max(dots) - min(dots) < 1e-9
    r = O.rotate_half(x, torch.tensor([7]), 8, 100.0)
    assert torch.equal(r[..., 8:], x[..., 8:]) and not torch.allclose(r[..., :8], x[..., :8])
    a = 7.0 * 100.0 ** (-2.0 * 1 / 8)          # pair (1, 5)
    assert abs(float(r[0, 0, 1]) - (float(x[0, 0, 1]) * math.cos(a) - float(x[0, 0, 5]) * math.sin(a))) < 1e-12
    assert abs(float(r[0, 0, 5]) - (float(x[0, 0, 5]) * math.cos(a) + float(x[0, 0, 1]) * math.sin(a))) < 1e-12


def test_router_weights_clamp_and_polynomial():
    z = torch.tensor([[0.1, 2.0, -1.0, 1.5]], dtype=torch.float64)
    ids, wt = O.route(torch.ones(1, 1, dtype=torch.float64), z.T.contiguous(), torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=torch.float64), 2)
    assert ids.tolist() == [[3, 1]]          # the bias is part of the logit: 2.5 beats 2.0
    assert torch.allclose(wt, torch.softmax(torch.tensor([[2.5, 2.0]], dtype=torch.float64), -1))
    one = torch.ones(1, 1, dtype=torch.float64)
    eye = torch.ones(1, 1, dtype=torch.float64)
    big = O.expert(one * 50.0, eye, eye, eye, 1.5)          # gate capped from above, up clamped on both sides
    assert abs(float(big) - 1.5 / (1 + math.exp(-1.702 * 1.5)) * 2.5) < 1e-12
    low = O.expert(one * -50.0, eye, eye, eye, 1.5)          # the gate is not clamped from below
    assert abs(float(low) - (-50.0) / (1 + math.exp(1.702 * 50.0)) * (-0.5)) < 1e-12
    v = torch.tensor([[1.0, -2.0, 3.0]], dtype=torch.float64)
    p = O.poly_norm(v, torch.tensor([2.0, 0.0, 0.0, 0.5], dtype=torch.float64), 0.0)
    assert torch.allclose(p, 2.0 * v / math.sqrt(14.0 / 3.0) + 0.5)
    p = O.poly_norm(v, torch.tensor([0.0, 0.0, 1.0, 0.0], dtype=torch.float64), 0.0)
    assert torch.allclose(p, v ** 3 / math.sqrt((1 + 64 + 729) / 3.0))


def test_one_stream_with_unit_coefficients_is_a_plain_residual():
    cfg = R.make_cfg(streams=1, mult=1.0, layers=[R.delta(mlp=R.dense(20))], taps=2)
    w = R.make_weights(cfg, 6)
    for q in ("1", "2"):
        w[f"l0.hc{q}.in"], w[f"l0.hc{q}.out"], w[f"l0.hc{q}.mix"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)
    ids = [3, 9, 27, 81, 5]
    st = []
    O.forward(cfg, w, ids, st)
    wd = {k: v.double() for k, v in w.items()}
    x = wd["embed"][torch.tensor(ids)] * 4.0
    h = O.layer_norm(x, wd["l0.norm1"], wd["l0.norm1.b"], 1e-5)
    x = x + wd["l0.ls1"] * O.delta_mixer(h + O.causal_conv(h, wd["l0.canon1"]), wd, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5)
    h = O.layer_norm(x, wd["l0.norm2"], wd["l0.norm2.b"], 1e-5)
    x = x + wd["l0.ls2"] * O.dense_ff(h + O.causal_conv(h, wd["l0.canon2"]), wd, "l0.mlp.", 1e-5)
    assert torch.allclose(st[0], x, atol=1e-12)
