"""GPU parity of the Futidra design against oracle/futidra_oracle.py: every mechanism alone through its per-kernel entry point
(with inputs built so that a key one place outside a window, a dropped unit of the denominator, a stale state or a wrong tail
shows), then whole models through the runner, externally scheduled steps of the engine, and its own scheduler.  32-bit mode is
held to the float64 oracle tightly; bf16 mode within bf16 noise, and to itself across schedules."""
import numpy as np
import pytest
import torch

import futidra_util as F
import stack_util as U
from conftest import pkg
from oracle import futidra_oracle as O

pytestmark = pytest.mark.gpu
F32_TOL = 2e-5
DEV = "cuda"
_KEEP = []


def lib():
    return pkg("_abi").lib()


def check(rc):
    pkg("_abi").check(rc)


def dev(t, dtype=None):
    d = t.to(device=DEV, dtype=dtype or t.dtype).contiguous()
    _KEEP.append(d)
    del _KEEP[:-96]
    return d


def i32(x):
    return dev(torch.tensor(x, dtype=torch.int32))


def sync():
    torch.cuda.synchronize()


def _prompt(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _adt(f32):
    return torch.float32 if f32 else torch.bfloat16


# ---- mechanisms alone ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("width", [40, 257, 1024])
def test_norm_after_the_sum_with_weight_and_bias(f32, width):
    g = torch.Generator().manual_seed(width)
    T, alpha, eps = 9, 3.0, 1e-5
    x = torch.randn(T, width, generator=g) * 2 + 0.7
    y = U.bf16_exact(torch.randn(T, width, generator=g))
    w, b = torch.randn(width, generator=g), torch.randn(width, generator=g)
    want = O.layer_norm(alpha * x.double() + y.double(), w.double(), b.double(), eps)
    xd, act = dev(x), torch.zeros(T, width, dtype=_adt(f32), device=DEV)
    check(lib().b200_postnorm_stream(f32, xd.data_ptr(), dev(y, _adt(f32)).data_ptr(), alpha, dev(w).data_ptr(), dev(b).data_ptr(), xd.data_ptr(),
                                     act.data_ptr(), None, T, width, eps, None))
    sync()
    assert torch.allclose(xd.cpu().double(), want, atol=2e-5)
    assert torch.allclose(act.float().cpu().double(), want, atol=2e-5 if f32 else 3e-2, rtol=0 if f32 else 1e-2)
    # the output norm: gathered rows, nothing added, not in place
    rows = [7, 0, 7, 3]
    out = torch.zeros(4, width, dtype=_adt(f32), device=DEV)
    check(lib().b200_postnorm_stream(f32, dev(x).data_ptr(), None, 1.0, dev(w).data_ptr(), dev(b).data_ptr(), None, out.data_ptr(),
                                     i32(rows).data_ptr(), 4, width, eps, None))
    sync()
    want = O.layer_norm(x[rows].double(), w.double(), b.double(), eps)
    assert torch.allclose(out.float().cpu().double(), want, atol=2e-5 if f32 else 3e-2, rtol=0 if f32 else 1e-2)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot_dims", [(4, 2, 24, 24, 16), (3, 3, 70, 66, 70), (2, 1, 8, 8, 0), (5, 1, 128, 128, 64)])
def test_head_norms_rotation_and_values_that_are_raw_keys(f32, heads, kv_heads, dim, vdim, rot_dims):
    g = torch.Generator().manual_seed(dim + heads)
    T, bs, n_blocks, eps, pad = 7, 4, 6, 1e-5, 3
    ld = (heads + kv_heads) * dim + pad
    qk = U.bf16_exact(torch.randn(T, ld, generator=g) * 1.5)
    qw, kw = 1 + 0.3 * torch.randn(dim, generator=g), 1 + 0.3 * torch.randn(dim, generator=g)
    pos = [5, 6, 7, 0, 1, 30, 2]
    slots = [21, 22, 23, 4, 5, 9, 0]
    rot = {"base": 900.0, "dims": rot_dims, "scaling": dict(factor=3.0, low=1.0, high=4.0, original=64)}
    table = None
    if rot_dims:
        spec = pkg("config").RotarySpec(base=900.0, dims=rot_dims, factor=3.0, original=64, fast=4.0, slow=1.0, scaled=True, kind="bands")
        table = dev(spec.table(32))
    q = O.rms_norm(qk[:, :heads * dim].double().reshape(T, heads, dim), qw.double(), eps)
    kraw = qk[:, heads * dim:(heads + kv_heads) * dim].double().reshape(T, kv_heads, dim)
    k = O.rms_norm(kraw, kw.double(), eps)
    if rot_dims:
        fr = O.rotary_frequencies(rot)
        q, k = O.rotate_pairs(q, torch.tensor(pos), fr), O.rotate_pairs(k, torch.tensor(pos), fr)
    qo = torch.zeros(T, heads * dim, device=DEV)
    kc = torch.full((n_blocks, kv_heads, bs, dim), 9.0, dtype=_adt(f32), device=DEV)
    vc = torch.full((n_blocks, kv_heads, bs, vdim), 9.0, dtype=_adt(f32), device=DEV)
    check(lib().b200_qk_headnorm_rotate_cache(f32, dev(qk, _adt(f32)).data_ptr(), ld, dev(qw).data_ptr(), dev(kw).data_ptr(), i32(pos).data_ptr(),
                                              i32(slots).data_ptr(), table.data_ptr() if table is not None else None, rot_dims, 32, qo.data_ptr(),
                                              kc.data_ptr(), vc.data_ptr(), T, heads, kv_heads, dim, vdim, bs, eps, None))
    sync()
    assert torch.allclose(qo.cpu().double().reshape(T, heads, dim), q, atol=2e-5)
    tol = dict(atol=2e-5) if f32 else dict(atol=2e-2, rtol=1e-2)
    for t, s in enumerate(slots):
        assert torch.allclose(kc[s // bs, :, s % bs].float().cpu().double(), k[t], **tol)
        assert torch.equal(vc[s // bs, :, s % bs].float().cpu().double(), kraw[t, :, :vdim])      # values: untouched projections
    assert float(kc[2, 0, 3, 0]) == 9.0       # slot 11 was never written


def _paged(rows, bs, n_blocks, order, dtype):
    """rows [n, kv_heads, d] laid into a paged cache [n_blocks][kv_heads][bs][d] through a shuffled block table."""
    n, G, d = rows.shape
    cache = torch.full((n_blocks, G, bs, d), 3.0)
    for j in range(n):
        cache[order[j // bs], :, j % bs] = rows[j]
    return dev(cache, dtype)


def _spiked(n, heads, kv_heads, dim, vdim, queries, window, seed):
    """Random q/k/v where, for every query position, the key just outside its window would dominate if it were seen and the key
    just inside it (the oldest one seen) carries real weight."""
    g = torch.Generator().manual_seed(seed)
    k = U.bf16_exact(torch.randn(n, kv_heads, dim, generator=g))
    v = U.bf16_exact(torch.randn(n, kv_heads, vdim, generator=g))
    q = torch.randn(len(queries), heads, dim, generator=g)
    for qi, p in enumerate(queries):
        out_j, in_j = p - window, p - window + 1
        for h in range(heads):
            gk = h // (heads // kv_heads)
            if out_j >= 0:
                q[qi, h] += 2.0 * k[out_j, gk] / k[out_j, gk].norm()
            if in_j >= 0:
                q[qi, h] += 1.0 * k[in_j, gk] / k[in_j, gk].norm()
    return q, k, v


def _attend(q, k, v, queries, window, scale, unit):
    """float64 attention of query rows at positions `queries` over keys 0 .. position, windowed."""
    Q, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(Q, H, v.shape[2], dtype=torch.float64)
    for qi, p in enumerate(queries):
        mask = torch.zeros(1, k.shape[0], dtype=torch.bool)
        mask[0, max(0, p - window + 1):p + 1] = True
        for h in range(H):
            gk = h // (H // G)
            s = (k[:, gk].double() @ q[qi, h].double())[None, :] * scale
            out[qi, h] = (O.windowed_softmax(s, mask, unit) @ v[:, gk].double())[0]
    return out


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("shared", [0, 1])
@pytest.mark.parametrize("window,bs", [(1, 16), (5, 16), (32, 16), (33, 64), (127, 64), (128, 16), (129, 8), (400, 64)])
def test_windowed_attention_at_window_tile_and_block_edges(f32, shared, window, bs):
    """A prompt portion of 40 rows ending at position 299 and three single rows, over a context of 300 keys in shuffled blocks.
    Windows of 1, around the 32-key and 128-key tiles, across block borders and wider than the context."""
    heads, kv_heads, dim, vdim, n, scale = 4, 2, 20, 12, 300, 0.4
    queries = list(range(260, 300)) + [window - 1 if window <= 300 else 17, 131, 64]
    q, k, v = _spiked(n, heads, kv_heads, dim, vdim, queries, window, window * 7 + bs)
    want = _attend(q, k, v, queries, window, scale, True)
    nb = (n + bs - 1) // bs
    order = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(1)).tolist()
    kc, vc = _paged(k, bs, nb + 3, order, _adt(f32)), _paged(v, bs, nb + 3, order, _adt(f32))
    T = len(queries)
    # four "sequences" over the same blocks: the portion, and the single rows
    bt = i32([order[:nb]] * 4)
    rts = [0] * 40 + [1, 2, 3]
    ctx = [p + 1 for p in queries]
    out = torch.zeros(T, heads * vdim, dtype=_adt(f32), device=DEV)
    ws = torch.zeros(lib().b200_paged_attn_anydim_workspace_bytes(T), dtype=torch.uint8, device=DEV)
    sink = dev(torch.zeros(heads))
    check(lib().b200_paged_attn_window(f32, dev(q.reshape(T, -1)).data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), nb, i32(rts).data_ptr(),
                                       i32(ctx).data_ptr(), i32(queries).data_ptr(), out.data_ptr(), T, heads, kv_heads, dim, vdim, bs, scale,
                                       shared, ws.data_ptr(), 0, 0, sink.data_ptr(), window, None))
    sync()
    got = out.float().cpu().double().reshape(T, heads, vdim)
    assert torch.allclose(got, want, atol=3e-5 if f32 else 2e-2, rtol=0 if f32 else 2e-2)
    # the key outside would have been decisive: seeing one more key changes the result visibly
    wider = _attend(q, k, v, queries, window + 1, scale, True)
    if window < 250:
        assert float((wider - want).abs().max()) > 0.05


@pytest.mark.parametrize("window,bs,heads", [(1, 16, 3), (9, 16, 2), (64, 64, 4), (65, 16, 1), (72, 64, 8), (130, 128, 5), (1000, 64, 3)])
def test_windowed_latent_attention_on_the_tensor_cores(window, bs, heads):
    """One kv head whose value is the key row itself, bf16 cache, windows around the 64-key tile."""
    rank, n, scale = 48, 300, 0.35
    queries = list(range(250, 300)) + [min(window, 299), 63, 64, 200]
    q, k, _ = _spiked(n, heads, 1, rank, rank, queries, window, window + heads)
    want = _attend(q, k, k, queries, window, scale, False)
    nb = (n + bs - 1) // bs
    order = torch.randperm(nb + 2, generator=torch.Generator().manual_seed(2)).tolist()
    cache = _paged(k, bs, nb + 2, order, torch.bfloat16)
    T = len(queries)
    bt = i32([order[:nb]] * 5)
    rts = [0] * 50 + [1, 2, 3, 4]
    ctx = [p + 1 for p in queries]
    assert lib().b200_latent_attn_supported(heads, rank, rank)
    out = torch.zeros(T, heads * rank, dtype=torch.bfloat16, device=DEV)
    ws = torch.zeros(lib().b200_paged_attn_anydim_workspace_bytes(T), dtype=torch.uint8, device=DEV)
    check(lib().b200_latent_attn_window(dev(q.reshape(T, -1)).data_ptr(), cache.data_ptr(), bt.data_ptr(), nb, i32(rts).data_ptr(),
                                        i32(ctx).data_ptr(), out.data_ptr(), T, heads, rank, rank, bs, scale, None, ws.data_ptr(), window, None))
    sync()
    got = out.float().cpu().double().reshape(T, heads, rank)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)
    if window < 250:
        assert float((_attend(q, k, k, queries, window + 1, scale, False) - want).abs().max()) > 0.05


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("window,bs,heads,kv_heads,dim,vdim", [(1, 16, 4, 2, 32, 32), (63, 16, 6, 2, 48, 32), (64, 64, 4, 4, 64, 64), (65, 128, 8, 2, 128, 128),
                                                               (200, 64, 5, 1, 16, 16), (1000, 16, 2, 1, 160, 144)])
def test_windowed_grouped_attention_on_the_tensor_cores(splits, window, bs, heads, kv_heads, dim, vdim):
    """Key and value caches of their own, query heads grouped over kv heads, the extra unit in the denominator, windows around
    the 64-key tile, the context split over CTAs and merged."""
    n, scale = 300, 0.3
    queries = list(range(255, 300)) + [min(window, 299), 63, 64, 128]
    q, k, v = _spiked(n, heads, kv_heads, dim, vdim, queries, window, window + heads)
    want = _attend(q, k, v, queries, window, scale, True)
    nb = (n + bs - 1) // bs
    order = torch.randperm(nb + 2, generator=torch.Generator().manual_seed(3)).tolist()
    kc, vc = _paged(k, bs, nb + 2, order, torch.bfloat16), _paged(v, bs, nb + 2, order, torch.bfloat16)
    T = len(queries)
    bt = i32([order[:nb]] * 5)
    rts = [0] * 45 + [1, 2, 3, 4]
    ctx = [p + 1 for p in queries]
    assert lib().b200_paged_attn_mma_supported(heads, kv_heads, dim, vdim)
    out = torch.zeros(T, heads * vdim, dtype=torch.bfloat16, device=DEV)
    ws = torch.zeros(lib().b200_paged_attn_anydim_workspace_bytes(T), dtype=torch.uint8, device=DEV)
    part = torch.zeros(T * heads * splits * (vdim + 2), device=DEV)
    check(lib().b200_paged_attn_mma(dev(q.reshape(T, -1)).data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), nb, i32(rts).data_ptr(),
                                    i32(ctx).data_ptr(), out.data_ptr(), T, heads, kv_heads, dim, vdim, bs, scale, dev(torch.zeros(heads)).data_ptr(),
                                    ws.data_ptr(), window, splits, part.data_ptr(), None))
    sync()
    got = out.float().cpu().double().reshape(T, heads, vdim)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)
    if window < 250:
        assert float((_attend(q, k, v, queries, window + 1, scale, True) - want).abs().max()) > 0.05


@pytest.mark.parametrize("f32", [1, 0])
def test_latent_norms_and_the_gate_of_one_number_per_head(f32):
    g = torch.Generator().manual_seed(8)
    T, qr, kr, heads, vdim, eps = 6, 36, 28, 3, 10, 1e-5
    ld = qr + kr + heads
    fused = U.bf16_exact(torch.randn(T, ld, generator=g) * 2)
    qw, kw = 1 + 0.3 * torch.randn(qr, generator=g), 1 + 0.3 * torch.randn(kr, generator=g)
    slots = [3, 9, 0, 1, 14, 2]
    cq = torch.zeros(T, qr, dtype=_adt(f32), device=DEV)
    cache = torch.full((16, kr), 5.0, dtype=_adt(f32), device=DEV)
    check(lib().b200_latent_norms(f32, dev(fused, _adt(f32)).data_ptr(), ld, qr, kr, dev(qw).data_ptr(), dev(kw).data_ptr(), i32(slots).data_ptr(),
                                  cq.data_ptr(), cache.data_ptr(), T, eps, None))
    sync()
    tol = dict(atol=2e-5) if f32 else dict(atol=3e-2, rtol=1e-2)
    assert torch.allclose(cq.float().cpu().double(), O.rms_norm(fused[:, :qr].double(), qw.double(), eps), **tol)
    assert torch.allclose(cache[slots].float().cpu().double(), O.rms_norm(fused[:, qr:qr + kr].double(), kw.double(), eps), **tol)
    assert float(cache[4, 0]) == 5.0
    # a layer that reads another layer's latents writes no cache row
    check(lib().b200_latent_norms(f32, dev(fused, _adt(f32)).data_ptr(), ld, qr, kr, dev(qw).data_ptr(), None, None, cq.data_ptr(), None, T, eps, None))
    sync()
    # expansion with the gate: y[t, h] = (W[h] x[t, h]) * sigmoid(gate[t, h])
    x = U.bf16_exact(torch.randn(T, heads * kr, generator=g))
    wv = U.bf16_exact(torch.randn(heads * vdim, kr, generator=g) * 0.3)
    y = torch.zeros(T, heads * vdim, dtype=_adt(f32), device=DEV)
    fd = dev(fused, _adt(f32))
    check(lib().b200_head_linear_head_gate(f32, dev(x, _adt(f32)).data_ptr(), heads * kr, kr, dev(wv, torch.bfloat16).data_ptr(), y.data_ptr(),
                                           heads * vdim, vdim, fd.data_ptr() + (qr + kr) * fd.element_size(), ld, T, heads, vdim, kr, None))
    sync()
    want = torch.einsum("thk,hvk->thv", x.double().reshape(T, heads, kr), wv.double().reshape(heads, vdim, kr))
    want = want * torch.sigmoid(fused[:, qr + kr:].double())[:, :, None]
    assert torch.allclose(y.float().cpu().double().reshape(T, heads, vdim), want, **(dict(atol=2e-5) if f32 else dict(atol=3e-2, rtol=2e-2)))


def _portions(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n))
        at += n
        i += 1
    return out


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 20, 12, 3), (1, 1, 72, 40, 1), (3, 3, 33, 70, 5), (2, 1, 130, 8, 2)])
def test_delta_rule_in_portions_with_two_sequences_and_dirty_slots(f32, heads, kv_heads, dim, vdim, taps):
    """Convolution tails shorter and longer than the portions, a state carried over many steps, key sizes across the 32-lane
    groups, a second sequence that starts later in a slot the first request of another shape left dirty.  The oracle runs each
    sequence whole; its output projection is the identity so that the comparison is of the gated, normed read-out."""
    W, ra, rg, eps = 48, 10, 6, 1e-5
    layer = F.delta(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=taps, a_rank=ra, g_rank=rg)
    cfg = F.make_cfg(width=W, layers=[layer])
    w = F.make_weights(cfg, dim + taps)
    w["l0.mix.o"] = torch.eye(heads * vdim)
    p = O.sub({k: v.double() for k, v in w.items()}, "l0.mix.")
    g = torch.Generator().manual_seed(3)
    n = {"a": 53, "b": 21}
    h = {k: U.bf16_exact(torch.randn(v, W, generator=g)) for k, v in n.items()}
    want = {k: O.channel_delta_mixer(h[k].double(), p, layer["mixer"], eps) for k in n}
    off = (pkg("_abi").C.c_int32 * 6)()
    qr = lib().b200_delta_fused_rows(heads, kv_heads, dim, vdim, ra, rg, off)
    Wf = torch.zeros(qr, W, dtype=torch.float64)
    for o, name in zip(off, ("q", "k", "v", "a1", "g1", "b")):
        Wf[o:o + p[name].shape[0]] = p[name]
    C, hd, av = 2 * kv_heads * dim + heads * vdim, heads * dim, heads * vdim
    tail_f = max(taps - 1, 0) * C
    slot_f = (tail_f + 3) // 4 * 4 + heads * vdim * dim + 8
    state = dev(torch.full((3, slot_f), 11.0))
    tails_ptr, rec_ptr = state.data_ptr(), state.data_ptr() + ((tail_f + 3) // 4 * 4) * 4
    conv = dev(torch.cat([p["q.conv"], p["k.conv"], p["v.conv"]]).float())
    sched = {"a": _portions(53, [1, 2, 1, 3, 17, 1, 1, 2, 9]), "b": _portions(21, [2, 1, 1, 6, 1, 3])}
    slot, got = {"a": 2, "b": 0}, {k: torch.zeros(v, av) for k, v in n.items()}
    adt = _adt(f32)
    for step in range(max(len(v) for v in sched.values()) + 2):
        names = [k for k in ("a", "b") if (k == "a" and step < len(sched["a"])) or (k == "b" and 2 <= step < len(sched["b"]) + 2)]
        if not names:
            continue
        rows, pos, rts, start = [], [], [], [0]
        for si, k in enumerate(names):
            lo, cnt = sched[k][step - (2 if k == "b" else 0)]
            rows.append(h[k][lo:lo + cnt])
            pos += list(range(lo, lo + cnt))
            rts += [si] * cnt
            start.append(start[-1] + cnt)
        x = torch.cat(rows).double()
        T, S = x.shape[0], len(names)
        fused = dev((x @ Wf.T).float(), adt)
        a2 = dev((fused[:, off[3]:off[3] + ra].double().cpu() @ p["a2"].T).float(), adt)
        g2 = dev((fused[:, off[4]:off[4] + rg].double().cpu() @ p["g2"].T).float(), adt)
        qn, kn = torch.zeros(T, kv_heads * dim, device=DEV), torch.zeros(T, kv_heads * dim, device=DEV)
        vn, beta, dec = torch.zeros(T, av, device=DEV), torch.zeros(T, heads, device=DEV), torch.zeros(T, hd, device=DEV)
        pos_d, rts_d, start_d, slots_d = i32(pos), i32(rts), i32(start), i32([slot[k] for k in names])
        check(lib().b200_delta_prep(f32, fused.data_ptr(), qr, a2.data_ptr(), conv.data_ptr(), dev(p["dt_bias"].float()).data_ptr(),
                                    dev(p["A_log"].float()).data_ptr(), pos_d.data_ptr(), rts_d.data_ptr(), start_d.data_ptr(), slots_d.data_ptr(),
                                    tails_ptr if taps > 1 else None, slot_f, qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), beta.data_ptr(),
                                    dec.data_ptr(), T, heads, kv_heads, dim, vdim, taps, ra, rg, None))
        if taps > 1:
            check(lib().b200_delta_tails(f32, fused.data_ptr(), qr, pos_d.data_ptr(), start_d.data_ptr(), slots_d.data_ptr(), tails_ptr, slot_f, S, C,
                                         taps, None))
        oraw = torch.zeros(T, av, device=DEV)
        check(lib().b200_delta_scan(qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), beta.data_ptr(), dec.data_ptr(), pos_d.data_ptr(), start_d.data_ptr(),
                                    slots_d.data_ptr(), rec_ptr, slot_f, oraw.data_ptr(), S, heads, kv_heads, dim, vdim, None))
        out = torch.zeros(T, av, dtype=adt, device=DEV)
        check(lib().b200_head_norm_gate(f32, oraw.data_ptr(), dev(p["norm"].float().repeat(heads)).data_ptr(), g2.data_ptr(), av, out.data_ptr(), T,
                                        heads, vdim, eps, None))
        sync()
        for si, k in enumerate(names):
            lo, cnt = sched[k][step - (2 if k == "b" else 0)]
            got[k][lo:lo + cnt] = out[start[si]:start[si + 1]].float().cpu()
    for k in n:
        if f32:
            assert torch.allclose(got[k].double(), want[k], atol=5e-5, rtol=1e-4), k
        else:      # inputs rounded to bf16 before the convolution and the gates
            err = (got[k].double() - want[k]).abs()
            assert float(err.mean()) < 0.02 and float(err.max()) < 0.3, (k, float(err.mean()), float(err.max()))
    assert float(state[1].min()) == 11.0 and float(state[1].max()) == 11.0          # the unused slot


# ---- whole models ----------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def model_a():
    cfg = F.make_cfg()
    return cfg, F.make_weights(cfg, 1)


ALONE = {
    "attention alone, grouped heads, window shorter than the prompt": [F.attention(mlp=F.dense())],
    "attention without rotation, window of one": [F.attention(window=1, rot_dims=0, heads=2, kv_heads=2)],
    "attention with every dimension turning, unscaled, window longer than the prompt": [F.attention(window=500, rot_dims=24, scaling=None)],
    "latent attention alone": [F.latent()],
    "latent attention reading the first layer's latents": [F.latent(window=4), F.latent(kv_from=0, heads=2, dim=8, vdim=16, q_rank=8, window=13)],
    "a latent layer of more heads than the shared-tile kernel takes, then attention that walks the step's run list":
        [F.latent(heads=12, dim=8, vdim=8, kv_rank=16, q_rank=16, window=20), F.attention()],
    "delta rule alone": [F.delta()],
    "delta rule, one tap, one q/k head for all heads": [F.delta(heads=3, kv_heads=1, conv=1, mlp=F.dense(24))],
}


@pytest.mark.parametrize("which", list(ALONE))
def test_one_mechanism_models_and_their_streams_fp32(which):
    cfg = F.make_cfg(width=64, layers=ALONE[which])
    w = F.make_weights(cfg, 4)
    ids = _prompt(cfg, 50, 1)
    r = F.make_runner(cfg, w, "float32")
    tap = r.set_stream_tap(True)
    got = U.replay(U.make_engine(r), [[("p", 50)]], {"p": ids})["p"]
    want, streams = O.forward(F.public_cfg(cfg), w, ids)
    assert U.rel_rms(got, want.numpy()).max() < F32_TOL
    L = len(cfg["layers"])
    t = tap[:L * 50 * 64].view(L, 50, 64).cpu().double()
    assert torch.allclose(t, streams, atol=1e-4, rtol=1e-5)
    r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["odd sizes", "tensor-core sizes", "one of each, alpha one"])
def test_other_sizes_and_constants(dtype, variant):
    """Widths, ranks and head sizes no vector access or TMA box fits; sizes that take every tensor-core path; constants that
    another model may make 1 or equal."""
    if variant == "odd sizes":
        cfg = F.make_cfg(width=100, vocab=131, alpha=0.5, eps=1e-3, layers=[
            F.delta(heads=1, kv_heads=1, dim=34, vdim=50, conv=2, a_rank=7, g_rank=3, mlp=F.dense(44)),
            F.latent(heads=5, dim=10, vdim=14, kv_rank=18, q_rank=22, window=3, mlp=F.dense(20)),
            F.attention(heads=6, kv_heads=2, dim=10, window=40, rot_dims=6, scaling=dict(factor=2.0, low=2.0, high=5.0, original=16)),
            F.latent(heads=1, dim=130, vdim=6, kv_rank=18, q_rank=5, window=100, kv_from=1)])
    elif variant == "tensor-core sizes":
        cfg = F.make_cfg(width=128, vocab=256, layers=[
            F.latent(heads=4, dim=32, vdim=32, kv_rank=64, q_rank=64, window=20, mlp=F.dense(128)),
            F.delta(heads=2, kv_heads=2, dim=64, vdim=64, conv=4, a_rank=16, g_rank=16),
            F.attention(heads=4, kv_heads=4, dim=64, window=33, rot_dims=64, mlp=F.dense(64)),
            F.latent(heads=17, dim=16, vdim=8, kv_rank=64, q_rank=32, window=70, kv_from=0)])
    else:
        cfg = F.make_cfg(width=48, alpha=1.0, layers=[F.attention(heads=1, kv_heads=1, dim=48, window=7, rot_dims=2),
                                                        F.delta(heads=1, kv_heads=1, dim=8, vdim=8, conv=8, a_rank=1, g_rank=1),
                                                        F.latent(heads=1, dim=8, vdim=8, kv_rank=8, q_rank=8, window=2)])
    w = F.make_weights(cfg, 6)
    ids = _prompt(cfg, 45, 2)
    want = O.forward(F.public_cfg(cfg), w, ids)[0].numpy()
    r = F.make_runner(cfg, w, dtype)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("p", 45)]], {"p": ids})["p"]
    cut = U.replay(eng, [[("p", n)] for n in (2, 7, 1, 1, 16, 2, 16)], {"p": ids})["p"]
    if dtype == "float32":
        assert U.rel_rms(whole, want).max() < F32_TOL and U.rel_rms(cut, want).max() < F32_TOL
    else:
        e = U.rel_rms(whole, want)
        assert np.median(e) < 0.03 and (e < 0.15).mean() > 0.9, (float(np.median(e)), float(e.max()))
        d = U.rel_rms(cut, whole)
        assert np.median(d) < 0.02 and (d < 0.15).mean() > 0.9, (float(np.median(d)), float(d.max()))
    r.close()


def test_every_schedule_gives_the_oracles_logits_fp32(model_a):
    """Prefill against token-by-token decoding, portions down to two tokens, unequal requests batched, a long decode tail that
    carries every window past the prompt, blocks and state slots that are freed and taken again (12 blocks of 16 where the four
    requests need 22; four slots for the requests of all schedules)."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3), "c": _prompt(cfg, 3, 4), "d": _prompt(cfg, 110, 5)}
    want = {n: O.forward(F.public_cfg(cfg), w, p)[0].numpy() for n, p in prompts.items()}
    r = F.make_runner(cfg, w, "float32", n_blocks=12, max_tokens=128)
    eng = U.make_engine(r)
    schedules = {
        "token by token": [[("c", 1)]] * 3 + [[("b", 1)]] * 37,
        "portions": [[("a", n)] for n in (2, 14, 1, 16, 17, 2, 2, 3, 13)],
        "prefill then a long decode": [[("d", 30)]] + [[("d", 1)]] * 80,
        "mixed": ([[("a", 33), ("c", 1)], [("c", 1), ("b", 2), ("a", 2)], [("b", 30), ("a", 1), ("c", 1)]] +
                  [[("a", 1), ("b", 1)]] * 5 + [[("a", 29)]] + [[("d", 64)], [("d", 2)], [("d", 44)]]),
    }
    for name, sched in schedules.items():
        got = U.replay(eng, sched, prompts)
        assert len(eng.blocks.free) == 12, name
        for n, l in got.items():
            assert l.shape[0] == len(prompts[n]), (name, n)
            assert U.rel_rms(l, want[n]).max() < F32_TOL, (name, n)
    r.close()


def test_a_request_left_out_of_steps_goes_on_where_it_stopped(model_a):
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 40, 21), "b": _prompt(cfg, 40, 22)}
    want = {n: O.forward(F.public_cfg(cfg), w, p)[0].numpy() for n, p in prompts.items()}
    r = F.make_runner(cfg, w, "float32")
    sched = [[("a", 7)], [("b", 9)], [("b", 1)], [("a", 2), ("b", 1)], [("b", 29)], [("a", 31)]]
    got = U.replay(U.make_engine(r), sched, prompts)
    for n in prompts:
        assert U.rel_rms(got[n], want[n]).max() < F32_TOL, n
    r.close()


def test_graph_replay_gives_the_same_logits_as_eager_steps(model_a):
    """Steps of equal shape replay one captured graph: sequence bounds, slots, windows and positions must come from the step's
    device metadata, not from what was captured."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 40, 7), "b": _prompt(cfg, 40, 8)}
    sched = [[("a", 8), ("b", 8)]] * 3 + [[("a", 1), ("b", 1)]] * 16
    out = []
    for graphs in (False, True):
        r = F.make_runner(cfg, w, "float32", graphs=graphs)
        out.append(U.replay(U.make_engine(r), sched, prompts))
        r.close()
    for n in prompts:
        assert np.array_equal(out[0][n], out[1][n]), n


def test_bf16_mode_within_bf16_noise_and_equal_across_schedules(model_a):
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3)}
    want = {n: O.forward(F.public_cfg(cfg), w, p)[0].numpy() for n, p in prompts.items()}
    r = F.make_runner(cfg, w, "bfloat16", n_blocks=12, max_tokens=128)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("a", 70)], [("b", 37)]], prompts)
    mixed = U.replay(eng, [[("a", 40), ("b", 2)], [("b", 20), ("a", 1)]] + [[("a", 1), ("b", 1)]] * 15 + [[("a", 14)]], prompts)
    for n in prompts:
        e = U.rel_rms(whole[n], want[n])
        assert np.median(e) < 0.03 and (e < 0.1).mean() > 0.9, (n, float(np.median(e)), float(e.max()))
        d = U.rel_rms(mixed[n], whole[n])
        assert np.median(d) < 0.02 and (d < 0.1).mean() > 0.9, (n, float(np.median(d)), float(d.max()))
    r.close()


def test_gate_activation_in_the_linears_epilogue_equals_the_separate_kernel(monkeypatch):
    """Feed-forward widths that are multiples of 64 take interleaved gate|up slabs and activate in the tcgen05 epilogue; relu of a
    bf16 value is exact, so the logits equal those of the plain linear followed by the activation kernel bit for bit."""
    cfg = F.make_cfg(width=128, vocab=256, layers=[F.latent(heads=4, dim=32, vdim=32, kv_rank=64, q_rank=64, window=20, mlp=F.dense(192)),
                                                   F.delta(heads=2, kv_heads=1, dim=32, vdim=32, mlp=F.dense(64)),
                                                   F.attention(heads=2, kv_heads=1, dim=32, window=12, mlp=F.dense(100))])
    w = F.make_weights(cfg, 9)
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 9, 3)}
    sched = [[("a", 40), ("b", 2)], [("b", 7), ("a", 1)]] + [[("a", 1)]] * 5 + [[("a", 24)]]
    out = []
    for fuse in ("1", "0"):
        monkeypatch.setenv("B200_STACK_FUSE_GATE_UP", fuse)
        r = F.make_runner(cfg, w, "bfloat16")
        assert r.fuse_gate_up == (fuse == "1")
        out.append(U.replay(U.make_engine(r), sched, prompts))
        r.close()
    for n in prompts:
        assert np.array_equal(out[0][n], out[1][n]), n
    want = O.forward(F.public_cfg(cfg), w, prompts["a"])[0].numpy()
    e = U.rel_rms(out[0]["a"], want)
    assert np.median(e) < 0.03 and e.max() < 0.15


def test_greedy_generation_through_the_engines_own_scheduler(model_a, tmp_path):
    """A checkpoint directory goes through the registry (which sizes the delta layers from the tensor shapes), the weight loader,
    LLMEngine.generate and the scheduler (which hands out blocks and state slots and overlaps steps); prompts of unequal length
    decode side by side, past every window."""
    cfg, w = model_a
    path = str(tmp_path / "ckpt")
    U.write_checkpoint(path, F.public_cfg(cfg), w)
    pc = pkg("config").load_model_config(path)
    assert type(pc).__name__ == "FutidraConfig"
    r = pkg("runner").make_runner(pc, dtype="float32", max_tokens=64, max_model_len=256, block_size=16, n_blocks=40, n_state_slots=4)
    r.load_weights(pkg("weights").load_safetensors_dir(path))
    eng = pkg("engine").LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=8, max_model_len=256)
    assert eng.scheduler.max_seqs == 3          # bounded by the state slots
    prompts = [_prompt(cfg, 21, 11), _prompt(cfg, 5, 12), _prompt(cfg, 70, 13), _prompt(cfg, 9, 14)]
    got = eng.generate(prompts, max_tokens=14)
    for p, out in zip(prompts, got):
        ids = list(p)
        for tok in out:      # every emitted token is the oracle's arg-max, or within fp32 noise of it
            z = O.forward(F.public_cfg(cfg), w, ids)[0][-1]
            assert tok == int(z.argmax()) or float(z.max() - z[tok]) < 1e-3 * float(z.abs().max())
            ids.append(tok)
    r.close()


def test_samplers_and_log_probabilities_read_the_steps_logits(model_a):
    """Sampled requests go through the framework's samplers after the step: with top_k = 1 a request at temperature 0.9 emits the
    greedy tokens; the log-probabilities of the emitted tokens are the oracle's log-softmax (the samplers read bf16 logits); a
    plain greedy request in the same batch is untouched by its neighbours."""
    cfg, w = model_a
    E = pkg("engine")
    r = F.make_runner(cfg, w, "float32", max_tokens=64, max_model_len=256, n_blocks=40)
    eng = E.LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=4, max_model_len=256)
    p = _prompt(cfg, 19, 31)
    greedy = eng.generate([p], max_tokens=10)[0]
    reqs = [E.Request("s", list(p), max_tokens=10, ignore_eos=True, temperature=0.9, top_k=1, seed=5),
            E.Request("l", list(p), max_tokens=10, ignore_eos=True, logprobs=2),
            E.Request("g", list(p), max_tokens=10, ignore_eos=True)]
    for q in reqs:
        eng.add_request(q)
    while eng.has_work():
        eng.step()
    assert reqs[0].output_ids == greedy and reqs[1].output_ids == greedy and reqs[2].output_ids == greedy
    ids = list(p)
    for tok, (lp, top) in zip(reqs[1].output_ids, reqs[1].logprob_data):
        z = torch.log_softmax(O.forward(F.public_cfg(cfg), w, ids)[0][-1], -1)
        assert abs(lp - float(z[tok])) < 0.05 and top[0][0] == int(z.argmax())
        ids.append(tok)
    r.close()
