"""GPU parity of the Rudolix design against oracle/rudolix_oracle.py: every mechanism alone through its per-kernel entry point
(with inputs built so that a lost far key, a sink left out, a stale state or a wrong tail shows), then whole models through the
runner, externally scheduled steps of the engine, and its own scheduler.  32-bit mode is held to the float64 oracle tightly; bf16
mode within bf16 noise, and to itself across schedules."""
import math

import numpy as np
import pytest
import torch

import rudolix_util as R
import stack_util as U
from conftest import pkg
from oracle import rudolix_oracle as O

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


def _portions(n, sizes):
    out, lo = [], 0
    for s in sizes:
        if lo >= n:
            break
        out.append((lo, min(s, n - lo)))
        lo += out[-1][1]
    if lo < n:
        out.append((lo, n - lo))
    return out


# ---- mechanisms alone ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("n,width", [(1, 40), (2, 257), (3, 64), (4, 1024), (8, 72)])
def test_streams_close_one_sublayer_and_open_the_next(f32, n, width):
    """The three uses of the kernel: the first launch of a step (every stream takes the embedding), a close with an activation row or
    with expert partial rows followed by an open, and the last launch over picked rows with unit read weights."""
    g = torch.Generator().manual_seed(n * 1000 + width)
    T, eps, mult, stride = 7, 1e-5, 0.3, 9 * width
    adt = _adt(f32)
    x0 = torch.randn(T, width, generator=g, dtype=torch.float64)
    a1, a2 = torch.randn(n, generator=g, dtype=torch.float64), torch.randn(n, generator=g, dtype=torch.float64)
    b1 = torch.randn(n, generator=g, dtype=torch.float64)
    M1 = torch.eye(n, dtype=torch.float64) + 0.3 * torch.randn(n, n, generator=g, dtype=torch.float64)
    w, b = 1 + 0.1 * torch.randn(width, generator=g, dtype=torch.float64), 0.2 * torch.randn(width, generator=g, dtype=torch.float64)
    ls = 1 + 0.3 * torch.randn(width, generator=g, dtype=torch.float64)
    X = dev(torch.full((n, 9, width), 7.0))
    X[0, :T] = x0.float().to(DEV)
    h = torch.zeros(T, width, device=DEV)
    hc1 = dev(torch.cat([a1, b1, M1.reshape(-1)]).float())
    wd, bd, lsd = dev(w.float()), dev(b.float()), dev(ls.float())
    check(lib().b200_hyper_step(f32, X.data_ptr(), stride, n, 1, None, None, 0, None, None, mult, hc1.data_ptr(), wd.data_ptr(), bd.data_ptr(), eps,
                                None, h.data_ptr(), None, None, T, width, None))
    sync()
    x0f = x0.float().double()
    assert torch.allclose(h.cpu().double(), O.layer_norm(a1.float().double().sum() * x0f, w.float().double(), b.float().double(), eps), atol=2e-5)
    assert all(torch.equal(X[s, :T].cpu(), x0.float()) for s in range(n)) and float(X[:, T:].min()) == 7.0
    # close with an activation row, open with other coefficients; the sum of the streams on the side
    xs = torch.randn(n, T, width, generator=g, dtype=torch.float64).float()
    X[:, :T] = xs.to(DEV)
    y = U.bf16_exact(torch.randn(T, width, generator=g))
    open2 = dev(a2.float())
    act, tot = torch.zeros(T, width, dtype=adt, device=DEV), torch.zeros(T, width, device=DEV)
    check(lib().b200_hyper_step(f32, X.data_ptr(), stride, n, 0, dev(y, adt).data_ptr(), None, 0, lsd.data_ptr(), hc1.data_ptr(), mult, open2.data_ptr(),
                                wd.data_ptr(), bd.data_ptr(), eps, None, None, act.data_ptr(), tot.data_ptr(), T, width, None))
    sync()
    c = {k: v.float().double() for k, v in dict(a2=a2, b1=b1, M1=M1, w=w, b=b, ls=ls).items()}
    new = [sum(c["M1"][s, t] * xs[s].double() for s in range(n)) + mult * c["b1"][t] * (y.double() * c["ls"]) for t in range(n)]
    for t in range(n):
        assert torch.allclose(X[t, :T].cpu().double(), new[t], atol=1e-5), t
    assert torch.allclose(tot.cpu().double(), sum(new), atol=1e-5)
    want = O.layer_norm(sum(c["a2"][t] * new[t] for t in range(n)), c["w"], c["b"], eps)
    assert torch.allclose(act.float().cpu().double(), want, atol=2e-5 if f32 else 3e-2)
    # close with partial rows over picked rows: the streams stay as they are, the read weights are ones
    X[:, :T] = xs.to(DEV)
    parts = torch.randn(T, 3, width, generator=g)
    rows = [5, 0, 6]
    out = torch.zeros(3, width, dtype=adt, device=DEV)
    check(lib().b200_hyper_step(f32, X.data_ptr(), stride, n, 0, None, dev(parts).data_ptr(), 3, lsd.data_ptr(), hc1.data_ptr(), mult, None, wd.data_ptr(),
                                bd.data_ptr(), eps, i32(rows).data_ptr(), None, out.data_ptr(), None, 3, width, None))
    sync()
    yp = parts.double().sum(1)
    new = [sum(c["M1"][s, t] * xs[s].double() for s in range(n)) + mult * c["b1"][t] * (yp * c["ls"]) for t in range(n)]
    want = O.layer_norm(sum(new)[rows], c["w"], c["b"], eps)
    assert torch.allclose(out.float().cpu().double(), want, atol=3e-5 if f32 else 3e-2)
    assert torch.equal(X[:, :T].cpu(), xs)


def _paged(T, bs, seed):
    """A shuffled block table for one sequence of T tokens and the slot of each token."""
    nb = (T + bs - 1) // bs
    perm = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(seed)).tolist()[:nb]
    return perm, [perm[t // bs] * bs + t % bs for t in range(T)], nb + 3


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot_dims,bs,T", [(4, 2, 24, 20, 16, 16, 150), (3, 3, 32, 48, 32, 64, 300), (2, 1, 16, 16, 0, 16, 33),
                                                                   (6, 2, 64, 32, 32, 128, 400), (5, 1, 40, 8, 2, 8, 70)])
def test_rotation_cache_and_attention_with_a_sink_and_a_far_key(f32, heads, kv_heads, dim, vdim, rot_dims, bs, T):
    """Rows go into the paged caches in portions (shuffled blocks), then every row attends.  The last rows ask for key 3, hundreds of
    places back: that key and those queries carry a large entry in a dimension that does not turn, so the far key outweighs all
    others together and the sink is of the same size as its score: a lost key or a dropped sink changes the output by order one."""
    g = torch.Generator().manual_seed(T + dim)
    scale, base = 0.25, 3000.0
    nq, nk = heads * dim, kv_heads * dim
    qkv = U.bf16_exact(torch.randn(T, nq + nk + kv_heads * vdim, generator=g))
    far = dim - 1 if rot_dims < dim else None
    sink = torch.randn(heads, generator=g)
    if far is not None:
        for kh in range(kv_heads):
            qkv[3, nq + kh * dim + far] = 8.0
        for h in range(heads):
            qkv[T - 2:, h * dim + far] = 8.0
        sink[:] = scale * 64.0 + torch.tensor([0.5, -0.5, 0.0, 1.0, -1.0, 0.3])[:heads]
    qkv = U.bf16_exact(qkv)
    pos = torch.arange(T)
    q = O.rotate_half(qkv[:, :nq].double().view(T, heads, dim), pos, rot_dims, base)
    k = O.rotate_half(qkv[:, nq:nq + nk].double().view(T, kv_heads, dim), pos, rot_dims, base)
    v = qkv[:, nq + nk:].double().view(T, kv_heads, vdim)
    want = O.sink_attention(q, k, v, scale, sink.double())
    if far is not None:      # the construction bites: without the sink, or without key 3, the last row differs by order one
        assert float((O.sink_attention(q, k, v, scale, sink.double() - 50.0)[-1] - want[-1]).abs().max()) > 0.1
    adt = _adt(f32)
    table, slots, nb = _paged(T, bs, T)
    kc = dev(torch.full((nb, kv_heads, bs, dim), 3.0, dtype=adt))
    vc = dev(torch.full((nb, kv_heads, bs, vdim), 3.0, dtype=adt))
    rot = dev(pkg("config").RotarySpec(base=base, dims=rot_dims).table(T + 5)) if rot_dims else None
    qout = torch.zeros(T, nq, device=DEV)
    fused = dev(qkv, adt)
    for lo, cnt in _portions(T, [1, 2, 13, 1, 50, 3]):
        check(lib().b200_qkv_rotate_cache(f32, fused[lo:].data_ptr(), fused.shape[1], i32(list(range(lo, lo + cnt))).data_ptr(),
                                          i32(slots[lo:lo + cnt]).data_ptr(), rot.data_ptr() if rot is not None else None, rot_dims, 1, T + 5,
                                          qout[lo:].data_ptr(), kc.data_ptr(), vc.data_ptr(), cnt, heads, kv_heads, dim, vdim, bs, None))
    sync()
    assert torch.allclose(qout.cpu().double().view(T, heads, dim), q, atol=1e-5)
    tol = 3e-5 if f32 else 3e-2
    bt, ctx, rts, posd = i32(table), i32(list(range(1, T + 1))), i32([0] * T), i32(list(range(T)))
    ws = dev(torch.zeros(lib().b200_paged_attn_anydim_workspace_bytes(T) // 4 + 4, dtype=torch.int32))
    sk = dev(sink)
    for shared in (0, 1):
        out = torch.zeros(T, heads * vdim, dtype=adt, device=DEV)
        check(lib().b200_paged_attn_window(f32, qout.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), len(table), rts.data_ptr(), ctx.data_ptr(),
                                           posd.data_ptr(), out.data_ptr(), T, heads, kv_heads, dim, vdim, bs, scale, shared, ws.data_ptr(), 0, 0,
                                           sk.data_ptr(), 0, None))
        sync()
        assert torch.allclose(out.float().cpu().double().view(T, heads, vdim), want, atol=tol, rtol=tol), shared
    if not f32 and lib().b200_paged_attn_mma_supported(heads, kv_heads, dim, vdim):
        for splits in (1, 3):
            out = torch.zeros(T, heads * vdim, dtype=adt, device=DEV)
            part = dev(torch.zeros(T * heads * splits * (vdim + 2)))
            check(lib().b200_paged_attn_mma(qout.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), len(table), rts.data_ptr(), ctx.data_ptr(),
                                            out.data_ptr(), T, heads, kv_heads, dim, vdim, bs, scale, sk.data_ptr(), ws.data_ptr(), 0, splits,
                                            part.data_ptr(), None))
            sync()
            assert torch.allclose(out.float().cpu().double().view(T, heads, vdim), want, atol=5e-2, rtol=5e-2), splits


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("taps", [1, 2, 4, 8, 9])
def test_input_convolution_over_long_steps_with_many_sequences(f32, taps):
    """Steps of a hundred rows and more take the kernel that slides a window of inputs along a run of rows: sequences of one, two and
    many rows side by side, runs that start in the middle of a sequence, then a second step that continues every sequence from its
    tail (slots shuffled, the unused slot dirty)."""
    g = torch.Generator().manual_seed(taps)
    width, hist = 70, taps - 1
    lens = [[1, 2, 3, 70, 5, 130, 17], [40, 1, 64, 2, 1, 33, 16]]
    n_seq = len(lens[0])
    h = [U.bf16_exact(torch.randn(lens[0][i] + lens[1][i], width, generator=g)) for i in range(n_seq)]
    w = U.bf16_exact(0.5 * torch.randn(width, taps, generator=g))
    want = [x.double() + O.causal_conv(x.double(), w.double()) for x in h]
    slot_f = hist * width + 4
    slots = [5, 0, 3, 1, 6, 2, 7]
    state = dev(torch.full((8, slot_f), 9.0))
    adt = _adt(f32)
    done = [0] * n_seq
    for step in range(2):
        rows, pos, rts, start = [], [], [], [0]
        for i in range(n_seq):
            n = lens[step][i]
            rows.append(h[i][done[i]:done[i] + n])
            pos += list(range(done[i], done[i] + n))
            rts += [i] * n
            start.append(start[-1] + n)
        x = dev(torch.cat(rows))
        T = x.shape[0]
        out = torch.zeros(T, width, dtype=adt, device=DEV)
        check(lib().b200_canon_conv(f32, x.data_ptr(), dev(w).data_ptr(), out.data_ptr(), T, width, taps, i32(pos).data_ptr(), i32(rts).data_ptr(),
                                    i32(start).data_ptr(), i32(slots).data_ptr(), state.data_ptr() if hist else None, slot_f, None))
        sync()
        for i in range(n_seq):
            n = lens[step][i]
            got = out[start[i]:start[i + 1]].float().cpu().double()
            assert torch.allclose(got, want[i][done[i]:done[i] + n], atol=1e-5 if f32 else 3e-2, rtol=0 if f32 else 1e-2), (step, i)
            done[i] += n
    assert float(state[4].min()) == 9.0 and float(state[4].max()) == 9.0


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("ff", [7, 64, 1000])
def test_polynomial_of_unit_rms_powers(f32, ff):
    g = torch.Generator().manual_seed(ff)
    z = U.bf16_exact(1.5 * torch.randn(9, ff, generator=g))
    coef = torch.tensor([0.9, 0.4, -0.3, 0.1])
    adt = _adt(f32)
    out = torch.zeros(9, ff, dtype=adt, device=DEV)
    check(lib().b200_polynorm(f32, dev(z, adt).data_ptr(), dev(coef).data_ptr(), out.data_ptr(), 9, ff, 1e-5, None))
    sync()
    want = O.poly_norm(z.double(), coef.double(), 1e-5)
    assert torch.allclose(out.float().cpu().double(), want, atol=1e-5 if f32 else 3e-2, rtol=1e-5 if f32 else 1e-2)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("ff", [7, 24, 1024])
def test_clamped_gate_activation_rows(f32, ff):
    g = torch.Generator().manual_seed(ff)
    gu = U.bf16_exact(2.0 * torch.randn(11, 2 * ff, generator=g))
    adt = _adt(f32)
    out = torch.zeros(11, ff, dtype=adt, device=DEV)
    check(lib().b200_ff_act_limit(f32, dev(gu, adt).data_ptr(), out.data_ptr(), 11, ff, 1, pkg("_abi").ACT_SWIGLU_CLAMP, 1.25, None))
    sync()
    a, b = gu[:, :ff].double().clamp(max=1.25), gu[:, ff:].double().clamp(-1.25, 1.25)
    want = a * torch.sigmoid(1.702 * a) * (b + 1.0)
    assert float((gu[:, :ff] > 1.25).sum()) > 0 and float((gu[:, ff:] < -1.25).sum()) > 0
    assert torch.allclose(out.float().cpu().double(), want, atol=1e-5 if f32 else 2e-2, rtol=1e-5 if f32 else 1e-2)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("T,width,experts,top,ff", [(5, 40, 6, 2, 24), (130, 64, 5, 5, 16), (70, 72, 9, 1, 40), (3, 33, 4, 3, 7)])
def test_chosen_softmax_router_and_clamped_experts(f32, T, width, experts, top, ff):
    """Logits with the bias inside, the largest win, weights over the winners alone; experts whose gate is capped from above and whose
    up value is clamped on both sides (inputs large enough that every clamp acts).  All three expert forms run: one CTA per pair,
    grouped tiles (many tokens), and in bf16 the tensor-core form where the sizes allow."""
    g = torch.Generator().manual_seed(T + width)
    limit = 0.8
    x = U.bf16_exact(torch.randn(T, width, generator=g))
    wr = U.bf16_exact(torch.randn(experts, width, generator=g) * 3.0 * width ** -0.5)
    bias = torch.randn(experts, generator=g)
    wg = U.bf16_exact(torch.randn(experts, ff, width, generator=g) * 2.0 * width ** -0.5)
    wu = U.bf16_exact(torch.randn(experts, ff, width, generator=g) * 2.0 * width ** -0.5)
    wd = U.bf16_exact(torch.randn(experts, width, ff, generator=g) * ff ** -0.5)
    ids_w, wt_w = O.route(x.double(), wr.double(), bias.double(), top)
    adt = _adt(f32)
    xd = dev(x, adt)
    ids, wts = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
    check(lib().b200_moe_route_chosen(f32, xd.data_ptr(), dev(wr, torch.bfloat16).data_ptr(), dev(bias).data_ptr(), T, width, experts, top,
                                      ids.data_ptr(), wts.data_ptr(), None))
    sync()
    assert torch.equal(ids.cpu().long(), ids_w) and torch.allclose(wts.cpu().double(), wt_w, atol=1e-5)
    assert torch.allclose(wts.sum(1).cpu(), torch.ones(T), atol=1e-5)
    gu = torch.cat([torch.cat([wg[e], wu[e]]) for e in range(experts)])
    ws = dev(torch.zeros(lib().b200_moe_workspace_bytes(T, top, experts, width, ff) // 4 + 64, dtype=torch.int32))
    parts = torch.zeros(T, top, width, device=DEV)
    check(lib().b200_moe_experts_limit(f32, xd.data_ptr(), dev(gu, torch.bfloat16).data_ptr(), dev(wd.reshape(-1, ff), torch.bfloat16).data_ptr(),
                                       ids.data_ptr(), wts.data_ptr(), T, width, ff, experts, top, parts.data_ptr(), ws.data_ptr(), 1,
                                       pkg("_abi").ACT_SWIGLU_CLAMP, limit, None))
    sync()
    want = torch.zeros(T, top, width, dtype=torch.float64)
    clamped = 0
    for t in range(T):
        for j in range(top):
            e = int(ids_w[t, j])
            want[t, j] = wt_w[t, j] * O.expert(x[t:t + 1].double(), wg[e].double(), wu[e].double(), wd[e].double(), limit)[0]
            clamped += int((x[t].double() @ wg[e].double().T > limit).sum())
    assert clamped > 0
    assert torch.allclose(parts.cpu().double(), want, atol=2e-5 if f32 else 4e-2, rtol=1e-4 if f32 else 3e-2)


def test_clamped_gate_in_the_grouped_linears_epilogue_agrees_with_the_separate_kernel():
    """bf16 experts whose ff is a multiple of 64: steps with small token tiles clamp and multiply in the gate|up linear's epilogue,
    steps with 128-row tiles run the activation kernel; the same six tokens get the same rows either way, and the oracle's."""
    g = torch.Generator().manual_seed(77)
    width, ff, experts, top, limit = 64, 128, 4, 2, 0.9
    x = U.bf16_exact(torch.randn(600, width, generator=g))
    wr = U.bf16_exact(torch.randn(experts, width, generator=g) * 3.0 * width ** -0.5)
    bias = torch.randn(experts, generator=g)
    wg = U.bf16_exact(torch.randn(experts, ff, width, generator=g) * 2.0 * width ** -0.5)
    wu = U.bf16_exact(torch.randn(experts, ff, width, generator=g) * 2.0 * width ** -0.5)
    wd = U.bf16_exact(torch.randn(experts, width, ff, generator=g) * ff ** -0.5)
    gu = dev(torch.cat([torch.cat([wg[e], wu[e]]) for e in range(experts)]), torch.bfloat16)
    dn = dev(wd.reshape(-1, ff), torch.bfloat16)
    ids_w, wt_w = O.route(x.double(), wr.double(), bias.double(), top)
    got = []
    for T in (6, 600):
        ids, wts = dev(ids_w[:T].int()), dev(wt_w[:T].float())
        ws = dev(torch.zeros(lib().b200_moe_workspace_bytes(T, top, experts, width, ff) // 4 + 64, dtype=torch.int32))
        parts = torch.zeros(T, top, width, device=DEV)
        check(lib().b200_moe_experts_limit(0, dev(x[:T], torch.bfloat16).data_ptr(), gu.data_ptr(), dn.data_ptr(), ids.data_ptr(), wts.data_ptr(), T,
                                           width, ff, experts, top, parts.data_ptr(), ws.data_ptr(), 1, pkg("_abi").ACT_SWIGLU_CLAMP, limit, None))
        sync()
        got.append(parts[:6].cpu().double())
    want = torch.zeros(6, top, width, dtype=torch.float64)
    for t in range(6):
        for j in range(top):
            e = int(ids_w[t, j])
            want[t, j] = wt_w[t, j] * O.expert(x[t:t + 1].double(), wg[e].double(), wu[e].double(), wd[e].double(), limit)[0]
    assert torch.allclose(got[0], got[1], atol=1e-6, rtol=1e-6)
    assert torch.allclose(got[0], want, atol=4e-2, rtol=3e-2)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 20, 12, 3), (1, 1, 72, 40, 1), (3, 3, 33, 70, 5), (2, 1, 130, 8, 2)])
def test_head_decay_delta_rule_in_portions_with_two_sequences_and_dirty_slots(f32, heads, kv_heads, dim, vdim, taps):
    """Convolution tails shorter and longer than the portions, a state carried over many steps, key sizes across the 32-lane groups,
    a second sequence that starts later in a dirty slot.  The oracle runs each sequence whole; its output projection is the
    identity, so the comparison is of the gated, normed read-out."""
    W, eps = 48, 1e-5
    layer = R.delta(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=taps)
    cfg = R.make_cfg(width=W, layers=[layer])
    w = R.make_weights(cfg, dim + taps)
    w["l0.mix.o"] = torch.eye(heads * vdim)
    wd = {k: v.double() for k, v in w.items()}
    g = torch.Generator().manual_seed(3)
    n = {"a": 53, "b": 21}
    h = {k: U.bf16_exact(torch.randn(v, W, generator=g)) for k, v in n.items()}
    want = {k: O.delta_mixer(h[k].double(), wd, "l0.mix.", layer["mixer"], eps) for k in n}
    Wf = torch.cat([wd["l0.mix." + x] for x in ("q", "k", "v", "g", "b", "a")])
    qr = Wf.shape[0]
    C, av = 2 * kv_heads * dim + heads * vdim, heads * vdim
    tail_f = max(taps - 1, 0) * C
    slot_f = (tail_f + 3) // 4 * 4 + heads * vdim * dim + 8
    state = dev(torch.full((3, slot_f), 11.0))
    tails_ptr, rec_ptr = state.data_ptr(), state.data_ptr() + ((tail_f + 3) // 4 * 4) * 4
    conv = dev(torch.cat([wd["l0.mix.q.conv"], wd["l0.mix.k.conv"], wd["l0.mix.v.conv"]]).float())
    dtb, alog, nw = dev(w["l0.mix.dt_bias"]), dev(w["l0.mix.A_log"]), dev(w["l0.mix.norm"].repeat(heads))
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
        qn, kn = torch.zeros(T, kv_heads * dim, device=DEV), torch.zeros(T, kv_heads * dim, device=DEV)
        vn, beta, dec = torch.zeros(T, av, device=DEV), torch.zeros(T, heads, device=DEV), torch.zeros(T, heads, device=DEV)
        pos_d, rts_d, start_d, slots_d = i32(pos), i32(rts), i32(start), i32([slot[k] for k in names])
        check(lib().b200_delta_prep_head(f32, fused.data_ptr(), qr, conv.data_ptr(), dtb.data_ptr(), alog.data_ptr(), pos_d.data_ptr(), rts_d.data_ptr(),
                                         start_d.data_ptr(), slots_d.data_ptr(), tails_ptr if taps > 1 else None, slot_f, qn.data_ptr(), kn.data_ptr(),
                                         vn.data_ptr(), beta.data_ptr(), dec.data_ptr(), T, heads, kv_heads, dim, vdim, taps, None))
        if taps > 1:
            check(lib().b200_delta_tails(f32, fused.data_ptr(), qr, pos_d.data_ptr(), start_d.data_ptr(), slots_d.data_ptr(), tails_ptr, slot_f, S, C,
                                         taps, None))
        oraw = torch.zeros(T, av, device=DEV)
        check(lib().b200_linear_scan(1, qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), beta.data_ptr(), dec.data_ptr(), heads, 1, 0, pos_d.data_ptr(),
                                     start_d.data_ptr(), slots_d.data_ptr(), rec_ptr, slot_f, oraw.data_ptr(), S, heads, kv_heads, dim, vdim, None))
        out = torch.zeros(T, av, dtype=adt, device=DEV)
        check(lib().b200_head_norm_gate_act(f32, oraw.data_ptr(), nw.data_ptr(), fused.data_ptr() + C * (4 if f32 else 2), qr, out.data_ptr(), T, heads,
                                            vdim, eps, 1, None))
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


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,groups,state,vdim,taps,ng", [(4, 2, 20, 12, 3, 2), (1, 1, 72, 40, 1, 1), (6, 3, 33, 35, 5, 6), (2, 1, 130, 8, 2, 4),
                                                              (8, 8, 16, 16, 4, 1)])
def test_state_space_recurrence_in_portions_with_two_sequences_and_dirty_slots(f32, heads, groups, state, vdim, taps, ng):
    """As above for the state-space mixer: convolution with bias over x | B | C, step sizes, decays, the recurrence without a
    correction term, the skip, the gate before the norm, the norm in parts."""
    W, eps = 48, 1e-5
    layer = R.mamba2(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=ng, conv=taps)
    cfg = R.make_cfg(width=W, layers=[layer])
    w = R.make_weights(cfg, state + taps)
    inner = heads * vdim
    w["l0.mix.o"] = torch.eye(inner)
    wd = {k: v.double() for k, v in w.items()}
    g = torch.Generator().manual_seed(5)
    n = {"a": 47, "b": 19}
    h = {k: U.bf16_exact(torch.randn(v, W, generator=g)) for k, v in n.items()}
    want = {k: O.mamba2_mixer(h[k].double(), wd, "l0.mix.", layer["mixer"], eps) for k in n}
    Wf = wd["l0.mix.in"]
    qr, gn = Wf.shape[0], groups * state
    C = inner + 2 * gn
    tail_f = max(taps - 1, 0) * C
    slot_f = (tail_f + 3) // 4 * 4 + inner * state + 8
    st = dev(torch.full((3, slot_f), -5.0))
    tails_ptr, rec_ptr = st.data_ptr(), st.data_ptr() + ((tail_f + 3) // 4 * 4) * 4
    conv, cb = dev(w["l0.mix.conv"]), dev(w["l0.mix.conv.b"])
    dtb, alog, skip, nw = dev(w["l0.mix.dt_bias"]), dev(w["l0.mix.A_log"]), dev(w["l0.mix.D"]), dev(w["l0.mix.norm"])
    sched = {"a": _portions(47, [2, 1, 1, 3, 17, 1, 2, 9]), "b": _portions(19, [1, 1, 2, 6, 1, 3])}
    slot, got = {"a": 1, "b": 2}, {k: torch.zeros(v, inner) for k, v in n.items()}
    adt, es = _adt(f32), 4 if f32 else 2
    for step in range(max(len(v) for v in sched.values()) + 3):
        names = [k for k in ("b", "a") if (k == "a" and step < len(sched["a"])) or (k == "b" and 3 <= step < len(sched["b"]) + 3)]
        if not names:
            continue
        rows, pos, rts, start = [], [], [], [0]
        for si, k in enumerate(names):
            lo, cnt = sched[k][step - (3 if k == "b" else 0)]
            rows.append(h[k][lo:lo + cnt])
            pos += list(range(lo, lo + cnt))
            rts += [si] * cnt
            start.append(start[-1] + cnt)
        x = torch.cat(rows).double()
        T, S = x.shape[0], len(names)
        fused = dev((x @ Wf.T).float(), adt)
        xn, bn, cn = torch.zeros(T, inner, device=DEV), torch.zeros(T, gn, device=DEV), torch.zeros(T, gn, device=DEV)
        dt, dec = torch.zeros(T, heads, device=DEV), torch.zeros(T, heads, device=DEV)
        pos_d, rts_d, start_d, slots_d = i32(pos), i32(rts), i32(start), i32([slot[k] for k in names])
        check(lib().b200_ssd_prep(f32, fused.data_ptr(), qr, conv.data_ptr(), cb.data_ptr(), dtb.data_ptr(), alog.data_ptr(), pos_d.data_ptr(),
                                  rts_d.data_ptr(), start_d.data_ptr(), slots_d.data_ptr(), tails_ptr if taps > 1 else None, slot_f, xn.data_ptr(),
                                  bn.data_ptr(), cn.data_ptr(), dt.data_ptr(), dec.data_ptr(), T, heads, groups, state, vdim, taps, None))
        if taps > 1:
            check(lib().b200_delta_tails(f32, fused.data_ptr() + inner * es, qr, pos_d.data_ptr(), start_d.data_ptr(), slots_d.data_ptr(), tails_ptr,
                                         slot_f, S, C, taps, None))
        oraw = torch.zeros(T, inner, device=DEV)
        check(lib().b200_linear_scan(0, cn.data_ptr(), bn.data_ptr(), xn.data_ptr(), dt.data_ptr(), dec.data_ptr(), heads, 1, 0, pos_d.data_ptr(),
                                     start_d.data_ptr(), slots_d.data_ptr(), rec_ptr, slot_f, oraw.data_ptr(), S, heads, groups, state, vdim, None))
        out = torch.zeros(T, inner, dtype=adt, device=DEV)
        check(lib().b200_ssd_gate_norm(f32, oraw.data_ptr(), xn.data_ptr(), skip.data_ptr(), fused.data_ptr(), qr, nw.data_ptr(), out.data_ptr(), T, heads,
                                       vdim, ng, eps, None))
        sync()
        for si, k in enumerate(names):
            lo, cnt = sched[k][step - (3 if k == "b" else 0)]
            got[k][lo:lo + cnt] = out[start[si]:start[si + 1]].float().cpu()
    for k in n:
        if f32:
            assert torch.allclose(got[k].double(), want[k], atol=5e-5, rtol=1e-4), k
        else:
            err = (got[k].double() - want[k]).abs()
            assert float(err.mean()) < 0.02 and float(err.max()) < 0.3, (k, float(err.mean()), float(err.max()))
    assert float(st[0].min()) == -5.0 and float(st[0].max()) == -5.0          # the unused slot


# ---- whole models ----------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def model_a():
    cfg = R.make_cfg()
    return cfg, R.make_weights(cfg, 1)


ALONE = {
    "attention alone, grouped heads, part of each head turning": [R.attention(mlp=R.dense())],
    "attention without rotation, one stream": [R.attention(rot_dims=0, heads=2, kv_heads=2)],
    "attention with every dimension turning and routed experts": [R.attention(rot_dims=24, vdim=24, mlp=R.moe())],
    "delta rule alone": [R.delta()],
    "delta rule, one tap, one q/k head for all heads": [R.delta(heads=3, kv_heads=1, conv=1, mlp=R.dense(24))],
    "state-space mixer alone": [R.mamba2()],
    "state-space mixer, one group, one norm part, every expert chosen": [R.mamba2(groups=1, norm_groups=1, conv=1, mlp=R.moe(3, 3, 8, 0.5))],
    "two layers without a feed-forward, then one with": [R.delta(), R.mamba2(), R.attention(mlp=R.moe(4, 1, 12, 2.0))],
}


@pytest.mark.parametrize("which", list(ALONE))
def test_one_mechanism_models_and_their_streams_fp32(which):
    one = "one stream" in which
    cfg = R.make_cfg(width=64, layers=ALONE[which], streams=1 if one else 3, taps=1 if one else 4)
    w = R.make_weights(cfg, 4)
    ids = _prompt(cfg, 50, 1)
    r = R.make_runner(cfg, w, "float32")
    tap = r.set_stream_tap(True)
    got = U.replay(U.make_engine(r), [[("p", 50)]], {"p": ids})["p"]
    streams = []
    want = O.forward(cfg, w, ids, streams)
    assert U.rel_rms(got, want.numpy()).max() < F32_TOL
    L = len(cfg["layers"])
    t = tap[:L * 50 * 64].view(L, 50, 64).cpu().double()
    assert torch.allclose(t, torch.stack(streams), atol=1e-4, rtol=1e-5)
    r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["odd sizes", "tensor-core sizes", "ones and equals", "eight streams"])
def test_other_sizes_and_constants(dtype, variant):
    """Widths and head sizes no vector access or TMA box fits; sizes that take every tensor-core path; constants that another
    model may make 1 or equal (one stream, one tap, multiplier and scale 1, as many key heads as heads, groups = heads)."""
    if variant == "odd sizes":
        cfg = R.make_cfg(width=100, vocab=131, eps=1e-3, streams=3, mult=1.7, taps=2, scale=1.0, layers=[
            R.delta(heads=1, kv_heads=1, dim=34, vdim=50, conv=2, mlp=R.dense(44)),
            R.mamba2(heads=5, vdim=14, state=18, groups=5, norm_groups=7, conv=6, mlp=R.moe(7, 3, 10, 0.3)),
            R.attention(heads=6, kv_heads=2, dim=10, vdim=14, rot_dims=6, mlp=R.dense(20)),
            R.mamba2(heads=1, vdim=6, state=130, groups=1, norm_groups=3, conv=2)])
    elif variant == "tensor-core sizes":
        cfg = R.make_cfg(width=128, vocab=256, streams=4, taps=4, layers=[
            R.attention(heads=4, kv_heads=2, dim=64, vdim=32, rot_dims=32, mlp=R.moe(8, 2, 64, 1.0)),
            R.delta(heads=2, kv_heads=2, dim=64, vdim=64, conv=4, mlp=R.dense(128)),
            R.mamba2(heads=4, vdim=32, state=64, groups=1, norm_groups=1, conv=4, mlp=R.moe(4, 4, 32, 2.0)),
            R.attention(heads=8, kv_heads=8, dim=16, vdim=16, rot_dims=16, mlp=R.dense(64))])
    elif variant == "ones and equals":
        cfg = R.make_cfg(width=48, streams=1, mult=1.0, taps=1, scale=1.0, layers=[
            R.attention(heads=1, kv_heads=1, dim=48, vdim=48, rot_dims=2), R.delta(heads=1, kv_heads=1, dim=8, vdim=8, conv=8),
            R.mamba2(heads=3, vdim=8, state=8, groups=3, norm_groups=3, conv=1, mlp=R.moe(1, 1, 8, 1.0))])
    else:
        cfg = R.make_cfg(width=40, streams=8, taps=8, layers=[R.mamba2(mlp=R.dense(16)), R.attention(mlp=R.moe()), R.delta(mlp=R.dense(8))])
    w = R.make_weights(cfg, 6)
    ids = _prompt(cfg, 45, 2)
    want = O.forward(cfg, w, ids).numpy()
    r = R.make_runner(cfg, w, dtype)
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
    """Prefill against token-by-token decoding, portions down to two tokens, unequal requests batched, a long decode tail, blocks and
    state slots that are freed and taken again (12 blocks of 16 where the four requests need 22; four slots for the requests of all
    schedules)."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3), "c": _prompt(cfg, 3, 4), "d": _prompt(cfg, 110, 5)}
    want = {n: O.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = R.make_runner(cfg, w, "float32", n_blocks=12, max_tokens=128)
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
    want = {n: O.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = R.make_runner(cfg, w, "float32")
    sched = [[("a", 7)], [("b", 9)], [("b", 1)], [("a", 2), ("b", 1)], [("b", 29)], [("a", 31)]]
    got = U.replay(U.make_engine(r), sched, prompts)
    for n in prompts:
        assert U.rel_rms(got[n], want[n]).max() < F32_TOL, n
    r.close()


def test_a_far_token_decides_after_hundreds_of_steps():
    """A sequence of 700 tokens whose last token's logits hang on the first tokens through every mixer: the recurrent layers are made
    to forget slowly, so the state written at the start still shows at the end; whole prompt, portions that cut pages and decoding
    agree with the oracle."""
    cfg = R.make_cfg(width=64, vocab=90, streams=2, taps=2, layers=[R.mamba2(mlp=R.dense(32)), R.delta(), R.attention(mlp=R.moe(4, 2, 16, 1.0))])
    w = R.make_weights(cfg, 12)
    w["l0.mix.A_log"], w["l0.mix.dt_bias"] = torch.full((4,), -6.0), torch.full((4,), -3.0)
    w["l1.mix.A_log"], w["l1.mix.dt_bias"] = torch.full((4,), -7.0), torch.full((4,), -3.0)
    w = {k: U.bf16_exact(v) for k, v in w.items()}
    ids = _prompt(cfg, 700, 9)
    want = O.forward(cfg, w, ids).numpy()
    other = O.forward(cfg, w, [(ids[0] + 1) % 90, (ids[1] + 7) % 90] + ids[2:]).numpy()
    assert U.rel_rms(other[-1:], want[-1:]).max() > 1e-3          # the start still shows at the end
    r = R.make_runner(cfg, w, "float32", max_tokens=768, max_model_len=768, block_size=64, n_blocks=12, max_logit_rows=768)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("p", 700)]], {"p": ids})["p"]
    cut = U.replay(eng, [[("p", n)] for n in (63, 2, 64, 129, 300, 110)] + [[("p", 1)]] * 32, {"p": ids})["p"]
    assert U.rel_rms(whole, want).max() < F32_TOL and U.rel_rms(cut, want).max() < F32_TOL
    r.close()


def test_graph_replay_gives_the_same_logits_as_eager_steps(model_a):
    """Steps of equal shape replay one captured graph: sequence bounds, slots and positions must come from the step's device
    metadata, not from what was captured."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 40, 7), "b": _prompt(cfg, 40, 8)}
    sched = [[("a", 8), ("b", 8)]] * 3 + [[("a", 1), ("b", 1)]] * 16
    out = []
    for graphs in (False, True):
        r = R.make_runner(cfg, w, "float32", graphs=graphs)
        out.append(U.replay(U.make_engine(r), sched, prompts))
        r.close()
    for n in prompts:
        assert np.array_equal(out[0][n], out[1][n]), n


def test_bf16_mode_within_bf16_noise_and_equal_across_schedules(model_a):
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3)}
    want = {n: O.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = R.make_runner(cfg, w, "bfloat16", n_blocks=12, max_tokens=128)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("a", 70)], [("b", 37)]], prompts)
    mixed = U.replay(eng, [[("a", 40), ("b", 2)], [("b", 20), ("a", 1)]] + [[("a", 1), ("b", 1)]] * 15 + [[("a", 14)]], prompts)
    for n in prompts:
        e = U.rel_rms(whole[n], want[n])
        assert np.median(e) < 0.03 and (e < 0.1).mean() > 0.9, (n, float(np.median(e)), float(e.max()))
        d = U.rel_rms(mixed[n], whole[n])
        assert np.median(d) < 0.02 and (d < 0.1).mean() > 0.9, (n, float(np.median(d)), float(d.max()))
    r.close()


def test_greedy_generation_through_the_engines_own_scheduler(model_a, tmp_path):
    """A checkpoint directory goes through the registry, the weight loader, LLMEngine.generate and the scheduler (which hands out
    blocks and state slots and overlaps steps); prompts of unequal length decode side by side."""
    cfg, w = model_a
    path = str(tmp_path / "ckpt")
    U.write_checkpoint(path, cfg, w)
    pc = pkg("config").load_model_config(path)
    assert type(pc).__name__ == "RudolixConfig"
    r = pkg("runner").make_runner(pc, dtype="float32", max_tokens=64, max_model_len=256, block_size=16, n_blocks=40, n_state_slots=4)
    r.load_weights(pkg("weights").load_safetensors_dir(path))
    eng = pkg("engine").LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=8, max_model_len=256)
    assert eng.scheduler.max_seqs == 3          # bounded by the state slots
    prompts = [_prompt(cfg, 21, 11), _prompt(cfg, 5, 12), _prompt(cfg, 70, 13), _prompt(cfg, 9, 14)]
    got = eng.generate(prompts, max_tokens=14)
    for p, out in zip(prompts, got):
        ids = list(p)
        for tok in out:      # every emitted token is the oracle's arg-max, or within fp32 noise of it
            z = O.forward(cfg, w, ids)[-1]
            assert tok == int(z.argmax()) or float(z.max() - z[tok]) < 1e-3 * float(z.abs().max())
            ids.append(tok)
    r.close()


def test_random_weights_of_the_benchmark_run(model_a):
    cfg, _ = model_a
    r = pkg("runner").make_runner(R.product_config(cfg), dtype="bfloat16", max_tokens=64, max_model_len=256, block_size=16, n_blocks=40, n_state_slots=4)
    r.init_random_weights(seed=3)
    eng = pkg("engine").LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=3, max_model_len=256)
    out = eng.generate([_prompt(cfg, 30, 1), _prompt(cfg, 4, 2)], max_tokens=6)
    assert [len(o) for o in out] == [6, 6] and all(0 <= t < cfg["vocab"] for o in out for t in o)
    r.close()


def test_samplers_and_log_probabilities_read_the_steps_logits(model_a):
    """Sampled requests go through the framework's samplers after the step: with top_k = 1 a request at temperature 0.9 emits the
    greedy tokens; the log-probabilities of the emitted tokens are the oracle's log-softmax (the samplers read bf16 logits); a
    plain greedy request in the same batch is untouched by its neighbours."""
    cfg, w = model_a
    E = pkg("engine")
    r = R.make_runner(cfg, w, "float32", max_tokens=64, max_model_len=256, n_blocks=40)
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
        z = torch.log_softmax(O.forward(cfg, w, ids)[-1], -1)
        assert abs(lp - float(z[tok])) < 0.05 and top[0][0] == int(z.argmax())
        ids.append(tok)
    r.close()
