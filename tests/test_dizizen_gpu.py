"""Dizizen on the GPU against the plain numpy restatement in tests/dizizen_oracle.py.

Small configurations of their own (sizes that differ from one another: head size, value size and rotated part all
different; grouped and single key/value heads; layers in several orders with dense, routed and no feed-forward; shared
caches; with and without identity slots, groups and a shared expert; two rotation bases in one model), random
bfloat16-exact weights.  float32 runs are held to a tight tolerance, bfloat16 runs to a loose one; the measure is the RMS
over the vocabulary of the mean-free difference of the logits, relative to the RMS of the logits.
"""
import json
import math

import numpy as np
import pytest

from tests import dizizen_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}


def A(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, kv_from=None, mlp=None):
    mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=dict(base=base, dims=rot_dims))
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def DENSE(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def MOE(experts, identity, top, count, keep, ff, shared=0):
    d = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


CFG_MIXED = {"architecture": "Dizizen", "vocab": 67, "width": 48, "residual_mult": 0.7, "embedding": {"scale": 2.5},
             "norm": {"eps": 1e-5},
             "layers": [A(4, 2, 12, 8, 0.3, 6, mlp=MOE(7, 2, 3, 3, 2, 20, shared=28)), A(3, 1, 10, 14, 0.25, 10, base=500.0),
                        A(4, 2, 12, 8, 0.3, 6, kv_from=0, mlp=DENSE(40, 1.2)),
                        A(3, 1, 10, 14, 0.25, 10, base=500.0, kv_from=1, mlp=MOE(5, 0, 2, 1, 1, 24))]}
CFG_ONES = {"architecture": "Dizizen", "vocab": 40, "width": 32, "residual_mult": 1.0, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6},
            "layers": [A(1, 1, 32, 2, 0.17, 32, base=300.0, mlp=MOE(1, 1, 1, 1, 1, 16)), A(1, 1, 6, 4, 0.4, 0, mlp=DENSE(8, 0.5)),
                       A(2, 2, 4, 6, 0.5, 2, mlp=MOE(0, 2, 2, 2, 2, 0, shared=12))]}
CFG_WIDE = {"architecture": "Dizizen", "vocab": 96, "width": 64, "residual_mult": 0.4, "embedding": {"scale": 4.0},
            "norm": {"eps": 1e-5},
            "layers": [A(8, 2, 16, 32, 0.25, 8, base=2e5, mlp=DENSE(72, 2.0)),
                       A(8, 2, 16, 32, 0.25, 8, base=2e5, kv_from=0, mlp=MOE(9, 3, 5, 4, 3, 40, shared=24)),
                       A(4, 4, 32, 16, 0.2, 32, mlp=MOE(6, 2, 2, 4, 2, 16))]}
CONFIGS = {"mixed": CFG_MIXED, "ones": CFG_ONES, "wide": CFG_WIDE}


def row_err(got, want):
    d = np.asarray(got, dtype=np.float64) - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1))


def rel_err(got, want, dtype="float32"):
    """float32: the worst row.  bfloat16: the row at the 90th percentile -- a rounding can flip the choice of an expert
    where two choice scores nearly tie, which moves that token by far more than rounding does and says nothing about
    the kernels; what a float32 run finds at one position only, it finds with the worst-row measure."""
    e = row_err(got, want)
    return float(np.max(e) if dtype == "float32" else np.quantile(e, 0.9))


def make(cfg_dict, dtype, seed=0, max_batch=4, max_seq=400, max_step_tokens=64, **kw):
    from zhilight_b200.dizizen import DizizenConfig, DizizenDecoder
    from zhilight_b200.safetensors_io import f32_to_bf16
    cfg = DizizenConfig.from_dict(cfg_dict)
    W = orc.random_weights(cfg, seed)
    m = DizizenDecoder(cfg, dtype=dtype, max_batch=max_batch, max_seq=max_seq, max_step_tokens=max_step_tokens, **kw)
    m.load_state_dict({k: f32_to_bf16(v) for k, v in W.items()})
    return cfg, {k: v.astype(np.float64) for k, v in W.items()}, m


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, n).tolist()


def dev(a, cuda, dtype=None):
    import torch
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(cuda)


def i32(a, cuda):
    import torch
    return torch.tensor(list(a), dtype=torch.int32, device=cuda)


def inv_freq(base, dims):
    return base ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gemm_clamped_unit_with_bias_and_grouped_relu2(cuda, lib, dtype):
    import torch
    from zhilight_b200 import ops
    td = getattr(torch, dtype)
    tol = 1e-5 if dtype == "float32" else 1e-2
    rng = np.random.default_rng(0)
    for m, f, k in ((5, 7, 16), (70, 65, 80), (3, 48, 64), (40, 10, 24)):     # few-rows kernel and tile kernel
        x = orc.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
        gate, up = (orc.bf16_round((rng.standard_normal((f, k)) / math.sqrt(k) * 2).astype(np.float32)) for _ in range(2))
        gb, ub = (orc.bf16_round(rng.standard_normal(f).astype(np.float32)) for _ in range(2))
        W = {"gate": gate, "gate.b": gb, "up": up, "up.b": ub, "down": np.eye(f), "down.b": np.zeros(f)}
        want = orc.clamped_gated_ff({k_: v.astype(np.float64) for k_, v in W.items()}, "", x.astype(np.float64), 0.9)
        w2 = np.empty((2 * f, k), np.float32)
        w2[0::2], w2[1::2] = gate, up
        b2 = np.empty(2 * f, np.float32)
        b2[0::2], b2[1::2] = gb, ub
        y = ops.gemm_nt_glu_clamp(dev(x, cuda, td), dev(w2, cuda, td), dev(b2, cuda), out_dtype=torch.float32, limit=0.9,
                                  alpha=1.702, beta=1.0)
        assert np.abs(y.cpu().numpy() - want).max() < tol * 4, (m, f, k)
    # grouped relu^2: 5 groups of unequal size (one empty, one larger than a tile), then a step of few rows
    for T, sizes in ((47, [0, 70, 3, 1, 67]), (6, [11, 0, 2, 4, 1])):
        G, K, F, top = 5, 40, 24, 3
        pairs = rng.permutation(T * top)
        off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
        x = orc.bf16_round(rng.standard_normal((T, K)).astype(np.float32))
        wu = orc.bf16_round((rng.standard_normal((G, F, K)) / math.sqrt(K)).astype(np.float32))
        wd = orc.bf16_round((rng.standard_normal((G, K, F)) / math.sqrt(F)).astype(np.float32))
        act = ops.gemm_nt_grouped(dev(x, cuda, td), dev(wu, cuda, td), dev(off, cuda), T * top, x_rows=i32(pairs // top, cuda),
                                  epilogue=ops.GEMM_EPI_RELU2)
        out = ops.gemm_nt_grouped(act, dev(wd, cuda, td), dev(off, cuda), T * top, y_rows=i32(pairs, cuda), out_dtype=torch.float32)
        act, out = act.float().cpu().numpy(), out.cpu().numpy()
        for g in range(G):
            for i in range(off[g], off[g + 1]):
                hid = np.maximum(wu[g].astype(np.float64) @ x[pairs[i] // top], 0.0) ** 2
                assert np.abs(act[i] - hid).max() < tol * 4 * max(1.0, hid.max()), (g, i)
                want = orc.relu2_expert({"up": wu[g].astype(np.float64), "down": wd[g].astype(np.float64)}, "", x[pairs[i] // top].astype(np.float64))
                assert np.abs(out[pairs[i]] - wd[g].astype(np.float64) @ act[i].astype(np.float64)).max() < tol * 4, (g, i)
                assert np.abs(out[pairs[i]] - want).max() < (1e-4 if dtype == "float32" else 0.1), (g, i)


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_tables_and_cache_append(cuda, lib, dtype, layout):
    """Queries / keys turn over the first `rot` of `d` dimensions, values over all of `vd`, each from its own table, at
    positions near 900 (a float angle would be off there), in both pairings."""
    import torch
    from zhilight_b200 import ops
    td = getattr(torch, dtype)
    H, G, d, vd, rot = 3, 1, 20, 12, 6
    rng = np.random.default_rng(1)
    slots, pos = [2, 2, 2, 0, 1], [898, 899, 900, 0, 37]
    T = len(pos)
    n_in = H * d + G * d + G * vd + 5
    proj = rng.standard_normal((T, n_in)).astype(np.float32)
    fq, fv = dev(inv_freq(10000.0, rot), cuda), dev(inv_freq(10000.0, vd), cuda)
    tq, tv = ops.rope_table(i32(pos, cuda), fq), ops.rope_table(i32(pos, cuda), fv)
    cq, sq = orc.half_tables(pos, rot, 10000.0)
    cv, sv = orc.half_tables(pos, vd, 10000.0)
    assert np.abs(tq.cpu().numpy()[..., 0] - cq).max() < 1e-7 and np.abs(tq.cpu().numpy()[..., 1] - sq).max() < 1e-7
    assert np.abs(tv.cpu().numpy()[..., 0] - cv).max() < 1e-7 and np.abs(tv.cpu().numpy()[..., 1] - sv).max() < 1e-7
    kc = torch.zeros((3, 1000, G * d), dtype=td, device=cuda)
    vc = torch.zeros((3, 1000, G * vd), dtype=td, device=cuda)
    q = ops.qkv_table_rope_append(dev(proj, cuda), 0, H * d, H * d + G * d, H, G, d, vd, tq, rot, tv, layout, ops.slot_table(kc),
                                  ops.slot_table(vc), i32(slots, cuda), i32(pos, cuda), td)
    p64 = proj.astype(np.float64)

    def turn(x, c, s, n):
        if layout == 0:
            return orc.rotate_halves(x, c, s, n)
        y = x.copy()                                   # adjacent pairs (2i, 2i + 1)
        a, b = x[..., 0:n:2], x[..., 1:n:2]
        y[..., 0:n:2] = a * c[:, None, :] - b * s[:, None, :]
        y[..., 1:n:2] = b * c[:, None, :] + a * s[:, None, :]
        return y

    wq = turn(p64[:, :H * d].reshape(T, H, d), cq, sq, rot).reshape(T, -1)
    wk = turn(p64[:, H * d:H * d + G * d].reshape(T, G, d), cq, sq, rot).reshape(T, -1)
    wv = turn(p64[:, H * d + G * d:H * d + G * d + G * vd].reshape(T, G, vd), cv, sv, vd).reshape(T, -1)
    tol = 2e-6 if dtype == "float32" else 2e-2
    for t in range(T):
        assert np.abs(q[t].float().cpu().numpy() - wq[t]).max() < tol
        assert np.abs(kc[slots[t], pos[t]].float().cpu().numpy() - wk[t]).max() < tol
        assert np.abs(vc[slots[t], pos[t]].float().cpu().numpy() - wv[t]).max() < tol
    assert float(kc[1, 36].abs().sum()) == 0 and float(kc[1, 38].abs().sum()) == 0       # no other row was touched
    # a layer that reads another layer's caches writes queries only
    kc.zero_(), vc.zero_()
    q2 = ops.qkv_table_rope_append(dev(proj, cuda), 0, -1, 0, H, G, d, vd, tq, rot, tv, layout, ops.slot_table(kc),
                                   ops.slot_table(vc), i32(slots, cuda), i32(pos, cuda), td)
    assert torch.equal(q2, q) and float(kc.abs().sum()) == 0 and float(vc.abs().sum()) == 0


@pytest.mark.parametrize("H,vd", [(6, 24), (8, 32), (8, 24), (2, 48)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_plain_softmax_rotated_values_far_key(cuda, lib, dtype, H, vd):
    """700 keys, values cached turned by their position, outputs turned back by the query's.  One far key is made to
    carry the softmax of one head (so the output there is that one value turned by the distance: a lost key or an
    output turned by a wrong position shows at full size); another head's scores are pushed far below zero, where a sink
    would take the denominator and an ordinary softmax must not care; rows past a token's position hold huge values; key
    splits 1 / 2 / 5 / 23; each query row alone and as runs (tile edges at 63 / 64 / 65 keys)."""
    import torch
    from zhilight_b200 import ops
    td = getattr(torch, dtype)
    G, d, n, scale, base = 2, 16, 700, 0.25, 700.0
    rng = np.random.default_rng(2)
    q = orc.bf16_round(rng.standard_normal((n, H, d)).astype(np.float32))
    k = orc.bf16_round(rng.standard_normal((n, G, d)).astype(np.float32))
    v = rng.standard_normal((n, G, vd))
    k[13, 0] = orc.bf16_round(np.sign(q[650, 1]) * 2.0)       # head 1 (group 0) of token 650 looks at key 13
    q[650, 1] *= 4
    q[651, H - 1] = orc.bf16_round(-8.0 * np.sign(k[:652, 1].sum(0)))
    cv, sv = orc.half_tables(np.arange(n), vd, base)
    vr = orc.bf16_round(orc.rotate_halves(v, cv, sv, vd).astype(np.float32))      # what the cache holds
    att = orc.causal_softmax_attention(q.astype(np.float64), k.astype(np.float64), vr.astype(np.float64), scale)
    want = orc.rotate_halves(att, cv, sv, vd, sign=-1.0)
    e = np.exp((k[:651, 0].astype(np.float64) @ q[650, 1]) * scale)
    assert e[13] / e.sum() > 0.9                                        # the far key does carry that head
    assert np.abs(want[650, 1] - att[650, 1]).max() > 0.3               # ... and the turn back matters there
    rows = [0, 1, 7, 8, 9, 63, 64, 65, 255, 256, 257, 511, 512, 650, 651, 699]
    kc = torch.full((2, n + 5, G * d), 3e4, dtype=td, device=cuda)
    vc = torch.full((2, n + 5, G * vd), 3e4, dtype=td, device=cuda)
    kc[1, :n] = dev(k.reshape(n, -1), cuda, td)
    vc[1, :n] = dev(vr.reshape(n, -1), cuda, td)
    fv = dev(inv_freq(base, vd), cuda)
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    for splits in (1, 2, 5, 23):
        kw = dict(no_sink=True, splits=splits)
        tab = ops.rope_table(i32(rows, cuda), fv)
        out = ops.sink_attention_ex(dev(q[rows].reshape(len(rows), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                    i32([1] * len(rows), cuda), i32(rows, cuda), scale, H, G, d, vd, out_table=tab, **kw)
        got = out.float().cpu().numpy().reshape(len(rows), H, vd)
        assert np.abs(got - want[rows]).max() < tol, (dtype, splits)
        ones = dict(run_row0=i32(range(len(rows)), cuda), run_len=i32([1] * len(rows), cuda), max_run_len=1)
        out = ops.sink_attention_ex(dev(q[rows].reshape(len(rows), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                    i32([1] * len(rows), cuda), i32(rows, cuda), scale, H, G, d, vd, out_table=tab, **kw, **ones)
        assert np.abs(out.float().cpu().numpy().reshape(len(rows), H, vd) - want[rows]).max() < tol, (dtype, splits, "runs of 1")
        seq = list(range(10)) + list(range(560, 700))
        out = ops.sink_attention_ex(dev(q[seq].reshape(len(seq), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                    i32([1] * len(seq), cuda), i32(seq, cuda), scale, H, G, d, vd,
                                    out_table=ops.rope_table(i32(seq, cuda), fv), run_row0=i32([0, 10], cuda),
                                    run_len=i32([10, 140], cuda), max_run_len=140, **kw)
        assert np.abs(out.float().cpu().numpy().reshape(len(seq), H, vd) - want[seq]).max() < tol, (dtype, splits, "two runs")
        # without the table the same call returns the sum as it is (the inverse turn is the only difference)
        out = ops.sink_attention_ex(dev(q[rows].reshape(len(rows), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                    i32([1] * len(rows), cuda), i32(rows, cuda), scale, H, G, d, vd, **kw, **ones)
        assert np.abs(out.float().cpu().numpy().reshape(len(rows), H, vd) - att[rows]).max() < tol, (dtype, splits, "no table")


def test_router_groups_identity_slots_and_weights(cuda, lib):
    """12 slots in 4 groups of which 2 count.  The correction decides which groups and slots are chosen but is no part of
    the weight; a slot with the largest choice value of all sits in a group that loses and must not be chosen; all choice
    values are negative (a dropped slot counts as minus infinity, not 0); the weights sum to 1; the lists sort the pairs
    by slot with the identity slots (9 .. 11) last; ready logits give the same as x and the router matrix."""
    from zhilight_b200 import ops
    rng = np.random.default_rng(3)
    T, D, S, top, groups, keep = 37, 24, 12, 3, 4, 2
    x = rng.standard_normal((T, D)).astype(np.float32)
    w = (3 * rng.standard_normal((S, D)) / math.sqrt(D)).astype(np.float32)
    corr = (-2.0 + 0.05 * rng.standard_normal(S)).astype(np.float32)
    corr[7] += 0.5                                                # group 2 (slots 6..8) always counts, slot 7 is always chosen
    te, tw, off, lt, lp = (t.cpu().numpy() for t in ops.moe_route_grouped(dev(x, cuda), dev(w, cuda), dev(corr, cuda), top, groups,
                                                                           keep, renorm_eps=1e-20))
    z = x.astype(np.float64) @ w.T.astype(np.float64)
    dropped_best = 0
    for t in range(T):
        chosen, weight = orc.grouped_route(z[t], corr.astype(np.float64), top, groups, keep)
        assert (te[t] == chosen).all(), t
        assert np.abs(tw[t] - weight).max() < 1e-6 and abs(tw[t].sum() - 1.0) < 1e-6
        e = np.exp(z[t] - z[t].max())
        c = e / e.sum() + corr
        assert (c < 0).all()
        rest = np.setdiff1d(np.arange(S), chosen)
        dropped_best += c[rest].max() > c[chosen].min()           # a better slot was left out because its group lost
    assert (te == 7).any(axis=1).all() and dropped_best > 5
    assert off[0] == 0 and off[-1] == T * top and (np.diff(off) >= 0).all() and len(off) == S + 1
    assert sorted(lp.tolist()) == list(range(T * top)) and (lt == lp // top).all()
    for s in range(S):
        assert (te.reshape(-1)[lp[off[s]:off[s + 1]]] == s).all()
    again = ops.moe_route_grouped(dev(z.astype(np.float32), cuda), None, dev(corr, cuda), top, groups, keep, renorm_eps=1e-20)
    assert (again[0].cpu().numpy() == te).all() and np.abs(again[1].cpu().numpy() - tw).max() < 1e-5
    # one group, every group kept, and top = all slots: the plain top-k of the framework's other router
    te1 = ops.moe_route_grouped(dev(x, cuda), dev(w, cuda), dev(corr, cuda), S, 3, 3)[0].cpu().numpy()
    assert (np.sort(te1, axis=1) == np.arange(S)).all()


@pytest.mark.parametrize("aligned", [True, False])
@pytest.mark.parametrize("D", [40, 300, 4100])
def test_gated_parallel_combine(cuda, lib, D, aligned):
    """aligned rows of a width up to 4096 take the kernel's register path, the others the channel-by-channel one."""
    import torch
    from zhilight_b200 import ops
    rng = np.random.default_rng(4)
    T, P, n_real, eps, mult = 9, 3, 5, 1e-5, 0.6
    ga, gf, wide = (4, D + 8, 2 * D + 12) if aligned else (3, D + 5, 2 * D + 7)
    x = rng.standard_normal((T, D)).astype(np.float32)
    gates = rng.standard_normal((T, wide)).astype(np.float32)
    a, fd = rng.standard_normal((T, D)).astype(np.float32), rng.standard_normal((T, D)).astype(np.float32)
    parts = rng.standard_normal((T, P, D)).astype(np.float32)
    coef = rng.random((T, P)).astype(np.float32)
    choice = rng.integers(0, 8, (T, P)).astype(np.int32)
    choice[0], choice[1] = [0, 1, 2], [7, 6, 5]                  # a token without and one with only handed-through parts
    parts[choice >= n_real] = np.nan                              # such rows are never read
    sa, sf, nw, nxt = (rng.standard_normal(D).astype(np.float32) for _ in range(4))
    h = orc.zero_centred_norm(x.astype(np.float64), nw.astype(np.float64) - 1.0, eps)
    f = fd.astype(np.float64).copy()
    for t in range(T):
        for p in range(P):
            f[t] += coef[t, p] * (parts[t, p] if choice[t, p] < n_real else h[t])
    g1, g2 = orc.sigmoid(gates[:, ga:ga + D].astype(np.float64)), orc.sigmoid(gates[:, gf:gf + D].astype(np.float64))
    want = x + mult * (sa * g1 * a + sf * g2 * f)
    xd = dev(x, cuda)
    hn = ops.gated_parallel_combine(xd, mult, dev(gates, cuda), ga, dev(a, cuda), dev(sa, cuda), eps, parts=dev(parts, cuda),
                                    coef=dev(coef, cuda), choice=dev(choice, cuda), n_real=n_real, f_dense=dev(fd, cuda),
                                    gf_off=gf, scale_f=dev(sf, cuda), norm_w=dev(nw, cuda), next_w=dev(nxt, cuda),
                                    act_dtype=torch.bfloat16)
    assert np.abs(xd.cpu().numpy() - want).max() < 3e-6 * np.abs(want).max()
    ref = orc.zero_centred_norm(want, nxt.astype(np.float64) - 1.0, eps)
    assert np.abs(hn.float().cpu().numpy() - ref).max() < 2.0 ** -8 * np.abs(ref).max()      # one bfloat16 rounding
    # no second sublayer, no next norm
    xd = dev(x, cuda)
    assert ops.gated_parallel_combine(xd, mult, dev(gates, cuda), ga, dev(a, cuda), dev(sa, cuda), eps) is None
    assert np.abs(xd.cpu().numpy() - (x + mult * sa * g1 * a)).max() < 3e-6 * np.abs(want).max()
    # only a dense second sublayer, float32 next norm
    xd = dev(x, cuda)
    hn = ops.gated_parallel_combine(xd, mult, dev(gates, cuda), ga, dev(a, cuda), dev(sa, cuda), eps, f_dense=dev(fd, cuda),
                                    gf_off=gf, scale_f=dev(sf, cuda), next_w=dev(nxt, cuda))
    want = x + mult * (sa * g1 * a + sf * g2 * fd)
    assert np.abs(xd.cpu().numpy() - want).max() < 3e-6 * np.abs(want).max()
    ref = orc.zero_centred_norm(want, nxt.astype(np.float64) - 1.0, eps)
    assert np.abs(hn.cpu().numpy() - ref).max() < 3e-6 * np.abs(ref).max()


# ---------------------------------------------------------------------------------------------- the whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_layers_caches_and_logits(cuda, lib, name, dtype):
    cfg, W, m = make(CONFIGS[name], dtype, seed=1, max_step_tokens=128)
    toks = tokens_for(cfg, 97, 5)
    want, streams, caches = orc.forward(cfg, W, toks)
    m.capture_layers(True)
    _, logits = m.step(toks, [2] * len(toks), range(len(toks)), range(len(toks)))
    got_streams = m.read_layers(len(toks))
    for i in range(len(cfg.layers)):   # the first layer that differs is the one to look at
        rows = np.abs(got_streams[i] - streams[i]).max(-1) / np.abs(streams[i]).max()
        d = rows.max() if dtype == "float32" else np.quantile(rows, 0.9)
        assert d < (1e-4 if dtype == "float32" else 6e-2), (name, dtype, "layer", i, d)
    for i, l in enumerate(cfg.layers):
        if l["kv_from"] >= 0:
            continue
        k, v = m.read_cache(i, 2, len(toks))
        for got, ref in ((k, caches[i][0]), (v, caches[i][1])):
            rows = np.abs(got - ref).max((-1, -2)) / np.abs(ref).max()
            d = rows.max() if dtype == "float32" else np.quantile(rows, 0.9)
            assert d < (1e-4 if dtype == "float32" else 6e-2), (name, dtype, "cache", i, d)
    assert rel_err(logits, want, dtype) < TOL[dtype]
    m.close()


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_vs_token_by_token_and_portions(cuda, lib, name, dtype):
    """The same prompt whole, token by token, and in portions down to two tokens: every position (the first tokens of the
    sequence among them) against the oracle and the three runs against one another."""
    from zhilight_b200.engine import Engine
    cfg, W, m = make(CONFIGS[name], dtype, seed=2, max_step_tokens=32)
    eng = Engine(m)
    toks = tokens_for(cfg, 75, 9)
    want = orc.forward(cfg, W, toks)[0]
    runs = {}
    for label, sizes in (("whole", [75]), ("single", [1] * 75), ("portions", [2, 3, 2, 17, 1, 2, 31, 5, 2, 10])):
        assert sum(sizes) == 75
        eng.open(label)
        rows, at = [], 0
        for s in sizes:
            rows.append(eng.forward_step([(label, toks[at:at + s], list(range(s)))])[label][1])
            at += s
        eng.close(label)
        runs[label] = np.concatenate(rows)
        assert rel_err(runs[label], want, dtype) < TOL[dtype], (name, dtype, label)
        assert rel_err(runs[label][:3], want[:3], "float32") < TOL[dtype], (name, dtype, label, "first tokens")
    cut = 1e-5 if dtype == "float32" else 2e-2      # the cuts change the order of sums, no more
    assert rel_err(runs["single"], runs["whole"].astype(np.float64), dtype) < cut
    assert rel_err(runs["portions"], runs["whole"].astype(np.float64), dtype) < cut
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone_and_slot_reuse(cuda, lib, dtype):
    """Three requests of different lengths share steps (prompt portions next to single decode tokens); afterwards their
    slots -- caches still in them -- are handed to new requests.  Every logit row equals the request run alone."""
    from zhilight_b200.engine import Engine
    cfg, W, m = make(CFG_MIXED, dtype, seed=3, max_batch=3, max_step_tokens=16)
    eng = Engine(m)
    prompts = {"a": tokens_for(cfg, 41, 1), "b": tokens_for(cfg, 9, 2), "c": tokens_for(cfg, 26, 3)}
    later = {"d": tokens_for(cfg, 30, 4), "e": tokens_for(cfg, 5, 5)}
    want = {k: orc.forward(cfg, W, v)[0] for k, v in {**prompts, **later}.items()}
    got = {k: [] for k in want}
    at = {k: 0 for k in want}
    for k in prompts:
        eng.open(k)
    plan = [{"a": 7, "b": 2, "c": 1}, {"a": 1, "b": 1, "c": 12}, {"a": 20, "b": 1, "c": 1}, {"a": 1, "b": 5, "c": 2},
            {"a": 12, "c": 10}]
    for step in plan:
        entries = [(k, prompts[k][at[k]:at[k] + n], list(range(n))) for k, n in step.items()]
        res = eng.forward_step(entries)
        for k, n in step.items():
            got[k].append(res[k][1])
            at[k] += n
    assert at == {"a": 41, "b": 9, "c": 26, "d": 0, "e": 0}
    used = {eng.seqs[k].slot for k in prompts}
    for k in prompts:
        eng.close(k)
    for k in later:
        assert eng.open(k).slot in used
    res = eng.forward_step([("d", later["d"][:11], list(range(11))), ("e", later["e"], list(range(5)))])
    got["d"].append(res["d"][1]); got["e"].append(res["e"][1])
    got["d"].append(eng.forward_step([("d", later["d"][11:], list(range(19)))])["d"][1])
    for k in want:
        assert rel_err(np.concatenate(got[k]), want[k], dtype) < TOL[dtype], (dtype, k)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_and_splits(cuda, lib, dtype):
    """A short prompt and then 330 single-token steps: the decode graph, the length buckets (256, 512) and the key splits
    of the attention kernel all change on the way, and every step's table of angles is made from positions on the device."""
    cfg, W, m = make(CFG_WIDE, dtype, seed=4, max_batch=2, max_seq=512, max_step_tokens=16)
    toks = tokens_for(cfg, 340, 11)
    want = orc.forward(cfg, W, toks)[0]
    _, first = m.step(toks[:10], [1] * 10, range(10), range(10))
    rows = [first]
    for p in range(10, 340):
        rows.append(m.step([toks[p]], [1], [p], [0])[1])
    assert rel_err(np.concatenate(rows), want, dtype) < TOL[dtype]
    assert m.stats()[1] > 0          # the single-token steps were replayed as graphs
    m.close()


def test_far_token_is_found_through_the_model(cuda, lib):
    """Token 7 of 300 moves the last logits by far more than the float32 tolerance (the oracle says so first), so a key
    lost far back, or a value turned by a wrong distance -- through prompt portions or through decoding -- fails."""
    cfg, W, m = make(CFG_WIDE, "float32", seed=5, max_batch=2, max_seq=320, max_step_tokens=64)
    toks = tokens_for(cfg, 300, 13)
    base = orc.forward(cfg, W, toks)[0][-1]
    other = list(toks)
    other[7] = (toks[7] + 1) % cfg.vocab
    moved = orc.forward(cfg, W, other)[0][-1]
    assert rel_err(moved[None], base[None]) > 10 * TOL["float32"]   # the oracle says token 7 matters at the end
    for seq, want in ((toks, base), (other, moved)):
        for c0 in range(0, 256, 64):
            m.step(seq[c0:c0 + 64], [0] * 64, range(c0, c0 + 64))
        for p in range(256, 299):
            m.step([seq[p]], [0], [p])
        got = m.step([seq[299]], [0], [299], [0])[1]
        assert rel_err(got, want[None]) < TOL["float32"]
    m.close()


def test_device_resident_decode_loop(cuda, lib):
    """set_state / step_device (greedy picks fed back on the device) give the tokens of step-by-step greedy decoding."""
    cfg, W, m = make(CFG_WIDE, "float32", seed=7, max_batch=2, max_seq=64, max_step_tokens=16)
    prompts = [tokens_for(cfg, 9, 1), tokens_for(cfg, 9, 2)]
    nxt = []
    for s, p in enumerate(prompts):
        nxt.append(int(m.step(p, [s] * 9, range(9), [8])[0][0]))
    ref = [list(p) + [n] for p, n in zip(prompts, nxt)]
    m.set_state(nxt, [9, 9])
    for _ in range(5):
        m.step_device(2)
    m.sync()
    for s in range(2):
        for _ in range(5):
            logits = orc.forward(cfg, W, ref[s])[0][-1]
            ref[s].append(int(np.argmax(logits)))
    # replay the same on the host path against the device loop's caches: position 14 sees what the loop wrote
    for s in range(2):
        got = m.step([ref[s][14]], [s], [14], [0])[1]
        want = orc.forward(cfg, W, ref[s][:15])[0][-1]
        assert rel_err(got, want[None]) < TOL["float32"], s
    m.close()


def test_greedy_generation_through_the_scheduler(cuda, lib):
    """Engine.generate (admission, portions, mixed steps, retiring, slot reuse: 5 prompts on 2 slots) against greedy
    decoding with the oracle; float32 so that near-ties do not flip."""
    from zhilight_b200.engine import Engine
    cfg, W, m = make(CFG_MIXED, "float32", seed=6, max_batch=2, max_seq=128, max_step_tokens=8)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (3, 19, 1, 11, 6)]
    seen = []
    outs = Engine(m).generate(prompts, max_new_tokens=7, on_step=lambda e: seen.append([len(t) for _, t, _ in e]))
    assert any(len(s) > 1 and max(s) > 1 and min(s) == 1 for s in seen)    # a prompt portion beside a decode token
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            logits = orc.forward(cfg, W, seq)[0][-1]
            top = np.sort(logits)[-2:]
            assert tok == int(np.argmax(logits)) or top[1] - top[0] < 1e-4
            seq.append(tok)
        assert len(out) == 7
    m.close()


def test_model_folder_registry_and_trace_replay(cuda, lib, tmp_path):
    """config.json + model.safetensors on disk -> registry -> trace replay: the written logits are the oracle's."""
    from zhilight_b200 import registry, safetensors_io, trace
    from zhilight_b200.dizizen import DizizenConfig
    cfg = DizizenConfig.from_dict(CFG_ONES)
    W = orc.random_weights(cfg, 8)
    (tmp_path / "m").mkdir()
    (tmp_path / "m" / "config.json").write_text(json.dumps(CFG_ONES))
    safetensors_io.save_file({k: safetensors_io.f32_to_bf16(v) for k, v in W.items()}, str(tmp_path / "m" / "model.safetensors"))
    model = registry.load_model(str(tmp_path / "m"), "float32", max_batch=2, max_seq=64, max_step_tokens=8)
    toks = tokens_for(cfg, 21, 3)
    lines = [json.dumps({"step": 0, "entries": [{"id": "x", "tokens": toks[:13], "want": [12, 0, 5]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "x", "tokens": toks[13:20], "want": []}], "end": []}),
             json.dumps({"step": 2, "entries": [{"id": "x", "tokens": toks[20:], "want": [0]}], "end": ["x"]})]
    said = []
    trace.replay(model, lines, str(tmp_path), emit=said.append)
    assert said == ["done 0", "done 1", "done 2"] and not (tmp_path / "1.f32").exists()
    want = orc.forward(cfg, {k: v.astype(np.float64) for k, v in W.items()}, toks)[0]
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(3, cfg.vocab)
    got2 = np.fromfile(tmp_path / "2.f32", dtype="<f4").reshape(1, cfg.vocab)
    assert rel_err(got0, want[[12, 0, 5]]) < TOL["float32"] and rel_err(got2, want[[20]]) < TOL["float32"]
    model.close()
