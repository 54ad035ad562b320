"""Dizizen pieces that need no GPU: the oracle's own consistency (mechanisms by hand), config parsing and validation,
tensor shapes, the registry entry and the family's source list."""
import copy
import math
import os

import numpy as np
import pytest

from tests import dizizen_oracle as orc
from tests.test_dizizen_gpu import CFG_MIXED, CFG_ONES, CFG_WIDE
from zhilight_b200.dizizen import DizizenConfig


def _weights(cfg, seed=0):
    return {k: v.astype(np.float64) for k, v in orc.random_weights(cfg, seed).items()}


def test_config_round_trip_and_shapes():
    for d in (CFG_MIXED, CFG_ONES, CFG_WIDE):
        cfg = DizizenConfig.from_dict(d)
        again = DizizenConfig.from_dict(cfg.to_dict())
        assert cfg.layers == again.layers
        assert (cfg.residual_mult, cfg.embed_scale, cfg.norm_eps) == (again.residual_mult, again.embed_scale, again.norm_eps)
        shapes = cfg.tensor_shapes()
        assert shapes["embed"] == (cfg.vocab, cfg.width) and shapes["final.norm"] == (cfg.width,)
    s = DizizenConfig.from_dict(CFG_MIXED).tensor_shapes()
    assert "l2.mix.k" not in s and "l2.mix.v.b" not in s and "l2.mix.q" in s        # a layer on another layer's cache
    assert "l1.ls2" not in s and "l1.rg2" not in s and "l1.rg1" in s                  # a layer without feed-forward
    assert s["l0.mlp.router"] == (9, 48) and s["l0.mlp.correction"] == (9,)           # experts + identity slots
    assert "l0.mlp.e6.up" in s and "l0.mlp.e7.up" not in s                            # identity slots have no tensors
    assert s["l0.mlp.shared.down"] == (48, 28) and "l3.mlp.shared.up" not in s
    assert s["l2.mlp.gate.b"] == (40,) and s["l1.mix.o"] == (48, 3 * 14) and s["l1.mix.v"] == (14, 48)
    s = DizizenConfig.from_dict(CFG_ONES).tensor_shapes()
    assert not any(n.startswith("l2.mlp.e") for n in s) and s["l2.mlp.router"] == (2, 32)   # identity slots only


def test_config_defaults():
    d = copy.deepcopy(CFG_WIDE)
    r = d["layers"][2]["mlp"]["router"]
    del r["groups"], r["identity"]
    del d["layers"][0]["mixer"]["kv_heads"], d["layers"][0]["mixer"]["vdim"]
    d["layers"][1]["mixer"].pop("kv_from")
    cfg = DizizenConfig.from_dict(d)
    assert (cfg.layers[2]["groups"], cfg.layers[2]["keep"], cfg.layers[2]["identity"]) == (1, 1, 0)
    assert cfg.layers[0]["kv_heads"] == 8 and cfg.layers[0]["vdim"] == 16 and cfg.layers[1]["kv_from"] == -1


def test_config_validation():
    def bad(edit):
        d = copy.deepcopy(CFG_MIXED)
        edit(d)
        with pytest.raises(ValueError):
            DizizenConfig.from_dict(d)

    bad(lambda d: d["layers"][0]["mixer"].update(kv_from=2))              # not an earlier layer
    bad(lambda d: d["layers"][3]["mixer"].update(kv_from=2))              # a layer that itself borrows has none to lend
    bad(lambda d: d["layers"][2]["mixer"].update(kv_from=1))              # another key / value shape
    bad(lambda d: d["layers"][0]["mixer"].update(kv_heads=3))
    bad(lambda d: d["layers"][0]["mixer"].update(vdim=7))                 # rotated values come in pairs
    bad(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=14))         # more than the head
    bad(lambda d: d["layers"][0].update(type="general_delta"))
    bad(lambda d: d["layers"][2]["mlp"].update(kind="glu"))
    bad(lambda d: d["layers"][0]["mlp"]["router"].update(top=10))
    bad(lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4))     # 9 slots do not split in 4
    bad(lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=4))
    bad(lambda d: d["layers"][0]["mlp"]["router"].update(top=7))          # two groups of three hold six


def test_registry_and_family_sources():
    from zhilight_b200 import build, registry
    assert "Dizizen" in registry.registered()
    assert registry.supported_dtypes(CFG_ONES) == ("bfloat16", "float32")
    for name in build.FAMILY_SOURCES["dizizen"]:
        assert os.path.exists(os.path.join(build.CSRC, name + ".cu")), name


# ---------------------------------------------------------------------------------------------- the oracle by hand
def test_norm_by_hand():
    x = np.array([[3.0, -4.0]])
    got = orc.zero_centred_norm(x, np.array([0.5, -1.0]), 0.0)
    assert np.allclose(got, [[3.0 / math.sqrt(12.5) * 1.5, 0.0]])
    assert np.allclose(orc.zero_centred_norm(np.zeros((1, 4)), np.zeros(4), 1e-5), 0.0)     # eps inside the root


def test_rotation_by_hand_and_relative_angle():
    # one pair (0, 2) of a 4-vector with 2 rotated dimensions... dims = 2: pair (0, 1); dims = 4: pairs (0, 2), (1, 3)
    c, s = orc.half_tables([1], 4, 100.0)
    assert np.allclose(c[0], [math.cos(1.0), math.cos(0.1)]) and np.allclose(s[0], [math.sin(1.0), math.sin(0.1)])
    x = np.array([[[1.0, 0.0, 0.0, 2.0, 9.0]]])
    y = orc.rotate_halves(x, c, s, 4)
    assert np.allclose(y[0, 0], [math.cos(1.0), -2 * math.sin(0.1), math.sin(1.0), 2 * math.cos(0.1), 9.0])
    # turning by position j and back by position i is a turn by j - i
    rng = np.random.default_rng(0)
    v = rng.standard_normal((1, 3, 6))
    cj, sj = orc.half_tables([11], 6, 50.0)
    ci, si = orc.half_tables([4], 6, 50.0)
    cd, sd = orc.half_tables([7], 6, 50.0)
    assert np.allclose(orc.rotate_halves(orc.rotate_halves(v, cj, sj, 6), ci, si, 6, sign=-1.0), orc.rotate_halves(v, cd, sd, 6))


def test_attention_by_hand():
    q = np.array([[[1.0, 0.0]], [[0.0, 2.0]]])
    k = np.array([[[3.0, 1.0]], [[1.0, 1.0]]])
    v = np.array([[[1.0, 10.0]], [[2.0, 20.0]]])
    o = orc.causal_softmax_attention(q, k, v, 0.5)
    assert np.allclose(o[0, 0], v[0, 0])                                   # the first token sees itself only
    e = np.exp(np.array([1.0, 1.0]))                                       # scores 0.5 * (2, 2): equal weights
    assert np.allclose(o[1, 0], (e[0] * v[0, 0] + e[1] * v[1, 0]) / e.sum())
    # grouped heads: 4 query heads on 2 key/value heads use heads 0, 0, 1, 1
    rng = np.random.default_rng(1)
    q, k, v = rng.standard_normal((5, 4, 3)), rng.standard_normal((5, 2, 3)), rng.standard_normal((5, 2, 2))
    o = orc.causal_softmax_attention(q, k, v, 0.7)
    alone = orc.causal_softmax_attention(q[:, 2:3], k[:, 1:2], v[:, 1:2], 0.7)
    assert np.allclose(o[:, 2], alone[:, 0])


def test_feed_forwards_by_hand():
    W = {"gate": np.array([[1.0], [1.0]]), "gate.b": np.array([0.0, 5.0]), "up": np.array([[2.0], [-9.0]]),
         "up.b": np.array([0.5, 0.0]), "down": np.eye(2), "down.b": np.array([0.0, 1.0])}
    y = orc.clamped_gated_ff(W, "", np.array([[1.0]]), 2.0)
    g0, g1 = 1.0, 2.0                                                      # the second gate is cut at the limit from above only
    want = [g0 * orc.sigmoid(1.702 * g0) * (2.0 + 1.0), g1 * orc.sigmoid(1.702 * g1) * (-2.0 + 1.0) + 1.0]   # up clamped both ways
    assert np.allclose(y[0], want)
    W["gate.b"] = np.array([-7.0, 0.0])                                    # a very negative gate passes
    y = orc.clamped_gated_ff(W, "", np.array([[1.0]]), 2.0)
    assert np.allclose(y[0, 0], -6.0 * orc.sigmoid(1.702 * -6.0) * 3.0)
    E = {"up": np.array([[1.0, 0.0], [0.0, -1.0]]), "down": np.array([[1.0, 1.0]])}
    assert np.allclose(orc.relu2_expert(E, "", np.array([3.0, 2.0])), [9.0])


def test_route_by_hand():
    z = np.log(np.array([4.0, 1.0, 1.0, 2.0, 1.0, 1.0]))                   # scores .4 .1 .1 .2 .1 .1
    none = np.zeros(6)
    ch, w = orc.grouped_route(z, none, 2, 1, 1)
    assert list(ch) == [0, 3] and np.allclose(w, [2 / 3, 1 / 3])
    ch, w = orc.grouped_route(z, none, 2, 3, 1)                            # groups (0,1) (2,3) (4,5): only the first counts
    assert list(ch) == [0, 1] and np.allclose(w, [0.8, 0.2])
    corr = np.array([0.0, 0.0, 0.0, 0.0, 0.35, 0.0])                       # slot 4 ranks first, its weight stays its score
    ch, w = orc.grouped_route(z, corr, 2, 3, 2)
    assert list(ch) == [4, 0] and np.allclose(w, [0.2, 0.8])
    neg = np.full(6, -5.0)                                                 # every choice value negative: dropped is -inf, not 0
    ch, _ = orc.grouped_route(z, neg, 3, 3, 2)
    assert sorted(ch) == [0, 1, 3] or sorted(ch) == [0, 2, 3]
    assert set(ch) <= {0, 1, 2, 3}


def test_identity_slots_and_shared_expert():
    cfg = DizizenConfig.from_dict(CFG_ONES)
    W = _weights(cfg, 3)
    l = cfg.layers[2]                                                      # no experts, two identity slots, a shared expert
    h = np.random.default_rng(2).standard_normal((4, cfg.width))
    got = orc.experts_ff(W, "l2.mlp.", l, h)
    shared = np.stack([orc.relu2_expert(W, "l2.mlp.shared.", r) for r in h])
    assert np.allclose(got, h + shared)                                    # both slots chosen: the weights sum to 1


def test_forward_is_causal_and_layers_add_up():
    cfg = DizizenConfig.from_dict(CFG_MIXED)
    W = _weights(cfg, 1)
    toks = np.random.default_rng(3).integers(0, cfg.vocab, 17).tolist()
    full, streams, caches = orc.forward(cfg, W, toks)
    part = orc.forward(cfg, W, toks[:9])[0]
    assert np.allclose(full[:9], part, rtol=0, atol=1e-10)
    assert streams.shape == (4, 17, cfg.width) and set(caches) == {0, 1, 2, 3}
    assert caches[2][0] is caches[0][0] and caches[3][1] is caches[1][1]   # the borrowed caches are the lender's
    # with every layer scale at zero nothing enters the stream
    Z = dict(W)
    for i in range(4):
        Z["l%d.ls1" % i] = np.zeros(cfg.width)
        if "l%d.ls2" % i in Z:
            Z["l%d.ls2" % i] = np.zeros(cfg.width)
    _, s0, _ = orc.forward(cfg, Z, toks)
    assert np.allclose(s0[-1], W["embed"][toks] * cfg.embed_scale)
