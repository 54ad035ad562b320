"""Lagelorn pieces that need no GPU: the oracle's own consistency, config parsing and validation, tensor shapes, and the
registry entry."""
import copy
import math

import numpy as np
import pytest

from tests import lagelorn_oracle as orc
from tests.test_lagelorn_gpu import CFG_MIXED, CFG_ONES, CFG_WIDE
from zhilight_b200.lagelorn import LagelornConfig


def _weights(cfg_dict, seed=0):
    shapes = LagelornConfig.from_dict(cfg_dict).tensor_shapes()
    return {k: v.astype(np.float64) for k, v in orc.random_weights(shapes, seed).items()}


def test_config_round_trip_and_shapes():
    for d in (CFG_MIXED, CFG_ONES, CFG_WIDE):
        cfg = LagelornConfig.from_dict(d)
        again = LagelornConfig.from_dict(cfg.to_dict())
        skip = ("l_rel_rows", "r_decay_rank")           # sizes of the checkpoint, not of config.json
        for a, b in zip(cfg.layers, again.layers):
            assert {k: v for k, v in a.items() if k not in skip} == {k: v for k, v in b.items() if k not in skip}
        assert not again.complete() or all(l["type"] == "delta" for l in again.layers)
        shapes = cfg.tensor_shapes()
        assert shapes["embed"] == (cfg.vocab, cfg.width) and shapes["pos"] == (cfg.max_positions, cfg.width)
        assert shapes["side.embed"] == (cfg.vocab, len(cfg.layers) * cfg.side_dim)
    s = LagelornConfig.from_dict(CFG_MIXED).tensor_shapes()
    assert "l1.norm2" not in s and "l1.mlp.gate" not in s and "l3.mlp.down.b" not in s      # layers without feed-forward
    assert s["l0.mix.left.q"] == (64, 48) and s["l0.mix.left.k.norm"] == (32,) and s["l0.mix.left.rel"] == (10, 4)
    assert s["l0.mix.right.w2"] == (48, 5) and s["l0.mix.right.u"] == (3, 16) and s["l3.mix.right.mu.w"] == (48,)
    assert s["l1.mix.q"] == (64, 48) and s["l1.mix.v.conv"] == (96, 4) and s["l1.mix.norm"] == (24,) and s["l1.mix.A_log"] == (4,)
    assert s["l2.mlp.gate.b"] == (24,) and s["l2.side.proj"] == (48, 6) and "l0.mix.left.v" not in s


def test_config_validation():
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        LagelornConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][0]["mixer"]["left"]["vdim"] = 8          # the values are the keys
    with pytest.raises(ValueError):
        LagelornConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][1]["type"] = "attention"
    with pytest.raises(ValueError):
        LagelornConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][1]["mixer"]["conv"] = 0
    with pytest.raises(ValueError):
        LagelornConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][2]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError):
        LagelornConfig.from_dict(bad)


def test_registry_knows_the_family():
    from zhilight_b200 import registry
    assert "Lagelorn" in registry.registered()
    assert registry.supported_dtypes(CFG_ONES) == ("bfloat16", "float32")


def test_oracle_is_causal_and_scans_compose():
    W = _weights(CFG_MIXED, 3)
    toks = np.random.default_rng(0).integers(0, CFG_MIXED["vocab"], 90).tolist()
    full = orc.forward(CFG_MIXED, W, toks)[0]
    part = orc.forward(CFG_MIXED, W, toks[:47])[0]
    assert np.abs(full[:47] - part).max() < 1e-9
    # the gated delta rule written with the decayed state equals its expanded form on the old state
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((12, 2, 6)) for _ in range(3))
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    beta, g = rng.random((12, 2)), rng.random((12, 2))
    o, S = orc.gated_delta_scan(q, k, v, beta, g)
    S2 = np.zeros((2, 6, 6))
    for t in range(12):
        for h in range(2):
            S2[h] = g[t, h] * S2[h] - g[t, h] * beta[t, h] * np.outer(k[t, h], k[t, h] @ S2[h]) + beta[t, h] * np.outer(k[t, h], v[t, h])
            assert np.abs(S2[h].T @ q[t, h] - o[t, h]).max() < 1e-12
    assert np.abs(S2 - S).max() < 1e-12
    # the read-out before the write: dot with the old state plus a scalar times the current value
    r, w, u = rng.standard_normal((12, 2, 6)), rng.random((12, 2, 6)), rng.standard_normal((2, 6))
    o, S = orc.bonus_decay_scan(r, k, v, w, u)
    S2 = np.zeros((2, 6, 6))
    for t in range(12):
        for h in range(2):
            assert np.abs(r[t, h] @ S2[h] + (r[t, h] * u[h] * k[t, h]).sum() * v[t, h] - o[t, h]).max() < 1e-12
            S2[h] = w[t, h][:, None] * S2[h] + np.outer(k[t, h], v[t, h])


def test_oracle_mechanisms_by_hand():
    # one key, no table: p = e^s / (e^sink + e^s)
    q, k, v = np.ones((1, 1, 2)), np.ones((1, 1, 2)), np.array([[[3.0, 5.0]]])
    out = orc.chunk_sink_attention(q, k, v, np.zeros((2, 1)), np.array([0.5]), 0.5, 0, 4.0)
    assert np.allclose(out[0, 0], np.array([3.0, 5.0]) * math.e / (math.exp(0.5) + math.e))
    # blocks of 2: token 2 sees only itself, token 3 sees 2 and 3; the table row is added after the scale
    q, k = np.zeros((4, 1, 1)), np.zeros((4, 1, 1))
    v = np.arange(4.0).reshape(4, 1, 1)
    table = np.array([[0.0], [math.log(3.0)]])
    out = orc.chunk_sink_attention(q, k, v, table, np.array([-1e9]), 7.0, 2, 3.0)
    assert np.allclose(out[:, 0, 0], [0.0, (0 * 3 + 1) / 4, 2.0, (2 * 3 + 3) / 4])
    # convolution: the last column weighs the current token, zeros before the start
    y = orc.short_conv(np.array([[1.0], [2.0], [4.0]]), np.array([[100.0, 10.0, 1.0]]))
    assert np.allclose(y[:, 0], [1.0, 12.0, 124.0])
    # norm after the sum and the side input on a width of 2
    assert np.allclose(orc.rms_norm(np.array([3.0, 4.0]), np.array([1.0, 2.0]), 0.0), [3 / math.sqrt(12.5), 8 / math.sqrt(12.5)])
    assert np.isclose(orc.gelu_tanh(1.0), 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715)))


def test_family_library_sources_exist():
    import os
    from zhilight_b200 import build
    names = build.FAMILY_SOURCES["lagelorn"]
    assert "lagelorn_runner" in names
    for n in names:
        assert os.path.exists(os.path.join(build.CSRC, n + ".cu")), n
