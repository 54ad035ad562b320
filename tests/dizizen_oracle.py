"""Plain, slow restatement of the Dizizen layer equations in numpy float64, one function per mechanism.

Nothing here is shared with the product path: attention is a loop over heads on a full score matrix, the experts a
loop over tokens and chosen experts, the rotations are written with explicit cos / sin tables.  A whole prompt is
computed at once; by causality the value at a position is also the truth for any way of cutting the prompt into
portions or decoding it token by token.
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def zero_centred_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the checkpoint keeps w, not the multiplier."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * (1.0 + w)


def half_tables(positions, dims, base):
    """cos, sin (n, dims / 2) of the angles p * base^(-2i / dims)."""
    i = np.arange(dims // 2, dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    return np.cos(ang), np.sin(ang)


def rotate_halves(x, cos, sin, dims, sign=1.0):
    """x (n, heads, d): dimension i < dims / 2 is paired with i + dims / 2 and the pair turns by sign * the angle;
    dimensions from `dims` on pass."""
    y = x.copy()
    hf = dims // 2
    a, b = x[..., :hf], x[..., hf:dims]
    c, s = cos[:, None, :], sign * sin[:, None, :]
    y[..., :hf] = a * c - b * s
    y[..., hf:dims] = b * c + a * s
    return y


def causal_softmax_attention(q, k, v, scale):
    """q (n, H, d), k (n, G, d), v (n, G, dv): query head h reads key/value head h // (H / G), position i sees j <= i."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    mask = np.tril(np.ones((n, n), dtype=bool))
    for h in range(H):
        g = h // (H // G)
        s = np.where(mask, (q[:, h] @ k[:, g].T) * scale, -np.inf)
        e = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, h] = (e / e.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out


def attention_mixer(W, p, l, h, shared):
    """l: the layer's parsed dict; shared: {layer index: (rotated keys, rotated values)} of the layers before.
    Values are turned by their own position before they are summed; the sum of a head is turned back by the query's."""
    n = h.shape[0]
    H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
    pos = np.arange(n)
    cq, sq = half_tables(pos, l["rot_dims"], l["rot_base"]) if l["rot_dims"] else (None, None)
    cv, sv = half_tables(pos, dv, l["rot_base"])
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(n, H, d)
    if l["rot_dims"]:
        q = rotate_halves(q, cq, sq, l["rot_dims"])
    if l["kv_from"] >= 0:
        k, v = shared[l["kv_from"]]
    else:
        k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(n, G, d)
        if l["rot_dims"]:
            k = rotate_halves(k, cq, sq, l["rot_dims"])
        v = rotate_halves((h @ W[p + "v"].T + W[p + "v.b"]).reshape(n, G, dv), cv, sv, dv)
    o = rotate_halves(causal_softmax_attention(q, k, v, l["scale"]), cv, sv, dv, sign=-1.0)
    return o.reshape(n, H * dv) @ W[p + "o"].T + W[p + "o.b"], (k, v)


def clamped_gated_ff(W, p, h, limit):
    g = np.minimum(h @ W[p + "gate"].T + W[p + "gate.b"], limit)
    u = np.clip(h @ W[p + "up"].T + W[p + "up.b"], -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T + W[p + "down.b"]


def relu2_expert(W, p, h):
    return W[p + "down"] @ (np.maximum(W[p + "up"] @ h, 0.0) ** 2)


def grouped_route(z, correction, top, groups, keep):
    """z (slots,) router logits of one token -> (chosen slots, weights).  softmax over all slots; the choice looks at
    score + correction, and only inside the `keep` groups (of `groups` equal runs of neighbours) whose largest such
    value is largest; the weights are the plain scores of the chosen, normalised."""
    e = np.exp(z - z.max())
    s = e / e.sum()
    c = s + correction
    per = len(z) // groups
    best = c.reshape(groups, per).max(axis=-1)
    kept = np.argsort(-best, kind="stable")[:keep]
    masked = np.full_like(c, -np.inf)
    for g in kept:
        masked[g * per:(g + 1) * per] = c[g * per:(g + 1) * per]
    chosen = np.argsort(-masked, kind="stable")[:top]
    return chosen, s[chosen] / (s[chosen].sum() + 1e-20)


def experts_ff(W, p, l, h):
    """Slots 0 .. experts-1 are small feed-forwards, the `identity` slots after them hand the input through."""
    out = np.zeros_like(h)
    z = h @ W[p + "router"].T
    for t in range(h.shape[0]):
        chosen, weight = grouped_route(z[t], W[p + "correction"], l["top"], l["groups"], l["keep"])
        for e, s in zip(chosen, weight):
            out[t] += s * (relu2_expert(W, p + "e%d." % e, h[t]) if e < l["experts"] else h[t])
        if l["shared_ff"]:
            out[t] += relu2_expert(W, p + "shared.", h[t])
    return out


def layer(cfg, W, i, x, shared):
    """One norm, both sublayers read it; each result times its layer scale and its sigmoid gate, the sum times m."""
    l, p = cfg.layers[i], "l%d." % i
    h = zero_centred_norm(x, W[p + "norm1"], cfg.norm_eps)
    a, shared[i] = attention_mixer(W, p + "mix.", l, h, shared)
    y = W[p + "ls1"] * sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"]) * a
    if l["ff_kind"]:
        f = clamped_gated_ff(W, p + "mlp.", h, l["limit"]) if l["ff_kind"] == "dense" else experts_ff(W, p + "mlp.", l, h)
        y = y + W[p + "ls2"] * sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"]) * f
    return x + cfg.residual_mult * y


def forward(cfg, W, tokens):
    """cfg: DizizenConfig; W: name -> float64 array.  -> (logits (n, vocab), residual stream after every layer
    (layers, n, width), {layer: (keys, values) as cached})."""
    x = W["embed"][np.asarray(tokens)] * cfg.embed_scale
    shared, per_layer = {}, []
    for i in range(len(cfg.layers)):
        x = layer(cfg, W, i, x, shared)
        per_layer.append(x.copy())
    return zero_centred_norm(x, W["final.norm"], cfg.norm_eps) @ W["head"].T, np.stack(per_layer), shared


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), still float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def random_weights(cfg, seed=0, router_gain=4.0):
    """name -> float32 array whose values are exact in bfloat16.  Router rows are scaled up so that the choice of
    experts does not hang on a rounding."""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shp in sorted(cfg.tensor_shapes().items()):
        last = name.rsplit(".", 1)[-1]
        if last == "norm1" or name == "final.norm":
            a = 0.1 * rng.standard_normal(shp)
        elif last in ("ls1", "ls2"):
            a = 1.0 + 0.3 * rng.standard_normal(shp)
        elif last == "correction":
            a = 0.05 * rng.standard_normal(shp)
        elif last == "b":
            a = 0.3 * rng.standard_normal(shp)
        elif name == "embed":
            a = rng.standard_normal(shp)
        elif last == "router":
            a = router_gain * rng.standard_normal(shp) / math.sqrt(shp[-1])
        else:
            a = rng.standard_normal(shp) / math.sqrt(shp[-1])
        W[name] = bf16_round(a.astype(np.float32))
    return W
