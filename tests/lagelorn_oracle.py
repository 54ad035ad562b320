"""Plain numpy float64 restatement of the Lagelorn family, one function per mechanism.

Nothing here is shared with the product path: attention works on full score matrices, the recurrences are explicit
loops over tokens with outer products, the convolution is a loop over taps.  `weights` maps checkpoint tensor names
to float64 arrays; `cfg` is the parsed config.json (a dict).
"""
import math

import numpy as np


def rms_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def distance_bucket(n, rows, far):
    """Row of the distance table for distance n >= 0: one row per distance below rows // 2, then rows - rows // 2
    logarithmic steps up to distance `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def chunk_sink_attention(q, k, v, table, sink, scale, chunk, far, pos0=0):
    """q (T, H, d), k (T, G, d), v (T, G, dv); token i at position pos0 + i sees j <= i of its own chunk of `chunk`
    positions (0: all); score = scale q.k + table[bucket(i - j), h]; the softmax denominator also holds exp(sink[h])."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // rep
        s = scale * (q[:, h] @ k[:, g].T)
        for i in range(T):
            logits = []
            idx = []
            for j in range(i + 1):
                if chunk and (pos0 + i) // chunk != (pos0 + j) // chunk:
                    continue
                logits.append(s[i, j] + table[distance_bucket(i - j, table.shape[0], far), h])
                idx.append(j)
            logits = np.array(logits)
            m = max(logits.max(), sink[h])
            e = np.exp(logits - m)
            den = e.sum() + math.exp(sink[h] - m)
            out[i, h] = (e / den) @ v[idx, g]
    return out


def left_mixer(h, W, p, mc, eps):
    H, G, d = mc["heads"], mc["kv_heads"], mc["dim"]
    q = h @ W[p + "q"].T + W[p + "q.b"]
    k = h @ W[p + "k"].T + W[p + "k.b"]
    v = k.copy()
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    T = h.shape[0]
    chunk = (mc.get("mask") or {}).get("size", 0)
    o = chunk_sink_attention(q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, d), W[p + "rel"], W[p + "sink"],
                             mc["scale"], chunk, mc["bias_max"])
    return o.reshape(T, -1) @ W[p + "o"].T


def shifted(h):
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    return prev


def bonus_decay_scan(r, k, v, w, u):
    """r, k, w (T, H, dk), v (T, H, dv), u (H, dk).  o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T."""
    T, H, dk = r.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv))
    S = np.zeros((H, dk, dv))
    for t in range(T):
        for h in range(H):
            kv = np.outer(k[t, h], v[t, h])
            out[t, h] = (S[h] + u[h][:, None] * kv).T @ r[t, h]
            S[h] = w[t, h][:, None] * S[h] + kv
    return out, S


def right_mixer(h, W, p, mc, eps, keep=None):
    H, d = mc["heads"], mc["dim"]
    T = h.shape[0]
    dx = shifted(h) - h
    mix = {s: h + dx * W[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[p + "r"].T).reshape(T, H, d)
    k = (mix["k"] @ W[p + "k"].T).reshape(T, H, d)
    v = (mix["v"] @ W[p + "v"].T).reshape(T, H, d)
    gate = silu(mix["g"] @ W[p + "g"].T)
    w = np.exp(-np.exp(np.tanh(mix["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, d)
    o, S = bonus_decay_scan(r, k, v, w, W[p + "u"])
    if keep is not None:
        keep.append(S)
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps)
    return (o.reshape(T, -1) * W[p + "norm"] * gate) @ W[p + "o"].T


def short_conv(x, taps_w):
    """x (T, C), taps_w (C, taps): y[t, c] = sum_j taps_w[c, j] x[t - (taps - 1 - j), c], zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += taps_w[:, j] * x[:T - back]
    return y


def gated_delta_scan(q, k, v, beta, g):
    """q, k (T, H, dk), v (T, H, dv), beta, g (T, H): S <- g S; e = beta (v - S^T k); S <- S + k e^T; o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv))
    S = np.zeros((H, dk, dv))
    for t in range(T):
        for h in range(H):
            S[h] *= g[t, h]
            e = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] += np.outer(k[t, h], e)
            out[t, h] = S[h].T @ q[t, h]
    return out, S


def delta_mixer(h, W, p, mc, eps, keep=None):
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    T = h.shape[0]
    rep = H // G
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    q = np.repeat(q, rep, axis=1)
    k = np.repeat(k, rep, axis=1)
    beta = sigmoid(h @ W[p + "b"].T)
    g = np.exp(-np.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    o, S = gated_delta_scan(q, k, v, beta, g)
    if keep is not None:
        keep.append(S)
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * W[p + "norm"]
    return (o.reshape(T, -1) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def dense_ff(h, W, p):
    a = gelu_tanh(h @ W[p + "gate"].T + W[p + "gate.b"]) * (h @ W[p + "up"].T + W[p + "up.b"])
    return a @ W[p + "down"].T + W[p + "down.b"]


def side_input(x, tokens, W, i, dim, eps):
    p = "l%d.side." % i
    e = W["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ W[p + "gate"].T) * e) @ W[p + "proj"].T
    return x + y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + eps) * W[p + "norm"]


def layer(x, tokens, W, cfg, i, keep=None):
    lc = cfg["layers"][i]
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    p = "l%d." % i
    if lc["type"] == "delta":
        m = delta_mixer(x, W, p + "mix.", lc["mixer"], eps, keep)
    else:
        mc = lc["mixer"]
        m = mc["left_scale"] * left_mixer(x, W, p + "mix.left.", mc["left"], eps) + \
            mc["right_scale"] * right_mixer(x, W, p + "mix.right.", mc["right"], eps, keep)
    x = rms_norm(alpha * x + m, W[p + "norm1"], eps)
    if lc.get("mlp") is not None:
        x = rms_norm(alpha * x + dense_ff(x, W, p + "mlp."), W[p + "norm2"], eps)
    return side_input(x, tokens, W, i, cfg["token_side"]["dim"], eps)


def model(tokens, W, cfg, return_layers=False):
    """Logits (T, vocab) of one sequence from position 0; with return_layers also the stream after every layer."""
    z, streams, _ = forward(cfg, W, tokens)
    return (z, streams) if return_layers else z


def forward(cfg, W, tokens):
    """-> (logits (T, vocab), the stream after every layer (L, T, width), the final recurrent state of every layer)."""
    tokens = np.asarray(tokens)
    x = W["embed"][tokens] + W["pos"][:len(tokens)]
    streams, states = [], []
    for i in range(len(cfg["layers"])):
        x = layer(x, tokens, W, cfg, i, states)
        streams.append(x)
    z = rms_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    cap = cfg["logit_softcap"]
    return cap * np.tanh(z / cap), np.stack(streams), states


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), still float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def random_weights(shapes, seed=0):
    """shapes: name -> shape.  -> name -> float32 array whose values are exact in bfloat16."""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shp in sorted(shapes.items()):
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2") and "side" not in name:
            a = 1.0 + 0.2 * rng.standard_normal(shp)
        elif name.endswith("side.norm"):
            a = 0.3 + 0.05 * rng.standard_normal(shp)
        elif ".mu." in name:
            a = rng.random(shp)
        elif last in ("b", "sink", "u", "dt_bias", "A_log") and len(shp) == 1 or last == "u":
            a = 0.5 * rng.standard_normal(shp)
        elif last == "w0":
            a = -1.5 + rng.standard_normal(shp)
        elif last == "rel":
            a = rng.standard_normal(shp)
        elif last == "conv":
            a = 0.5 * rng.standard_normal(shp)
        elif name in ("embed", "side.embed"):
            a = rng.standard_normal(shp)
        elif name == "pos":
            a = 0.3 * rng.standard_normal(shp)
        else:
            a = rng.standard_normal(shp) / math.sqrt(shp[-1])
        W[name] = bf16_round(a.astype(np.float32))
    return W
