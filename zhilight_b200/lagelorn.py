"""Lagelorn front end (zl_lagelorn_* C-ABI): configuration from config.json, weight loading, and the step call.

Lagelorn is a decoder-only family with learned positions, x = embed[token] + pos[p], and norm after the sum:
x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)) with plain-weight RMS norms on an fp32 residual stream; the
sublayers read x itself.  After every layer the layer's slice e of a second token embedding enters:
y = W_proj (gelu_tanh(W_gate x) * e), x <- x + rms(y) * w.  config.json lists the layers one by one:

  * "delta": a gated delta rule.  q, k (kv_heads x dim) and v (heads x vdim) pass a causal convolution of `conv` taps per
    channel and silu; q and k become unit vectors per head (q also times dim^-1/2); per head a rate beta = sigmoid(W_b x)
    and a decay g = exp(-exp(A_log) softplus(W_a x + dt_bias)); S <- g S, e = beta (v - S^T k), S <- S + k e^T, o = S^T q;
    then RMS norm per head, a weight of size vdim, a silu gate, W_o.
  * "parallel": left_scale * A(x) + right_scale * R(x).  A is attention inside blocks of mask.size positions with grouped
    key heads, biased q / k projections normed over the whole projection, the projected keys as values, a learned bias
    per head by bucketed distance (rows of `rel`, logarithmic buckets up to bias_max), and a learned sink per head in the
    softmax denominator.  R reads five mixes x + (x_prev - x) mu_s of the token with its predecessor and keeps a
    decaying state per head: o = (S + diag(u) k v^T)^T r, S <- diag(w) S + k v^T with w = exp(-exp(W_w2 tanh(W_w1 .) + w0));
    then RMS norm per head, a weight, a silu gate, W_o.

The feed-forward ("mlp": {"kind": "dense", "ff"} or null) is W_down (gelu_tanh(W_gate x) * (W_up x)) with biases.  The
logits are head . norm(x), soft-capped: cap * tanh(z / cap).

    {"architecture": "Lagelorn", "vocab": V, "width": D, "max_positions": P, "norm": {"eps": e}, "postln_alpha": a,
     "token_side": {"dim": s}, "logit_softcap": c,
     "layers": [{"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...},
                {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "bias_max",
                                                        "mask": {"size"}},
                                               "right": {"heads", "dim"}, "left_scale", "right_scale"}, "mlp": ...}]}

Checkpoint tensors: embed, pos, side.embed (vocab, layers * s), head, final.norm; per layer l<i>.norm1 / norm2,
l<i>.side.{gate, proj, norm}, l<i>.mlp.{gate, up, down}(+ .b); delta l<i>.mix.{q, k, v, q.conv, k.conv, v.conv, b, a, A_log,
dt_bias, g, norm, o}; parallel l<i>.mix.left.{q, q.b, k, k.b, q.norm, k.norm, rel, sink, o} and l<i>.mix.right.{mu.r, mu.k,
mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o}.  Linears are (out, in).  The row count of `rel` and the inner size of
the decay path (rows of w1) come from the checkpoint.
"""
import ctypes

import numpy as np

from . import _lib
from .safetensors_io import is_bf16

LAYER_TYPES = {"delta": 0, "parallel": 1}


class LagelornLayer(ctypes.Structure):
    """zl_lagelorn_layer_t"""
    _fields_ = [("type", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("dim", ctypes.c_int),
                ("vdim", ctypes.c_int), ("conv", ctypes.c_int), ("l_heads", ctypes.c_int), ("l_kv_heads", ctypes.c_int),
                ("l_dim", ctypes.c_int), ("l_chunk", ctypes.c_int), ("l_rel_rows", ctypes.c_int),
                ("l_bias_max", ctypes.c_float), ("l_scale", ctypes.c_float), ("r_heads", ctypes.c_int),
                ("r_dim", ctypes.c_int), ("r_decay_rank", ctypes.c_int), ("left_scale", ctypes.c_float),
                ("right_scale", ctypes.c_float), ("ff", ctypes.c_int)]


class LagelornCConfig(ctypes.Structure):
    """zl_lagelorn_config_t"""
    _fields_ = [("num_layers", ctypes.c_int), ("width", ctypes.c_int), ("vocab", ctypes.c_int),
                ("max_positions", ctypes.c_int), ("side_dim", ctypes.c_int), ("eps", ctypes.c_float),
                ("postln_alpha", ctypes.c_float), ("logit_softcap", ctypes.c_float), ("dtype", ctypes.c_int),
                ("max_batch", ctypes.c_int), ("max_seq", ctypes.c_int), ("max_step_tokens", ctypes.c_int),
                ("use_pdl", ctypes.c_int), ("use_graph", ctypes.c_int)]


_LAYER_DEFAULTS = dict(heads=0, kv_heads=0, dim=0, vdim=0, conv=0, l_heads=0, l_kv_heads=0, l_dim=0, l_chunk=0, l_rel_rows=0,
                       l_bias_max=0.0, l_scale=0.0, r_heads=0, r_dim=0, r_decay_rank=0, left_scale=0.0, right_scale=0.0, ff=0)


class LagelornConfig:
    """Parsed config.json of a Lagelorn model.  `layers` is a list of dicts with every key of zl_lagelorn_layer_t;
    l_rel_rows / r_decay_rank 0 mean "take it from the checkpoint"."""

    def __init__(self, vocab, width, layers, max_positions, side_dim, norm_eps=1e-6, postln_alpha=1.0, logit_softcap=30.0):
        self.vocab, self.width, self.max_positions, self.side_dim = int(vocab), int(width), int(max_positions), int(side_dim)
        self.norm_eps, self.postln_alpha, self.logit_softcap = float(norm_eps), float(postln_alpha), float(logit_softcap)
        self.layers = layers
        if self.logit_softcap <= 0:
            raise ValueError("logit_softcap must be positive")
        for i, l in enumerate(layers):
            if l["type"] == "delta":
                if l["heads"] <= 0 or l["kv_heads"] <= 0 or l["heads"] % l["kv_heads"]:
                    raise ValueError("layer %d: heads is not a multiple of kv_heads" % i)
                if l["conv"] < 1:
                    raise ValueError("layer %d: conv must be at least 1" % i)
            else:
                if l["l_heads"] <= 0 or l["l_kv_heads"] <= 0 or l["l_heads"] % l["l_kv_heads"]:
                    raise ValueError("layer %d: left.heads is not a multiple of left.kv_heads" % i)
                if l["l_chunk"] < 0:
                    raise ValueError("layer %d: mask.size must not be negative" % i)

    @classmethod
    def from_dict(cls, d):
        layers = []
        for i, l in enumerate(d["layers"]):
            kind = l.get("type")
            if kind not in LAYER_TYPES:
                raise ValueError("layer %d: unknown layer type %r" % (i, kind))
            mx, mlp = l["mixer"], l.get("mlp")
            out = dict(_LAYER_DEFAULTS, type=kind)
            if kind == "delta":
                out.update(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                           vdim=int(mx.get("vdim", mx["dim"])), conv=int(mx["conv"]))
            else:
                lf, rt = mx["left"], mx["right"]
                if int(lf.get("vdim", lf["dim"])) != int(lf["dim"]):
                    raise ValueError("layer %d: the values of the left mixer are its keys: vdim must equal dim" % i)
                out.update(l_heads=int(lf["heads"]), l_kv_heads=int(lf.get("kv_heads", lf["heads"])), l_dim=int(lf["dim"]),
                           l_chunk=int((lf.get("mask") or {}).get("size", 0)), l_rel_rows=int(lf.get("rel_rows", 0)),
                           l_bias_max=float(lf["bias_max"]), l_scale=float(lf["scale"]), r_heads=int(rt["heads"]),
                           r_dim=int(rt["dim"]), r_decay_rank=int(rt.get("decay_rank", 0)),
                           left_scale=float(mx["left_scale"]), right_scale=float(mx["right_scale"]))
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ValueError("layer %d: unknown feed-forward kind %r" % (i, mlp.get("kind")))
                out.update(ff=int(mlp["ff"]))
            layers.append(out)
        return cls(d["vocab"], d["width"], layers, d["max_positions"], d["token_side"]["dim"],
                   (d.get("norm") or {}).get("eps", 1e-6), d.get("postln_alpha", 1.0), d["logit_softcap"])

    def to_dict(self):
        out = []
        for l in self.layers:
            if l["type"] == "delta":
                mx = {k: l[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            else:
                left = {"heads": l["l_heads"], "kv_heads": l["l_kv_heads"], "dim": l["l_dim"], "vdim": l["l_dim"],
                        "scale": l["l_scale"], "bias_max": l["l_bias_max"], "mask": {"size": l["l_chunk"]}}
                mx = {"left": left, "right": {"heads": l["r_heads"], "dim": l["r_dim"]}, "left_scale": l["left_scale"],
                      "right_scale": l["right_scale"]}
            out.append({"type": l["type"], "mixer": mx, "mlp": {"kind": "dense", "ff": l["ff"]} if l["ff"] else None})
        return {"architecture": "Lagelorn", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "layers": out, "norm": {"eps": self.norm_eps}, "postln_alpha": self.postln_alpha,
                "token_side": {"dim": self.side_dim}, "logit_softcap": self.logit_softcap}

    def complete(self):
        return all(l["type"] == "delta" or (l["l_rel_rows"] > 0 and l["r_decay_rank"] > 0) for l in self.layers)

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor (the sizes taken from the checkpoint must be known)."""
        D, sd, s = self.width, self.side_dim, {}
        s["embed"] = s["head"] = (self.vocab, D)
        s["pos"] = (self.max_positions, D)
        s["side.embed"] = (self.vocab, len(self.layers) * sd)
        s["final.norm"] = (D,)
        for i, l in enumerate(self.layers):
            p = "l%d." % i
            s[p + "norm1"] = (D,)
            if l["type"] == "delta":
                H, G, d, vd, taps = l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["conv"]
                m = p + "mix."
                s[m + "q"] = s[m + "k"] = (G * d, D)
                s[m + "v"] = s[m + "g"] = (H * vd, D)
                s[m + "q.conv"] = s[m + "k.conv"] = (G * d, taps)
                s[m + "v.conv"] = (H * vd, taps)
                s[m + "b"] = s[m + "a"] = (H, D)
                s[m + "A_log"] = s[m + "dt_bias"] = (H,)
                s[m + "norm"] = (vd,)
                s[m + "o"] = (D, H * vd)
            else:
                H, G, d = l["l_heads"], l["l_kv_heads"], l["l_dim"]
                m = p + "mix.left."
                s[m + "q"], s[m + "q.b"], s[m + "q.norm"] = (H * d, D), (H * d,), (H * d,)
                s[m + "k"], s[m + "k.b"], s[m + "k.norm"] = (G * d, D), (G * d,), (G * d,)
                s[m + "rel"], s[m + "sink"], s[m + "o"] = (l["l_rel_rows"], H), (H,), (D, H * d)
                RH, rd, R = l["r_heads"], l["r_dim"], l["r_decay_rank"]
                m = p + "mix.right."
                for n in "rkvgw":
                    s[m + "mu." + n] = (D,)
                for n in "rkvg":
                    s[m + n] = (RH * rd, D)
                s[m + "w1"], s[m + "w2"], s[m + "w0"] = (R, D), (RH * rd, R), (RH * rd,)
                s[m + "u"], s[m + "norm"], s[m + "o"] = (RH, rd), (RH * rd,), (D, RH * rd)
            if l["ff"]:
                F = l["ff"]
                s[p + "norm2"] = (D,)
                s[p + "mlp.gate"] = s[p + "mlp.up"] = (F, D)
                s[p + "mlp.gate.b"] = s[p + "mlp.up.b"] = (F,)
                s[p + "mlp.down"], s[p + "mlp.down.b"] = (D, F), (D,)
            s[p + "side.gate"], s[p + "side.proj"], s[p + "side.norm"] = (sd, D), (D, sd), (D,)
        return s


DTYPES = {"bf16": 1, "bfloat16": 1, "f32": 2, "float32": 2}


class LagelornDecoder:
    """One model instance on the current CUDA device.  Slots (0..max_batch-1) each own `max_seq` key / value rows per
    parallel layer, the recurrent states of both kinds of layer, the convolutions' last inputs and the last token of the
    predecessor mixes; the engine's scheduler decides which sequence lives in which slot.  The native model is created
    when the sizes are complete: at once if the table rows and decay ranks are given, otherwise when load_state_dict sees
    the checkpoint."""

    architecture = "Lagelorn"
    supports_dtypes = ("bfloat16", "float32")
    supports_ragged_steps = True

    def __init__(self, config, dtype="bf16", max_batch=1, max_seq=512, max_step_tokens=512, use_pdl=True, use_graph=True):
        self.lib = _lib.load()
        self.config = config
        self.vocab_size = config.vocab
        self.dtype = dtype
        self.max_batch = int(max_batch)
        self.max_seq = min(int(max_seq), config.max_positions)      # a position needs a row of the position table
        self.max_step_tokens = max(int(max_step_tokens), self.max_batch)
        self.use_pdl, self.use_graph = use_pdl, use_graph
        self.h = None
        if config.complete():
            self._create()

    def _create(self):
        c = self.config
        self.cfg = LagelornCConfig(len(c.layers), c.width, c.vocab, c.max_positions, c.side_dim, c.norm_eps, c.postln_alpha,
                                   c.logit_softcap, DTYPES[self.dtype], self.max_batch, self.max_seq, self.max_step_tokens,
                                   int(self.use_pdl), int(self.use_graph))
        arr = (LagelornLayer * len(c.layers))()
        for i, l in enumerate(c.layers):
            arr[i] = LagelornLayer(LAYER_TYPES[l["type"]], *[l[k] for k, _ in LagelornLayer._fields_[1:]])
        h = ctypes.c_void_p()
        _lib.check(self.lib.zl_lagelorn_create(ctypes.byref(self.cfg), arr, ctypes.byref(h)))
        self.h = h

    @classmethod
    def from_config_dict(cls, d, **kw):
        return cls(LagelornConfig.from_dict(d), **kw)

    def close(self):
        if getattr(self, "h", None):
            self.lib.zl_lagelorn_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_state_dict(self, state_dict):
        """name -> numpy array: bfloat16 bit patterns (safetensors_io.Bf16Array) or float32."""
        for i, l in enumerate(self.config.layers):
            if l["type"] != "parallel":
                continue
            for key, name in (("l_rel_rows", "l%d.mix.left.rel" % i), ("r_decay_rank", "l%d.mix.right.w1" % i)):
                if l[key] <= 0:
                    if name not in state_dict:
                        raise ValueError("tensor %s is missing" % name)
                    l[key] = int(np.asarray(state_dict[name]).shape[0])
        if self.h is None:
            self._create()
        needed = self.config.tensor_shapes()
        for name, arr in state_dict.items():
            a = np.ascontiguousarray(arr)
            if name not in needed:
                continue                      # a checkpoint may carry tensors this family does not use
            if not (is_bf16(arr) or a.dtype == np.float32):
                raise ValueError("tensor %s: expected bfloat16 or float32, got %s" % (name, a.dtype))
            if tuple(a.shape) != tuple(needed[name]):
                raise ValueError("tensor %s: shape %s, expected %s" % (name, tuple(a.shape), tuple(needed[name])))
            rows, cols = (1, a.size) if a.ndim <= 1 else (a.shape[0], a.size // a.shape[0])
            _lib.check(self.lib.zl_lagelorn_load_tensor(self.h, name.encode(), a.ctypes.data_as(ctypes.c_void_p), rows, cols,
                                                        a.itemsize))
        _lib.check(self.lib.zl_lagelorn_finalize(self.h))

    def init_synthetic(self, seed=0):
        for l in self.config.layers:
            if l["type"] == "parallel":
                if l["l_rel_rows"] <= 0:
                    l["l_rel_rows"] = 32
                if l["r_decay_rank"] <= 0:
                    l["r_decay_rank"] = 64
        if self.h is None:
            self._create()
        _lib.check(self.lib.zl_lagelorn_init_synthetic(self.h, seed))

    def step(self, tokens, slots, positions, want_rows=(), want_logits=True):
        """One step over T rows.  Returns (next tokens (n_want), logits (n_want, vocab) or None) for the wanted rows."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        s = np.ascontiguousarray(slots, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        w = np.ascontiguousarray(want_rows, dtype=np.int32)
        nxt = np.empty(w.size, dtype=np.int32)
        logits = np.empty((w.size, self.vocab_size), dtype=np.float32) if want_logits else None
        _lib.check(self.lib.zl_lagelorn_step(
            self.h, t.ctypes.data_as(ctypes.c_void_p), s.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
            t.size, w.ctypes.data_as(ctypes.c_void_p) if w.size else None, w.size,
            logits.ctypes.data_as(ctypes.c_void_p) if (want_logits and w.size) else None,
            nxt.ctypes.data_as(ctypes.c_void_p) if w.size else None))
        return nxt, logits

    # the two calls LlamaDecoder offers, on top of step()
    def prefill(self, task, tokens, pos0=0, want_logits=False):
        n = len(tokens)
        nxt, logits = None, None
        for c0 in range(0, n, self.max_step_tokens):
            chunk = tokens[c0:c0 + self.max_step_tokens]
            last = c0 + len(chunk) == n
            nxt, logits = self.step(chunk, [task] * len(chunk), range(pos0 + c0, pos0 + c0 + len(chunk)),
                                    [len(chunk) - 1] if last else [], want_logits)
        return (int(nxt[0]), logits) if want_logits else int(nxt[0])

    def decode(self, tokens, positions, want_logits=False):
        b = len(tokens)
        nxt, logits = self.step(tokens, range(b), positions, range(b), want_logits)
        return (nxt, logits) if want_logits else nxt

    def set_state(self, tokens, positions):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        _lib.check(self.lib.zl_lagelorn_set_state(self.h, t.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
                                                  t.size))

    def step_device(self, b):
        _lib.check(self.lib.zl_lagelorn_step_device(self.h, b))

    def sync(self):
        _lib.check(self.lib.zl_lagelorn_sync(self.h))

    def stream(self):
        return self.lib.zl_lagelorn_stream(self.h)

    def capture_layers(self, on=True):
        _lib.check(self.lib.zl_lagelorn_capture_layers(self.h, int(on)))

    def read_layers(self, n_tokens):
        out = np.empty((len(self.config.layers), n_tokens, self.config.width), dtype=np.float32)
        _lib.check(self.lib.zl_lagelorn_read_layers(self.h, out.ctypes.data_as(ctypes.c_void_p), n_tokens))
        return out

    def read_state(self, layer, slot):
        l = self.config.layers[layer]
        shape = (l["heads"], l["dim"], l["vdim"]) if l["type"] == "delta" else (l["r_heads"], l["r_dim"], l["r_dim"])
        out = np.empty(shape, dtype=np.float32)
        _lib.check(self.lib.zl_lagelorn_read_state(self.h, layer, slot, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def stats(self):
        wb, kn = ctypes.c_double(), ctypes.c_int()
        _lib.check(self.lib.zl_lagelorn_stats(self.h, ctypes.byref(wb), ctypes.byref(kn)))
        return wb.value, kn.value
