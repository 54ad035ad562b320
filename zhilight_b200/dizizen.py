"""Dizizen front end (zl_dizizen_* C-ABI): configuration from config.json, weight loading, and the step call.

Dizizen is a decoder-only family whose config.json lists the layers one by one.  The residual stream is fp32,
x = embedding.scale * embed[token].  A layer is *parallel*: one RMS norm (weight 1 + w) h = norm1(x) feeds the mixer and
the feed-forward, and

    x += residual_mult * (ls1 * sigmoid(W_rg1 h + b_rg1) * mixer(h) + ls2 * sigmoid(W_rg2 h + b_rg2) * ff(h))

with per-channel layer scales ls1 / ls2 and a full-width sigmoid gate per sublayer.  The mixer:

  * "attention": grouped key/value heads, biased q / k / v / o projections, rotation of the first rot.dims dimensions of
    q and k in halves (i with i + dims / 2), **rotated values**: the value at position j is turned by j over all vdim
    dimensions (same pairing, frequencies base^(-2m / vdim)) and cached so, and a head's output at position i is turned
    back by i; plain causal softmax with the configured score scale; "kv_from": j reads layer j's caches.

The feed-forward is absent (mlp null), "dense": W_down (g sigmoid(1.702 g) (u + 1)) with g = min(W_gate h, limit),
u = clamp(W_up h, +-limit) and biases, or "moe": relu^2 experts W_down relu(W_up h)^2 without biases, of which `top` are
chosen per token.  Router scores are a softmax over experts + identity slots; the choice looks at score + correction
inside the groups.keep best of groups.count equal groups of neighbouring slots (a group's rank is its largest score +
correction); the weights are the chosen slots' plain scores over their sum.  The last router.identity slots have no
tensors: they return h itself.  A shared expert of the same form (mlp.shared.ff) is added for every token.  config.json:

    {"architecture": "Dizizen", "vocab": V, "width": D, "residual_mult": m, "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", optional "kv_from", "rot": {"base", "dims"}},
                 "mlp": null | {"kind": "dense", "ff", "limit"}
                      | {"kind": "moe", "expert": {"ff"}, "shared": {"ff"} or absent,
                         "router": {"experts", "identity", "top", "groups": {"count", "keep"}}}}, ...]}

Checkpoint tensors: embed, head, final.norm, per layer l<i>.norm1, l<i>.ls1, l<i>.rg1, l<i>.rg1.b (and ls2, rg2, rg2.b
with a feed-forward), l<i>.mix.{q, q.b, k, k.b, v, v.b, o, o.b} (no k / v with kv_from), dense l<i>.mlp.{gate, gate.b, up,
up.b, down, down.b}, experts l<i>.mlp.{router (experts + identity rows), correction, e<j>.up, e<j>.down, shared.up,
shared.down}; Linears are (out, in).
"""
import ctypes

import numpy as np

from . import _lib
from .safetensors_io import is_bf16

FF_KINDS = {None: 0, "dense": 1, "moe": 2}


class DizizenLayer(ctypes.Structure):
    """zl_dizizen_layer_t"""
    _fields_ = [("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("dim", ctypes.c_int), ("vdim", ctypes.c_int),
                ("kv_from", ctypes.c_int), ("rot_dims", ctypes.c_int), ("rot_base", ctypes.c_float), ("scale", ctypes.c_float),
                ("ff_kind", ctypes.c_int), ("ff", ctypes.c_int), ("limit", ctypes.c_float), ("experts", ctypes.c_int),
                ("identity", ctypes.c_int), ("top", ctypes.c_int), ("groups", ctypes.c_int), ("keep", ctypes.c_int),
                ("shared_ff", ctypes.c_int)]


class DizizenCConfig(ctypes.Structure):
    """zl_dizizen_config_t"""
    _fields_ = [("num_layers", ctypes.c_int), ("width", ctypes.c_int), ("vocab", ctypes.c_int), ("eps", ctypes.c_float),
                ("embed_scale", ctypes.c_float), ("residual_mult", ctypes.c_float), ("dtype", ctypes.c_int),
                ("max_batch", ctypes.c_int), ("max_seq", ctypes.c_int), ("max_step_tokens", ctypes.c_int),
                ("use_pdl", ctypes.c_int), ("use_graph", ctypes.c_int)]


class DizizenConfig:
    """Parsed config.json of a Dizizen model.  `layers` is a list of dicts with every key of zl_dizizen_layer_t
    (ff_kind is None, "dense" or "moe")."""

    def __init__(self, vocab, width, layers, norm_eps=1e-5, embed_scale=1.0, residual_mult=1.0):
        self.vocab, self.width = int(vocab), int(width)
        self.norm_eps, self.embed_scale, self.residual_mult = float(norm_eps), float(embed_scale), float(residual_mult)
        self.layers = layers
        for i, l in enumerate(layers):
            if l["heads"] % l["kv_heads"]:
                raise ValueError("layer %d: heads is not a multiple of kv_heads" % i)
            if l["rot_dims"] % 2 or l["rot_dims"] > l["dim"]:
                raise ValueError("layer %d: rot.dims must be even and at most dim" % i)
            if l["vdim"] % 2:
                raise ValueError("layer %d: rotated values need an even vdim" % i)
            j = l["kv_from"]
            if j >= 0:
                s = layers[j] if j < i else None
                if not (s and s["kv_from"] < 0 and all(s[k] == l[k] for k in ("kv_heads", "dim", "vdim"))):
                    raise ValueError("layer %d: kv_from must name an earlier layer with keys and values of its own and the "
                                     "same shape" % i)
            if l["ff_kind"] == "moe":
                slots = l["experts"] + l["identity"]
                if not 0 < l["top"] <= slots:
                    raise ValueError("layer %d: router.top must be between 1 and experts + identity" % i)
                if l["groups"] < 1 or slots % l["groups"] or not 0 < l["keep"] <= l["groups"]:
                    raise ValueError("layer %d: groups.count must divide experts + identity and keep lie in 1..count" % i)
                if l["keep"] * (slots // l["groups"]) < l["top"]:
                    raise ValueError("layer %d: the kept groups hold fewer slots than router.top" % i)

    @classmethod
    def from_dict(cls, d):
        layers = []
        for i, l in enumerate(d["layers"]):
            if l.get("type") != "attention":
                raise ValueError("layer %d: unknown mixer type %r" % (i, l.get("type")))
            mx, mlp = l["mixer"], l.get("mlp")
            rot = mx.get("rot") or {}
            kv_from = mx.get("kv_from")
            out = dict(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                       vdim=int(mx.get("vdim", mx["dim"])), kv_from=-1 if kv_from is None else int(kv_from),
                       rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                       scale=float(mx.get("scale", int(mx["dim"]) ** -0.5)), ff_kind=None, ff=0, limit=0.0, experts=0,
                       identity=0, top=0, groups=1, keep=1, shared_ff=0)
            if mlp is not None:
                kind = mlp.get("kind")
                if kind == "dense":
                    out.update(ff_kind="dense", ff=int(mlp["ff"]), limit=float(mlp["limit"]))
                elif kind == "moe":
                    r = mlp["router"]
                    g = r.get("groups") or {}
                    out.update(ff_kind="moe", ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]),
                               identity=int(r.get("identity", 0)), top=int(r["top"]), groups=int(g.get("count", 1)),
                               keep=int(g.get("keep", g.get("count", 1))), shared_ff=int((mlp.get("shared") or {}).get("ff", 0)))
                else:
                    raise ValueError("layer %d: unknown feed-forward kind %r" % (i, kind))
            layers.append(out)
        return cls(d["vocab"], d["width"], layers, (d.get("norm") or {}).get("eps", 1e-5),
                   (d.get("embedding") or {}).get("scale", 1.0), d.get("residual_mult", 1.0))

    def to_dict(self):
        out = []
        for l in self.layers:
            mx = {k: l[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")}
            mx["rot"] = {"base": l["rot_base"], "dims": l["rot_dims"]}
            if l["kv_from"] >= 0:
                mx["kv_from"] = l["kv_from"]
            mlp = None
            if l["ff_kind"] == "dense":
                mlp = {"kind": "dense", "ff": l["ff"], "limit": l["limit"]}
            elif l["ff_kind"] == "moe":
                mlp = {"kind": "moe", "expert": {"ff": l["ff"]},
                       "router": {"experts": l["experts"], "identity": l["identity"], "top": l["top"],
                                  "groups": {"count": l["groups"], "keep": l["keep"]}}}
                if l["shared_ff"]:
                    mlp["shared"] = {"ff": l["shared_ff"]}
            out.append({"type": "attention", "mixer": mx, "mlp": mlp})
        return {"architecture": "Dizizen", "vocab": self.vocab, "width": self.width, "layers": out,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embed_scale}, "residual_mult": self.residual_mult}

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor."""
        D, s = self.width, {}
        s["embed"] = s["head"] = (self.vocab, D)
        s["final.norm"] = (D,)
        for i, l in enumerate(self.layers):
            p, H, G, d, vd = "l%d." % i, l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            s[p + "norm1"] = s[p + "ls1"] = s[p + "rg1.b"] = (D,)
            s[p + "rg1"] = (D, D)
            s[p + "mix.q"], s[p + "mix.q.b"] = (H * d, D), (H * d,)
            if l["kv_from"] < 0:
                s[p + "mix.k"], s[p + "mix.k.b"] = (G * d, D), (G * d,)
                s[p + "mix.v"], s[p + "mix.v.b"] = (G * vd, D), (G * vd,)
            s[p + "mix.o"], s[p + "mix.o.b"] = (D, H * vd), (D,)
            if l["ff_kind"]:
                s[p + "ls2"] = s[p + "rg2.b"] = (D,)
                s[p + "rg2"] = (D, D)
            if l["ff_kind"] == "dense":
                s[p + "mlp.gate"] = s[p + "mlp.up"] = (l["ff"], D)
                s[p + "mlp.gate.b"] = s[p + "mlp.up.b"] = (l["ff"],)
                s[p + "mlp.down"], s[p + "mlp.down.b"] = (D, l["ff"]), (D,)
            elif l["ff_kind"] == "moe":
                slots = l["experts"] + l["identity"]
                s[p + "mlp.router"], s[p + "mlp.correction"] = (slots, D), (slots,)
                for e in range(l["experts"]):
                    s[p + "mlp.e%d.up" % e], s[p + "mlp.e%d.down" % e] = (l["ff"], D), (D, l["ff"])
                if l["shared_ff"]:
                    s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = (l["shared_ff"], D), (D, l["shared_ff"])
        return s


DTYPES = {"bf16": 1, "bfloat16": 1, "f32": 2, "float32": 2}


class DizizenDecoder:
    """One model instance on the current CUDA device.  Slots (0..max_batch-1) each own `max_seq` key / value rows per
    layer that has keys and values of its own; the engine's scheduler decides which sequence lives in which slot."""

    architecture = "Dizizen"
    supports_dtypes = ("bfloat16", "float32")
    supports_ragged_steps = True

    def __init__(self, config, dtype="bf16", max_batch=1, max_seq=512, max_step_tokens=512, use_pdl=True, use_graph=True):
        self.lib = _lib.load()
        self.config = config
        self.vocab_size = config.vocab
        self.dtype = dtype
        self.max_batch, self.max_seq = int(max_batch), int(max_seq)
        self.max_step_tokens = max(int(max_step_tokens), self.max_batch)
        c = config
        self.cfg = DizizenCConfig(len(c.layers), c.width, c.vocab, c.norm_eps, c.embed_scale, c.residual_mult, DTYPES[dtype],
                                  self.max_batch, self.max_seq, self.max_step_tokens, int(use_pdl), int(use_graph))
        arr = (DizizenLayer * len(c.layers))()
        for i, l in enumerate(c.layers):
            arr[i] = DizizenLayer(l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["kv_from"], l["rot_dims"], l["rot_base"],
                                  l["scale"], FF_KINDS[l["ff_kind"]], l["ff"], l["limit"], l["experts"], l["identity"], l["top"],
                                  l["groups"], l["keep"], l["shared_ff"])
        h = ctypes.c_void_p()
        _lib.check(self.lib.zl_dizizen_create(ctypes.byref(self.cfg), arr, ctypes.byref(h)))
        self.h = h

    @classmethod
    def from_config_dict(cls, d, **kw):
        return cls(DizizenConfig.from_dict(d), **kw)

    def close(self):
        if getattr(self, "h", None):
            self.lib.zl_dizizen_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_state_dict(self, state_dict):
        """name -> numpy array: bfloat16 bit patterns (safetensors_io.Bf16Array) or float32."""
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
            _lib.check(self.lib.zl_dizizen_load_tensor(self.h, name.encode(), a.ctypes.data_as(ctypes.c_void_p), rows, cols,
                                                       a.itemsize))
        _lib.check(self.lib.zl_dizizen_finalize(self.h))

    def init_synthetic(self, seed=0):
        _lib.check(self.lib.zl_dizizen_init_synthetic(self.h, seed))

    def step(self, tokens, slots, positions, want_rows=(), want_logits=True):
        """One step over T rows.  Returns (next tokens (n_want), logits (n_want, vocab) or None) for the wanted rows."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        s = np.ascontiguousarray(slots, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        w = np.ascontiguousarray(want_rows, dtype=np.int32)
        nxt = np.empty(w.size, dtype=np.int32)
        logits = np.empty((w.size, self.vocab_size), dtype=np.float32) if want_logits else None
        _lib.check(self.lib.zl_dizizen_step(
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
        _lib.check(self.lib.zl_dizizen_set_state(self.h, t.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
                                                 t.size))

    def step_device(self, b):
        _lib.check(self.lib.zl_dizizen_step_device(self.h, b))

    def sync(self):
        _lib.check(self.lib.zl_dizizen_sync(self.h))

    def stream(self):
        return self.lib.zl_dizizen_stream(self.h)

    def capture_layers(self, on=True):
        _lib.check(self.lib.zl_dizizen_capture_layers(self.h, int(on)))

    def read_layers(self, n_tokens):
        out = np.empty((len(self.config.layers), n_tokens, self.config.width), dtype=np.float32)
        _lib.check(self.lib.zl_dizizen_read_layers(self.h, out.ctypes.data_as(ctypes.c_void_p), n_tokens))
        return out

    def read_cache(self, layer, slot, n_rows):
        """(keys (n_rows, kv_heads, dim), values (n_rows, kv_heads, vdim)) of a layer that owns its caches, as float32."""
        l = self.config.layers[layer]
        k = np.empty((n_rows, l["kv_heads"], l["dim"]), dtype=np.float32)
        v = np.empty((n_rows, l["kv_heads"], l["vdim"]), dtype=np.float32)
        _lib.check(self.lib.zl_dizizen_read_cache(self.h, layer, slot, n_rows, k.ctypes.data_as(ctypes.c_void_p),
                                                  v.ctypes.data_as(ctypes.c_void_p)))
        return k, v

    def stats(self):
        wb, kn = ctypes.c_double(), ctypes.c_int()
        _lib.check(self.lib.zl_dizizen_stats(self.h, ctypes.byref(wb), ctypes.byref(kn)))
        return wb.value, kn.value
