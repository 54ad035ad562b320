"""Model registry: config.json -> decoder class, and loading a model folder (config.json + *.safetensors).

A builder takes the parsed config.json and the runtime sizes and returns a decoder that offers
`step(tokens, slots, positions, want_rows, want_logits)`, `load_state_dict`, `max_batch`, `max_seq`,
`max_step_tokens`, `vocab_size` and `supports_dtypes` -- the interface the engine schedules against.
"""
import glob
import json
import os
import re

import numpy as np

from . import safetensors_io

_BUILDERS = {}


def register(name, builder, dtypes=("bfloat16",)):
    """builder(config_dict, dtype, max_batch, max_seq, max_step_tokens, **kw) -> decoder; dtypes it can run in."""
    _BUILDERS[name] = (builder, tuple(dtypes))


def architecture_of(config):
    """The registry key a config.json selects: its "architecture", or the first of HF's "architectures"."""
    if "architecture" in config:
        return config["architecture"]
    archs = config.get("architectures") or []
    if archs:
        return archs[0]
    if "model_type" in config:
        return config["model_type"]
    raise ValueError("config.json names no architecture")


def registered():
    return sorted(_BUILDERS)


def build_model(config, dtype="bfloat16", max_batch=1, max_seq=512, max_step_tokens=512, **kw):
    arch = architecture_of(config)
    if arch not in _BUILDERS:
        raise ValueError("unknown architecture %r (registered: %s)" % (arch, ", ".join(registered())))
    return _BUILDERS[arch][0](config, dtype, max_batch, max_seq, max_step_tokens, **kw)


def supported_dtypes(config):
    arch = architecture_of(config)
    if arch not in _BUILDERS:
        raise ValueError("unknown architecture %r" % arch)
    return _BUILDERS[arch][1]


def load_model(model_dir, dtype="bfloat16", max_batch=1, max_seq=512, max_step_tokens=512, **kw):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    model = build_model(config, dtype, max_batch, max_seq, max_step_tokens, **kw)
    tensors = {}
    for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        tensors.update(safetensors_io.load_file(path))
    if not tensors:
        raise FileNotFoundError("no *.safetensors in %s" % model_dir)
    model.load_state_dict(tensors)
    return model


# ---- Dekipel ---------------------------------------------------------------------------------------------------------
def _build_dekipel(config, dtype, max_batch, max_seq, max_step_tokens, **kw):
    from .dekipel import DekipelDecoder
    return DekipelDecoder.from_config_dict(config, dtype=dtype, max_batch=max_batch, max_seq=max_seq,
                                           max_step_tokens=max_step_tokens, **kw)


register("Dekipel", _build_dekipel, ("bfloat16", "float32"))


# ---- Kodupel ---------------------------------------------------------------------------------------------------------
def _build_kodupel(config, dtype, max_batch, max_seq, max_step_tokens, **kw):
    from .kodupel import KodupelDecoder
    return KodupelDecoder.from_config_dict(config, dtype=dtype, max_batch=max_batch, max_seq=max_seq,
                                           max_step_tokens=max_step_tokens, **kw)


register("Kodupel", _build_kodupel, ("bfloat16", "float32"))


# ---- Lagelorn --------------------------------------------------------------------------------------------------------
def _build_lagelorn(config, dtype, max_batch, max_seq, max_step_tokens, **kw):
    from .lagelorn import LagelornDecoder
    return LagelornDecoder.from_config_dict(config, dtype=dtype, max_batch=max_batch, max_seq=max_seq,
                                            max_step_tokens=max_step_tokens, **kw)


register("Lagelorn", _build_lagelorn, ("bfloat16", "float32"))


# ---- Dizizen ---------------------------------------------------------------------------------------------------------
def _build_dizizen(config, dtype, max_batch, max_seq, max_step_tokens, **kw):
    from .dizizen import DizizenDecoder
    return DizizenDecoder.from_config_dict(config, dtype=dtype, max_batch=max_batch, max_seq=max_seq,
                                           max_step_tokens=max_step_tokens, **kw)


register("Dizizen", _build_dizizen, ("bfloat16", "float32"))


# ---- Llama (HF folder) -----------------------------------------------------------------------------------------------
_HF_LLAMA_NAMES = [
    (r"^model\.embed_tokens\.weight$", "token_embedding.weight"),
    (r"^model\.norm\.weight$", "output_layernorm.weight"),
    (r"^lm_head\.weight$", "lm_head.weight"),
    (r"^model\.layers\.(\d+)\.input_layernorm\.weight$", r"layers.\1.ln_attn.weight"),
    (r"^model\.layers\.(\d+)\.post_attention_layernorm\.weight$", r"layers.\1.ln_ff.weight"),
    (r"^model\.layers\.(\d+)\.self_attn\.q_proj\.(.+)$", r"layers.\1.attn.project_q.\2"),
    (r"^model\.layers\.(\d+)\.self_attn\.k_proj\.(.+)$", r"layers.\1.attn.project_k.\2"),
    (r"^model\.layers\.(\d+)\.self_attn\.v_proj\.(.+)$", r"layers.\1.attn.project_v.\2"),
    (r"^model\.layers\.(\d+)\.self_attn\.o_proj\.(.+)$", r"layers.\1.attn.attn_out.\2"),
    (r"^model\.layers\.(\d+)\.mlp\.gate_proj\.(.+)$", r"layers.\1.ff.w_in.\2"),
    (r"^model\.layers\.(\d+)\.mlp\.up_proj\.(.+)$", r"layers.\1.ff.w_gated.\2"),
    (r"^model\.layers\.(\d+)\.mlp\.down_proj\.(.+)$", r"layers.\1.ff.w_out.\2"),
]


def hf_llama_name(name):
    """HF Llama tensor name -> the driver's name (zhilight/loader.py:250-358 naming), or None."""
    for pat, rep in _HF_LLAMA_NAMES:
        if re.match(pat, name):
            return re.sub(pat, rep, name)
    return None


class _LlamaModel:
    """LlamaDecoder behind the engine's step interface.  Its decode call addresses slots 0..B-1 in order; any other
    set of rows goes through the chunked-prefill call slot by slot, and only a run's last row can be wanted."""

    architecture = "llama"
    supports_dtypes = ("bfloat16", "float16")
    supports_ragged_steps = False

    def __init__(self, config, dtype, max_batch, max_seq, max_step_tokens, **kw):
        from .llama import LlamaDecoder
        d = config
        nh = d["num_attention_heads"]
        rs = d.get("rope_scaling") or {}
        l3 = None
        if rs.get("rope_type", rs.get("type")) == "llama3":
            l3 = dict(factor=rs["factor"], low=rs["low_freq_factor"], high=rs["high_freq_factor"],
                      orig=rs["original_max_position_embeddings"])
        self.max_batch, self.max_seq = max_batch, max_seq
        self.max_step_tokens = min(max(max_step_tokens, 1), 2048)
        self.vocab_size = d["vocab_size"]
        self.dec = LlamaDecoder(d["num_hidden_layers"], d["hidden_size"], nh, d.get("num_key_value_heads", nh),
                                d.get("head_dim", d["hidden_size"] // nh), d["intermediate_size"], d["vocab_size"],
                                eps=d.get("rms_norm_eps", 1e-5), rope_theta=d.get("rope_theta", 10000.0), rope_llama3=l3,
                                dtype={"bfloat16": "bf16", "float16": "f16"}[dtype], max_batch=max_batch, max_seq=max_seq,
                                prefill_chunk=self.max_step_tokens, **kw)

    def load_state_dict(self, tensors):
        sd = {}
        for name, a in tensors.items():
            mapped = hf_llama_name(name) or name
            sd[mapped] = np.asarray(a).view(np.uint16) if safetensors_io.is_bf16(a) else a
        self.dec.load_state_dict(sd)

    def init_synthetic(self, seed=0):
        self.dec.init_synthetic(seed)

    def step(self, tokens, slots, positions, want_rows=(), want_logits=True):
        tokens, slots, positions, want = list(tokens), list(slots), list(positions), list(want_rows)
        n = len(tokens)
        if slots == list(range(n)) and want == list(range(n)):
            r = self.dec.decode(tokens, positions, want_logits=want_logits)
            return r if want_logits else (r, None)
        nxt, logits, i = {}, {}, 0
        while i < n:
            j = i
            while j + 1 < n and slots[j + 1] == slots[i]:
                j += 1
            r = self.dec.prefill(slots[i], tokens[i:j + 1], positions[i], want_logits=want_logits)
            nxt[j], logits[j] = (r[0], r[1][0]) if want_logits else (r, None)
            i = j + 1
        if any(w not in nxt for w in want):
            raise ValueError("this model returns logits for the last row of a slot's run only")
        return (np.array([nxt[w] for w in want], dtype=np.int32),
                np.stack([logits[w] for w in want]) if (want_logits and want) else None)

    def close(self):
        self.dec.close()


for _name in ("LlamaForCausalLM", "llama"):
    register(_name, _LlamaModel, ("bfloat16", "float16"))
