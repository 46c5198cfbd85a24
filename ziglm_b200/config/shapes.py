"""config.json dictionaries of a few members of the Llama family and of the other designs, for models with random weights.

The reference's ``synthetic`` stage writes one fixed 2-layer sample (src/synthetic.zig:9-18); these are the
shapes the measurements of this library name, so that the command line and ``bench.py`` agree on them.
No checkpoint is read: ``Engine.from_config`` fills the weights from a seed.
"""
from __future__ import annotations

import copy
import math
from typing import Any, Dict


def _llama3(factor: float) -> Dict[str, Any]:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 8192}


SHAPES: Dict[str, Dict[str, Any]] = {
    # the reference's sample model (src/synthetic.zig:9-18)
    "tiny": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 32,
        "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 128, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False, "attention_bias": False,
    },
    "llama-1b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
        "rope_theta": 500000.0, "rope_scaling": _llama3(32.0), "max_position_embeddings": 131072,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": False,
    },
    "llama-8b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
        "rope_theta": 500000.0, "rope_scaling": _llama3(8.0), "max_position_embeddings": 131072,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False,
    },
    "llama-13b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 5120, "intermediate_size": 13824, "num_hidden_layers": 40,
        "num_attention_heads": 40, "num_key_value_heads": 40, "head_dim": 128, "vocab_size": 32000,
        "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 4096,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False,
    },
}


def _tumatar(width: int, vocab: int, pairs: int, heads: int, ff: int, experts: int, expert_ff: int) -> Dict[str, Any]:
    """A Tumatar stack of ``pairs`` times (recurrence + dense feed-forward, latent attention + experts) at the
    width of a Llama shape: heads of 128 with a key/value latent of 128 (what the tensor-core attention takes),
    a query latent of three eighths of the width, a recurrence as wide as the model in blocks of 128 channels."""
    rec = {"type": "rglru", "mixer": {"width": width, "blocks": width // 128, "conv": 4},
           "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}}
    att = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": 128, "vdim": 128, "q_rank": 3 * width // 8, "kv_rank": 128, "scale": 128 ** -0.5},
           "mlp": {"kind": "moe", "expert": {"ff": expert_ff},
                   "router": {"experts": experts, "top": 2, "groups": {"count": 4, "keep": 2}}}}
    return {"architecture": "Tumatar", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "logit_scale": 1.0, "loop": None,
            "layers": [copy.deepcopy(x) for _ in range(pairs) for x in (rec, att)]}


# the new design at the widths of the 1B and 8B Llama shapes (as many layer runs, the same vocabulary)
SHAPES["tumatar-1b"] = _tumatar(2048, 128256, 8, 16, 8192, 16, 2048)
SHAPES["tumatar-8b"] = _tumatar(4096, 128256, 16, 32, 14336, 16, 3584)


def _tikalix(width: int, vocab: int, pairs: int, heads: int, kv_heads: int, dim: int, ff: int, experts: int,
             expert_ff: int) -> Dict[str, Any]:
    """A Tikalix stack of ``pairs`` times (attention + dense feed-forward, attention + experts with a shared one) with
    the heads of the Llama shape of that width: keys and values of one size, the whole head rotated and stretched
    fourfold, a soft cap of 50."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
             "rot": {"dims": dim, "base": 500000.0, "scaling": {"factor": 4.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    dense = {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}}
    moe = {"type": "attention", "mixer": mixer,
           "mlp": {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0}, "router": {"experts": experts, "top": 2},
                   "shared": {"ff": expert_ff, "limit": 7.0}}}
    return {"architecture": "Tikalix", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": [copy.deepcopy(x) for _ in range(pairs) for x in (dense, moe)]}


SHAPES["tikalix-1b"] = _tikalix(2048, 128256, 8, 32, 8, 64, 8192, 16, 2048)
SHAPES["tikalix-8b"] = _tikalix(4096, 128256, 16, 32, 8, 128, 14336, 16, 3584)


def _vilazen(width: int, vocab: int, groups: int, heads: int, kv_heads: int, dim: int, ff: int) -> Dict[str, Any]:
    """A Vilazen stack of ``groups`` times (side-by-side attention and decayed linear attention, windowed attention
    with mixed values, latent attention, windowed attention with mixed values) with the heads of the Llama shape of
    that width: keys and values of one size, half of every head rotated, windows of 1,024 positions that keep the
    first 64, a key/value latent of 96 beside 32 rotated dimensions (what the tensor-core attention takes), linear
    attention over heads of 128 with decays between exp(-1/4) and exp(-1/1024)."""
    rot = {"dims": dim // 2, "base": 500000.0}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": dict(rot),
           "mask": {"size": 1024, "keep_first": 64}, "v_mix": True}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": dict(rot)}
    lin_heads = width // 256
    right = {"heads": lin_heads, "dim": 128, "vdim": 128,
             "decay": [math.exp(-1.0 / 4.0 ** (1 + 4.0 * i / max(1, lin_heads - 1))) for i in range(lin_heads)]}
    lat = {"heads": width // 128, "dim": 96, "rot_dim": 32, "vdim": 128, "kv_rank": 96, "scale": 128 ** -0.5,
           "rot": {"dims": 32, "base": 500000.0}, "mask": {"size": 1024}}
    mlp = {"kind": "dense", "ff": ff}
    four = ({"type": "parallel", "mixer": {"left": left, "left_scale": 1.0, "right": right, "right_scale": 1.0}, "mlp": mlp},
            {"type": "attention", "mixer": att, "mlp": mlp},
            {"type": "latent_attention", "mixer": lat, "mlp": mlp},
            {"type": "attention", "mixer": att, "mlp": mlp})
    return {"architecture": "Vilazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "layers": [copy.deepcopy(x) for _ in range(groups) for x in four]}


SHAPES["vilazen-1b"] = _vilazen(2048, 128256, 4, 32, 8, 64, 8192)
SHAPES["vilazen-8b"] = _vilazen(4096, 128256, 8, 32, 8, 128, 14336)


def _lipadra(width: int, vocab: int, groups: int, heads: int, kv_heads: int, dim: int, experts: int, expert_ff: int) -> Dict[str, Any]:
    """A Lipadra stack of ``groups`` times (retention, selective scan, chunked attention, retention; the fourth layer
    runs with the first one's tensors) with the heads of the Llama shape of that width: keys and values of one size,
    half of every head rotated, chunks of 1,024 positions, retention over heads of 128 with decays between exp(-1/4)
    and exp(-1/1024), a scan twice as wide as the model with 16 states a channel, and in every layer sixteen experts
    and two identity experts in six groups of three, two a token, beside a shared expert."""
    ret_heads = width // 128
    ret = {"heads": ret_heads, "dim": 128, "vdim": 128, "rot": {"dims": 64, "base": 500000.0},
           "decay": [math.exp(-1.0 / 4.0 ** (1 + 4.0 * i / max(1, ret_heads - 1))) for i in range(ret_heads)]}
    scan = {"inner": 2 * width, "state": 16, "conv": 4, "dt_rank": width // 16}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
           "rot": {"dims": dim // 2, "base": 500000.0}, "mask": {"size": 1024}}
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": expert_ff},
           "router": {"experts": experts, "identity": 2, "top": 2, "scale": 2.0, "groups": {"count": 6, "keep": 3}}}
    layers = []
    for g in range(groups):
        first = len(layers)
        layers += [{"type": "retention", "mixer": copy.deepcopy(ret), "mlp": copy.deepcopy(mlp)},
                   {"type": "mamba1", "mixer": copy.deepcopy(scan), "mlp": copy.deepcopy(mlp)},
                   {"type": "attention", "mixer": copy.deepcopy(att), "mlp": copy.deepcopy(mlp)},
                   {"type": "retention", "mixer": copy.deepcopy(ret), "mlp": copy.deepcopy(mlp), "weights_of": first}]
    return {"architecture": "Lipadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "layers": layers}


SHAPES["lipadra-1b"] = _lipadra(2048, 128256, 4, 32, 8, 64, 16, 2048)
SHAPES["lipadra-8b"] = _lipadra(4096, 128256, 8, 32, 8, 128, 16, 3584)


def shape(name: str) -> Dict[str, Any]:
    """A copy of the named config.json dictionary."""
    try:
        return copy.deepcopy(SHAPES[name])
    except KeyError:
        raise KeyError(f"no shape named {name!r} (known: {', '.join(sorted(SHAPES))})") from None
