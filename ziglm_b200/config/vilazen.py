"""Typed configuration of the Vilazen decoder, read from config.json.

The design: the embedded tokens are normed; every layer has ONE norm h = norm(x) that its mixer and its
feed-forward both read, ``x += mixer(h) + ff(h)``; every norm over the model width is an RMS norm whose stored
weight is its gain minus one.  A layer's mixer is one of three:

``attention``         grouped-query attention: q and k, each as one long vector, are RMS-normed with a weight before
                      the rotation; rotary positions over the first part of each head, dimension 2i paired with
                      2i + 1; a sliding window that also keeps the first tokens of the sequence; optionally the
                      values are mixed with those of the first such layer, (1 - l) v + l v_first with a learned l;
                      one sigmoid gate a head on the heads' outputs.
``latent_attention``  keys and values are made per head from a normed low-rank latent, beside one rotated key part
                      that all heads share; queries have an unrotated and a rotated part; a sliding window.
``parallel``          two mixers side by side on the same input, summed with a factor each: ``left`` is causal
                      grouped-query attention with biases, rotary positions, a learned number per head in the
                      softmax's denominator and a gate per head; ``right`` is linear attention with a fixed decay per
                      head (S <- a S + k v^T, o = S^T q over silu'd q, k, v), its heads RMS-normed together and gated
                      element by element.
The feed-forward is dense with the exact gelu.  The head is a matrix of its own behind a final norm.

config.json keys
----------------
architecture            "Vilazen"
vocab, width            sizes of the embedding table
norm.eps                epsilon of every norm
layers[i].type          "attention", "latent_attention" or "parallel"
layers[i].mixer         attention: heads, kv_heads, dim, vdim, scale, rot.dims, rot.base, mask.size, mask.keep_first
                        (absent: 0; mask absent or null: causal), v_mix (absent: false)
                        latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot.base, mask.size
                        parallel: left (heads, kv_heads, dim, vdim, scale, rot), left_scale, right (heads, dim, vdim,
                        decay: a number per head), right_scale
layers[i].mlp           null, or kind "dense" with ff

Every size and constant is read from here; nothing is inferred from tensor shapes (the loader checks the shapes
against this configuration).  Tensor names: ``embed``, ``embed.norm``, ``head``, ``final.norm`` and, under
``l<i>.``, ``norm1``, ``mlp.up``/``mlp.down`` and the mixer's tensors ``mix.*`` (``mix.left.*``, ``mix.right.*``).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .common import ConfigError, architecture_name
from .spec import FeedForwardSpec, HookSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .tumatar import _int, _num, _obj

LAYER_TYPES = ("attention", "latent_attention", "parallel")
VALUE_MIX_BUFFER = "value_mix_first"      # the step's scratch in which the first value-mixing layer leaves its values


def _rot(m: Mapping[str, Any], where: str, dim: int) -> None:
    rot = _obj(m, "rot", where)
    R = _int(rot, "dims", where + "rot.")
    if R % 2 or R > dim:
        raise ConfigError(f"config.json: {where}rot.dims {R} must be even and at most the head's {dim}")
    if _num(rot, "base", where + "rot.") == 1.0:
        raise ConfigError(f"config.json: {where}rot.base must differ from 1")


def _mask(m: Mapping[str, Any], where: str, keep: bool) -> None:
    mask = _obj(m, "mask", where, optional=True)
    if mask is not None:
        _int(mask, "size", where + "mask.")
        if keep and mask.get("keep_first") is not None:
            _int(mask, "keep_first", where + "mask.", minimum=0)


def _grouped(m: Mapping[str, Any], where: str) -> None:
    H, G = _int(m, "heads", where), _int(m, "kv_heads", where)
    if H % G:
        raise ConfigError(f"config.json: {where}heads {H} is not a multiple of kv_heads {G}")
    D = _int(m, "dim", where)
    _int(m, "vdim", where)
    _num(m, "scale", where)
    _rot(m, where, D)


@dataclass(frozen=True)
class VilazenConfig:
    ARCHITECTURE = "Vilazen"

    raw: Mapping[str, Any]          # the checked dictionary, as it was read
    vocab: int
    width: int
    eps: float
    layers: Tuple[Mapping[str, Any], ...]

    @property
    def architecture(self) -> str:
        return self.ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return ()

    # -------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VilazenConfig":
        if architecture_name(d) != cls.ARCHITECTURE:
            raise ConfigError(f"config.json names the architecture {architecture_name(d)!r}, not {cls.ARCHITECTURE!r}")
        vocab = _int(d, "vocab", "")
        width = _int(d, "width", "")
        norm = _obj(d, "norm", "")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        mixed_values = None
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            m = _obj(layer, "mixer", where)
            mw = where + "mixer."
            if kind == "attention":
                _grouped(m, mw)
                _mask(m, mw, keep=True)
                mix = m.get("v_mix")
                if mix is not None and not isinstance(mix, bool):
                    raise ConfigError(f"config.json: {mw}'v_mix' must be true or false, found {mix!r}")
                if mix:
                    size = m["kv_heads"] * m["vdim"]
                    if mixed_values is not None and mixed_values != size:
                        raise ConfigError(f"config.json: {mw}v_mix: this layer has {size} values a token, the first "
                                          f"value-mixing layer {mixed_values}")
                    mixed_values = size
            elif kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    _int(m, key, mw)
                if _int(m, "rot_dim", mw) % 2:
                    raise ConfigError(f"config.json: {mw}rot_dim must be even")
                _num(m, "scale", mw)
                if _num(_obj(m, "rot", mw), "base", mw + "rot.") == 1.0:
                    raise ConfigError(f"config.json: {mw}rot.base must differ from 1")
                _mask(m, mw, keep=False)
            elif kind == "parallel":
                _grouped(_obj(m, "left", mw), mw + "left.")
                r = _obj(m, "right", mw)
                H = _int(r, "heads", mw + "right.")
                _int(r, "dim", mw + "right.")
                _int(r, "vdim", mw + "right.")
                decay = r.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != H:
                    raise ConfigError(f"config.json: {mw}right.decay must hold one number for each of the {H} heads")
                for a in decay:
                    if isinstance(a, bool) or not isinstance(a, (int, float)) or not 0.0 < float(a) <= 1.0:
                        raise ConfigError(f"config.json: {mw}right.decay must hold numbers in (0, 1], found {a!r}")
                _num(m, "left_scale", mw, positive=False)
                _num(m, "right_scale", mw, positive=False)
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known ({', '.join(LAYER_TYPES)})")
            mlp = _obj(layer, "mlp", where, optional=True)
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind')!r} is not known (dense)")
                _int(mlp, "ff", where + "mlp.")
            checked.append(copy.deepcopy(dict(layer)))
        return cls(raw=copy.deepcopy(dict(d)), vocab=vocab, width=width, eps=_num(norm, "eps", "norm."),
                   layers=tuple(checked))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ layout
    @staticmethod
    def _position(dims: int, base: float) -> PositionSpec:
        return PositionSpec(kind="rope", rotary_dim=int(dims), theta=float(base), options={"pairs": "adjacent"})

    def _grouped_spec(self, m: Mapping[str, Any], names: Dict[str, str], at: str, under: str, *, bias: bool,
                      whole_norm: bool, sink: bool, value_mix: Optional[str], out_scale: float) -> MixerSpec:
        """The grouped-query attention of a layer: ``at`` is the prefix of the part's local names, ``under`` that of
        the tensors' names in the files."""
        mask = m.get("mask") or {}
        opts: Dict[str, Any] = {"value_dim": m["vdim"], "gate": "sigmoid_head", "out_scale": float(out_scale)}
        for p in ("q", "k", "v", "g", "o"):
            names[f"{at}{p}.weight"] = f"{under}{p}"
        if bias:
            for p in ("q", "k", "v"):
                names[f"{at}{p}.bias"] = f"{under}{p}.b"
        if whole_norm:
            opts["qk_norm"] = "whole"
            opts["qk_norm_eps"] = self.eps
            names[f"{at}q_norm.weight"] = f"{under}q.norm"
            names[f"{at}k_norm.weight"] = f"{under}k.norm"
        if sink:
            opts["sink"] = True
            names[f"{at}sink"] = f"{under}sink"
        if mask.get("size") is not None:
            opts["keep_first"] = int(mask.get("keep_first") or 0)
        if value_mix is not None:
            opts["value_mix"] = value_mix
            opts["value_mix_buffer"] = VALUE_MIX_BUFFER
            names[f"{at}vmix"] = f"{under}vmix"
        return MixerSpec(kind="capped_attention", width=self.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"],
                         head_dim=m["dim"], bias=bias, scale=float(m["scale"]), window=mask.get("size"),
                         position=self._position(m["rot"]["dims"], m["rot"]["base"]), options=opts)

    def model_spec(self) -> ModelSpec:
        d, eps = self.width, self.eps
        norm = NormSpec("rmsnorm", d, eps, options={"unit_offset": True})
        layers = []
        seen_value_mix = False
        for i, layer in enumerate(self.layers):
            m, kind = layer["mixer"], layer["type"]
            names: Dict[str, str] = {"mixer_norm.weight": "norm1"}
            if kind == "attention":
                role = None
                if m.get("v_mix"):
                    role = "mix" if seen_value_mix else "first"
                    seen_value_mix = True
                mixer = self._grouped_spec(m, names, "mixer.", "mix.", bias=False, whole_norm=True, sink=False,
                                           value_mix=role, out_scale=1.0)
            elif kind == "latent_attention":
                mask = m.get("mask") or {}
                for p in ("q", "dkv", "uk", "uv", "o"):
                    names[f"mixer.{p}.weight"] = f"mix.{p}"
                names["mixer.dkv_norm.weight"] = "mix.dkv.norm"
                mixer = MixerSpec(kind="latent_attention", width=d, n_heads=m["heads"], head_dim=m["dim"],
                                  scale=float(m["scale"]), window=mask.get("size"),
                                  position=self._position(m["rot_dim"], m["rot"]["base"]),
                                  options={"value_dim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": None,
                                           "rot_dim": m["rot_dim"], "gate": None, "norm_eps": eps})
            else:
                left = self._grouped_spec(m["left"], names, "mixer.left.", "mix.left.", bias=True, whole_norm=False,
                                          sink=True, value_mix=None, out_scale=float(m["left_scale"]))
                r = m["right"]
                for p in ("q", "k", "v", "g", "o"):
                    names[f"mixer.right.{p}.weight"] = f"mix.right.{p}"
                names["mixer.right.norm.weight"] = "mix.right.norm"
                right = MixerSpec(kind="decayed_linear_attention", width=d, n_heads=r["heads"], head_dim=r["dim"],
                                  options={"value_dim": r["vdim"], "decay": tuple(float(a) for a in r["decay"]),
                                           "activation": "silu", "norm_eps": eps, "gate": "sigmoid",
                                           "out_scale": float(m["right_scale"])})
                mixer = MixerSpec(kind="side_by_side", width=d, options={"parts": (("left.", left), ("right.", right))})
            mlp = layer.get("mlp")
            ffn = None
            if mlp is not None:
                ffn = FeedForwardSpec(kind="mlp", width=d, intermediate=mlp["ff"], activation="gelu")
                names["ffn.up.weight"] = "mlp.up"
                names["ffn.down.weight"] = "mlp.down"
            layers.append(LayerSpec(block="shared_norm", prefix=f"l{i}.", mixer_norm=norm, mixer=mixer, ffn_norm=None,
                                    ffn=ffn, names=names))
        embed_norm = HookSpec("rmsnorm", options={"width": d, "eps": eps, "unit_offset": True},
                              names={"weight": "embed.norm"})
        return ModelSpec(
            architecture=self.ARCHITECTURE, width=d, vocab_size=self.vocab, layers=tuple(layers),
            schedule=tuple(range(len(layers))), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", head_name="head", embedding_scale=1.0, max_positions=0, embed_hook=embed_norm,
            # a file may hold the mixing weight of an attention layer that mixes no values
            options={"ignored_tensors": ("l*.mix.vmix",)})
