"""Typed configuration of the Lipadra decoder, read from config.json.

The design: the residual stream x is normed BEHIND every sum, ``x <- norm1(alpha x + mixer(x))`` and
``x <- norm2(alpha x + ff(x))`` with RMS norms of plain weight, and the sublayers read x itself.  A layer may run
with the tensors of another layer (``weights_of``) while keeping keys, values and states of its own.  A layer's
mixer is one of three:

``attention``   grouped-query attention with biases on q, k, v; every q and k head RMS-normed with a weight of one
                head's length (one for all query heads, one for all key heads) before the rotation; rotary positions
                over the first part of each head, dimension i paired with i + dims/2; a query sees the earlier keys
                of its own chunk of ``mask.size`` positions only, chunks counted from the start of the sequence; the
                softmax's denominator holds one more 1 (as if one more key of score zero that carries nothing were always seen).
``retention``   linear attention with a fixed decay per head: rotated q and k, k times dim^(-1/2) after the rotation,
                S <- a S + k v^T, o = S^T q, every head's o divided by its own root mean square (no weight), the
                heads times silu(W_g h).
``mamba1``      a selective scan behind a short causal convolution with silu, beside a silu gate.
The feed-forward is a mixture of experts: softmax scores over experts and identity experts together, a learned
offset that enters the choice only, a choice restricted to the best groups of neighbours (a group scored by its
largest choice score), weights = score times ``router.scale`` without renormalising, identity experts that return
their input, and a shared expert times sigmoid(w_sg . h).  The head is the embedding table behind a final norm.

config.json keys
----------------
architecture            "Lipadra"
vocab, width            sizes of the embedding table
norm.eps                epsilon of every norm
postln_alpha            alpha above
layers[i].type          "attention", "retention" or "mamba1"
layers[i].weights_of    absent, or the index of the layer whose tensors this layer runs with (its entry is then equal
                        to that layer's in every other key)
layers[i].mixer         attention: heads, kv_heads, dim, vdim, scale, rot.dims, rot.base, mask.size (mask absent or
                        null: causal)
                        retention: heads, dim, vdim, decay (a number per head), rot.dims, rot.base
                        mamba1: inner, state, conv, dt_rank
layers[i].mlp           null, or kind "moe" with expert.ff, router (experts, identity, top, scale, groups.count,
                        groups.keep; groups absent or null: one group) and shared (null, or ff)

Every size and constant is read from here; nothing is inferred from tensor shapes (the loader checks the shapes
against this configuration).  Tensor names: ``embed``, ``final.norm`` and, under ``l<i>.``, ``norm1``, ``norm2``,
``mix.*`` and ``mlp.*`` (``mlp.e<j>.gate|up|down``, ``mlp.router``, ``mlp.correction``, ``mlp.shared.gate|up|down|sg``).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Tuple

from .common import ConfigError, architecture_name
from .spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .tumatar import _int, _num, _obj

LAYER_TYPES = ("attention", "retention", "mamba1")


def _rot(m: Mapping[str, Any], where: str, dim: int) -> None:
    rot = _obj(m, "rot", where)
    R = _int(rot, "dims", where + "rot.")
    if R % 2 or R > dim:
        raise ConfigError(f"config.json: {where}rot.dims {R} must be even and at most the head's {dim}")
    if _num(rot, "base", where + "rot.") == 1.0:
        raise ConfigError(f"config.json: {where}rot.base must differ from 1")


def _check_mixer(kind: Any, m: Mapping[str, Any], mw: str) -> None:
    if kind == "attention":
        H, G = _int(m, "heads", mw), _int(m, "kv_heads", mw)
        if H % G:
            raise ConfigError(f"config.json: {mw}heads {H} is not a multiple of kv_heads {G}")
        D = _int(m, "dim", mw)
        _int(m, "vdim", mw)
        _num(m, "scale", mw)
        _rot(m, mw, D)
        mask = _obj(m, "mask", mw, optional=True)
        if mask is not None:
            _int(mask, "size", mw + "mask.")
    elif kind == "retention":
        H, D = _int(m, "heads", mw), _int(m, "dim", mw)
        _int(m, "vdim", mw)
        _rot(m, mw, D)
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != H:
            raise ConfigError(f"config.json: {mw}decay must hold one number for each of the {H} heads")
        for a in decay:
            if isinstance(a, bool) or not isinstance(a, (int, float)) or not 0.0 < float(a) <= 1.0:
                raise ConfigError(f"config.json: {mw}decay must hold numbers in (0, 1], found {a!r}")
    elif kind == "mamba1":
        for key in ("inner", "state", "dt_rank"):
            _int(m, key, mw)
        _int(m, "conv", mw)
    else:
        raise ConfigError(f"config.json: {mw[:-len('mixer.')]}type {kind!r} is not known ({', '.join(LAYER_TYPES)})")


def _check_mlp(mlp: Mapping[str, Any], fw: str) -> None:
    if mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {fw}kind {mlp.get('kind')!r} is not known (moe)")
    _int(_obj(mlp, "expert", fw), "ff", fw + "expert.")
    r = _obj(mlp, "router", fw)
    rw = fw + "router."
    E, top = _int(r, "experts", rw), _int(r, "top", rw)
    identity = 0 if r.get("identity") is None else _int(r, "identity", rw, minimum=0)
    _num(r, "scale", rw)
    groups = _obj(r, "groups", rw, optional=True)
    count, keep = (1, 1) if groups is None else (_int(groups, "count", rw + "groups."), _int(groups, "keep", rw + "groups."))
    routed = E + identity
    if routed % count or keep > count or top > keep * (routed // count):
        raise ConfigError(f"config.json: {rw}{routed} router outputs in {count} groups of which {keep} are kept "
                          f"cannot give {top} a token")
    shared = _obj(mlp, "shared", fw, optional=True)
    if shared is not None:
        _int(shared, "ff", fw + "shared.")


@dataclass(frozen=True)
class LipadraConfig:
    ARCHITECTURE = "Lipadra"

    raw: Mapping[str, Any]          # the checked dictionary, as it was read
    vocab: int
    width: int
    eps: float
    alpha: float
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
    def from_dict(cls, d: Mapping[str, Any]) -> "LipadraConfig":
        if architecture_name(d) != cls.ARCHITECTURE:
            raise ConfigError(f"config.json names the architecture {architecture_name(d)!r}, not {cls.ARCHITECTURE!r}")
        vocab = _int(d, "vocab", "")
        width = _int(d, "width", "")
        norm = _obj(d, "norm", "")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            _check_mixer(layer.get("type"), _obj(layer, "mixer", where), where + "mixer.")
            mlp = _obj(layer, "mlp", where, optional=True)
            if mlp is not None:
                _check_mlp(mlp, where + "mlp.")
            owner = layer.get("weights_of")
            if owner is not None:
                if isinstance(owner, bool) or not isinstance(owner, int) or not 0 <= owner < len(layers) or owner == i:
                    raise ConfigError(f"config.json: {where}weights_of must name another layer, found {owner!r}")
                other = layers[owner]
                if not isinstance(other, Mapping) or other.get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}weights_of names layer {owner}, which has no tensors of its own")
                if layer.get("type") != other.get("type") or (layer.get("mlp") is None) != (other.get("mlp") is None):
                    raise ConfigError(f"config.json: {where}weights_of: the layer is of another kind than layer {owner}, "
                                      f"whose tensors it runs with")
            checked.append(copy.deepcopy(dict(layer)))
        return cls(raw=copy.deepcopy(dict(d)), vocab=vocab, width=width, eps=_num(norm, "eps", "norm."),
                   alpha=_num(d, "postln_alpha", "", positive=False), layers=tuple(checked))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ layout
    def _mixer(self, kind: str, m: Mapping[str, Any], names: Dict[str, str]) -> MixerSpec:
        d, eps = self.width, self.eps
        if kind == "attention":
            for p in ("q", "k", "v"):
                names[f"mixer.{p}.weight"] = f"mix.{p}"
                names[f"mixer.{p}.bias"] = f"mix.{p}.b"
            names["mixer.o.weight"] = "mix.o"
            names["mixer.q_norm.weight"] = "mix.q.norm"
            names["mixer.k_norm.weight"] = "mix.k.norm"
            mask = m.get("mask") or {}
            return MixerSpec(kind="capped_attention", width=d, n_heads=m["heads"], n_kv_heads=m["kv_heads"],
                             head_dim=m["dim"], bias=True, scale=float(m["scale"]),
                             position=PositionSpec(kind="rope", rotary_dim=int(m["rot"]["dims"]), theta=float(m["rot"]["base"])),
                             options={"value_dim": m["vdim"], "qk_norm": "head_first", "qk_norm_eps": eps,
                                      "chunk": mask.get("size"), "sink": "zero"})
        if kind == "retention":
            for p in ("q", "k", "v", "g", "o"):
                names[f"mixer.{p}.weight"] = f"mix.{p}"
            return MixerSpec(kind="decayed_linear_attention", width=d, n_heads=m["heads"], head_dim=m["dim"],
                             position=PositionSpec(kind="rope", rotary_dim=int(m["rot"]["dims"]), theta=float(m["rot"]["base"])),
                             options={"value_dim": m["vdim"], "decay": tuple(float(a) for a in m["decay"]),
                                      "activation": None, "norm": "head", "norm_eps": eps, "gate": "silu",
                                      "key_scale": float(m["dim"]) ** -0.5})
        names.update({"mixer.in.weight": "mix.in", "mixer.conv.weight": "mix.conv", "mixer.conv.bias": "mix.conv.b",
                      "mixer.x.weight": "mix.x", "mixer.dt.weight": "mix.dt", "mixer.dt.bias": "mix.dt.b",
                      "mixer.A_log": "mix.A_log", "mixer.D": "mix.D", "mixer.o.weight": "mix.o"})
        return MixerSpec(kind="selective_scan", width=d,
                         options={"channels": m["inner"], "states": m["state"], "taps": m["conv"], "dt_rank": m["dt_rank"]})

    def _feed_forward(self, mlp: Mapping[str, Any], names: Dict[str, str]) -> FeedForwardSpec:
        d = self.width
        r, ex, sh = mlp["router"], mlp["expert"], mlp.get("shared")
        groups = r.get("groups") or {"count": 1, "keep": 1}
        E = r["experts"]
        opts: Dict[str, Any] = {"experts": E, "identity": int(r.get("identity") or 0), "top": r["top"], "score": "softmax",
                                "correction": True, "groups": groups["count"], "keep_groups": groups["keep"],
                                "group_best": 1, "renormalize": False, "weight_scale": float(r["scale"])}
        names["ffn.router.weight"] = "mlp.router"
        names["ffn.correction"] = "mlp.correction"
        for e in range(E):
            for part in ("gate", "up", "down"):
                names[f"ffn.e{e}.{part}.weight"] = f"mlp.e{e}.{part}"
        if sh is not None:
            opts["shared"] = FeedForwardSpec(kind="gated_mlp", width=d, intermediate=sh["ff"], activation="silu")
            opts["shared_gate"] = True
            for part in ("gate", "up", "down"):
                names[f"ffn.shared.{part}.weight"] = f"mlp.shared.{part}"
            names["ffn.shared_gate.weight"] = "mlp.shared.sg"
        return FeedForwardSpec(kind="moe", width=d, intermediate=ex["ff"], activation="silu", options=opts)

    def _layer(self, layer: Mapping[str, Any], prefix: str) -> LayerSpec:
        names: Dict[str, str] = {"mixer_post_norm.weight": "norm1"}
        norm = NormSpec("rmsnorm", self.width, self.eps)
        mixer = self._mixer(layer["type"], layer["mixer"], names)
        options: Dict[str, Any] = {"mixer_post_norm": norm, "residual_mult": self.alpha}
        ffn = None
        if layer.get("mlp") is not None:
            options["ffn_post_norm"] = norm
            names["ffn_post_norm.weight"] = "norm2"
            ffn = self._feed_forward(layer["mlp"], names)
        return LayerSpec(block="sum_norm", prefix=prefix, mixer_norm=None, mixer=mixer, ffn_norm=None, ffn=ffn,
                         names=names, options=options)

    def model_spec(self) -> ModelSpec:
        """A layer that runs with another layer's tensors is that layer's spec once more in the schedule (storage
        belongs to places of the schedule, so it keeps keys, values and states of its own).  Should its entry differ
        from the owner's in a constant, it becomes a spec of its own over the owner's tensor names."""
        d = self.width
        layers = []
        index_of: Dict[int, int] = {}           # layer of config.json with tensors of its own -> its LayerSpec
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is None:
                index_of[i] = len(layers)
                layers.append(self._layer(layer, f"l{i}."))
        schedule = []
        for i, layer in enumerate(self.layers):
            owner = layer.get("weights_of")
            if owner is None:
                schedule.append(index_of[i])
            elif {k: v for k, v in layer.items() if k != "weights_of"} == dict(self.layers[owner]):
                schedule.append(index_of[owner])
            else:
                schedule.append(len(layers))
                layers.append(self._layer(layer, f"l{owner}."))
        return ModelSpec(
            architecture=self.ARCHITECTURE, width=d, vocab_size=self.vocab, layers=tuple(layers),
            schedule=tuple(schedule), final_norm=NormSpec("rmsnorm", d, self.eps), embedding_name="embed",
            final_norm_name="final.norm", head_name=None, embedding_scale=1.0, max_positions=0)
