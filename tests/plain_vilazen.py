"""A plain, slow statement of the Vilazen decoder in PyTorch on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations and sharing no code with the library's product
path.  ``dtype`` float32 computes everything in float32 (float64 with ``wide=True``); bfloat16 rounds where the
library may: the operands and results of the projections and the activations next to them, while positions,
angles, scores, softmax, norms, the recurrent state and the residual stream stay float32.

Notation: d model width, H query heads, G key/value heads, D query/key size, V value size, R rotated dimensions,
T tokens of one sequence, W a window's size, F the number of first tokens a window keeps, C the size of a latent.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Mapping, Optional

import torch


class Plain:
    """How numbers are held: ``act`` is the type of projections' inputs and outputs, ``acc`` the type of
    everything the design computes in 32-bit (float64 stands in for it when a tighter oracle is wanted)."""

    def __init__(self, dtype: torch.dtype = torch.float32, wide: bool = False):
        self.act = dtype
        self.acc = torch.float64 if wide else torch.float32

    def round(self, x: torch.Tensor) -> torch.Tensor:
        return x.to(self.act).to(self.acc)

    def linear(self, x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y = W x (+ b): operands rounded to ``act``, summed in ``acc``, result rounded to ``act``."""
        y = self.round(x) @ self.round(w).t()
        if b is not None:
            y = y + self.round(b)
        return self.round(y)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the gain minus one."""
    return rms_unit(x, eps) * (1.0 + w.to(x.dtype))


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the gain."""
    return rms_unit(x, eps) * w.to(x.dtype)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Mapping[str, Any]) -> torch.Tensor:
    """x: [T, heads, D]; the first R dimensions of every head are turned, dimension 2i together with 2i + 1, by the
    angle position * base^(-2i/R)."""
    R, base = int(rot["dims"]), float(rot["base"])
    freq = torch.tensor([base ** (-2.0 * i / R) for i in range(R // 2)], dtype=torch.float64)
    # the angle is formed in 32-bit from a 32-bit frequency, as position * frequency
    ang = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(x.dtype)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:R:2], x[..., 1:R:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., R:]], dim=-1)


def visible(query_pos: torch.Tensor, key_pos: torch.Tensor, window: Optional[int], keep_first: int = 0) -> torch.Tensor:
    """[T, keys] true where a query may see a key: the key is not ahead of it and lies inside the window (the
    query's own position counts as the window's first) or among the first ``keep_first`` positions."""
    i, j = query_pos[:, None], key_pos[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_rows(s: torch.Tensor, seen: torch.Tensor, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax over the seen keys; with ``sink`` (one number) the denominator also holds exp(sink), which belongs
    to no key."""
    s = s.masked_fill(~seen, float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.reshape(1, 1).to(s.dtype))
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(s.dtype) - m)
    return e / den


def _keep(past: Optional[Dict[str, torch.Tensor]], name: str, new: torch.Tensor) -> torch.Tensor:
    """All rows of ``name`` so far: what ``past`` holds, then ``new`` (and ``past`` is brought up to date)."""
    if past is None:
        return new
    if name in past:
        new = torch.cat([past[name], new], dim=0)
    past[name] = new
    return new


def grouped_attention(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
                      past: Optional[Dict[str, torch.Tensor]], first_position: int, biases: bool, whole_norm: bool,
                      sink: bool, shared: Optional[Dict[str, Any]] = None) -> torch.Tensor:
    """Grouped-query attention with a per-head output gate.  ``whole_norm``: q and k, each as one long vector, are
    RMS-normed with a weight before the rotation.  ``sink``: the softmax's denominator holds exp(w['sink'][head]).
    ``shared``: what the layers of one pass hand on (the values of the first value-mixing layer)."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = p.linear(h, w["q"], w["q.b"] if biases else None)
    k = p.linear(h, w["k"], w["k.b"] if biases else None)
    v = p.linear(h, w["v"], w["v.b"] if biases else None)
    if whole_norm:
        q, k = norm_plain(q, w["q.norm"], eps), norm_plain(k, w["k.norm"], eps)
    pos = torch.arange(first_position, first_position + T)
    q = rotate_pairs(q.view(T, H, D), pos, m["rot"])
    k = rotate_pairs(k.view(T, G, D), pos, m["rot"])
    if m.get("v_mix") and shared is not None:
        if "v_first" in shared:
            lam = w["vmix"].to(p.acc)
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    v = v.view(T, G, V)
    if p.act != torch.float32:
        q, k, v = p.round(q), p.round(k), p.round(v)       # what the cache holds and the score product reads
    k, v = _keep(past, "k", k), _keep(past, "v", v)
    mask = m.get("mask") or {}
    seen = visible(pos, torch.arange(k.shape[0]), mask.get("size"), int(mask.get("keep_first", 0)))
    out = torch.zeros(T, H, V, dtype=p.acc)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].t()) * float(m["scale"])
        out[:, head, :] = softmax_rows(s, seen, w["sink"][head] if sink else None) @ v[:, g, :]
    gate = torch.sigmoid(p.linear(h, w["g"]))                # [T, H]: one number a head
    out = out * gate[:, :, None]
    return out.reshape(T, H * V)


def decayed_linear_attention(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
                             past: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
    """Per head S_t = a S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu of their projections; the heads
    together are RMS-normed with a weight and multiplied by sigmoid(W_g h)."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    silu = torch.nn.functional.silu
    q = p.round(silu(p.linear(h, w["q"]))).view(T, H, D)
    k = p.round(silu(p.linear(h, w["k"]))).view(T, H, D)
    v = p.round(silu(p.linear(h, w["v"]))).view(T, H, V)
    S = past["S"] if past is not None and "S" in past else torch.zeros(H, D, V, dtype=p.acc)
    decay = torch.tensor([float(a) for a in m["decay"]], dtype=p.acc)
    out = torch.zeros(T, H, V, dtype=p.acc)
    for t in range(T):
        S = decay[:, None, None] * S + k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    if past is not None:
        past["S"] = S
    out = norm_plain(out.reshape(T, H * V), w["norm"], eps)
    return out * torch.sigmoid(p.linear(h, w["g"]))


def latent_attention(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
                     past: Optional[Dict[str, torch.Tensor]], first_position: int) -> torch.Tensor:
    """Keys and values made from a normed latent c; one rotated key part shared by all heads; a sliding window."""
    T = h.shape[0]
    H, D, Rr, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(first_position, first_position + T)
    q = p.linear(h, w["q"]).view(T, H, D + Rr)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, {"dims": Rr, "base": m["rot"]["base"]})
    down = p.linear(h, w["dkv"])
    c = p.round(norm_plain(down[:, :C], w["dkv.norm"], eps))
    k_rot = p.round(rotate_pairs(down[:, None, C:], pos, {"dims": Rr, "base": m["rot"]["base"]})[:, 0, :])
    c, k_rot = _keep(past, "c", c), _keep(past, "k_rot", k_rot)
    n = c.shape[0]
    k_plain = p.linear(c, w["uk"]).view(n, H, D)
    v = p.linear(c, w["uv"]).view(n, H, V)
    seen = visible(pos, torch.arange(n), (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, V, dtype=p.acc)
    for head in range(H):
        s = (q_plain[:, head, :] @ k_plain[:, head, :].t() + p.round(q_rot[:, head, :]) @ k_rot.t()) * float(m["scale"])
        out[:, head, :] = softmax_rows(s, seen) @ v[:, head, :]
    return out.reshape(T, H * V)


def dense_ff(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    return p.linear(gelu_erf(p.linear(h, w["up"])), w["down"])


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PlainVilazen:
    """The whole model over one sequence at a time, with keys, values, latents and states kept between calls."""

    def __init__(self, config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor],
                 dtype: torch.dtype = torch.float32, wide: bool = False):
        self.c = config
        self.p = Plain(dtype, wide)
        self.w = {k: (v if v.dtype in (torch.int32, torch.int64) else v.to(self.p.acc)) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])

    def new_state(self) -> List[Dict[str, torch.Tensor]]:
        return [{"left": {}, "right": {}} for _ in self.c["layers"]]

    def mixer(self, kind: str, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any],
              past: Optional[Dict[str, Any]], first_position: int, shared: Dict[str, Any]) -> torch.Tensor:
        p, eps = self.p, self.eps
        if kind == "attention":
            heads = grouped_attention(p, h, w, m, eps, None if past is None else past["left"], first_position,
                                      biases=False, whole_norm=True, sink=False, shared=shared)
            return p.linear(heads, w["o"])
        if kind == "latent_attention":
            heads = latent_attention(p, h, w, m, eps, None if past is None else past["left"], first_position)
            return p.linear(heads, w["o"])
        if kind == "parallel":
            lw, rw = _sub(w, "left."), _sub(w, "right.")
            left = grouped_attention(p, h, lw, m["left"], eps, None if past is None else past["left"], first_position,
                                     biases=True, whole_norm=False, sink=True)
            right = decayed_linear_attention(p, h, rw, m["right"], eps, None if past is None else past["right"])
            return float(m["left_scale"]) * p.linear(left, lw["o"]) + float(m["right_scale"]) * p.linear(right, rw["o"])
        raise ValueError(f"layer type {kind!r} is not part of the design")

    def forward(self, tokens: List[int], state: Optional[List[Dict[str, Any]]] = None,
                first_position: int = 0, layers_out: Optional[list] = None) -> torch.Tensor:
        """Logits [T, vocab] of the given tokens, which follow ``first_position`` tokens held in ``state``."""
        c, p, w = self.c, self.p, self.w
        x = norm_around_zero(w["embed"][torch.tensor(tokens, dtype=torch.long)], w["embed.norm"], self.eps)
        shared: Dict[str, Any] = {}
        for i, layer in enumerate(c["layers"]):
            lw = _sub(w, f"l{i}.")
            h = norm_around_zero(x, lw["norm1"], self.eps)
            y = self.mixer(layer["type"], h, _sub(lw, "mix."), layer["mixer"], None if state is None else state[i],
                           first_position, shared)
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp["kind"] != "dense":
                    raise ValueError(f"feed-forward kind {mlp['kind']!r} is not part of the design")
                y = y + dense_ff(p, h, _sub(lw, "mlp."))
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        h = norm_around_zero(x, w["final.norm"], self.eps)
        return (p.round(h) @ p.round(w["head"]).t()).to(torch.float32)
