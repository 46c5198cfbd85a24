"""A plain, slow statement of the Lipadra decoder in PyTorch on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations and sharing no code with the library's product
path.  ``dtype`` float32 computes everything in float32 (float64 with ``wide=True``); bfloat16 rounds where the
library may: the operands and results of the projections, the short convolution and the activations next to them,
while positions, angles, scores, softmax, norms, routers, decays, step sizes, recurrent states and the residual
stream stay float32.

The design.  x is the residual stream, one row a token.  Every layer is
    x <- norm1(alpha x + mixer(x)),   x <- norm2(alpha x + ff(x))
with RMS norms (plain weight) BEHIND the sums, so the stream is normed after every sublayer and the sublayers read
x itself.  A layer may name another layer whose tensors it runs with (``weights_of``), with keys, values and states
of its own.  Mixers: ``attention`` (grouped queries, biases, a weighted RMS norm of every q and k head before the
rotation, rotation of the first part of a head in halves, keys visible only inside the query's chunk of
``mask.size`` positions, a softmax whose denominator holds one more 1), ``retention`` (linear attention with a fixed
decay a head, rotated q and k, k scaled, every head's output divided by its root mean square, a silu gate) and
``mamba1`` (a selective scan behind a short causal convolution).  The feed-forward is a mixture of experts with a
softmax router over real and identity experts, a learned offset in the choice, groups of experts, an unrenormed
weight times a factor, and a shared expert behind a sigmoid gate of one number a token.  The head is the embedding.

Notation: d model width, H query heads, G key/value heads, D query/key size, V value size, R rotated dimensions,
T tokens of one sequence, C channels, N states a channel, K taps, E real experts, I identity experts.
"""
from __future__ import annotations

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

    def linear_wide(self, x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The same product with the sums left in ``acc`` (router logits, step sizes)."""
        y = self.round(x) @ self.round(w).t()
        return y if b is None else y + b.to(self.acc)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w.to(x.dtype)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rot: Mapping[str, Any]) -> torch.Tensor:
    """x: [T, heads, D]; of every head's first R dimensions, dimension i turns together with i + R/2 by the angle
    position * base^(-2i/R); the dimensions from R on are left alone."""
    R, base = int(rot["dims"]), float(rot["base"])
    half = R // 2
    f = torch.tensor([base ** (-2.0 * i / R) for i in range(half)], dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                      # [T, R/2]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:R]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., R:]], dim=-1)


def same_chunk(query_pos: torch.Tensor, key_pos: torch.Tensor, size: Optional[int]) -> torch.Tensor:
    """[Tq, Tk] booleans: key j is seen by query i when j <= i and, with chunks, both lie in the same chunk of
    ``size`` positions counted from the start of the sequence."""
    i, j = query_pos[:, None], key_pos[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return seen


def softmax_one_more(s: torch.Tensor, seen: torch.Tensor) -> torch.Tensor:
    """p_j = exp(s_j) / (1 + sum over the seen j of exp(s_j)): the denominator counts one more key, of score zero, that
    carries nothing."""
    s = s.masked_fill(~seen, float("-inf"))
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))


def _keep(past: Optional[Dict[str, torch.Tensor]], name: str, new: torch.Tensor) -> torch.Tensor:
    """Append ``new`` (rows of tokens) to what ``past`` holds under ``name`` and return all rows."""
    if past is None:
        return new
    rows = new if name not in past else torch.cat([past[name], new], dim=0)
    past[name] = rows
    return rows


def chunked_attention(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
                      past: Optional[Dict[str, torch.Tensor]], first_position: int) -> torch.Tensor:
    """The concatenated heads [T, H V] before W_o."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(first_position, first_position + T)
    q = p.linear(h, w["q"], w["q.b"]).reshape(T, H, D)
    k = p.linear(h, w["k"], w["k.b"]).reshape(T, G, D)
    v = p.linear(h, w["v"], w["v.b"]).reshape(T, G, V)
    q = rms_unit(q, eps) * w["q.norm"].to(q.dtype)
    k = rms_unit(k, eps) * w["k.norm"].to(k.dtype)
    q = rotate_halves(q, pos, m["rot"])
    k = p.round(rotate_halves(k, pos, m["rot"]))          # keys and values are kept in the storage type
    q = p.round(q)
    k_all = _keep(past, "k", k)
    v_all = _keep(past, "v", v)
    key_pos = torch.arange(k_all.shape[0])
    mask = m.get("mask") or {}
    seen = same_chunk(pos, key_pos, mask.get("size"))
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k_all[:, g].t()) * float(m["scale"])
        out[:, head] = softmax_one_more(s, seen) @ v_all[:, g]
    return p.round(out.reshape(T, H * V))


def retention(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
              past: Optional[Dict[str, torch.Tensor]], first_position: int) -> torch.Tensor:
    """The gated heads [T, H V] before W_o: S_t = a S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(first_position, first_position + T)
    q = rotate_halves(p.linear(h, w["q"]).reshape(T, H, D), pos, m["rot"])
    k = rotate_halves(p.linear(h, w["k"]).reshape(T, H, D), pos, m["rot"]) * (D ** -0.5)
    v = p.linear(h, w["v"]).reshape(T, H, V)
    a = torch.tensor([float(x) for x in m["decay"]], dtype=q.dtype)
    S = torch.zeros(H, D, V, dtype=q.dtype) if past is None or "S" not in past else past["S"]
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for t in range(T):
        S = a[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    if past is not None:
        past["S"] = S
    out = rms_unit(out, eps).reshape(T, H * V)
    return p.round(out * silu(p.linear(h, w["g"])))


def causal_conv(p: Plain, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor,
                past: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
    """Per channel: y_t = b + sum_j w[:, j] x_(t - (K-1) + j), zeros before the start of the sequence; the last
    column of w meets the current token."""
    T, C = x.shape
    K = w.shape[1]
    before = torch.zeros(K - 1, C, dtype=x.dtype) if past is None or "conv" not in past else past["conv"]
    rows = torch.cat([before, x], dim=0)
    if past is not None:
        past["conv"] = rows[rows.shape[0] - (K - 1):].clone()
    y = torch.zeros(T, C, dtype=x.dtype) + p.round(b)[None, :]
    wr = p.round(w)
    for j in range(K):
        y = y + rows[j:j + T] * wr[:, j][None, :]
    return y


def selective_scan(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any],
                   past: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
    """The gated channels [T, C] before W_o."""
    T = h.shape[0]
    C, N, rank = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = p.linear(h, w["in"])
    x, z = xz[:, :C], xz[:, C:]
    x = p.round(silu(p.round(causal_conv(p, x, w["conv"], w["conv.b"], past))))
    dbc = p.linear(x, w["x"])
    dt = softplus(p.linear_wide(dbc[:, :rank], w["dt"], w["dt.b"]))            # [T, C]
    B, Cm = dbc[:, rank:rank + N], dbc[:, rank + N:rank + 2 * N]
    A = -torch.exp(w["A_log"].to(x.dtype))                                      # [C, N]
    S = torch.zeros(C, N, dtype=x.dtype) if past is None or "S" not in past else past["S"]
    y = torch.zeros(T, C, dtype=x.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + w["D"].to(x.dtype) * x[t]
    if past is not None:
        past["S"] = S
    return p.round(y * silu(z))


def expert(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    return p.linear(p.round(silu(p.linear(h, w["gate"])) * p.linear(h, w["up"])), w["down"])


def route(z: torch.Tensor, correction: torch.Tensor, r: Mapping[str, Any]) -> Dict[str, torch.Tensor]:
    """z: router logits [T, E + I].  ids [T, top] of the chosen outputs and their weights."""
    n, top = z.shape[1], int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    s = torch.softmax(z, dim=-1)
    choice = s + correction.to(s.dtype)[None, :]
    best = choice.reshape(-1, count, n // count).max(dim=-1).values                 # [T, count]
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    choice = choice.masked_fill(~kept.repeat_interleave(n // count, dim=1), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    return {"ids": ids, "weights": s.gather(1, ids) * float(r["scale"])}


def mixture(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], mlp: Mapping[str, Any]) -> torch.Tensor:
    r = mlp["router"]
    E, I = int(r["experts"]), int(r.get("identity") or 0)
    z = p.linear_wide(h, w["router"])
    chosen = route(z, w["correction"], r)
    hr = p.round(h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen["ids"][t].tolist(), chosen["weights"][t]):
            y = hr[t] if e >= E else expert(p, h[t:t + 1], _sub(w, f"e{e}."))[0]
            out[t] = out[t] + g * y
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(p.linear_wide(h, w["shared.sg"]))                       # [T, 1]
        out = out + gate * expert(p, h, _sub(w, "shared."))
    return out


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PlainLipadra:
    """The whole model over one sequence at a time, with keys, values and states kept between calls."""

    def __init__(self, config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor],
                 dtype: torch.dtype = torch.float32, wide: bool = False):
        self.c = config
        self.p = Plain(dtype, wide)
        self.w = {k: (v if v.dtype in (torch.int32, torch.int64) else v.to(self.p.acc)) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.alpha = float(config["postln_alpha"])

    def new_state(self) -> List[Dict[str, torch.Tensor]]:
        return [{} for _ in self.c["layers"]]

    def mixer(self, kind: str, x: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any],
              past: Optional[Dict[str, Any]], first_position: int) -> torch.Tensor:
        p = self.p
        if kind == "attention":
            return p.linear(chunked_attention(p, x, w, m, self.eps, past, first_position), w["o"])
        if kind == "retention":
            return p.linear(retention(p, x, w, m, self.eps, past, first_position), w["o"])
        if kind == "mamba1":
            return p.linear(selective_scan(p, x, w, m, past), w["o"])
        raise ValueError(f"layer type {kind!r} is not part of the design")

    def forward(self, tokens: List[int], state: Optional[List[Dict[str, Any]]] = None,
                first_position: int = 0, layers_out: Optional[list] = None) -> torch.Tensor:
        """Logits [T, vocab] of the given tokens, which follow ``first_position`` tokens held in ``state``."""
        c, w = self.c, self.w
        x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
        for i, layer in enumerate(c["layers"]):
            owner = layer.get("weights_of")
            lw = _sub(w, f"l{i if owner is None else owner}.")
            y = self.mixer(layer["type"], x, _sub(lw, "mix."), layer["mixer"], None if state is None else state[i],
                           first_position)
            x = norm_plain(self.alpha * x + y, lw["norm1"], self.eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp["kind"] != "moe":
                    raise ValueError(f"feed-forward kind {mlp['kind']!r} is not part of the design")
                x = norm_plain(self.alpha * x + mixture(self.p, x, _sub(lw, "mlp."), mlp), lw["norm2"], self.eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        h = norm_plain(x, w["final.norm"], self.eps)
        return (self.p.round(h) @ self.p.round(w["embed"]).t()).to(torch.float32)
