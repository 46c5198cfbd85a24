"""Grouped-query attention with the options of newer decoders, each of which may be left out.

For the rows h the mixer reads, H query heads, G key/value heads, query/key size D and value size V:
    q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v
    q, k <- q / rms(q) * w_q, k / rms(k) * w_k  q (all heads as one vector) and k likewise  (``qk_norm`` "whole")
    q, k <- rotate(q, k; position)              the first ``rotary_dim`` dimensions of a head, in the pairs of the
                                                position encoding; cosines and sines times its amplitude
    q, k <- q / rms(q), k / rms(k)              per head over D, no weight        (``qk_norm`` "head": the default
                                                when ``qk_norm_eps`` is given; None: left out)
                                                (``qk_norm`` "head_first": per head over D BEFORE the rotation, times a
                                                weight of D numbers that all query heads share, and one for the keys)
    v <- (1 - l) v + l v_first                  v_first: the values of the same tokens in the first layer that takes
                                                part (``value_mix`` "mix"; that layer itself says "first"); l learned
    s_ij = (q_i . k_j) * scale;  s <- c tanh(s / c)                               (``softcap`` c; None: left out)
    j visible to i:  j <= i and (i - j < window or j < keep_first)                (``MixerSpec.window``, ``keep_first``)
                     or j <= i and floor(i / c) = floor(j / c)                    (``chunk`` c instead of a window)
    p = softmax over the visible j, with exp(sink_h) also in the denominator       (``sink``: a learned number a head;
                                                                                  "zero": the fixed number 0, so that
                                                                                  the denominator holds one more 1)
    o_i = sum_j p_ij v_j
    out = W_o (concat(o) * sigmoid(W_g h))      one gate an element (``gate`` "sigmoid") or one a head
                                                (``gate`` "sigmoid_head", times ``out_scale``); None: left out
``value_dim`` V may differ from ``head_dim`` D.  The projections of h are one matrix product over the concatenated
weight [q; k; v; g].

Keys and values share the cache's head size: both are kept with max(D, V) elements a head (rounded up to a
multiple of 8), the shorter of the two with zeros behind it, which add nothing to a score and whose part of the
result is zero.  The padding is built into the weights when they are bound (zero rows of W_k or W_v, zero columns
of W_o), so every kernel sees one head size; the norms divide by the true element counts.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, position_class, register_mixer
from .linear import Linear


def _pad_heads(w: torch.Tensor, heads: int, size: int, padded: int) -> torch.Tensor:
    """[heads * size, ...] -> [heads * padded, ...] with zero rows behind every head."""
    if size == padded:
        return w
    rest = tuple(w.shape[1:])
    out = w.new_zeros((heads, padded) + rest)
    out[:, :size] = w.reshape((heads, size) + rest)
    return out.reshape((heads * padded,) + rest)


def _order_heads(w: torch.Tensor, heads: int, size: int, order) -> torch.Tensor:
    """[heads * size, ...] with the rows of every head taken in ``order`` (None: as they are)."""
    if order is None:
        return w
    rest = tuple(w.shape[1:])
    idx = torch.tensor(order, dtype=torch.long, device=w.device)
    return w.reshape((heads, size) + rest).index_select(1, idx).reshape((heads * size,) + rest)


class CappedAttention(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} heads cannot share {spec.n_kv_heads} key/value heads")
        if spec.scale is None:
            raise ValueError("capped_attention: the spec must give the factor on the scores")
        if spec.cache_from is not None:
            raise ValueError("capped_attention: shared caches are not part of this mixer")
        self.n_heads, self.n_kv, self.dim = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.value_dim = int(o.get("value_dim", spec.head_dim))
        self.scale = float(spec.scale)
        self.softcap = float(o["softcap"]) if o.get("softcap") else 0.0
        self.norm_eps = None if o.get("qk_norm_eps") is None else float(o["qk_norm_eps"])
        self.norm_kind = None if self.norm_eps is None else o.get("qk_norm", "head")
        if self.norm_kind not in (None, "head", "whole", "head_first"):
            raise ValueError(f"capped_attention: norm of q and k {self.norm_kind!r} is not known (head, whole, head_first)")
        self.gate = o.get("gate")
        if self.gate not in (None, "sigmoid", "sigmoid_head"):
            raise ValueError(f"capped_attention: output gate {self.gate!r} is not known (sigmoid, sigmoid_head)")
        self.gated = self.gate is not None
        self.out_scale = float(o.get("out_scale", 1.0))
        if self.out_scale != 1.0 and self.gate != "sigmoid_head":
            raise ValueError("capped_attention: a factor on the output rides on the gate of a head (sigmoid_head)")
        self.window = None if spec.window is None else int(spec.window)
        self.keep_first = int(o.get("keep_first") or 0) if self.window is not None else 0
        self.chunk = None if o.get("chunk") is None else int(o["chunk"])
        if self.chunk is not None and (self.chunk <= 0 or self.window is not None):
            raise ValueError("capped_attention: chunks have a positive size and do not go with a window")
        if o.get("sink") not in (None, False, True, "zero"):
            raise ValueError(f"capped_attention: sink {o.get('sink')!r} is not known (true, \"zero\")")
        self.has_sink = bool(o.get("sink"))
        self.sink_learned = o.get("sink") is True
        self.value_mix = o.get("value_mix")
        if self.value_mix not in (None, "first", "mix"):
            raise ValueError(f"capped_attention: value_mix {self.value_mix!r} is not known (first, mix)")
        self.value_mix_buffer = str(o.get("value_mix_buffer", "value_mix_first"))
        self.kept = self.kept_head_size(self.dim, self.value_dim, dtype)
        if self.kept > 512:
            raise ValueError(f"capped_attention: heads of {max(self.dim, self.value_dim)} elements are not supported (at most 512)")
        self.position = position_class(spec.position.kind)(spec.position, dtype, device)
        # the gate's columns of the product: one an element, or one a head (kept as a multiple of 8 columns)
        self.gate_cols = 0 if not self.gated else (self.n_heads * self.kept if self.gate == "sigmoid"
                                                   else -(-self.n_heads // 8) * 8)
        self.proj: Optional[Linear] = None      # [q; k; v; g] with every head padded to ``kept``
        self.o: Optional[Linear] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None
        self.mix = 0.0

    @staticmethod
    def kept_head_size(dim: int, value_dim: int, dtype: torch.dtype) -> int:
        """The one head size keys, values and queries are held with: the larger of the two, as a multiple of 8; in
        bfloat16 the next size the tensor-core attention kernels take (64, 128) when that is at most a quarter more."""
        kept = -(-max(dim, value_dim) // 8) * 8
        if dtype == torch.bfloat16:
            for fast in (64, 128):
                if kept <= fast and fast * 4 <= kept * 5:
                    return fast
        return kept

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        H, G, D, d = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.width
        o = spec.options
        V = int(o.get("value_dim", D))
        p = {"q.weight": ParamDecl((H * D, d)), "k.weight": ParamDecl((G * D, d)), "v.weight": ParamDecl((G * V, d)),
             "o.weight": ParamDecl((d, H * V))}
        if spec.bias:
            p.update({"q.bias": ParamDecl((H * D,)), "k.bias": ParamDecl((G * D,)), "v.bias": ParamDecl((G * V,))})
        if o.get("gate") == "sigmoid":
            p["g.weight"] = ParamDecl((H * V, d))
        elif o.get("gate") == "sigmoid_head":
            p["g.weight"] = ParamDecl((H, d))
        if o.get("qk_norm_eps") is not None and o.get("qk_norm") == "whole":
            p["q_norm.weight"] = ParamDecl((H * D,), init="ones")
            p["k_norm.weight"] = ParamDecl((G * D,), init="ones")
        if o.get("qk_norm_eps") is not None and o.get("qk_norm") == "head_first":
            p["q_norm.weight"] = ParamDecl((D,), init="ones")
            p["k_norm.weight"] = ParamDecl((D,), init="ones")
        if o.get("sink") is True:
            p["sink"] = ParamDecl((H,))
        if o.get("value_mix") is not None:
            p["vmix"] = ParamDecl(())        # the layer that only leaves its values owns one too, and does not use it
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        H, G, D, V, P = self.n_heads, self.n_kv, self.dim, self.value_dim, self.kept
        order = self.position.head_order(D) if hasattr(self.position, "head_order") else None
        parts = [("q", H, D, order), ("k", G, D, order), ("v", G, V, None)]
        ws = [tensors[f"{n}.weight"] for n, _, _, _ in parts] + ([tensors["g.weight"]] if self.gated else [])
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        blocks = [_pad_heads(_order_heads(tensors[f"{n}.weight"].to(wide), heads, size, ordr), heads, size, P)
                  for n, heads, size, ordr in parts]
        if self.gate == "sigmoid":
            blocks.append(_pad_heads(tensors["g.weight"].to(wide), H, V, P))
        elif self.gate == "sigmoid_head":
            g = tensors["g.weight"].to(wide)
            blocks.append(torch.cat([g, g.new_zeros(self.gate_cols - H, g.shape[1])], dim=0))
        weight = torch.cat(blocks, dim=0)
        bias = None
        if self.spec.bias:
            bs = []
            for n, heads, size, ordr in parts:
                b = tensors.get(f"{n}.bias")
                b = b if b is not None else ws[0].new_zeros(heads * size)
                bs.append(_pad_heads(_order_heads(b.to(torch.float32), heads, size, ordr), heads, size, P))
            if self.gated:
                bs.append(bs[0].new_zeros(self.gate_cols))
            bias = torch.cat(bs, dim=0)
        self.proj = Linear(weight, bias)
        w_o = tensors["o.weight"]
        if V != P:
            w_o = _pad_heads(w_o.t().contiguous(), H, V, P).t().contiguous()
        self.o = Linear(w_o)
        if self.norm_kind == "whole":
            self.q_norm_w = _pad_heads(_order_heads(tensors["q_norm.weight"].float(), H, D, order), H, D, P).contiguous()
            self.k_norm_w = _pad_heads(_order_heads(tensors["k_norm.weight"].float(), G, D, order), G, D, P).contiguous()
        if self.norm_kind == "head_first":
            self.q_norm_w = _pad_heads(_order_heads(tensors["q_norm.weight"].float(), 1, D, order), 1, D, P).contiguous()
            self.k_norm_w = _pad_heads(_order_heads(tensors["k_norm.weight"].float(), 1, D, order), 1, D, P).contiguous()
        if self.has_sink:
            self.sinks = (tensors["sink"].float().contiguous() if self.sink_learned
                          else torch.zeros(H, dtype=torch.float32, device=w_o.device))
        if self.value_mix == "mix":
            self.mix = float(tensors["vmix"].float().item())

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("attention", "elementwise")
        libs += kernels.fast_attention_libraries(self.dtype, self.kept, self.n_heads, self.n_kv, softcap=self.softcap,
                                                 keep_first=self.keep_first, sinks=self.has_sink)
        for lin in (self.proj, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return KVNeed(self.n_kv, self.kept, self.window, keep_first=self.keep_first, chunk=self.chunk)

    def state_needs(self) -> Optional[StateNeed]:
        return None

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T = residual.shape[0]
        H, G, P = self.n_heads, self.n_kv, self.kept
        heads_width = (H + 2 * G) * P
        proj = step.ws.buf("cattn_proj", (T, heads_width + self.gate_cols), self.dtype)
        self.proj(h, proj)
        table = self.position.rotary_table()
        inv_freq, rot = table if table is not None else (None, 0)
        amplitude = float(getattr(self.position, "amplitude", 1.0))
        k_pages, v_pages = (io.k_pages, io.v_pages) if io.writes_cache else (None, None)
        if self.norm_kind == "whole" or self.value_mix is not None:
            if amplitude != 1.0:
                raise ValueError("capped_attention: an amplitude on the rotation is not combined with a norm of the "
                                 "whole q and k or with mixed values")
            mix_buf = None
            if self.value_mix is not None:
                mix_buf = step.ws.buf(self.value_mix_buffer, (T, G * self.value_dim), self.dtype)
            whole = self.norm_kind == "whole"
            kernels.qk_prep(proj, H, G, P, rot, inv_freq, self.q_norm_w if whole else None,
                            self.k_norm_w if whole else None, H * self.dim, G * self.dim, self.norm_eps or 0.0,
                            {None: 0, "first": 1, "mix": 2}[self.value_mix], self.mix, mix_buf, self.value_dim,
                            step.positions, step.seq_of_token, io.block_table, k_pages, v_pages, io.page_size)
        else:
            head_norm = self.norm_kind in ("head", "head_first")
            first = self.norm_kind == "head_first"
            kernels.rope_norm_store(proj, H, G, P, rot, inv_freq, amplitude, self.dim if head_norm else 0,
                                    (self.norm_eps or 0.0) if head_norm else 0.0, step.positions, step.seq_of_token,
                                    io.block_table, k_pages, v_pages, io.page_size, norm_first=first,
                                    q_weight=self.q_norm_w if first else None, k_weight=self.k_norm_w if first else None)
        out = step.ws.buf("attn_out", (T, H * P), self.dtype)
        gate = proj[:, heads_width:] if self.gate == "sigmoid" else None
        # the flat decode kernel multiplies by an element gate's sigmoid as it stores, the decode kernel that splits a
        # sequence's keys by a head's gate where it combines the splits; behind the others a kernel does
        head_gate = proj[:, heads_width:heads_width + H] if self.gate == "sigmoid_head" else None
        gated = kernels.attention(step, proj, out, H, G, P, self.scale, self.window, io, softcap=self.softcap, gate=gate,
                                  keep_first=self.keep_first, sinks=self.sinks, head_gate=head_gate,
                                  head_gate_mult=self.out_scale, chunk=self.chunk)
        if self.gate == "sigmoid" and not gated:
            kernels.sigmoid_mul(out, gate, out)
        elif self.gate == "sigmoid_head" and not gated:
            kernels.gate_heads(out, head_gate, out, H, self.out_scale)
        self.o(out, residual, accumulate=accumulate)
        return None


register_mixer("capped_attention", CappedAttention)
