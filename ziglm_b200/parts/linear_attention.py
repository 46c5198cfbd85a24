"""Linear attention with a fixed decay per head: a matrix-valued state per sequence instead of a cache of keys.

For the rows h the mixer reads, H heads of query/key size D and value size V, decays a_h in (0, 1]:
    q = act(W_q h),  k = act(W_k h),  v = act(W_v h)        laid out head by head (``activation``: "silu" or None)
    S_t = a_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t          S: [D, V] per head, zero where a sequence starts
    out = W_o (norm(concat(o)) * sigmoid(W_g h) * out_scale)   the heads RMS-normed together with a weight
                                                              (``gate`` None: without the sigmoid)
Options beside these: ``MixerSpec.position`` (rotary positions on q and k: the first rotated dimensions of every
head are turned before the recurrence), ``key_scale`` (k times a factor, after the rotation), ``norm`` "heads" (the
default: the heads normed together with the weight ``norm.weight``) or "head" (every head divided by its own root
mean square, no weight), ``gate`` "sigmoid", "silu" (g * sigmoid(g)) or None.  The rotation and the factor on k are
applied to the float32 copies of q and k the recurrence's kernel works on.
There is no other factor on the scores and no softmax.  A sequence carries [H, D, V] float32 from step to step
(``StateNeed``); the recurrence, the scores q . k with their decays and the outputs are float32 in both precisions
(the kernel works through a step in chunks of tokens, a decoded token being a chunk of one).  The four projections of
h are one matrix product; the activation is applied as the kernel reads q, k and v.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, position_class, register_mixer
from .linear import Linear


class DecayedLinearAttention(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.n_heads, self.dim = spec.n_heads, spec.head_dim
        self.value_dim = int(o.get("value_dim", spec.head_dim))
        self.decay = tuple(float(a) for a in o["decay"])
        if len(self.decay) != self.n_heads or any(not 0.0 < a <= 1.0 for a in self.decay):
            raise ValueError(f"decayed_linear_attention: one decay in (0, 1] is needed for each of the {self.n_heads} heads")
        if self.dim > 512:
            raise ValueError(f"decayed_linear_attention: keys of {self.dim} elements are not supported (at most 512)")
        self.activation = o.get("activation")
        if self.activation not in (None, "silu"):
            raise ValueError(f"decayed_linear_attention: activation {self.activation!r} is not known (silu)")
        self.gate = o.get("gate")
        if self.gate not in (None, "sigmoid", "silu"):
            raise ValueError(f"decayed_linear_attention: output gate {self.gate!r} is not known (sigmoid, silu)")
        self.norm_kind = o.get("norm", "heads")
        if self.norm_kind not in ("heads", "head"):
            raise ValueError(f"decayed_linear_attention: norm {self.norm_kind!r} is not known (heads, head)")
        self.key_scale = float(o.get("key_scale", 1.0))
        self.position = position_class(spec.position.kind)(spec.position, dtype, device)
        table = self.position.rotary_table()
        if table is not None and getattr(self.position, "head_order", lambda d: None)(self.dim) is not None:
            raise ValueError("decayed_linear_attention: rotary positions turn the halves of a head's rotated part")
        self.prepared = table is not None or self.key_scale != 1.0
        if self.prepared and self.activation is not None:
            raise ValueError("decayed_linear_attention: an activation on q, k and v is not combined with a rotation "
                             "or a factor on k")
        self.eps = float(o["norm_eps"])
        self.out_scale = float(o.get("out_scale", 1.0))
        self.proj: Optional[Linear] = None       # [q; k; v; g]
        self.o: Optional[Linear] = None
        self.norm_w: Optional[torch.Tensor] = None
        self.pows: Optional[torch.Tensor] = None  # [H, chunk + 1]: decay_h^n, rounded once from float64

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        H, D, d = spec.n_heads, spec.head_dim, spec.width
        V = int(spec.options.get("value_dim", D))
        p = {"q.weight": ParamDecl((H * D, d)), "k.weight": ParamDecl((H * D, d)), "v.weight": ParamDecl((H * V, d)),
             "o.weight": ParamDecl((d, H * V))}
        if spec.options.get("norm", "heads") == "heads":
            p["norm.weight"] = ParamDecl((H * V,), init="ones")
        if spec.options.get("gate") is not None:
            p["g.weight"] = ParamDecl((H * V, d))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        names = ["q", "k", "v"] + (["g"] if self.gate else [])
        ws = [tensors[f"{n}.weight"] for n in names]
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(wide) for w in ws], dim=0))
        self.o = Linear(tensors["o.weight"])
        self.norm_w = tensors["norm.weight"].float().contiguous() if self.norm_kind == "heads" else None
        chunk = kernels.linear_attention_chunk()
        table = torch.tensor([[a ** n for n in range(chunk + 1)] for a in self.decay], dtype=torch.float64)
        self.pows = table.to(torch.float32).to(self.o.weight.device).contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("linear_attention", "elementwise")
        for lin in (self.proj, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return None

    def state_needs(self) -> Optional[StateNeed]:
        return StateNeed((self.n_heads, self.dim, self.value_dim), torch.float32)

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T = residual.shape[0]
        H, D, V = self.n_heads, self.dim, self.value_dim
        qk, hv = H * D, H * V
        proj = step.ws.buf("lin_proj", (T, 2 * qk + hv + (hv if self.gate else 0)), self.dtype)
        self.proj(h, proj)
        mixed = step.ws.buf("lin_mixed", (T, hv), torch.float32)
        # a rotation and a factor on k are applied to the kernel's own float32 copies of q and k
        table = self.position.rotary_table()
        inv_freq, rot = table if table is not None else (None, 0)
        kernels.decayed_linear_attention(proj, 0, qk, 2 * qk, H, D, V, self.activation, self.pows, io.state, step, mixed,
                                         rotary_dim=rot, inv_freq=inv_freq, key_scale=self.key_scale)
        out = step.ws.buf("lin_out", (T, hv), self.dtype)
        gate = proj[:, 2 * qk + hv:] if self.gate else None
        if self.norm_kind == "heads" and self.gate != "silu":
            kernels.norm_gate(mixed, self.norm_w, gate, out, self.eps, self.out_scale)
        else:
            kernels.head_norm_gate(mixed, self.norm_w, gate, out, 1 if self.norm_kind == "heads" else H, self.eps,
                                   self.gate, self.out_scale)
        self.o(out, residual, accumulate=accumulate)
        return None


register_mixer("decayed_linear_attention", DecayedLinearAttention)
