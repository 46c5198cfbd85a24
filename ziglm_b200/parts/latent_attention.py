"""Attention through a low-rank latent, with a sigmoid gate on the heads' outputs, a query latent, rotary positions
on a part of the keys that all heads share, and a sliding window, each of which may be left out.

For the normed input h of a layer with H heads of query/key size D (unrotated) and Rr (rotated), value size V and
latent sizes Rq, R:
    c_q = norm(W_dq h)            q  = W_uq c_q            [H, D + Rr]     (``q_rank`` None: q = W_q h)
    [c | r] = W_dkv h             c <- norm(c)             R and Rr elements a position (r is not normed)
    k_j = W_uk c_j,  v_j = W_uv c_j                        [H, D], [H, V]   (j: a position)
    s_ij = (q_i[:D] . k_j + rot(q_i[D:], i) . rot(r_j, j)) * scale,  j <= i and i - j < window
    p = softmax_j(s);  o_i = sum_j p_ij v_j
    out = W_o (o * sigmoid(W_g h))                                          (``gate`` None: out = W_o o)
Only c and the rotated r are kept per position: one vector of Rr + R elements that is key and value at once
(``KVNeed(values_are_keys=True)``).  The products with W_uk and W_uv are moved to the other side of the
attention, head by head:
    q'_i = [rot(q_i[D:]) | W_uk[h]^T q_i[:D]]  (Rr + R elements per head),   s_ij = (q'_i . [rot(r_j) | c_j]) * scale,
    l_i  = sum_j p_ij [rot(r_j) | c_j],                                      o_i  = W_uv[h] l_i[Rr:],
so the attention itself is the library's attention of H query heads over one key/value head of size Rr + R
whose keys and values are the same pages, and the two per-head products are block-diagonal products (the first also
moves the rotated part of a query to the front of its head, in the order that makes the encoding's pairs the halves
the rotation kernel turns; the second skips the first Rr elements).  The projections of h that are normed or gated
(W_dq, W_dkv, W_g) are one matrix product with a float32 result: the norms of the latents and the gate's sigmoid
read it in float32.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec, NormSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, norm_class, position_class, register_mixer
from .linear import Linear


class LatentAttention(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.n_heads, self.dim = spec.n_heads, spec.head_dim
        self.value_dim, self.kv_rank = int(o["value_dim"]), int(o["kv_rank"])
        self.q_rank = None if o.get("q_rank") is None else int(o["q_rank"])
        self.rot_dim = int(o.get("rot_dim") or 0)
        if spec.scale is None:
            raise ValueError("latent_attention: the spec must give the factor on the scores")
        self.scale = float(spec.scale)
        self.gate = o.get("gate", "sigmoid")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"latent_attention: output gate {self.gate!r} is not known (sigmoid)")
        self.window = None if spec.window is None else int(spec.window)
        # the attention kernels take head sizes that are multiples of 8: a latent of another size is kept with
        # zeros behind it (they add nothing to a score and their part of the result is not read)
        self.kept = -(-(self.rot_dim + self.kv_rank) // 8) * 8
        if self.kept > 512:
            raise ValueError(f"latent_attention: a key/value latent of {self.kv_rank} elements beside {self.rot_dim} "
                             "rotated ones is not supported (at most 512 together)")
        self.position = position_class(spec.position.kind)(spec.position, dtype, device)
        table = self.position.rotary_table()
        if self.rot_dim and (table is None or table[1] != self.rot_dim):
            raise ValueError("latent_attention: the position encoding must turn exactly the rotated part of the keys")
        if not self.rot_dim and table is not None:
            raise ValueError("latent_attention: a rotation needs a rotated part of the keys (rot_dim)")
        eps = float(o["norm_eps"])
        norm_kind = o.get("norm", "rmsnorm")
        self.q_norm = (norm_class(norm_kind)(NormSpec(norm_kind, self.q_rank, eps), dtype, device)
                       if self.q_rank is not None else None)
        self.kv_norm = norm_class(norm_kind)(NormSpec(norm_kind, self.kv_rank, eps), dtype, device)
        self.down: Optional[Linear] = None       # [W_dq; W_dkv; W_g], whichever exist
        self.uq: Optional[Linear] = None         # W_uq, or W_q when there is no query latent
        self.o: Optional[Linear] = None
        self.uk_t: Optional[torch.Tensor] = None  # [H, kept, D + Rr]: per head, a query into the latent's space
        self.uv: Optional[torch.Tensor] = None    # [H, V, kept]

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        o = spec.options
        H, D, V, R, d = spec.n_heads, spec.head_dim, int(o["value_dim"]), int(o["kv_rank"]), spec.width
        Rr = int(o.get("rot_dim") or 0)
        p = {"dkv.weight": ParamDecl((R + Rr, d)), "dkv_norm.weight": ParamDecl((R,), init="ones"),
             "uk.weight": ParamDecl((H * D, R)), "uv.weight": ParamDecl((H * V, R)), "o.weight": ParamDecl((d, H * V))}
        if o.get("q_rank") is not None:
            Rq = int(o["q_rank"])
            p.update({"dq.weight": ParamDecl((Rq, d)), "dq_norm.weight": ParamDecl((Rq,), init="ones"),
                      "uq.weight": ParamDecl((H * (D + Rr), Rq))})
        else:
            p["q.weight"] = ParamDecl((H * (D + Rr), d))
        if o.get("gate", "sigmoid") == "sigmoid":
            p["g.weight"] = ParamDecl((H * V, d))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        H, D, V, R, Rr, K = self.n_heads, self.dim, self.value_dim, self.kv_rank, self.rot_dim, self.kept
        order = self.position.head_order(Rr) if Rr and hasattr(self.position, "head_order") else None
        order = list(order) if order is not None else list(range(Rr))
        dkv = tensors["dkv.weight"]
        if Rr:
            # the rotated rows in the order that makes the encoding's pairs the halves the kernel turns
            idx = torch.tensor(list(range(R)) + [R + i for i in order], dtype=torch.long, device=dkv.device)
            dkv = dkv.index_select(0, idx)
        ws = ([tensors["dq.weight"]] if self.q_rank is not None else []) + [dkv]
        ws += [tensors["g.weight"]] if self.gate else []
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.down = Linear(torch.cat([w.to(wide) for w in ws], dim=0))
        self.uq = Linear(tensors["uq.weight"] if self.q_rank is not None else tensors["q.weight"])
        self.o = Linear(tensors["o.weight"])
        if self.q_norm is not None:
            self.q_norm.bind({"weight": tensors["dq_norm.weight"]})
        self.kv_norm.bind({"weight": tensors["dkv_norm.weight"]})
        uk = tensors["uk.weight"].view(H, D, R)
        into = uk.new_zeros(H, K, D + Rr)                    # row r of a head: what element r of q' is made of
        for r, src in enumerate(order):
            into[:, r, D + src] = 1.0                        # the rotated part moves to the front, exactly
        into[:, Rr:Rr + R, :D] = uk.transpose(1, 2)
        uv = tensors["uv.weight"].view(H, V, R)
        out_of = uv.new_zeros(H, V, K)
        out_of[:, :, Rr:Rr + R] = uv
        self.uk_t = into.contiguous()
        self.uv = out_of.contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("elementwise", "block_linear", "attention")
        libs += kernels.fast_attention_libraries(self.dtype, self.kept, min(self.n_heads, self.HEADS_AT_ONCE), 1)
        for lin in (self.down, self.uq, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return KVNeed(1, self.kept, self.window, values_are_keys=True)

    def state_needs(self) -> Optional[StateNeed]:
        return None

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T = residual.shape[0]
        H, D, V, Rn, Rr, K = self.n_heads, self.dim, self.value_dim, self.kv_rank, self.rot_dim, self.kept
        Rq = self.q_rank or 0
        proj = step.ws.buf("lat_proj", (T, Rq + Rn + Rr + (H * V if self.gate else 0)), torch.float32)
        self.down(h, proj)
        q = step.ws.buf("lat_q", (T, H * (D + Rr)), self.dtype)
        if self.q_norm is not None:
            cq = step.ws.buf("lat_cq", (T, Rq), self.dtype)
            self.q_norm.forward_rows(proj[:, :Rq], cq)
            self.uq(cq, q)
        else:
            self.uq(h, q)
        # a row of ``qc``: the H queries in the latent's space, then the token's key/value head: [rotated | latent]
        qc = step.ws.buf("lat_qc", (T, (H + 1) * K), self.dtype)
        self.kv_norm.forward_rows(proj[:, Rq:Rq + Rn], qc[:, H * K + Rr:H * K + Rr + Rn])
        if Rr:
            kernels.convert_rows(proj[:, Rq + Rn:Rq + Rn + Rr], qc[:, H * K:H * K + Rr])
        if K != Rr + Rn:
            qc[:, H * K + Rr + Rn:].zero_()
        kernels.block_linear(q, self.uk_t, qc[:, :H * K])
        table = self.position.rotary_table()
        kernels.rope_store(qc, H, 1, K, Rr, table[0] if table is not None else None, step.positions, step.seq_of_token,
                           io.block_table, io.k_pages, None, io.page_size, keys_only=True)
        heads = step.ws.buf("lat_heads", (T, H * V), self.dtype)
        gate = proj[:, Rq + Rn + Rr:] if self.gate else None
        # all heads read the one key/value head; the tensor-core kernels take up to 16 query heads a key/value head,
        # so more heads go through them 16 at a time (the queries are a column slice of the rows, the latent pages
        # are the same)
        n = self.HEADS_AT_ONCE if (H > self.HEADS_AT_ONCE and kernels.fast_attention_libraries(
            self.dtype, K, self.HEADS_AT_ONCE, 1)) else H
        for h0 in range(0, H, n):
            h1 = min(H, h0 + n)
            mixed = step.ws.buf("lat_mixed", (T, (h1 - h0) * K), self.dtype)
            kernels.attention(step, qc[:, h0 * K:h1 * K], mixed, h1 - h0, 1, K, self.scale, self.window, io)
            if self.gate:
                kernels.block_linear(mixed, self.uv[h0:h1], heads[:, h0 * V:h1 * V], epilogue="sigmoid_gate",
                                     gate=gate[:, h0 * V:h1 * V])
            else:
                kernels.block_linear(mixed, self.uv[h0:h1], heads[:, h0 * V:h1 * V])
        self.o(heads, residual, accumulate=accumulate)
        return None

    HEADS_AT_ONCE = 16


register_mixer("latent_attention", LatentAttention)
