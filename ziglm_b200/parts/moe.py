"""Mixture of experts: a router picks ``top`` of E small gated feed-forwards for every token.

    z = W_r h (float32)              score = sigmoid(z) (or softmax)         choice = score + correction
    the experts form ``groups`` equal groups of neighbours, a group is scored by the sum of its ``group_best``
    best choice scores, and only experts of the ``keep_groups`` best groups can be chosen;
    out = sum over the chosen e of score_e * W_down[e] (act(W_gate[e] h) * (W_up[e] h))
(the weights are divided by their sum only with ``renormalize``).  Options of the spec: ``experts``, ``top``,
``groups``, ``keep_groups``, ``group_best``, ``score`` ("sigmoid", "softmax", or "softmax_chosen": the experts with
the largest logits, weighted by the softmax over the chosen logits alone), ``correction`` (whether a learned offset
per expert enters the choice), ``renormalize``.  The experts' activation is silu(gate) * up, or with
``activation`` "swish_clamped" and the options ``limit`` and ``slope`` the clamped form
min(g, L) sigmoid(slope min(g, L)) (clamp(u, -L, L) + 1).  ``shared``: the spec of a feed-forward that runs for
every token and is added to the experts' sum (its tensors under ``shared.``); with ``shared_gate`` it is added times
sigmoid(w_sg . h), one number a token (the tensor ``shared_gate.weight`` [1, d], whose product rides on the router's).
``identity``: that many further outputs of the router, behind the experts', stand for identity experts, which have no
tensors and whose output is the token's row h itself (times the weight); scores, offsets, groups and the choice run
over experts and identity experts together.  ``weight_scale``: a factor on the chosen experts' weights.

The (token, choice) pairs are grouped by expert on the device (nothing is read back, so a decode step stays a
replayable graph), the experts' products run over the groups, each pair's result lands in a float32 row of its
own, and a token's rows are summed in the order of its choices.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import FeedForwardSpec
from .base import ParamDecl, Part, feed_forward_class, register_feed_forward
from .linear import Linear


class MixtureOfExperts(Part):
    can_overwrite = True

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.n_experts, self.top = int(o["experts"]), int(o["top"])
        self.identity = int(o.get("identity") or 0)
        if self.identity < 0:
            raise ValueError("moe: the number of identity experts cannot be negative")
        self.n_routed = self.n_experts + self.identity       # outputs of the router
        self.weight_scale = float(o.get("weight_scale", 1.0))
        self.shared_gate = bool(o.get("shared_gate", False))
        if self.shared_gate and o.get("shared") is None:
            raise ValueError("moe: a gate on the shared expert needs a shared expert")
        self.groups, self.keep_groups = int(o.get("groups", 1)), int(o.get("keep_groups", o.get("groups", 1)))
        self.group_best = int(o.get("group_best", 2))
        if o.get("score", "sigmoid") not in self.SCORES:
            raise ValueError(f"moe: router score {o.get('score')!r} is not known ({', '.join(self.SCORES)})")
        self.softmax = self.SCORES[o.get("score", "sigmoid")]
        self.renormalize = bool(o.get("renormalize", False))
        if spec.activation not in ("silu", "swish_clamped"):
            raise ValueError(f"moe: expert activation {spec.activation!r} is not known (silu, swish_clamped)")
        # the clamped form: a positive limit switches the kernels' silu to it
        self.limit = float(o.get("limit", 0.0)) if spec.activation == "swish_clamped" else 0.0
        self.slope = float(o.get("slope", 1.0)) if spec.activation == "swish_clamped" else 1.0
        if spec.activation == "swish_clamped" and not self.limit > 0.0:
            raise ValueError("moe: the clamped activation needs a positive limit")
        if self.softmax == 2 and (o.get("correction") or int(o.get("groups", 1)) != 1):
            raise ValueError("moe: the softmax over the chosen logits goes with neither a correction nor groups")
        shared = o.get("shared")
        self.shared = feed_forward_class(shared.kind)(shared, dtype, device) if shared is not None else None
        E, G = self.n_routed, self.groups
        if E % G or not 1 <= self.keep_groups <= G or not 1 <= self.top <= self.keep_groups * (E // G):
            raise ValueError(f"moe: {E} experts in {G} groups of which {self.keep_groups} are kept cannot give "
                             f"{self.top} experts a token")
        self.ff = spec.intermediate
        self.router: Optional[Linear] = None
        self.correction: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None     # [E, 2 ff, d]
        self.down: Optional[torch.Tensor] = None        # [E, d, ff]
        self.interleaved = False                        # gate and up rows of an expert alternate (bfloat16)
        self._host_offs = None                          # the experts' offsets read back for a prompt step

    @classmethod
    def declare(cls, spec: FeedForwardSpec) -> Dict[str, ParamDecl]:
        o = spec.options
        E, ff, d = int(o["experts"]), spec.intermediate, spec.width
        routed = E + int(o.get("identity") or 0)
        p = {"router.weight": ParamDecl((routed, d))}
        if o.get("correction", False):
            p["correction"] = ParamDecl((routed,))
        if o.get("shared_gate", False):
            p["shared_gate.weight"] = ParamDecl((1, d))
        for e in range(E):
            p[f"e{e}.gate.weight"] = ParamDecl((ff, d))
            p[f"e{e}.up.weight"] = ParamDecl((ff, d))
            p[f"e{e}.down.weight"] = ParamDecl((d, ff))
        shared = o.get("shared")
        if shared is not None:
            for name, decl in feed_forward_class(shared.kind).declare(shared).items():
                p["shared." + name] = decl
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = self.n_experts
        router = tensors["router.weight"]
        if self.shared_gate:
            # the gate's one row rides behind the router's: one product gives the logits and the gate's number
            sg = tensors["shared_gate.weight"]
            wide_r = torch.float32 if torch.float32 in (router.dtype, sg.dtype) else router.dtype
            router = torch.cat([router.to(wide_r), sg.to(wide_r).reshape(1, -1)], dim=0).contiguous()
        self.router = Linear(router)
        self.correction = tensors["correction"].float().contiguous() if "correction" in tensors else None
        mats = [tensors[f"e{e}.{n}.weight"] for e in range(E) for n in ("gate", "up", "down")]
        wide = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        # bfloat16: gate and up rows alternate, which is what the tensor-core product's gated epilogue reads
        self.interleaved = self.dtype == torch.bfloat16 and wide == torch.bfloat16
        join = (lambda g, u: torch.stack([g, u], dim=1).reshape(2 * g.shape[0], -1)) if self.interleaved \
            else (lambda g, u: torch.cat([g, u], dim=0))
        self.gate_up = torch.stack([join(tensors[f"e{e}.gate.weight"].to(wide), tensors[f"e{e}.up.weight"].to(wide))
                                    for e in range(E)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down.weight"].to(wide) for e in range(E)]).contiguous()
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in tensors.items() if k.startswith("shared.")})

    SCORES = {"sigmoid": 0, "softmax": 1, "softmax_chosen": 2}

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("moe",) + (kernels.fast_gemm_libraries() if self.interleaved else ())
        if self.shared is not None:
            libs += self.shared.kernel_libraries()
        return libs + (self.router.libraries(self.dtype) if self.router is not None else ("gemm_generic",))

    def forward(self, step, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T, d = residual.shape
        E, top, ff = self.n_routed, self.top, self.ff
        n_extra = 1 if self.shared_gate else 0
        P = T * top
        ws = step.ws
        ids = ws.buf("moe_ids", (T, top), torch.int32)
        weights = ws.buf("moe_weights", (T, top), torch.float32)
        route = dict(softmax_scores=self.softmax, renormalize=self.renormalize, weight_scale=self.weight_scale,
                     n_extra=n_extra)
        gate = None                             # the shared expert's gate: one float32 number a token
        if T <= self.SKINNY_TOKENS and h.dtype == self.router.weight.dtype and (3 * E + h.shape[1]) * 4 < 40 * 1024:
            # few tokens: the router's product is taken inside the routing kernel
            gate = ws.buf("moe_shared_gate", (T, 1), torch.float32) if n_extra else None
            kernels.moe_route(None, self.correction, top, self.groups, self.keep_groups, self.group_best, ids, weights,
                              h=h, router=self.router.weight, extra_out=gate, **route)
        else:
            z = ws.buf("moe_logits", (T, E + n_extra), torch.float32)
            self.router(h, z)                   # float32 sums of the rows' products (on the tensor cores in bfloat16)
            kernels.moe_route(z, self.correction, top, self.groups, self.keep_groups, self.group_best, ids, weights,
                              **route)
            gate = z[:, E:] if n_extra else None
        extras = {}
        if self.identity:
            extras.update(ids=ids, n_real=self.n_experts, h=h)
        if self.shared_gate:
            shared_y = ws.buf("moe_shared_y", (T, d), torch.float32)
            self.shared.forward(step, h, shared_y, accumulate=False)
            extras.update(shared=shared_y, gate=gate)
        max_tiles = kernels.moe_max_tiles(P, E)
        offs = ws.buf("moe_offs", (E + 1,), torch.int32)
        order = ws.buf("moe_order", (P,), torch.int32)
        tile_expert = ws.buf("moe_tile_expert", (max_tiles,), torch.int32)
        tile_row = ws.buf("moe_tile_row", (max_tiles,), torch.int32)
        n_tiles = ws.buf("moe_n_tiles", (1,), torch.int32)
        place = ws.buf("moe_place", (P,), torch.int32)
        kernels.moe_group(ids.view(-1), E, offs, order, place, tile_expert, tile_row, n_tiles, n_real=self.n_experts)
        groups = (offs, order, tile_expert, tile_row, n_tiles)
        act = ws.buf("moe_act", (P, ff), self.dtype)
        y = ws.buf("moe_y", (P, d), torch.float32)
        # a step of one token a sequence may be captured as a graph, whatever its size: nothing is read back in it
        single = bool(getattr(step, "single_token", False))
        if (self.interleaved and T >= self.TENSOR_CORE_TOKENS and not single
                and self._on_tensor_cores(step, h, offs, order, act, y)):
            kernels.moe_combine(y, weights, residual, accumulate, place=place, **extras)
            return self._add_shared(step, h, residual)
        skinny = T <= self.SKINNY_TOKENS or single or (self.interleaved and T < self.TENSOR_CORE_TOKENS)
        kernels.moe_grouped(h, self.gate_up, act, True, P, top, *groups, interleaved=self.interleaved, skinny=skinny,
                            limit=self.limit, slope=self.slope)
        kernels.moe_grouped(act, self.down, y, False, P, top, *groups, skinny=skinny)
        kernels.moe_combine(y, weights, residual, accumulate, **extras)
        return self._add_shared(step, h, residual)

    def _add_shared(self, step, h: torch.Tensor, residual: torch.Tensor):
        """The shared feed-forward's output, added to what the experts left in ``residual``."""
        if self.shared is not None and not self.shared_gate:     # a gated one was added where the pairs were summed
            self.shared.forward(step, h, residual)
        return None

    TENSOR_CORE_TOKENS = 128      # from this many tokens on a prompt step's experts run on the tensor cores
    SKINNY_TOKENS = 64            # up to this many tokens (in bfloat16: up to where the tensor cores take over, and in
                                  # every step of one token a sequence) an expert's weights are streamed against its rows

    def _on_tensor_cores(self, step, h, offs, order, act, y) -> bool:
        """A prompt step in bfloat16: the tokens' rows are gathered into grouped order and every expert that has
        rows runs the library's tensor-core product on its run of them (gate/up with the activation in the
        epilogue, then down into float32 rows in grouped order).  The runs' lengths are known on the device only,
        so the experts' offsets are read back: one small copy and one wait of the host per layer, which a step of
        hundreds of tokens hides and a decode step (captured as a graph) never takes."""
        import ctypes
        E, top = self.n_routed, self.top       # the offsets count the identity experts' runs too; they lie last
        P = order.numel()
        rows = step.ws.buf("moe_rows", (P, h.shape[1]), self.dtype)
        kernels.moe_gather(h, order, top, rows)
        if self._host_offs is None:
            self._host_offs = torch.empty(E + 1, dtype=torch.int32).pin_memory()
        self._host_offs.copy_(offs, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        host = ctypes.c_void_p(self._host_offs.data_ptr())
        if not kernels.gemm_tc_groups(rows, self.gate_up, act, host, glu="silu", limit=self.limit, slope=self.slope):
            return False
        return kernels.gemm_tc_groups(act, self.down, y, host)


register_feed_forward("moe", MixtureOfExperts)
