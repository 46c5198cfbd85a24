"""A selective state-space mixer: a scan whose step sizes and input/output maps depend on the token, behind a short
causal convolution, beside a silu gate.

For the rows h the mixer reads, with C channels, N states a channel, a convolution of K taps and a step-size rank r:
    [x | z] = W_in h                                   x, z: C channels each
    x <- silu(conv(x) + b_conv)                        per channel, K taps, zeros before the start of the sequence
    [dt' | B | C] = W_x x                              r + N + N numbers a token
    dt = softplus(W_dt dt' + b_dt)                     one step size a channel, float32
    S_t[c, n] = exp(dt_c A[c, n]) S_(t-1)[c, n] + dt_c x_c B_n,   A = -exp(A_log)
    y_c = sum_n S_t[c, n] C_n + D_c x_c
    out = W_o (y * silu(z))
A sequence carries [K - 1 + N, C] float32 from step to step (``StateNeed``): the convolution's last K - 1 inputs, then
S, which starts at zero.  Step sizes, decays, the products that enter the recurrence and the state are float32 in
both precisions; the scan runs in chunks of tokens whose maps are composed, a decoded token being one chunk.
Options of the spec: ``channels``, ``states``, ``taps``, ``dt_rank``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, register_mixer
from .linear import Linear


class SelectiveScan(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.channels, self.states = int(o["channels"]), int(o["states"])
        self.taps, self.rank = int(o["taps"]), int(o["dt_rank"])
        if min(self.channels, self.states, self.taps, self.rank) <= 0:
            raise ValueError("selective_scan: channels, states, taps and dt_rank must be positive")
        if self.states > 256:
            raise ValueError(f"selective_scan: {self.states} states a channel are not supported (at most 256)")
        self.in_proj: Optional[Linear] = None
        self.x_proj: Optional[Linear] = None
        self.dt_proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.conv_w = self.conv_b = self.a_t = self.d = None

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        o = spec.options
        C, N, K, r, d = int(o["channels"]), int(o["states"]), int(o["taps"]), int(o["dt_rank"]), spec.width
        return {"in.weight": ParamDecl((2 * C, d)), "conv.weight": ParamDecl((C, K)), "conv.bias": ParamDecl((C,)),
                "x.weight": ParamDecl((r + 2 * N, C)), "dt.weight": ParamDecl((C, r)), "dt.bias": ParamDecl((C,)),
                "A_log": ParamDecl((C, N)), "D": ParamDecl((C,)), "o.weight": ParamDecl((d, C))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.in_proj = Linear(tensors["in.weight"])
        self.x_proj = Linear(tensors["x.weight"])
        self.dt_proj = Linear(tensors["dt.weight"], tensors["dt.bias"].float())
        self.o = Linear(tensors["o.weight"])
        self.conv_w = tensors["conv.weight"].float().t().contiguous()          # [taps, channels]: a row per tap
        self.conv_b = tensors["conv.bias"].float().contiguous()
        # [states, channels], times log2(e): the kernel's exp(dt A) is one multiplication and one exp2
        self.a_t = (-torch.exp(tensors["A_log"].float()) * math.log2(math.e)).t().contiguous()
        self.d = tensors["D"].float().contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("recurrent",)
        for lin in (self.in_proj, self.x_proj, self.dt_proj, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return None

    def state_needs(self) -> Optional[StateNeed]:
        return StateNeed((self.taps - 1 + self.states, self.channels), torch.float32)

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T, C, N, r = residual.shape[0], self.channels, self.states, self.rank
        proj = step.ws.buf("ssm_proj", (T, 2 * C), self.dtype)
        self.in_proj(h, proj)
        x, z = proj[:, :C], proj[:, C:]
        u = step.ws.buf("ssm_u", (T, C), self.dtype)
        kernels.causal_conv(x, self.conv_w, self.conv_b, io.state, step, u, activation="silu")
        dbc = step.ws.buf("ssm_dbc", (T, r + 2 * N), self.dtype)
        self.x_proj(u, dbc)
        dt_pre = step.ws.buf("ssm_dt", (T, C), torch.float32)
        self.dt_proj(dbc[:, :r], dt_pre)
        out = step.ws.buf("ssm_out", (T, C), self.dtype)
        kernels.selective_scan(u, dt_pre, dbc, r, r + N, N, z, x, self.a_t, self.d, self.taps, io.state, step, out)
        self.o(out, residual, accumulate=accumulate)
        return None


register_mixer("selective_scan", SelectiveScan)
