"""RMSNorm: y_i = x_i / sqrt(mean(x^2) + eps) * w_i, statistics in float32.

The reference computes ``ss = sum x^2; inv = 1/sqrt(ss/n + eps); y = (x*inv)*w``
(src/math.zig:850-945, src/cuda_bridge.cu:1475-1534) and adds 1 to the weight
only for Gemma (src/types.zig:279-283); that offset is the ``unit_offset`` option
here and is off unless a spec asks for it.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import NormSpec
from .base import ParamDecl, Part, register_norm


class RMSNorm(Part):
    fusable = True

    def __init__(self, spec: NormSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.width = spec.width
        self.eps = float(spec.eps)
        self.weight_offset = 1.0 if spec.options.get("unit_offset") else 0.0
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def declare(cls, spec: NormSpec) -> Dict[str, ParamDecl]:
        # a weight kept as the gain minus one lies around zero
        return {"weight": ParamDecl((spec.width,), init="zeros" if spec.options.get("unit_offset") else "ones")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("elementwise",)

    def forward(self, step, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                name: str = "norm_out") -> torch.Tensor:
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        if out is None:
            out = step.ws.buf(name, (n, self.width), self.dtype)
        kernels.rmsnorm(x, self.weight, out, self.eps, rows=rows, weight_offset=self.weight_offset)
        return out

    def add_normed(self, step, branch: torch.Tensor, residual: torch.Tensor) -> None:
        """residual += norm(branch), both float32 [T, width]: a norm behind a sublayer, summed into the residual
        stream by the kernel that takes it."""
        kernels.rmsnorm_rows(branch, self.weight, residual, self.eps, add=True, weight_offset=self.weight_offset)

    def add_scaled(self, step, branch: torch.Tensor, residual: torch.Tensor, mult: float,
                   rows_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """residual += mult * norm(branch), both float32 [T, width]; with ``rows_out`` the new rows of the residual
        are also left there in its type (what a sublayer that reads the residual itself takes next)."""
        kernels.norm_add_scaled(branch, self.weight, self.eps, mult, residual, rows_out, weight_offset=self.weight_offset)
        return rows_out

    def sum_normed(self, step, branch: torch.Tensor, residual: torch.Tensor, alpha: float,
                   rows_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """residual = norm(alpha * residual + branch), both float32 [T, width], in place: the norm behind a sum, which
        norms the residual stream itself; with ``rows_out`` the new rows are also left there in its type."""
        kernels.sum_norm(branch, self.weight, self.eps, alpha, residual, rows_out, weight_offset=self.weight_offset)
        return rows_out

    def add_normed_then(self, step, branch: torch.Tensor, residual: torch.Tensor, nxt: "RMSNorm",
                        name: str = "norm_out") -> torch.Tensor:
        """residual += norm(branch), and the rows of the norm ``nxt`` of the new residual (the input of the next
        sublayer), in one kernel where the row fits its shared memory, else in two."""
        out = step.ws.buf(name, tuple(residual.shape), self.dtype)
        if (isinstance(nxt, RMSNorm) and nxt.weight.dtype == self.weight.dtype
                and kernels.norm_add_norm(branch, self.weight, self.eps, residual, nxt.weight, nxt.eps, out,
                                          off1=self.weight_offset, off2=nxt.weight_offset)):
            return out
        self.add_normed(step, branch, residual)
        return nxt.forward(step, residual, out=out)

    def forward_rows(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """The norm of float32 rows that may be a column slice of a wider matrix, into rows that may be one too."""
        kernels.rmsnorm_rows(x, self.weight, out, self.eps, weight_offset=self.weight_offset)
        return out


class CastRows(Part):
    """No norm at all: the rows of the float32 residual in the step's storage type.  It stands where an arrangement
    whose sublayers read the residual stream itself has no norm before a sublayer; it owns no tensor."""
    fusable = False

    def __init__(self, spec: Optional[NormSpec], dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.eps = 0.0

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("elementwise",)

    def forward(self, step, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                name: str = "cast_out") -> torch.Tensor:
        if rows is not None:
            raise ValueError("cast: a choice of rows is not supported")
        if out is None:
            if self.dtype == torch.float32:
                return x
            out = step.ws.buf(name, tuple(x.shape), self.dtype)
        kernels.convert(x, out)
        return out


register_norm("rmsnorm", RMSNorm)
register_norm("cast", CastRows)
