"""Small parts that run once per step outside the layers, or between two places of the schedule.

``add_row``   x[t, :] += table[row, :] for every token of the step: a learned vector added to the residual
              stream at a fixed place (the start of a pass through a repeated run of layers).  Options:
              ``rows`` and ``width`` (the table's shape), ``row``.
``scale``     logits *= factor.  Option: ``factor``.
``rmsnorm``   x <- x / sqrt(mean(x^2) + eps) * (w + offset) over every row, in place and in float32: a norm of the
              embedded tokens before the first layer.  Options: ``width``, ``eps``, ``unit_offset`` (the stored weight
              is the gain minus one).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import HookSpec
from .base import ParamDecl, Part, register_hook


class AddRow(Part):
    def __init__(self, spec: HookSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.row_index = int(spec.options["row"])
        if not 0 <= self.row_index < int(spec.options["rows"]):
            raise ValueError(f"add_row: row {self.row_index} is outside the table of {spec.options['rows']} rows")
        self.row: Optional[torch.Tensor] = None

    @classmethod
    def declare(cls, spec: HookSpec) -> Dict[str, ParamDecl]:
        return {"table": ParamDecl((int(spec.options["rows"]), int(spec.options["width"])))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.row = tensors["table"][self.row_index].contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("elementwise",)

    def forward(self, step, x: torch.Tensor) -> None:
        kernels.add_row(x, self.row)


class Scale(Part):
    def __init__(self, spec: HookSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.factor = float(spec.options["factor"])

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("elementwise",)

    def forward(self, step, x: torch.Tensor) -> None:
        kernels.scale_(x, self.factor)


class NormRows(Part):
    def __init__(self, spec: HookSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.width = int(spec.options["width"])
        self.eps = float(spec.options["eps"])
        self.weight_offset = 1.0 if spec.options.get("unit_offset") else 0.0
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def declare(cls, spec: HookSpec) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((int(spec.options["width"]),), init="zeros" if spec.options.get("unit_offset") else "ones")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("elementwise",)

    def forward(self, step, x: torch.Tensor) -> None:
        if x.shape[-1] != self.width:
            raise ValueError(f"rmsnorm hook: rows of {x.shape[-1]} elements, the norm is over {self.width}")
        # every element is read and written by the same thread, after the row's sum is known: in place is safe
        kernels.rmsnorm_rows(x, self.weight, x, self.eps, weight_offset=self.weight_offset)


register_hook("add_row", AddRow)
register_hook("rmsnorm", NormRows)
register_hook("scale", Scale)
