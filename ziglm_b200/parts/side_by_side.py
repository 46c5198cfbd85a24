"""Several mixers side by side: all read the same rows and their outputs are summed.

``MixerSpec.options["parts"]`` lists (prefix, MixerSpec) pairs; a part's tensors are declared under its prefix, and a
factor on a part's output is that part's own option (it rides where the part rounds its heads before its output
projection, so the sum itself is plain).  At most one part may keep keys and values and at most one a state per
sequence: the place of the schedule owns one set of pages and one state tensor, which go to the part that asked.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, mixer_class, register_mixer


class SideBySide(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        parts = spec.options.get("parts")
        if not parts:
            raise ValueError("side_by_side: the spec must list the mixers that run side by side")
        self.parts: List[Tuple[str, Part]] = [(prefix, mixer_class(sub.kind)(sub, dtype, device)) for prefix, sub in parts]
        if sum(1 for _, p in self.parts if p.cache_needs() is not None) > 1:
            raise ValueError("side_by_side: only one of the mixers may keep keys and values")
        if sum(1 for _, p in self.parts if p.state_needs() is not None) > 1:
            raise ValueError("side_by_side: only one of the mixers may keep a state per sequence")

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        out: Dict[str, ParamDecl] = {}
        for prefix, sub in spec.options["parts"]:
            for name, decl in mixer_class(sub.kind).declare(sub).items():
                out[prefix + name] = decl
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self.parts:
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs: Tuple[str, ...] = ()
        for _, part in self.parts:
            libs += part.kernel_libraries()
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        for _, part in self.parts:
            need = part.cache_needs()
            if need is not None:
                return need
        return None

    def state_needs(self) -> Optional[StateNeed]:
        for _, part in self.parts:
            need = part.state_needs()
            if need is not None:
                return need
        return None

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        for i, (_, part) in enumerate(self.parts):
            if i == 0 and not accumulate:
                if part.can_overwrite:
                    part.forward(step, io, h, residual, accumulate=False)
                    continue
                residual.zero_()
            part.forward(step, io, h, residual)
        return None


register_mixer("side_by_side", SideBySide)
