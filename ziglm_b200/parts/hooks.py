"""Small parts that run once per step outside the layers, or between two places of the schedule.

``add_row``   x[t, :] += table[row, :] for every token of the step: a learned vector added to the residual
              stream at a fixed place (the start of a pass through a repeated run of layers).  Options:
              ``rows`` and ``width`` (the table's shape), ``row``.
``scale``     logits *= factor.  Option: ``factor``.
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


register_hook("add_row", AddRow)
register_hook("scale", Scale)
