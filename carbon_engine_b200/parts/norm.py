"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * weight, the weight used as stored (no "+1")
(src/model/layers.rs:117-146), or, with ``unit_offset``, stored as the deviation from 1 and used as 1 + weight.  The weight is
held in float32 whatever it was stored in; the sum of squares and the scaling are float32.  ``add_into`` is the norm
of a sublayer's OUTPUT added into the residual (designs that normalise what a sublayer returns, not what it reads).

:class:`GroupedRMSNorm` takes the norm in equal consecutive parts of the width, each part divided by its
own root mean square, and can read a residual kept as several streams: the weighted (or plain) sum of the
streams is formed, normalised and scaled in one kernel."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Norm, TensorGetter, TensorSpec, register_init_kind


register_init_kind("norm_offset", 0.0, 0.1, True)


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, name: str, unit_offset: bool = False):
        """``unit_offset``: the stored weight is the deviation from 1; 1 + weight is formed once, at load, in float32."""
        self.width, self.eps, self.name, self.unit_offset = int(width), float(eps), name, bool(unit_offset)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), "norm_offset" if self.unit_offset else "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        w = get(self.name).to(device).to(torch.float32)
        self.weight = (w + 1.0 if self.unit_offset else w).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, out, self.eps, rows)

    def add_into(self, y: torch.Tensor, x: torch.Tensor, rounded: Optional[torch.Tensor] = None) -> None:
        """x += norm(y); both float32 [T, width].  ``rounded`` (bfloat16) receives the new x rounded."""
        ops.rmsnorm_add(y, self.weight, x, self.eps, rounded)


class GroupedRMSNorm(Norm):
    """y = w * concat_g(part_g / sqrt(mean(part_g^2) + eps)) over ``groups`` equal parts of the width.  ``x`` may
    be [T, width] or [T, streams, width]; with streams, ``coef`` [streams] weights their sum (None: plain sum)."""

    def __init__(self, width: int, eps: float, name: str, groups: int = 1):
        if groups <= 0 or width % groups:
            raise ValueError(f"a width of {width} cannot be normalised in {groups} equal parts")
        self.width, self.eps, self.name, self.groups = int(width), float(eps), name, int(groups)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.weight = get(self.name).to(device).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                coef: Optional[torch.Tensor] = None) -> None:
        ops.streams_norm(x, self.weight, out, self.eps, self.groups, coef, rows)


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations; weight and bias in float32."""

    def __init__(self, width: int, eps: float, name: str, bias_name: Optional[str] = None):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.bias_name = bias_name or f"{name}.b"
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), "norm"), TensorSpec(self.bias_name, (self.width,), "bias")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.weight = get(self.name).to(device).to(torch.float32).contiguous()
        self.bias = get(self.bias_name).to(device).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        ops.layernorm(x, self.weight, self.bias, out, self.eps, rows)
