"""Gated feed-forward: down(act(gate(h)) * up(h)), added into the residual stream
(src/model/layers.rs:568, 625-648; src/model/mod.rs:649).  The activation is SiLU or ReLU; the gate and up
weights are held as one matrix so that one product with a gated epilogue serves both.
Dense feed-forward without a gate: down(act(up(h))), act the square of ReLU, the up product's epilogue."""
from __future__ import annotations

from typing import List, Sequence

import torch

from .base import FeedForward, Part
from .linear import ACCUM, RELU2, RELUGLU, STORE_F32, SWIGLU, Linear

_EPILOGUES = {"silu": SWIGLU, "relu": RELUGLU}


class GatedMLP(FeedForward):
    can_store = True

    def __init__(self, hidden: int, intermediate: int, prefix: str, activation: str = "silu",
                 names: Sequence[str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        """``names``: the gate, up and down tensors' names under ``prefix``."""
        if activation not in _EPILOGUES:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(sorted(_EPILOGUES))})")
        self.epilogue = _EPILOGUES[activation]
        self.hidden, self.intermediate, self.prefix = hidden, intermediate, prefix
        gate, up, down = names
        self.gate_up = Linear(hidden, [intermediate, intermediate], [f"{prefix}.{gate}", f"{prefix}.{up}"])
        self.down = Linear(intermediate, [hidden], [f"{prefix}.{down}"])

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * self.intermediate * element_size

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, accumulate: bool = True) -> None:
        act = ctx.buffer((h.shape[0], self.intermediate))
        self.gate_up.forward(h, act, self.epilogue)
        self.down.forward(act, x, ACCUM if accumulate else STORE_F32)


class DenseMLP(FeedForward):
    """down(act(up(h))) with act = relu(z)^2 (``activation`` "relu2")."""
    can_store = True
    _ACTS = {"relu2": RELU2}

    def __init__(self, hidden: int, intermediate: int, prefix: str, activation: str = "relu2", names: Sequence[str] = ("up", "down")):
        if activation not in self._ACTS:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(sorted(self._ACTS))})")
        self.epilogue = self._ACTS[activation]
        self.hidden, self.intermediate, self.prefix = hidden, intermediate, prefix
        up, down = names
        self.up = Linear(hidden, [intermediate], [f"{prefix}.{up}"])
        self.down = Linear(intermediate, [hidden], [f"{prefix}.{down}"])

    def children(self) -> List[Part]:
        return [self.up, self.down]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * self.intermediate * element_size

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, accumulate: bool = True) -> None:
        act = ctx.buffer((h.shape[0], self.intermediate))
        self.up.forward(h, act, self.epilogue)
        self.down.forward(act, x, ACCUM if accumulate else STORE_F32)
