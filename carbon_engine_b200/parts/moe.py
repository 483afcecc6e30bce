"""Mixture-of-experts feed-forward: a router picks ``top`` of ``experts`` small feed-forward layers for every token, and
their outputs are summed with the router's weights; a shared expert may run for every token beside them.

    z = W_router h (float32);  s = softmax(z) over all experts
    experts form ``groups`` equal groups of neighbours; a group's score is its largest s; only experts of the ``keep``
    best groups are eligible; the ``top`` eligible experts with the largest s are chosen
    weight_e = s_e / (sum of the chosen s + 1e-20) * scale
    y = sum_e weight_e W_down,e act(W_up,e h)  +  sigmoid(W_sg h) * W_down,s act(W_up,s h)        act = relu^2

The experts' matrices are held as two stacks [experts, ff, hidden] and [experts, hidden, ff].  A step's (token, expert)
pairs are laid out by expert on the device (every expert's rows start a tile), the two products run as grouped products
over that layout, and a last kernel sums each token's rows in the order of its picks.  Nothing of the routing reaches
the host, so a step of a given size launches the same grids whatever the router says (a decode step can be captured).
In bfloat16, with sizes the kernel takes, the products run on the tcgen05 grouped kernel of ``gemm_tc.cu`` (tiles of 16 rows
in steps of single tokens, of 64 or 128 rows in steps of many); it loads its rows by TMA, so the tokens' rows are first
copied into the layout's order.  Other sizes and float32 take the kernels of ``moe.cu``, which read the tokens' rows where
they lie.  The shared expert is two ordinary products.
The router's product also yields the shared expert's gate logit (its row is appended to the router's).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops, ops_tensor
from .base import FeedForward, Part, TensorGetter, TensorSpec, to_device
from .linear import RELU2, STORE, STORE_F32, Linear


class RoutedExperts(FeedForward):
    can_store = True
    #: pairs per expert up to which a step's layout uses tiles of 16 rows (steps of single tokens) instead of 64
    SMALL_TILE_MAX = 16

    def __init__(self, hidden: int, experts: int, top: int, ff: int, prefix: str, groups: int = 1, keep_groups: int = 1,
                 scale: float = 1.0, activation: str = "relu2", shared_ff: int = 0, shared_gate: bool = True):
        """Tensors ``prefix.router`` [experts, hidden], ``prefix.e<i>.up`` [ff, hidden], ``prefix.e<i>.down`` [hidden, ff] and,
        with ``shared_ff`` > 0, ``prefix.shared.up`` / ``.down`` and (with ``shared_gate``) ``prefix.shared.sg`` [1, hidden]."""
        if activation not in ops.MOE_ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(sorted(ops.MOE_ACTIVATIONS))})")
        if not 0 < top <= experts:
            raise ValueError(f"top {top} of {experts} experts")
        if groups <= 0 or experts % groups or not 0 < keep_groups <= groups or keep_groups * (experts // groups) < top:
            raise ValueError(f"{experts} experts in {groups} groups of which {keep_groups} are kept cannot give {top} experts")
        self.hidden, self.experts, self.top, self.ff, self.prefix = int(hidden), int(experts), int(top), int(ff), prefix
        self.groups, self.keep_groups, self.scale, self.activation = int(groups), int(keep_groups), float(scale), activation
        self.shared_ff, self.shared_gate = int(shared_ff), bool(shared_gate) and shared_ff > 0
        sizes, names = [experts], [f"{prefix}.router"]
        if self.shared_gate:
            sizes.append(1); names.append(f"{prefix}.shared.sg")
        self.router = Linear(hidden, sizes, names, pad_rows_to=4)
        self.up: Optional[torch.Tensor] = None            # [experts, ff, hidden]
        self.down: Optional[torch.Tensor] = None          # [experts, hidden, ff]
        # the shared expert is two ordinary products (the activation is the first one's epilogue)
        self.shared_up = Linear(hidden, [self.shared_ff], [f"{prefix}.shared.up"]) if self.shared_ff > 0 else None
        self.shared_down = Linear(self.shared_ff, [hidden], [f"{prefix}.shared.down"]) if self.shared_ff > 0 else None

    def children(self) -> List[Part]:
        return [c for c in (self.router, self.shared_up, self.shared_down) if c is not None]

    def tensor_specs(self) -> List[TensorSpec]:
        p = self.prefix
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(f"{p}.e{e}.up", (self.ff, self.hidden)), TensorSpec(f"{p}.e{e}.down", (self.hidden, self.ff))]
        return specs

    def load(self, get: TensorGetter, device, dtype) -> None:
        p = self.prefix
        self.up = torch.empty((self.experts, self.ff, self.hidden), dtype=dtype, device=device)
        self.down = torch.empty((self.experts, self.hidden, self.ff), dtype=dtype, device=device)
        for e in range(self.experts):
            self.up[e].copy_(to_device(get(f"{p}.e{e}.up"), device, dtype))
            self.down[e].copy_(to_device(get(f"{p}.e{e}.down"), device, dtype))

    def tile_for(self, tokens: int, dtype=None) -> int:
        """Rows of a tile of the layout: 16 for steps of single tokens; else 64, or 128 where the tensor-core product takes
        the sizes and the experts have rows enough to fill such tiles."""
        pairs = tokens * self.top
        if pairs <= self.SMALL_TILE_MAX * self.experts:
            return 16
        if pairs >= 128 * self.experts and self._fast(128, dtype):
            return 128
        return 64

    def _fast(self, tile: int, dtype) -> bool:
        return ops_tensor.grouped_bf16_supported(tile, self.ff, self.hidden, self.hidden, self.ff, dtype) and \
            ops_tensor.grouped_bf16_supported(tile, self.hidden, self.ff, self.ff, self.hidden, dtype)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        rows = max(ops.moe_max_tiles(tokens * self.top, self.experts, tile) * tile for tile in (16, 64, 128))
        return rows * (self.ff + 2 * self.hidden) * element_size + tokens * (self.shared_ff + self.hidden) * element_size \
            + tokens * (self.router.padded_out + 3 * self.top + 1) * 4 + rows * 4

    def _product(self, x, w, out, tile, activation, fast, row_token=None, tile_expert=None, n_tiles=None) -> None:
        if fast and row_token is None and ops_tensor.grouped_bf16(x, w, out, tile, ops.MOE_ACTIVATIONS[activation], tile_expert, n_tiles):
            return
        ops.moe_matmul(x, w, out, tile, activation, row_token, tile_expert, n_tiles)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, accumulate: bool = True) -> None:
        T, E, top = h.shape[0], self.experts, self.top
        i32 = lambda n: ctx.buffer((n,), torch.int32)
        z = ctx.buffer((T, self.router.padded_out), torch.float32)
        self.router.forward(h, z, STORE_F32)
        ids, weights = ctx.buffer((T, top), torch.int32), ctx.buffer((T, top), torch.float32)
        sgate = ctx.buffer((T,), torch.float32) if self.shared_gate else None
        ops.moe_route(z, E, top, self.groups, self.keep_groups, self.scale, ids, weights, sgate)
        tile = self.tile_for(T, h.dtype)
        fast = self._fast(tile, h.dtype)
        tiles = ops.moe_max_tiles(T * top, E, tile)
        row_token, pair_row, tile_expert, n_tiles = i32(tiles * tile), i32(T * top), i32(tiles), i32(1)
        ops.moe_align(ids, E, tile, row_token, pair_row, tile_expert, n_tiles)
        act = ctx.buffer((tiles * tile, self.ff))
        if fast:
            laid = ctx.buffer((tiles * tile, self.hidden))
            ops.moe_gather(h, row_token, n_tiles, tile, laid)
            self._product(laid, self.up, act, tile, self.activation, True, None, tile_expert, n_tiles)
        else:
            ops.moe_matmul(h, self.up, act, tile, self.activation, row_token, tile_expert, n_tiles)
        rows = ctx.buffer((tiles * tile, self.hidden))
        self._product(act, self.down, rows, tile, "none", fast, None, tile_expert, n_tiles)
        shared = None
        if self.shared_ff > 0:
            sact = ctx.buffer((T, self.shared_ff))
            self.shared_up.forward(h, sact, RELU2 if self.activation == "relu2" else STORE)
            shared = ctx.buffer((T, self.hidden))
            self.shared_down.forward(sact, shared, STORE)
        ops.moe_combine(rows, pair_row, weights, x, shared, sgate, accumulate)
