"""Retention: linear attention with a fixed decay per head, without softmax and without a denominator.

Per head, with S [dim, vdim] (key channel x value channel) carried from token to token in float32:

    S_t = decay_h S_{t-1} + k_t v_t^T,      o_t = S_t^T q_t

q and k (``heads`` heads of ``dim``) are projections of the mixer's input, rotated by the token's position over their first
rotary elements (element i with i + rotary_dim/2; ``position`` None: no rotation); k is multiplied by dim^-1/2 after the
rotation; v (``heads`` heads of ``vdim``) is used as projected.  Every head's o_t is divided by its root mean square over
vdim (no weight), the heads are concatenated and multiplied by an activation of a gate projection (SiLU), then projected.
The decays are constants of the configuration, one per head.

Kept per request: the state [heads, dim, vdim], float32 in both precisions.  One product gives q | k | v | g in float32; the
recurrence runs on the kernels the delta rule uses (csrc/kernels/gated_delta.cu: prepare, walk, finish) with the write
u_t = v_t instead of the delta rule's correction.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .base import Mixer, Part, StateCacheSpec, TensorGetter
from .linear import ACCUM, STORE_F32, Linear
from .rope import PositionEncoding


class Retention(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, decay: Sequence[float], prefix: str, eps: float,
                 position: Optional[PositionEncoding] = None, gate: str = "silu", out_scale: float = 1.0):
        """Tensors ``prefix.q``, ``.k``, ``.v``, ``.g``, ``.o``.  ``decay``: one number per head."""
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"gate '{gate}' (silu, sigmoid)")
        self.hidden, self.heads, self.dim, self.vdim = hidden, heads, dim, vdim
        self.decay = [float(g) for g in decay]
        self.prefix, self.eps, self.position, self.gate, self.out_scale = prefix, float(eps), position, gate, float(out_scale)
        p = prefix
        self.inp = Linear(hidden, [heads * dim, heads * dim, heads * vdim, heads * vdim], [f"{p}.{t}" for t in ("q", "k", "v", "g")],
                          pad_rows_to=4)
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"])
        self.decay_dev: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.inp, self.o]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=device)
        if self.position is not None and self.position.cos is None:
            self.position.prepare(device)

    def cache_spec(self):
        return StateCacheSpec((self.heads, self.dim, self.vdim), torch.float32)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        H, d, dv = self.heads, self.dim, self.vdim
        prep = 2 * H * d + H * dv + H * d + H + 3
        return tokens * ((self.inp.padded_out + prep + H * dv) * 4 + H * dv * element_size)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, d, dv = self.heads, self.dim, self.vdim
        proj = ctx.buffer((T, self.inp.padded_out), torch.float32)
        self.inp.forward(h, proj, STORE_F32)
        off_g = 2 * H * d + H * dv
        gz = proj[:, off_g:off_g + H * dv]
        pos = self.position
        cos = pos.cos if pos is not None else None
        if cos is not None and ctx.max_position >= cos.shape[0]:
            raise ValueError(f"position {ctx.max_position} is beyond the rotary table ({cos.shape[0]}): raise max_seq_len")
        rotation = (cos, pos.sin if pos is not None else None, pos.rotary_dim if cos is not None else 0, ctx.positions, ctx.status)
        prep = ctx.buffer((T, ops.gated_delta_prep_width(H, H, d, dv)), torch.float32)
        raw = ctx.buffer((T, H * dv), torch.float32)
        out = ctx.buffer((T, H * dv))
        prof = ops.profiling()
        if prof is not None:
            prof.note_work(T * (3 * H * d + 2 * H * dv + H) * 4 + 2 * ctx.B * H * d * dv * 4, 4 * T * H * d * dv)
        ops.gated_delta(proj, None, gz, None, self.decay_dev, None, None, prep, raw, cache.state, None, out,
                        ctx.seq_of_token, ctx.seq_slot, ctx.q_start, ctx.B, 0, 0, H, H, d, dv, 1, self.eps,
                        decay=ops.DECAY_CONSTANT, gate=ops.GATE_SILU if self.gate == "silu" else ops.GATE_SIGMOID, delta=False,
                        out_scale=self.out_scale, rotation=rotation)
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
