"""The gated delta rule: a recurrent mixer with a matrix state per head, with a decay per head and key channel
(:class:`ChannelGatedDelta`) or one decay per head (:class:`HeadGatedDelta`).

Per head, with S [dim, vdim] (key channel x value channel) carried from token to token in float32:

    S <- diag(g_t) S;    u_t = beta_t (v_t - S^T k_t);    S <- S + k_t u_t^T;    o_t = S^T q_t

q, k (``kv_heads`` heads of ``dim``) and v (``heads`` heads of ``vdim``) are projections of the mixer's input that pass
a short causal convolution over time per channel (``taps`` taps, zeros before the sequence's start) and SiLU; q and k
are then unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^-1/2; value head h reads query/key head
h // (heads / kv_heads).  beta_t = sigmoid(W_b h), one per head.  The decay, one per head and key channel:
g_t = exp(-exp(A_h) softplus(W_a2 (W_a1 h) + bias)).  Every head's o_t is divided by its root mean square over vdim,
multiplied by a weight of size vdim that the heads share and by sigmoid(W_g2 (W_g1 h)), then projected.

Kept per request: the state [heads, dim, vdim] and the convolution's last ``taps - 1`` inputs, both float32 in both
precisions.  One product gives q | k | v | beta | a1 | g1 in float32; the two narrow second products are ordinary
``Linear``s; then four kernels (csrc/kernels/gated_delta.cu): prepare, keep, walk, finish.

With one decay per head, g_t = exp(-exp(A_h) softplus(W_a h + bias_h)) multiplies every row of the head's state alike, and
the gate is an activation (SiLU or sigmoid) of a projection of full rank: one product gives q | k | v | beta | a | g.

``out_scale`` multiplies the heads' outputs before the output product (the mixer's weight where mixers are summed).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import BundleCacheSpec, Mixer, Part, StateCacheSpec, TensorGetter, TensorSpec, register_init_kind
from .linear import ACCUM, STORE_F32, Linear

register_init_kind("conv_taps", 0.0, 0.5, True)
register_init_kind("decay_log", 0.0, 0.5, True)
register_init_kind("narrow", 0.0, 0.3, False)


class ChannelGatedDelta(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, prefix: str, eps: float,
                 decay_rank: int = -1, gate_rank: int = -1, out_scale: float = 1.0):
        """``decay_rank`` / ``gate_rank``: widths of the two narrow projections; -1 takes them from the stored tensors."""
        self.out_scale = float(out_scale)
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} query/key heads")
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = hidden, heads, kv_heads, dim, vdim, int(taps)
        self.prefix, self.eps = prefix, float(eps)
        p = prefix
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.inp = Linear(hidden, [kv_heads * dim, kv_heads * dim, heads * vdim, heads, int(decay_rank), int(gate_rank)],
                          [f"{p}.{t}" for t in ("q", "k", "v", "b", "a1", "g1")], pad_rows_to=4)
        self.a2 = Linear(int(decay_rank), [heads * dim], [f"{p}.a2"], init="narrow")
        self.g2 = Linear(int(gate_rank), [heads * vdim], [f"{p}.g2"], init="narrow")
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"])
        self.conv_w: Optional[torch.Tensor] = None       # [channels, taps] float32: q, k, v rows
        self.a_log: Optional[torch.Tensor] = None
        self.dt_bias: Optional[torch.Tensor] = None
        self.norm_w: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.inp, self.a2, self.g2, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        p, G, H, d, dv, K = self.prefix, self.kv_heads, self.heads, self.dim, self.vdim, self.taps
        return [TensorSpec(f"{p}.q.conv", (G * d, K), "conv_taps"), TensorSpec(f"{p}.k.conv", (G * d, K), "conv_taps"),
                TensorSpec(f"{p}.v.conv", (H * dv, K), "conv_taps"), TensorSpec(f"{p}.A_log", (H,), "decay_log"),
                TensorSpec(f"{p}.dt_bias", (H * d,), "bias"), TensorSpec(f"{p}.norm", (dv,), "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        f32 = lambda name: get(f"{self.prefix}.{name}").to(device).to(torch.float32).contiguous()
        self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")
        self.a2.in_features = int(get(f"{self.prefix}.a2").shape[1])        # ranks given as -1 are the stored tensors'
        self.g2.in_features = int(get(f"{self.prefix}.g2").shape[1])

    def cache_spec(self):
        state = StateCacheSpec((self.heads, self.dim, self.vdim), torch.float32)
        if self.taps == 1:
            return state
        return BundleCacheSpec(state, (("conv", StateCacheSpec((self.taps - 1, self.channels), torch.float32)),))

    def step_bytes(self, tokens: int, element_size: int) -> int:
        H, d, dv = self.heads, self.dim, self.vdim
        prep = self.channels + H * d + H + 3
        return tokens * ((self.inp.padded_out + prep + H * d + 2 * H * dv) * 4 + (H * dv + 64) * element_size)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        proj = ctx.buffer((T, self.inp.padded_out), torch.float32)
        self.inp.forward(h, proj, STORE_F32)
        off_b = self.channels
        ra, rg = self.inp.out_features[4], self.inp.out_features[5]
        narrow = ctx.buffer((T, ra + rg))
        ops.copy_cols(proj, off_b + H, ra + rg, narrow)
        dec, gz = ctx.buffer((T, H * d), torch.float32), ctx.buffer((T, H * dv), torch.float32)
        self.a2.forward(narrow[:, :ra], dec, STORE_F32)
        self.g2.forward(narrow[:, ra:], gz, STORE_F32)
        prep = ctx.buffer((T, ops.gated_delta_prep_width(H, G, d, dv)), torch.float32)
        raw = ctx.buffer((T, H * dv), torch.float32)
        out = ctx.buffer((T, H * dv))
        prof = ops.profiling()
        if prof is not None:         # what the walk reads and writes once, the state of every sequence twice
            prof.note_work(T * (3 * H * d + 2 * H * dv + H) * 4 + 2 * ctx.B * H * d * dv * 4, 6 * T * H * d * dv)
        kept = cache.extra["conv"] if self.taps > 1 else None
        ops.gated_delta(proj, dec, gz, self.conv_w, self.a_log, self.dt_bias, self.norm_w, prep, raw, cache.state, kept, out,
                        ctx.seq_of_token, ctx.seq_slot, ctx.q_start, ctx.B, 0, off_b, H, G, d, dv, self.taps, self.eps,
                        out_scale=self.out_scale)
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)


class HeadGatedDelta(Mixer):
    """The gated delta rule with one decay per head and a gate of full rank.  Tensors ``prefix.q|k|v`` (+ ``.conv``), ``.b``,
    ``.a``, ``.A_log`` [heads], ``.dt_bias`` [heads], ``.g``, ``.norm`` [vdim], ``.o``."""
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, prefix: str, eps: float,
                 gate: str = "silu", out_scale: float = 1.0):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} query/key heads")
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"gate '{gate}' (silu, sigmoid)")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = hidden, heads, kv_heads, dim, vdim, int(taps)
        self.prefix, self.eps, self.gate, self.out_scale = prefix, float(eps), gate, float(out_scale)
        p = prefix
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.inp = Linear(hidden, [kv_heads * dim, kv_heads * dim, heads * vdim, heads, heads, heads * vdim],
                          [f"{p}.{t}" for t in ("q", "k", "v", "b", "a", "g")], pad_rows_to=4)
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"])
        self.conv_w: Optional[torch.Tensor] = None       # [channels, taps] float32: q, k, v rows
        self.a_log: Optional[torch.Tensor] = None
        self.dt_bias: Optional[torch.Tensor] = None
        self.norm_w: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.inp, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        p, G, H, d, dv, K = self.prefix, self.kv_heads, self.heads, self.dim, self.vdim, self.taps
        return [TensorSpec(f"{p}.q.conv", (G * d, K), "conv_taps"), TensorSpec(f"{p}.k.conv", (G * d, K), "conv_taps"),
                TensorSpec(f"{p}.v.conv", (H * dv, K), "conv_taps"), TensorSpec(f"{p}.A_log", (H,), "decay_log"),
                TensorSpec(f"{p}.dt_bias", (H,), "bias"), TensorSpec(f"{p}.norm", (dv,), "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        f32 = lambda name: get(f"{self.prefix}.{name}").to(device).to(torch.float32).contiguous()
        self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")

    def cache_spec(self):
        state = StateCacheSpec((self.heads, self.dim, self.vdim), torch.float32)
        if self.taps == 1:
            return state
        return BundleCacheSpec(state, (("conv", StateCacheSpec((self.taps - 1, self.channels), torch.float32)),))

    def step_bytes(self, tokens: int, element_size: int) -> int:
        H, d, dv = self.heads, self.dim, self.vdim
        prep = self.channels + H * d + H + 3
        return tokens * ((self.inp.padded_out + prep + H * dv) * 4 + H * dv * element_size)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        proj = ctx.buffer((T, self.inp.padded_out), torch.float32)
        self.inp.forward(h, proj, STORE_F32)
        off_b = self.channels
        dec, gz = proj[:, off_b + H:off_b + 2 * H], proj[:, off_b + 2 * H:off_b + 2 * H + H * dv]
        prep = ctx.buffer((T, ops.gated_delta_prep_width(H, G, d, dv)), torch.float32)
        raw = ctx.buffer((T, H * dv), torch.float32)
        out = ctx.buffer((T, H * dv))
        prof = ops.profiling()
        if prof is not None:
            prof.note_work(T * (3 * H * d + 2 * H * dv + H) * 4 + 2 * ctx.B * H * d * dv * 4, 6 * T * H * d * dv)
        kept = cache.extra["conv"] if self.taps > 1 else None
        ops.gated_delta(proj, dec, gz, self.conv_w, self.a_log, self.dt_bias, self.norm_w, prep, raw, cache.state, kept, out,
                        ctx.seq_of_token, ctx.seq_slot, ctx.q_start, ctx.B, 0, off_b, H, G, d, dv, self.taps, self.eps,
                        decay=ops.DECAY_PER_HEAD, gate=ops.GATE_SILU if self.gate == "silu" else ops.GATE_SIGMOID,
                        out_scale=self.out_scale)
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
