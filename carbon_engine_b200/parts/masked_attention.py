"""Grouped-query softmax attention over the paged cache without rotation, with separate key and value head sizes and
these options, each a parameter: a tanh cap on the scores (``softcap * tanh(score / softcap)``), a sliding window
that may keep the sequence's first ``keep_first`` tokens visible for every later query, a sigmoid gate on the
concatenated heads computed from the mixer's input, and a blend of the layer's values with the values that another
layer computed for the same tokens earlier in the step (``v <- (1 - lam) v + lam v_first``; the blended values are
what the cache holds).

One product gives q | k | v | gate logits.  A layer whose window keeps first tokens holds all its pages (the kept
tokens must stay readable); a plain window gives pages back as it moves on.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from .base import Mixer, PagedCacheSpec, Part, TensorGetter, TensorSpec, register_init_kind
from .linear import ACCUM, STORE, STORE_F32, Linear

register_init_kind("blend", 0.3, 0.1, True)


class MaskedAttentionPlan:
    def __init__(self, tiles, n_tiles):
        self.tiles, self.n_tiles = tiles, n_tiles
        self.graph_key = None            # a decode step of B sequences is always B tiles


def plan_query_tiles(ctx, section: str, tile: int) -> MaskedAttentionPlan:
    """The step's tiles of up to ``tile`` query tokens as (sequence, first token) pairs, of every sequence (a
    one-token sequence is a tile of one row)."""
    tiles = ctx.bufs.host_section(section)
    n = 0
    for b in range(ctx.B):
        for q0 in range(0, ctx.h_q_start[b + 1] - ctx.h_q_start[b], tile):
            tiles[2 * n], tiles[2 * n + 1] = b, q0
            n += 1
    return MaskedAttentionPlan(ctx.bufs.dev_section(section), n)


def attend(ctx, plan, q, q_head, cache, ldk, ldv, v_pool, gate, out, table, nh, nkv, d, dv, window, keep_first, scale, softcap,
           sinks=None, out_scale=1.0):
    """The attention of both mixers of this family: the tensor-core kernel where it takes the sizes (bfloat16), else
    the float32-arithmetic kernel.  ``sinks`` (float32 [nh] or None): a learned number per head whose exponential joins
    the softmax's denominator without a key or a value.  ``out_scale`` multiplies what is stored."""
    prof = ops.profiling()
    if prof is not None:
        el, keys, pairs = q.element_size(), 0, 0
        for b in range(ctx.B):
            n, before = ctx.h_q_start[b + 1] - ctx.h_q_start[b], ctx.h_ctx_before[b]
            for p in range(before, before + n):
                seen = p + 1 if window <= 0 else min(p + 1, window) + max(0, min(keep_first, p - window + 1))
                pairs += seen
            keys += (before + n) if window <= 0 else min(before + n, window + n + keep_first)
        prof.note_work((keys * nkv * (d + (dv if v_pool is not cache.k_pool else 0)) + ctx.T * nh * (d + dv)) * el,
                       2 * pairs * nh * (d + dv))
    if q.dtype == torch.bfloat16 and ctx.fast_attention and plan is not None and \
            ops.masked_attention_mma_supported(d, dv, q.stride(0), q_head, ldk, ldv, v_pool is cache.k_pool):
        ops.masked_attention_mma(q, q_head, cache.k_pool, v_pool, ldk, ldv, gate, out, ctx.positions, ctx.seq_slot, ctx.q_start,
                                 table, plan.tiles, plan.n_tiles, ctx.status, nh, nkv, d, dv, cache.page_size, window, keep_first,
                                 scale, softcap, sinks, out_scale)
        return
    ops.masked_attention(q, q_head, cache.k_pool, v_pool, ldk, ldv, gate, out, ctx.positions, ctx.seq_of_token, ctx.seq_slot,
                         table, ctx.status, nh, nkv, d, dv, cache.page_size, window, keep_first, scale, softcap, sinks, out_scale)


class GatedWindowAttention(Mixer):
    graph_safe = True
    plan_key = "masked_attention"
    TILE = 64               # query tokens a block of the tensor-core kernel takes

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, prefix: str, scale: Optional[float] = None,
                 softcap: float = 0.0, window: int = 0, keep_first: int = 0, gate: bool = True, value_mix: Optional[str] = None,
                 mix_key: str = "values", page_size: Optional[int] = None):
        """``value_mix``: None, "source" (this layer's values are kept for the later layers of the step) or "blend"
        (its values are blended with the source layer's; ``prefix.vmix`` is the blend's weight).  Tensors ``prefix.q``,
        ``.k``, ``.v``, ``.g`` (with ``gate``), ``.o`` and, with ``value_mix``, ``.vmix``."""
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix '{value_mix}' (source, blend or None)")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = hidden, heads, kv_heads, dim, vdim
        self.prefix, self.softcap, self.window, self.keep_first = prefix, float(softcap or 0.0), int(window), int(keep_first)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(dim)
        self.gate, self.value_mix, self.mix_key, self.page_size = bool(gate), value_mix, mix_key, page_size
        p = prefix
        sizes, names = [heads * dim, kv_heads * dim, kv_heads * vdim], [f"{p}.q", f"{p}.k", f"{p}.v"]
        if gate:
            sizes.append(heads * vdim); names.append(f"{p}.g")
        self.qkvg = Linear(hidden, sizes, names, pad_rows_to=8)         # the row stride keeps 16-byte alignment
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"])
        self.lam = 0.0

    def children(self) -> List[Part]:
        return [self.qkvg, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.prefix}.vmix", (), "blend")] if self.value_mix else []

    def load(self, get: TensorGetter, device, dtype) -> None:
        if self.value_mix == "blend":
            self.lam = float(get(f"{self.prefix}.vmix").to(torch.float32))

    def cache_spec(self) -> PagedCacheSpec:
        # kept first tokens stay readable only if no page is given back
        window = self.window if self.keep_first == 0 else 0
        return PagedCacheSpec(self.kv_heads, self.dim, window, self.page_size, v_heads=self.kv_heads, v_head_dim=self.vdim)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * (self.qkvg.padded_out + self.heads * self.vdim) * element_size

    def step_sections(self, max_tokens: int, max_seqs: int):
        return [("masked_attention.tiles", 2 * (max_seqs + max_tokens // self.TILE + 1))]

    def plan_step(self, ctx) -> MaskedAttentionPlan:
        return plan_query_tiles(ctx, "masked_attention.tiles", self.TILE)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        qkvg = ctx.buffer((T, self.qkvg.padded_out))
        self.qkvg.forward(h, qkvg, STORE)
        v_off = (H + G) * d
        if self.value_mix == "source":
            ctx.shared[self.mix_key] = (qkvg, v_off, G * dv)
        elif self.value_mix == "blend":
            first, first_off, n = ctx.shared[self.mix_key]
            if n != G * dv:
                raise ValueError(f"{self.prefix}: values of {G * dv} numbers cannot be blended with values of {n}")
            ops.value_mix(qkvg, v_off, n, first, first_off, self.lam)
        table = ctx.block_tables[cache.group]
        ops.bias_rope_kvwrite(qkvg, cache.k_pool, cache.v_pool, None, None, None, ctx.positions, ctx.seq_of_token, ctx.seq_slot,
                              table, ctx.status, H, G, G, d, dv, 0, cache.page_size, write_kv=cache.writes)
        gate = qkvg[:, v_off + G * dv:] if self.gate else None
        out = ctx.buffer((T, H * dv))
        attend(ctx, ctx.plans.get(self.plan_key), qkvg, d, cache, d, dv, cache.v_pool, gate, out, table, H, G, d, dv, self.window,
               self.keep_first, self.scale, self.softcap)
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
