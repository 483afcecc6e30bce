"""Grouped-query softmax attention over the paged cache with a norm per head, a rotation, and these options, each a
parameter: values that are the keys as projected (no value projection), a temperature per head on the scores, and a sink
per head in the softmax's denominator.

Order of operations: one product gives q | k (| v) in float32; every head of q and k is divided by its root mean square and
multiplied by a weight of ``dim`` shared by the heads (``qk_norm``), then rotated over its first rotary elements (element i
with i + rotary_dim/2); score = <q, k> scale temp_h (``head_temperature``: a stored number per head, folded into the query);
the query at position i sees every key j <= i, or the last ``window`` of them; softmax whose denominator also holds
exp(sink_h) (``sink``: a stored number per head that has no key and no value and is neither scaled nor multiplied by the
temperature); the heads' weighted sums of the values; the output product.  With ``tied_values`` the values are the key
projection's output itself, before the norm and the rotation, so the value size is ``dim`` and there is no ``.v`` tensor.

Where values and keys have one size, bfloat16 steps run the kernels of :class:`carbon_engine_b200.parts.attention.PagedAttention`
(the split-KV decode kernel fed by TMA and the tcgen05 flash kernel, which take the sink and the output's factor at the point
where a row's sums are inverted); float32 steps, other head sizes and values of another size run the masked-attention family's
kernels (``parts/masked_attention.py:attend``).  ``out_scale`` multiplies the heads' outputs before the output product (the
mixer's weight where mixers are summed).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from .base import Mixer, PagedCacheSpec, Part, TensorGetter, TensorSpec, register_init_kind
from .linear import ACCUM, STORE_F32, Linear
from .attention import PagedAttention
from .masked_attention import attend, plan_query_tiles
from .rope import PositionEncoding

register_init_kind("sink", 0.0, 1.0, True)
register_init_kind("temperature", 1.0, 0.2, True)


class SinkAttention(Mixer):
    graph_safe = True
    can_store = True
    TILE, TILE_TC = PagedAttention.TILE, PagedAttention.TILE_TC       # tokens per tile of the flash kernels

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, prefix: str, eps: float, vdim: Optional[int] = None,
                 position: Optional[PositionEncoding] = None, scale: Optional[float] = None, window: int = 0, qk_norm: bool = True,
                 tied_values: bool = False, head_temperature: bool = False, sink: bool = False, out_scale: float = 1.0,
                 page_size: Optional[int] = None):
        """Tensors ``prefix.q``, ``.k``, ``.v`` (unless ``tied_values``), ``.q.norm`` and ``.k.norm`` [dim] (with ``qk_norm``),
        ``.temp`` [heads] (with ``head_temperature``), ``.sink`` [heads] (with ``sink``), ``.o``."""
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        vdim = dim if vdim is None else int(vdim)
        if tied_values and vdim != dim:
            raise ValueError(f"values that are the projected keys have the keys' size {dim}, not {vdim}")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = hidden, heads, kv_heads, dim, vdim
        self.prefix, self.eps, self.position, self.window = prefix, float(eps), position, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(dim)
        self.qk_norm, self.tied_values, self.head_temperature, self.sink = bool(qk_norm), bool(tied_values), bool(head_temperature), bool(sink)
        self.out_scale, self.page_size = float(out_scale), page_size
        # values of the keys' size: the step is planned for, and runs on, the paged attention's kernels
        self.plan_key = PagedAttention.plan_key if vdim == dim else "masked_attention"
        p = prefix
        sizes, names = [heads * dim, kv_heads * dim], [f"{p}.q", f"{p}.k"]
        if not tied_values:
            sizes.append(kv_heads * vdim); names.append(f"{p}.v")
        self.qkv = Linear(hidden, sizes, names, pad_rows_to=4)
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"])
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.temp: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.qkv, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        p, specs = self.prefix, []
        if self.qk_norm:
            specs += [TensorSpec(f"{p}.q.norm", (self.dim,), "norm"), TensorSpec(f"{p}.k.norm", (self.dim,), "norm")]
        if self.head_temperature:
            specs.append(TensorSpec(f"{p}.temp", (self.heads,), "temperature"))
        if self.sink:
            specs.append(TensorSpec(f"{p}.sink", (self.heads,), "sink"))
        return specs

    def load(self, get: TensorGetter, device, dtype) -> None:
        f32 = lambda name: get(f"{self.prefix}.{name}").to(device).to(torch.float32).contiguous()
        if self.qk_norm:
            self.q_norm_w, self.k_norm_w = f32("q.norm"), f32("k.norm")
        self.temp = f32("temp") if self.head_temperature else None
        self.sinks = f32("sink") if self.sink else None
        if self.position is not None and self.position.cos is None:
            self.position.prepare(device)

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(self.kv_heads, self.dim, self.window, self.page_size, v_heads=self.kv_heads, v_head_dim=self.vdim)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * (self.qkv.padded_out * 4 + self.heads * (self.dim + self.vdim) * element_size)

    def step_sections(self, max_tokens: int, max_seqs: int):
        if self.plan_key == PagedAttention.plan_key:
            return PagedAttention.step_sections(self, max_tokens, max_seqs)
        return [("masked_attention.tiles", 2 * (max_seqs + max_tokens // 64 + 1))]

    def plan_step(self, ctx):
        if self.plan_key == PagedAttention.plan_key:
            return PagedAttention.plan_step(self, ctx)
        return plan_query_tiles(ctx, "masked_attention.tiles", 64)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        proj = ctx.buffer((T, self.qkv.padded_out), torch.float32)
        self.qkv.forward(h, proj, STORE_F32)
        pos = self.position
        cos = pos.cos if pos is not None else None
        if cos is not None and ctx.max_position >= cos.shape[0]:
            raise ValueError(f"position {ctx.max_position} is beyond the rotary table ({cos.shape[0]}): raise max_seq_len")
        table = ctx.block_tables[cache.group]
        q = ctx.buffer((T, H * d))
        off_k = H * d
        off_v = off_k if self.tied_values else off_k + G * d
        ops.norm_rope_kvwrite(proj, q, cache.k_pool, cache.v_pool, self.q_norm_w, self.k_norm_w, self.temp, cos,
                              pos.sin if pos is not None else None, ctx.positions, ctx.seq_of_token, ctx.seq_slot, table, ctx.status,
                              0, off_k, off_v, H, G, d, dv, pos.rotary_dim if cos is not None else 0, cache.page_size, self.eps,
                              write_kv=cache.writes)
        out = ctx.buffer((T, H * dv))
        plan = ctx.plans.get(self.plan_key)
        fast = self.plan_key == PagedAttention.plan_key
        if fast and q.dtype == torch.bfloat16 and ctx.fast_attention and plan is not None:
            from .. import ops_tensor
            prof = ops.profiling()
            if prof is not None:         # keys and values of every sequence once, queries and outputs; causal flops
                keys = pairs = 0
                for b in range(ctx.B):
                    n, before = ctx.h_q_start[b + 1] - ctx.h_q_start[b], ctx.h_ctx_before[b]
                    keys += before + n
                    pairs += n * before + n * (n + 1) // 2
                prof.note_work((2 * keys * G * d + 2 * ctx.T * H * d) * 2, 4 * pairs * H * d)
            if ops_tensor.attention_bf16(ctx, plan, q, out, cache, table, H, G, d, self.window, self.scale, sinks=self.sinks,
                                         out_scale=self.out_scale):
                self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
                return
        attend(ctx, None if fast else plan, q, d, cache, d, dv, cache.v_pool, None, out, table, H, G, d, dv, self.window, 0,
               self.scale, 0.0, sinks=self.sinks, out_scale=self.out_scale)
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
