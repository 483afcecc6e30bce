"""Latent attention: queries, keys and values go through low-rank latents, and the cache holds ONE row per token,
[latent c (kv_rank) | rotated key part (rot_dim)], whatever the number of heads.

    c_q = rms_norm(W_dq h) * w_q;      q = W_uq c_q, head by head [dim unrotated | rot_dim rotated]
    W_dkv h = [kv_rank | rot_dim]:     c = rms_norm(first part) * w_kv;   the second part is a key part all heads share
    per head: key = [W_uk c | rotated part], value = W_uv c;  score = <q, key> * scale;  causal, optionally a window
    output = W_o (concatenated heads * sigmoid(W_g h))

Options, each a parameter: queries without a latent (``q_rank`` 0: q = W_q h); a learned number per head whose
exponential joins the softmax's denominator without a key or a value (``sink``); the gate as one number per head
instead of one per output element (``gate="head"``); a layer without a down-projection of its own that reads the rows
another layer cached (``own_kv=False``: the model's schedule gives it that layer's cache, read-only).

The rotation turns the first ``rotary_dim`` elements of the rotated parts in half pairs.  The keys and values of a
head are never formed: with W_uk moved to the query side, <q_plain, W_uk c> = <W_uk^T q_plain, c>, so every head
attends over the cached rows themselves with a query of size kv_rank + rot_dim, the weighted sum of the rows' latent
parts comes out (size kv_rank), and W_uv is applied to that sum.  The two per-head products are one kernel each.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from .base import Mixer, PagedCacheSpec, Part, TensorGetter, TensorSpec, register_init_kind, to_device
from .linear import ACCUM, STORE, STORE_F32, Linear
from .masked_attention import attend, plan_query_tiles
from .rope import PositionEncoding

register_init_kind("sink", 0.0, 1.0, True)


class LatentAttention(Mixer):
    graph_safe = True
    can_store = True
    plan_key = "masked_attention"            # the same tiles as the other mixer of the family
    TILE = 64

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, prefix: str,
                 eps: float, position: Optional[PositionEncoding] = None, scale: Optional[float] = None, window: int = 0,
                 gate=True, page_size: Optional[int] = None, sink: bool = False, own_kv: bool = True):
        """``gate``: False / None, True or "element" (sigmoid(W_g h) per output element, W_g [heads * vdim, hidden]) or "head"
        (one per head, W_g [heads, hidden]).  Tensors under ``prefix``: ``dq``, ``dq.norm``, ``uq`` (or ``q`` with ``q_rank`` 0),
        ``dkv``, ``dkv.norm`` (with ``own_kv``), ``uk``, ``uv``, ``g``, ``sink`` [heads], ``o``."""
        gate = "element" if gate is True else (gate or None)
        if gate not in (None, "element", "head"):
            raise ValueError(f"gate '{gate}' (element, head or None)")
        self.hidden, self.heads, self.dim, self.rot_dim, self.vdim = hidden, heads, dim, rot_dim, vdim
        self.q_rank, self.kv_rank, self.prefix, self.eps, self.position = int(q_rank), kv_rank, prefix, float(eps), position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(dim + rot_dim)
        self.window, self.gate, self.page_size = int(window), gate, page_size
        self.sink, self.own_kv = bool(sink), bool(own_kv)
        p = prefix
        # one product into float32 for what a norm or a sigmoid reads next: query latent | key/value row | gate logits
        sizes, names = [], []
        if self.q_rank > 0:
            sizes.append(self.q_rank); names.append(f"{p}.dq")
        if self.own_kv:
            sizes.append(kv_rank + rot_dim); names.append(f"{p}.dkv")
        self.gate_off = sum(sizes)
        if gate:
            sizes.append(heads * vdim if gate == "element" else heads); names.append(f"{p}.g")
        self.inp = Linear(hidden, sizes, names, pad_rows_to=4) if sizes else None
        q_size = heads * (dim + rot_dim)
        self.uq = Linear(self.q_rank, [q_size], [f"{p}.uq"]) if self.q_rank > 0 else Linear(hidden, [q_size], [f"{p}.q"])
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"])
        self.wq: Optional[torch.Tensor] = None
        self.wkv: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None        # float32 [heads]
        self.uk_t: Optional[torch.Tensor] = None         # [heads, kv_rank, dim]: W_uk of every head, transposed
        self.uv: Optional[torch.Tensor] = None           # [heads, vdim, kv_rank]

    def children(self) -> List[Part]:
        return [c for c in (self.inp, self.uq, self.o) if c is not None]

    def tensor_specs(self) -> List[TensorSpec]:
        p = self.prefix
        specs = [TensorSpec(f"{p}.uk", (self.heads * self.dim, self.kv_rank)), TensorSpec(f"{p}.uv", (self.heads * self.vdim, self.kv_rank))]
        if self.q_rank > 0:
            specs.append(TensorSpec(f"{p}.dq.norm", (self.q_rank,), "norm"))
        if self.own_kv:
            specs.append(TensorSpec(f"{p}.dkv.norm", (self.kv_rank,), "norm"))
        if self.sink:
            specs.append(TensorSpec(f"{p}.sink", (self.heads,), "sink"))
        return specs

    def load(self, get: TensorGetter, device, dtype) -> None:
        p = self.prefix
        f32 = lambda name: get(name).to(device).to(torch.float32).contiguous()
        self.wq = f32(f"{p}.dq.norm") if self.q_rank > 0 else None
        self.wkv = f32(f"{p}.dkv.norm") if self.own_kv else None
        self.sinks = f32(f"{p}.sink") if self.sink else None
        uk = to_device(get(f"{p}.uk"), device, dtype)
        self.uk_t = uk.view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = to_device(get(f"{p}.uv"), device, dtype).view(self.heads, self.vdim, self.kv_rank)
        if self.position is not None and self.position.cos is None:
            self.position.prepare(device)

    def cache_spec(self) -> PagedCacheSpec:
        # one key head of kv_rank + rot_dim per token and no value pool: the values are the rows' leading part
        return PagedCacheSpec(1, self.kv_rank + self.rot_dim, self.window, self.page_size, v_heads=1, v_head_dim=0)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        H, row = self.heads, self.kv_rank + self.rot_dim
        proj = self.inp.padded_out * 4 if self.inp is not None else 0
        return tokens * (proj + (self.q_rank + H * (self.dim + self.rot_dim) + H * row + H * self.kv_rank
                                 + H * self.vdim) * element_size)

    def step_sections(self, max_tokens: int, max_seqs: int):
        return [("masked_attention.tiles", 2 * (max_seqs + max_tokens // self.TILE + 1))]

    def plan_step(self, ctx):
        return plan_query_tiles(ctx, "masked_attention.tiles", self.TILE)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, d, dr, dv, r, qr = self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank, self.q_rank
        row = r + dr
        pos = self.position
        cos = pos.cos if pos is not None else None
        sin = pos.sin if pos is not None else None
        rd = pos.rotary_dim if cos is not None else 0
        if cos is not None and ctx.max_position >= cos.shape[0]:
            raise ValueError(f"position {ctx.max_position} is beyond the rotary table ({cos.shape[0]}): raise max_seq_len")
        if cache.writes and not self.own_kv:
            raise ValueError(f"{self.prefix}: a layer without a down-projection of its own can only read another layer's cache")
        writes = cache.writes and self.own_kv
        proj = None
        if self.inp is not None:
            proj = ctx.buffer((T, self.inp.padded_out), torch.float32)
            self.inp.forward(h, proj, STORE_F32)
        table = ctx.block_tables[cache.group]
        cq = ctx.buffer((T, qr)) if qr > 0 else None
        if qr > 0 or writes:
            ops.latent_prepare(proj, self.wq, self.wkv, cq, cache.k_pool, cos, sin, ctx.positions, ctx.seq_of_token, ctx.seq_slot,
                               table, ctx.status, 0, qr, qr, r, dr, rd, cache.page_size, self.eps, write_kv=writes)
        q = ctx.buffer((T, H * (d + dr)))
        self.uq.forward(cq if qr > 0 else h, q, STORE)
        qa = ctx.buffer((T, H * row))
        ops.head_matmul(q, d + dr, self.uk_t, qa, row, H, r, d)
        ops.rope_part(q, d + dr, d, qa, row, r, cos, sin, ctx.positions, ctx.status, H, dr, rd)
        lat = ctx.buffer((T, H * r))
        attend(ctx, ctx.plans.get(self.plan_key), qa, row, cache, row, row, cache.k_pool, None, lat, table, H, 1, row, r,
               self.window, 0, self.scale, 0.0, self.sinks)
        out = ctx.buffer((T, H * dv))
        ops.head_matmul(lat, r, self.uv, out, dv, H, dv, r, gate=proj[:, self.gate_off:] if self.gate else None,
                        gate_per_head=self.gate == "head")
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
