"""Arrangements of parts in a layer.  Pre-norm: x += mixer(norm1(x)); x += ffn(norm2(x))
(src/model/mod.rs:645-650).  Output-norm: x += norm1(mixer(x)); x += norm2(ffn(x)).  Parallel: h = norm1(x);
x += mixer(h) + ffn(h)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Block, BundleCacheSpec, FeedForward, Mixer, Norm, Part


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None, ffn: Optional[FeedForward] = None,
                 after: Optional[Part] = None):
        """``ffn`` None: the layer has only the mixer.  ``after``: a part with ``forward(ctx, x)`` that adds into the
        residual once the sublayers are done (a per-layer token input, for instance)."""
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.after = mixer_norm, mixer, ffn_norm, ffn, after

    def children(self) -> List[Part]:
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.after) if p is not None]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        h = tokens * self.mixer_norm.width * element_size if hasattr(self.mixer_norm, "width") else 0
        parts = [self.mixer.step_bytes(tokens, element_size)]
        parts += [p.step_bytes(tokens, element_size) for p in (self.ffn, self.after) if p is not None]
        return h + max(parts)

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        h = ctx.buffer(tuple(x.shape))
        self.mixer_norm.forward(x, h)
        self.mixer.forward(ctx, h, x, cache)
        if self.ffn is not None:
            self.ffn_norm.forward(x, h)
            self.ffn.forward(ctx, h, x)
        if self.after is not None:
            self.after.forward(ctx, x)


class ParallelBlock(Block):
    """One norm, and both sublayers read its output: h = norm(x); x += mixer(h) + ffn(h).  ``ffn`` None: the layer has only the
    mixer.  Both sublayers add into the float32 residual, the mixer first."""

    def __init__(self, norm: Norm, mixer: Mixer, ffn: Optional[FeedForward] = None):
        self.norm, self.mixer, self.ffn = norm, mixer, ffn

    def children(self) -> List[Part]:
        return [p for p in (self.norm, self.mixer, self.ffn) if p is not None]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        h = tokens * self.norm.width * element_size if hasattr(self.norm, "width") else 0
        ffn = self.ffn.step_bytes(tokens, element_size) if self.ffn is not None else 0
        return h + max(self.mixer.step_bytes(tokens, element_size), ffn)

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        h = ctx.buffer(tuple(x.shape))
        self.norm.forward(x, h)
        self.mixer.forward(ctx, h, x, cache)
        if self.ffn is not None:
            self.ffn.forward(ctx, h, x)


class OutputNormBlock(Block):
    """The norm sits on each sublayer's OUTPUT: x += norm1(mixer(x)); x += norm2(ffn(x)).  The sublayers read the
    residual itself, rounded to the compute dtype (in float32 they read it in place).  The sublayers STORE their result
    in a float32 buffer (``can_store``), and the norm's kernel adds its normalised rows into the residual."""

    def __init__(self, width: int, mixer: Mixer, mixer_norm: Norm, ffn: Optional[FeedForward] = None, ffn_norm: Optional[Norm] = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        for part in (mixer, ffn):
            if part is not None and not getattr(part, "can_store", False):
                raise ValueError(f"{type(part).__name__} cannot store its output, which a norm on the output needs")
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and not hasattr(norm, "add_into"):
                raise ValueError(f"{type(norm).__name__} cannot add its output into the residual")
        self.width, self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = int(width), mixer, mixer_norm, ffn, ffn_norm

    def children(self) -> List[Part]:
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        ffn = self.ffn.step_bytes(tokens, element_size) if self.ffn is not None else 0
        return tokens * self.width * (element_size + 4) + max(self.mixer.step_bytes(tokens, element_size), ffn)

    #: what the norm before left in ``ctx.shared``: the residual rounded to bfloat16, and whose rounding it is
    ROUNDED = "residual.rounded"

    def _read(self, ctx, x: torch.Tensor) -> torch.Tensor:
        if ctx.dtype == torch.float32:
            return x
        left = ctx.shared.pop(self.ROUNDED, None)
        if left is not None and left[1] == x.data_ptr() and left[0].shape == x.shape:
            return left[0]
        h = ctx.buffer(tuple(x.shape))
        ops.copy_cols(x, 0, x.shape[1], h)
        return h

    def _add(self, ctx, norm: Norm, y: torch.Tensor, x: torch.Tensor) -> None:
        """x += norm(y); in bfloat16 the norm's kernel also leaves the new residual rounded for the sublayer that reads it
        next (this block's feed-forward, or the next block's mixer)."""
        if ctx.dtype != torch.bfloat16:
            norm.add_into(y, x)
            return
        h = ctx.buffer(tuple(x.shape))
        norm.add_into(y, x, rounded=h)
        ctx.shared[self.ROUNDED] = (h, x.data_ptr())

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        y = ctx.buffer(tuple(x.shape), torch.float32)
        owed = self.mixer.forward(ctx, self._read(ctx, x), y, cache, accumulate=False)
        if owed is not None:
            ops.add_bias(y, owed)
        self._add(ctx, self.mixer_norm, y, x)
        if self.ffn is None:
            return
        owed = self.ffn.forward(ctx, self._read(ctx, x), y, accumulate=False)
        if owed is not None:
            ops.add_bias(y, owed)
        self._add(ctx, self.ffn_norm, y, x)


class StreamBlock(Block):
    """Pre-norm with the options of a residual kept as several streams and of a token shift before the mixer:

        u = sum_s c_in[s] x_s (or x);  h = norm(u);  h <- shift(h) (mixer only);  y = sublayer(h);
        x_t <- sum_s mix[s, t] x_s + c_out[t] y   (or x += y)

    ``ffn`` None: the layer has only the mixer.  ``connections``: the two sublayers' hyper-connections (None: a
    plain residual [T, width]).  ``shift``: the token shift (None: the mixer reads the norm's output); its state,
    the last normed row of every request, is kept beside the mixer's cache (``BundleCacheSpec``).  The norms take
    ``coef=`` (:class:`carbon_engine_b200.parts.norm.GroupedRMSNorm`)."""

    def __init__(self, width: int, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None, connections=None, shift=None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        if connections is not None and len(connections) != (2 if ffn is not None else 1):
            raise ValueError("one hyper-connection per sublayer")
        self.width = int(width)
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.connections, self.shift = connections, shift
        for part in (mixer, ffn):
            if connections is not None and part is not None and not getattr(part, "can_store", False):
                raise ValueError(f"{type(part).__name__} cannot store its output, which a residual in streams needs")

    def children(self) -> List[Part]:
        parts = [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.shift, *(self.connections or [])]
        return [p for p in parts if p is not None]

    def cache_spec(self):
        main = self.mixer.cache_spec()
        if self.shift is None:
            return main
        return BundleCacheSpec(main, (("shift", self.shift.state_spec()),))

    def step_bytes(self, tokens: int, element_size: int) -> int:
        h = tokens * self.width * (element_size + 4 + (4 if self.connections is not None else 0))
        ffn = self.ffn.step_bytes(tokens, element_size) if self.ffn is not None else 0
        return h + max(self.mixer.step_bytes(tokens, element_size), ffn)

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        T, W = x.shape[0], self.width
        hc = self.connections
        # the mixer
        coef = hc[0].c_in if hc is not None else None
        h = ctx.buffer((T, W))
        if self.shift is not None:
            hn = ctx.buffer((T, W), torch.float32)
            self.mixer_norm.forward(x, hn, coef=coef)
            self.shift.forward(ctx, hn, h, cache.extra["shift"])
        else:
            self.mixer_norm.forward(x, h, coef=coef)
        if hc is None:
            self.mixer.forward(ctx, h, x, cache)
        else:
            y = ctx.buffer((T, W), torch.float32)
            owed = self.mixer.forward(ctx, h, y, cache, accumulate=False)
            hc[0].write(x, y, owed)
        # the feed-forward
        if self.ffn is None:
            return
        self.ffn_norm.forward(x, h, coef=hc[1].c_in if hc is not None else None)
        if hc is None:
            self.ffn.forward(ctx, h, x)
        else:
            owed = self.ffn.forward(ctx, h, y, accumulate=False)
            hc[1].write(x, y, owed)
