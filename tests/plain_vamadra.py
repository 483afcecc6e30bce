"""A plain, slow implementation of the Vamadra design: whole sequences, float64, one function per mechanism.

It shares no code with the engine: it takes the configuration as the dict config.json holds and the weights
as a dict name -> tensor, runs one sequence from its first token, and keeps nothing between calls.  Keys and
values of every head are formed in full (no product is moved to the query side), experts are looped over.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

F = torch.float64


# ---------------------------------------------------------------------------------------------------------------
# reading a model folder
# ---------------------------------------------------------------------------------------------------------------
def read_model(folder: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor of model.safetensors in float64 (integer tables stay integers)."""
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw, shape = data[lo:hi], tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy()).to(F)
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.float32).copy()).to(F)
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.int32).copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = t.reshape(shape)
    return cfg, out


# ---------------------------------------------------------------------------------------------------------------
# norms and activations
# ---------------------------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain_weight(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def norm_zero_centred(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' and the model's norm: the stored weight is the deviation from 1."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


# ---------------------------------------------------------------------------------------------------------------
# rotation
# ---------------------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> Tuple[List[float], float]:
    """The dims/2 angular steps per position and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return freq, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, size]: element i of the first rot.dims turns with element i + dims/2; the rest passes."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, mag = rotary_frequencies(rot)
    ang = positions.to(F)[:, None] * torch.tensor(freq, dtype=F)[None, :]
    cos, sin = (ang.cos() * mag)[:, None, :], (ang.sin() * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------------------------
# latent attention
# ---------------------------------------------------------------------------------------------------------------
def latent_rows(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, positions: torch.Tensor, eps: float):
    """What a layer with a down-projection of its own keeps per token: the latent c [T, kv_rank] and the rotated key
    part shared by the heads [T, rot_dim]."""
    r = int(m["kv_rank"])
    z = h @ w[f"{p}.dkv"].T
    c = norm_plain_weight(z[:, :r], w[f"{p}.dkv.norm"], eps)
    k_rot = rotate(z[:, None, r:], positions, m["rot"])[:, 0]
    return c, k_rot


def sink_softmax(scores: torch.Tensor, sink: float) -> torch.Tensor:
    """Causal softmax over a [T, T] score table whose denominator holds exp(sink) once more."""
    T = scores.shape[0]
    out = torch.zeros_like(scores)
    for i in range(T):
        row = scores[i, :i + 1]
        top = max(float(row.max()), sink)
        e = torch.exp(row - top)
        out[i, :i + 1] = e / (e.sum() + math.exp(sink - top))
    return out


def latent_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, positions: torch.Tensor, eps: float,
                     kept: dict, layer: int) -> torch.Tensor:
    T = h.shape[0]
    H, d, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    if m.get("kv_from") is None:
        kept[layer] = latent_rows(w, p, m, h, positions, eps)
        c, k_rot = kept[layer]
    else:
        c, k_rot = kept[int(m["kv_from"])]
    q = (h @ w[f"{p}.q"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, m["rot"])
    k_plain = (c @ w[f"{p}.uk"].T).view(T, H, d)
    v = (c @ w[f"{p}.uv"].T).view(T, H, dv)
    gate = torch.sigmoid(h @ w[f"{p}.g"].T)                 # [T, H]
    heads = []
    for i in range(H):
        s = (q_plain[:, i] @ k_plain[:, i].T + q_rot[:, i] @ k_rot.T) * float(m["scale"])
        pr = sink_softmax(s, float(w[f"{p}.sink"][i]))
        heads.append((pr @ v[:, i]) * gate[:, i:i + 1])
    return torch.cat(heads, dim=-1) @ w[f"{p}.o"].T


# ---------------------------------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------------------------------
def dense_ffn(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def small_expert(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return relu_squared(h @ w[f"{p}.up"].T) @ w[f"{p}.down"].T


def route(z: torch.Tensor, router: dict, margin: Optional[list] = None) -> Tuple[List[int], List[float]]:
    """One token's router logits -> the chosen experts and their weights.  ``margin`` receives how clear the choice was:
    the smallest gap between something chosen and something not (the last kept group and the first dropped one; the last
    chosen expert and the first one passed over), in logits."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.softmax(z, dim=-1)
    allowed = list(range(E))
    groups = router.get("groups")
    gap = math.inf
    if groups:
        n, size, keep = int(groups["count"]), E // int(groups["count"]), int(groups["keep"])
        order = sorted(range(n), key=lambda g: -float(s[g * size:(g + 1) * size].max()))
        best = order[:keep]
        allowed = [e for e in range(E) if e // size in best]
        if keep < n:
            gap = float(z[order[keep - 1] * size:(order[keep - 1] + 1) * size].max() - z[order[keep] * size:(order[keep] + 1) * size].max())
    ranked = sorted(allowed, key=lambda e: -float(s[e]))
    chosen = ranked[:top]
    if top < len(ranked):
        gap = min(gap, float(z[ranked[top - 1]] - z[ranked[top]]))
    if margin is not None:
        margin.append(gap)
    total = sum(float(s[e]) for e in chosen) + 1e-20
    scale = float(router.get("scale", 1.0))
    return chosen, [float(s[e]) / total * scale for e in chosen]


def moe_ffn(w: Dict[str, torch.Tensor], p: str, mlp: dict, h: torch.Tensor, margins: Optional[list] = None) -> torch.Tensor:
    """``margins`` receives one number per token: the gap of :func:`route` as a fraction of the size of what a router
    logit is summed from (the root of the sum of its terms' squares: a rounding of the input moves a logit by a small
    fraction of that)."""
    out = torch.zeros_like(h)
    z = h @ w[f"{p}.router"].T
    for t in range(h.shape[0]):
        gap: list = []
        chosen, weights = route(z[t], mlp["router"], gap)
        if margins is not None:
            size = float(torch.sqrt(((h[t][None, :] * w[f"{p}.router"]) ** 2).sum(-1)).max())
            margins.append(gap[0] / max(size, 1e-30))
        for e, g in zip(chosen, weights):
            out[t] += g * small_expert(w, f"{p}.e{e}", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + small_expert(w, f"{p}.shared", h) * torch.sigmoid(h @ w[f"{p}.shared.sg"].T)
    return out


# ---------------------------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], tap: Optional[Callable] = None,
            round_input: Optional[Callable] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token.  ``tap(i, x)`` sees the residual after layer i.
    ``round_input``: applied to what the sublayers read (to see what a rounding of the activations does).
    ``margins`` receives, per mixture layer, a list with every token's router margin (:func:`route`)."""
    eps = float(cfg["norm"]["eps"])
    rd = round_input or (lambda t: t)
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)].to(F)
    positions = torch.arange(len(tokens))
    kept: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']}")
        y = latent_attention(w, f"{p}.mix", layer["mixer"], rd(x), positions, eps, kept, i)
        x = x + norm_zero_centred(y, w[f"{p}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = dense_ffn(w, f"{p}.mlp", rd(x))
            else:
                per_token: list = []
                y = moe_ffn(w, f"{p}.mlp", mlp, rd(x), per_token)
                if margins is not None:
                    margins.append(per_token)
            x = x + norm_zero_centred(y, w[f"{p}.norm2"], eps)
        if tap is not None:
            tap(i, x)
    return norm_zero_centred(x, w["final.norm"], eps) @ w["head"].T
