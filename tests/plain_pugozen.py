"""A plain, slow implementation of the Pugozen design: whole sequences, float64, one function per mechanism.

It shares no code with the engine: it takes the configuration as the dict config.json holds and the weights
as a dict name -> tensor, runs one sequence from its first token, and keeps nothing between calls.  The tests
compare the engine's logits, residual streams and single mechanisms with it.

A layer normalises once and both sublayers read that: x <- x + mixer(norm1(x)) + ff(norm1(x)).  The mixers:
``retention`` (linear attention with a fixed decay per head, rotated queries and keys), ``delta`` (the gated delta rule
with a decay per head), ``parallel`` (softmax attention whose values are the projected keys, with a sink and a
temperature per head, beside the gated delta rule with a decay per head and key channel; a weighted sum of the two).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_half_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, size]: element i of the first ``dims`` turns with element i + dims/2 by the angle
    position * base^(-2i/dims); the rest passes unchanged."""
    if dims <= 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K] (the last column weighs the current token, zeros before the start) -> silu(conv) [T, C]."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros((K - 1, C), dtype=F), x], dim=0)
    y = torch.zeros((T, C), dtype=F)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j][None, :]
    return silu(y)


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule_walk(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """One head: q, k [T, d], v [T, dv], g [T, d] (a decay per key channel; a decay per head is a constant row),
    beta [T] -> o [T, dv].  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, d = q.shape
    dv = v.shape[1]
    S = torch.zeros((d, dv), dtype=F)
    out = torch.zeros((T, dv), dtype=F)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def retention_walk(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: float) -> torch.Tensor:
    """One head: S <- decay S + k v^T; o = S^T q."""
    T, d = q.shape
    S = torch.zeros((d, v.shape[1]), dtype=F)
    out = torch.zeros((T, v.shape[1]), dtype=F)
    for t in range(T):
        S = decay * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out


def retention_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate_half_pairs((h @ w[f"{p}.q"].T).reshape(T, H, d), pos, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = rotate_half_pairs((h @ w[f"{p}.k"].T).reshape(T, H, d), pos, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = k * d ** -0.5
    v = (h @ w[f"{p}.v"].T).reshape(T, H, dv)
    out = torch.stack([retention_walk(q[:, i], k[:, i], v[:, i], float(m["decay"][i])) for i in range(H)], dim=1)
    out = rms_norm(out, None, eps).reshape(T, H * dv) * silu(h @ w[f"{p}.g"].T)
    return out @ w[f"{p}.o"].T


def _delta_inputs(w, p, m, h):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"]).reshape(T, G, d)
    k = causal_conv_silu(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"]).reshape(T, G, d)
    v = causal_conv_silu(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"]).reshape(T, H, dv)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)
    return q, k, v, beta


def head_delta_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The gated delta rule with one decay per head and a SiLU gate of full rank."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v, beta = _delta_inputs(w, p, m, h)
    g = torch.exp(-torch.exp(w[f"{p}.A_log"])[None, :] * softplus(h @ w[f"{p}.a"].T + w[f"{p}.dt_bias"][None, :]))     # [T, H]
    out = torch.zeros((T, H, dv), dtype=F)
    for i in range(H):
        j = i // (H // G)
        out[:, i] = delta_rule_walk(q[:, j], k[:, j], v[:, i], g[:, i][:, None].expand(T, d), beta[:, i])
    out = (rms_norm(out, w[f"{p}.norm"], eps)).reshape(T, H * dv) * silu(h @ w[f"{p}.g"].T)
    return out @ w[f"{p}.o"].T


def channel_delta_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel and a sigmoid gate through a narrow pair of matrices."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v, beta = _delta_inputs(w, p, m, h)
    z = (h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.dt_bias"][None, :]
    g = torch.exp(-torch.exp(w[f"{p}.A_log"])[None, :, None] * softplus(z).reshape(T, H, d))
    out = torch.zeros((T, H, dv), dtype=F)
    for i in range(H):
        j = i // (H // G)
        out[:, i] = delta_rule_walk(q[:, j], k[:, j], v[:, i], g[:, i], beta[:, i])
    gate = torch.sigmoid((h @ w[f"{p}.g1"].T) @ w[f"{p}.g2"].T)
    out = rms_norm(out, w[f"{p}.norm"], eps).reshape(T, H * dv) * gate
    return out @ w[f"{p}.o"].T


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, temp: torch.Tensor,
                           sink: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; score = q.k scale temp_h; exp(sink_h) joins the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    for i in range(H):
        j = i // (H // G)
        s = (q[:, i] @ k[:, j].T) * scale * temp[i]
        s = s.masked_fill(torch.triu(torch.ones((T, T), dtype=torch.bool), diagonal=1), float("-inf"))
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[i].reshape(1, 1))
        e = torch.exp(s - top)
        out[:, i] = (e @ v[:, j]) / (e.sum(-1, keepdim=True) + torch.exp(sink[i] - top))
    return out


def tied_attention_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Softmax attention whose values are the keys as projected (before their norm and rotation)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    q = (h @ w[f"{p}.q"].T).reshape(T, H, d)
    k = (h @ w[f"{p}.k"].T).reshape(T, G, d)
    v = k
    rot = m.get("rot") or {}
    q = rotate_half_pairs(rms_norm(q, w[f"{p}.q.norm"], eps), pos, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = rotate_half_pairs(rms_norm(k, w[f"{p}.k.norm"], eps), pos, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    out = sink_softmax_attention(q, k, v, float(m["scale"]), w[f"{p}.temp"], w[f"{p}.sink"])
    return out.reshape(T, H * d) @ w[f"{p}.o"].T


def pair_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    left = tied_attention_mixer(w, f"{p}.left", m["left"], h, eps)
    right = channel_delta_mixer(w, f"{p}.right", m["right"], h, eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def dense_ff(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ w[f"{p}.up"].T) ** 2) @ w[f"{p}.down"].T


MIXERS = {"retention": retention_mixer, "delta": head_delta_mixer, "parallel": pair_mixer}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the residual after every layer."""
    w = {k: v.to(F) if v.is_floating_point() else v for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    x = w["embed"][tok] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer['weights_of']}" if layer.get("weights_of") is not None else f"l{i}"
        h = rms_norm(x, w[f"{p}.norm1"], eps)
        y = MIXERS[layer["type"]](w, f"{p}.mix", layer["mixer"], h, eps)
        if layer.get("mlp") is not None:
            y = y + dense_ff(w, f"{p}.mlp", h)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def read_model(folder: str):
    """(config dict, weights dict) of a model folder: config.json and model.safetensors (an 8-byte little-endian header
    length, a JSON header name -> dtype, shape, data_offsets, then the data)."""
    import json
    import os
    import struct
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        blob = fh.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode())
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = {"F32": torch.float32, "BF16": torch.bfloat16, "I32": torch.int32}[meta["dtype"]]
        weights[name] = torch.frombuffer(bytearray(blob[8 + n + lo:8 + n + hi]), dtype=dt).reshape(meta["shape"]).clone()
    return cfg, weights
