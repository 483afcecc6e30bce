"""Typed configuration of the Pugozen architecture.

config.json names the design with ``"architecture": "Pugozen"`` and describes the model layer by layer:

* ``vocab``, ``width``: vocabulary and residual width; ``embedding`` = ``{"scale"}`` multiplies the embedding rows;
* ``layers``: a list of ``{"type", "mixer", "mlp"}`` and optionally ``"weights_of": j`` (the layer has no tensors of its own
  and runs layer j's, with a cache of its own; sizes and constants are then layer j's).  ``kv_heads`` left out means as
  many as ``heads``.  ``type`` is
  ``"retention"`` (linear attention with a fixed decay per head: ``heads``, ``dim``, ``vdim``, ``decay`` = one number per
  head, ``rot`` = ``{"dims", "base"}``),
  ``"delta"`` (the gated delta rule with one decay per head: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps) or
  ``"parallel"`` (two mixers side by side: ``left`` = softmax attention whose values are the projected keys, with ``heads``,
  ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot``; ``right`` = the gated delta rule with a decay per head and key
  channel, with ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``; ``left_scale``, ``right_scale`` weigh their sum);
  ``mlp`` is ``{"kind": "dense", "ff"}`` or null;
* ``norm`` = ``{"eps"}``: the epsilon of the layers' RMS norms and of the mixers' own.

What config.json does not give is taken from the stored tensors' shapes (the ranks of the right mixer's two narrow
projections), unless the mixer's entry names them (``a_rank``, ``g_rank``), which a model with random weights needs.
``max_position_embeddings`` and ``eos_token_id`` are optional additions of this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from .base import ConfigError, ModelConfig, token_id_list

RETENTION, DELTA, PARALLEL = "retention", "delta", "parallel"
DEFAULT_MAX_POSITIONS = 32768


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer >= {minimum}, got {v!r}")
    return v


def _float(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _rot(m: Dict[str, Any], where: str) -> None:
    rot = m.get("rot")
    if rot is None:
        return
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}'rot' must be an object with 'dims' and 'base'")
    dims = _int(rot, "dims", where + "rot: ", 2)
    if dims % 2 or dims > m["dim"]:
        raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most dim={m['dim']}")
    if _float(rot, "base", where + "rot: ") <= 0.0:
        raise ConfigError(f"config.json: {where}rot.base must be positive")


def _delta(m: Any, where: str, ranks: bool) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where}an object is expected")
    m.setdefault("kv_heads", m.get("heads"))
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} kv_heads")
    _int(m, "dim", where); _int(m, "vdim", where); _int(m, "conv", where)
    if ranks:
        for key in ("a_rank", "g_rank"):
            if m.get(key) is not None:
                _int(m, key, where)


def _check_layer(i: int, layer: Any) -> Dict[str, Any]:
    where = f"layers[{i}]: "
    if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
        raise ConfigError(f"config.json: {where}an object with 'type', 'mixer' and 'mlp' is expected")
    layer = copy.deepcopy(layer)
    kind, m = layer.get("type"), layer["mixer"]
    if kind == RETENTION:
        heads = _int(m, "heads", where)
        _int(m, "dim", where); _int(m, "vdim", where)
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or \
                any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
            raise ConfigError(f"config.json: {where}'decay' must list one number per head ({heads}), got {decay!r}")
        _rot(m, where)
    elif kind == DELTA:
        _delta(m, where, ranks=False)
    elif kind == PARALLEL:
        left = m.get("left")
        if not isinstance(left, dict):
            raise ConfigError(f"config.json: {where}'left' must be an object")
        left.setdefault("kv_heads", left.get("heads"))
        heads, kv = _int(left, "heads", where + "left: "), _int(left, "kv_heads", where + "left: ")
        if heads % kv:
            raise ConfigError(f"config.json: {where}left: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(left, "dim", where + "left: ")
        if left.get("vdim") is not None and _int(left, "vdim", where + "left: ") != dim:
            raise ConfigError(f"config.json: {where}left: the values are the projected keys, so vdim must equal dim={dim}")
        _float(left, "scale", where + "left: ")
        _rot(left, where + "left: ")
        _delta(m.get("right"), where + "right: ", ranks=True)
        _float(m, "left_scale", where); _float(m, "right_scale", where)
    else:
        raise ConfigError(f"config.json: {where}unknown layer type {kind!r} ({RETENTION}, {DELTA}, {PARALLEL})")
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense', got {mlp!r}")
        _int(mlp, "ff", where + "mlp: ")
    out = {"type": kind, "mixer": m, "mlp": mlp}
    if layer.get("weights_of") is not None:
        out["weights_of"] = _int(layer, "weights_of", where, 0)
    return out


def weight_owner(layers, i: int) -> int:
    """The layer whose tensors layer ``i`` runs (itself, unless it names another with ``weights_of``)."""
    seen = set()
    while layers[i].get("weights_of") is not None:
        if i in seen:
            raise ConfigError(f"config.json: layers[{i}]: 'weights_of' goes in a circle")
        seen.add(i)
        i = layers[i]["weights_of"]
    return i


@dataclass(frozen=True)
class PugozenConfig(ModelConfig):
    width: int = 0
    layers: Tuple[Dict[str, Any], ...] = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PugozenConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        checked = tuple(_check_layer(i, layer) for i, layer in enumerate(layers))
        for i, layer in enumerate(checked):
            j = layer.get("weights_of")
            if j is None:
                continue
            if j >= len(checked) or j == i:
                raise ConfigError(f"config.json: layers[{i}]: 'weights_of' must name another layer, got {j}")
            weight_owner(checked, i)           # refuses a circle
            # the layer's own entry is taken to equal its owner's: sizes and constants are the owner's, whose tensors it runs
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _float(norm, "eps", "norm: ")
        if eps <= 0.0:
            raise ConfigError(f"config.json: norm eps={eps} must be positive")
        scale = 1.0
        if raw.get("embedding") is not None:
            if not isinstance(raw["embedding"], dict):
                raise ConfigError("config.json: 'embedding' must be an object with 'scale'")
            scale = _float(raw["embedding"], "scale", "embedding: ")
        max_pos = raw.get("max_position_embeddings")
        max_pos = DEFAULT_MAX_POSITIONS if max_pos is None else _int(raw, "max_position_embeddings", "")
        eos = token_id_list(raw.get("eos_token_id"))
        for t in raw.get("_generation_eos_token_ids", []):
            if t not in eos:
                eos.append(t)
        return cls(architecture="Pugozen", vocab_size=vocab, max_position_embeddings=max_pos, eos_token_ids=tuple(eos),
                   width=width, layers=checked, norm_eps=eps, embedding_scale=scale)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": "Pugozen", "vocab": self.vocab_size, "width": self.width,
                               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale}}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out


def sketch_config(vocab: int, width: int, n_layers: int, heads: int, kv_heads: int, head_dim: int, ff: int,
                  max_positions: int = DEFAULT_MAX_POSITIONS, eps: float = 1e-5, rope_base: float = 10000.0,
                  shared_from: int = 0) -> PugozenConfig:
    """A configuration of the usual proportions from a few sizes, for random-weight models (the command line's
    ``tiny-model``, measurements): layers go delta rule, parallel, parallel, retention and again; state heads of ``head_dim``
    filling the width; attention heads of ``head_dim`` rotated over a quarter of it.  ``shared_from`` > 0: the layers from
    that index on run the weights of the layer that many places before them."""
    state_heads = max(1, width // head_dim)
    key_heads = max(1, state_heads // 2) if state_heads % 2 == 0 else state_heads
    rot = max(2, head_dim // 8 * 2)
    kinds = (DELTA, PARALLEL, PARALLEL, RETENTION)
    layers = []
    for i in range(n_layers):
        kind = kinds[i % 4]
        if kind == DELTA:
            m = {"heads": state_heads, "kv_heads": key_heads, "dim": head_dim, "vdim": head_dim, "conv": 4}
        elif kind == RETENTION:
            m = {"heads": state_heads, "dim": head_dim, "vdim": head_dim,
                 "decay": [1.0 - 2.0 ** (-5 - (5 * j) // state_heads) for j in range(state_heads)],
                 "rot": {"dims": head_dim // 2 * 2, "base": rope_base}}
        else:
            m = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                          "rot": {"dims": rot, "base": rope_base}},
                 "right": {"heads": state_heads, "kv_heads": state_heads, "dim": head_dim, "vdim": head_dim, "conv": 3,
                           "a_rank": max(8, width // 32 * 2), "g_rank": max(8, width // 32 * 2)},
                 "left_scale": 0.7, "right_scale": 0.6}
        layer = {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff}}
        if shared_from > 0 and i >= shared_from:
            layer["weights_of"] = i - shared_from
        layers.append(layer)
    return PugozenConfig.from_dict({"architecture": "Pugozen", "vocab": vocab, "width": width, "layers": layers,
                                    "norm": {"eps": eps}, "embedding": {"scale": float(width) ** 0.5},
                                    "max_position_embeddings": max_positions})
