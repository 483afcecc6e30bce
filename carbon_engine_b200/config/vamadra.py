"""Typed configuration of the Vamadra architecture.

config.json names the design with ``"architecture": "Vamadra"`` and describes the model layer by layer:

* ``vocab``, ``width``: vocabulary and residual width;
* ``norm`` = ``{"eps"}``: the epsilon of every RMS norm;
* ``layers``: a list of ``{"type", "mixer", "mlp"}``.  ``type`` is ``"latent_attention"``; its ``mixer`` gives ``heads``,
  ``dim`` (unrotated query/key size per head), ``rot_dim`` (rotated size), ``vdim``, ``kv_rank``, ``scale``,
  ``rot`` = ``{"dims", "base", "scaling": {"factor", "original", "fast", "slow"}}`` (``scaling`` optional) and optionally
  ``kv_from``: the index of an earlier layer whose cached rows this layer reads instead of projecting its own;
  ``mlp`` is null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top",
  "groups": {"count", "keep"}, "scale"}, "shared": {"ff"}}`` (``groups``, ``scale`` and ``shared`` optional).

``max_position_embeddings`` and ``eos_token_id`` are optional additions of this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, token_id_list

LATENT_ATTENTION = "latent_attention"
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


def _check_rot(m: Dict[str, Any], where: str) -> None:
    rot = m.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}'rot' must be an object with 'dims' and 'base'")
    dims = _int(rot, "dims", where + "rot: ", 2)
    if dims % 2 or dims > m["rot_dim"]:
        raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most rot_dim={m['rot_dim']}")
    if _float(rot, "base", where + "rot: ") <= 1.0:
        raise ConfigError(f"config.json: {where}rot.base must be above 1")
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}rot.scaling must be an object with 'factor', 'original', 'fast' and 'slow'")
        for key in ("factor", "original", "fast", "slow"):
            if _float(sc, key, where + "rot.scaling: ") <= 0.0:
                raise ConfigError(f"config.json: {where}rot.scaling.{key} must be positive")


def _check_mlp(mlp: Any, where: str) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        _int(mlp, "ff", where + "mlp: ")
        return
    if not isinstance(mlp.get("expert"), dict) or not isinstance(mlp.get("router"), dict):
        raise ConfigError(f"config.json: {where}a mixture of experts needs 'expert' and 'router' objects")
    _int(mlp["expert"], "ff", where + "mlp.expert: ")
    r = mlp["router"]
    experts, top = _int(r, "experts", where + "mlp.router: "), _int(r, "top", where + "mlp.router: ")
    if top > experts:
        raise ConfigError(f"config.json: {where}top={top} of {experts} experts")
    groups = r.get("groups")
    if groups is not None:
        if not isinstance(groups, dict):
            raise ConfigError(f"config.json: {where}mlp.router.groups must be an object with 'count' and 'keep'")
        count, keep = _int(groups, "count", where + "mlp.router.groups: "), _int(groups, "keep", where + "mlp.router.groups: ")
        if experts % count or keep > count or keep * (experts // count) < top:
            raise ConfigError(f"config.json: {where}{experts} experts in {count} groups of which {keep} are kept cannot give {top}")
    if r.get("scale") is not None:
        _float(r, "scale", where + "mlp.router: ")
    if mlp.get("shared") is not None:
        if not isinstance(mlp["shared"], dict):
            raise ConfigError(f"config.json: {where}mlp.shared must be an object with 'ff'")
        _int(mlp["shared"], "ff", where + "mlp.shared: ")


def _check_layer(i: int, layer: Any, earlier: list) -> Dict[str, Any]:
    where = f"layers[{i}]: "
    if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
        raise ConfigError(f"config.json: {where}an object with 'type', 'mixer' and 'mlp' is expected")
    kind, m = layer.get("type"), layer["mixer"]
    if kind != LATENT_ATTENTION:
        raise ConfigError(f"config.json: {where}unknown layer type {kind!r} ({LATENT_ATTENTION})")
    for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
        _int(m, key, where)
    _float(m, "scale", where)
    _check_rot(m, where)
    src = m.get("kv_from")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
            raise ConfigError(f"config.json: {where}kv_from={src!r} must name an earlier layer")
        other = earlier[src]["mixer"]
        if other.get("kv_from") is not None:
            raise ConfigError(f"config.json: {where}kv_from={src}: that layer has no down-projection of its own")
        if any(other[k] != m[k] for k in ("kv_rank", "rot_dim", "rot")):
            raise ConfigError(f"config.json: {where}kv_from={src}: kv_rank, rot_dim and rot must equal that layer's")
    _check_mlp(layer.get("mlp"), where)
    return {"type": kind, "mixer": copy.deepcopy(m), "mlp": copy.deepcopy(layer.get("mlp"))}


@dataclass(frozen=True)
class VamadraConfig(ModelConfig):
    width: int = 0
    layers: Tuple[Dict[str, Any], ...] = ()
    norm_eps: float = 1e-6

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VamadraConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        checked: list = []
        for i, layer in enumerate(layers):
            checked.append(_check_layer(i, layer, checked))
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _float(norm, "eps", "norm: ")
        if eps <= 0.0:
            raise ConfigError(f"config.json: norm eps={eps} must be positive")
        max_pos = raw.get("max_position_embeddings")
        max_pos = DEFAULT_MAX_POSITIONS if max_pos is None else _int(raw, "max_position_embeddings", "")
        eos = token_id_list(raw.get("eos_token_id"))
        for t in raw.get("_generation_eos_token_ids", []):
            if t not in eos:
                eos.append(t)
        return cls(architecture="Vamadra", vocab_size=vocab, max_position_embeddings=max_pos, eos_token_ids=tuple(eos),
                   width=width, layers=tuple(checked), norm_eps=eps)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": "Vamadra", "vocab": self.vocab_size, "width": self.width,
                               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out


def sketch_config(vocab: int, width: int, n_layers: int, heads: int, head_dim: int, ff: int, kv_rank: Optional[int] = None,
                  experts: int = 16, top: int = 4, expert_ff: Optional[int] = None, shared_ff: Optional[int] = None,
                  groups: Tuple[int, int] = (4, 2), share_every: int = 2, max_positions: int = DEFAULT_MAX_POSITIONS,
                  eps: float = 1e-6, rope_base: float = 10000.0, yarn_factor: float = 0.0) -> VamadraConfig:
    """A configuration of the usual proportions from a few sizes, for random-weight models (the command line's
    ``tiny-model``, measurements): heads of ``head_dim`` unrotated and half as many rotated elements, values of ``head_dim``,
    a latent of ``kv_rank`` (default: a quarter of the width); the first layer dense, the others alternating mixtures of
    experts and dense; of every ``share_every`` layers the first projects rows and the others read them."""
    rot = max(2, head_dim // 4 * 2)
    r = kv_rank or max(8, width // 32 * 8)
    eff = expert_ff or max(8, ff // top // 8 * 8)
    rotation: Dict[str, Any] = {"dims": rot, "base": rope_base}
    if yarn_factor > 0.0:
        rotation["scaling"] = {"factor": yarn_factor, "original": 4096, "fast": 32.0, "slow": 1.0}
    layers = []
    for i in range(n_layers):
        m: Dict[str, Any] = {"heads": heads, "dim": head_dim, "rot_dim": rot, "vdim": head_dim, "kv_rank": r,
                             "scale": (head_dim + rot) ** -0.5, "rot": copy.deepcopy(rotation)}
        if share_every > 1 and i % share_every:
            m["kv_from"] = i - i % share_every
        if i % 2 == 0:
            mlp: Dict[str, Any] = {"kind": "dense", "ff": ff}
        else:
            mlp = {"kind": "moe", "expert": {"ff": eff},
                   "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}, "scale": 2.5},
                   "shared": {"ff": shared_ff or eff * 2}}
        layers.append({"type": LATENT_ATTENTION, "mixer": m, "mlp": mlp})
    raw = {"architecture": "Vamadra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "max_position_embeddings": max_positions}
    return VamadraConfig.from_dict(raw)
