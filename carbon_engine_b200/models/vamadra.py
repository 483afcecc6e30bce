"""The Vamadra decoder, put together from the package's parts.

Every layer normalises what its sublayers RETURN: x += norm1(mixer(x)); x += norm2(ff(x)) (``parts/block.py``
``OutputNormBlock``), with RMS norms whose stored weights are deviations from 1 (``RMSNorm(unit_offset=True)``).  The mixer is
latent attention (``parts/latent_attention.py``) without a query latent, with a sink per head in the softmax, one gate per
head and a rotation whose frequencies are stretched the YaRN way; a layer may read the rows an earlier layer cached instead
of projecting its own, which the model's schedule expresses as a call that reads that layer's cache.  The feed-forward is
gated with SiLU (``parts/mlp.py``) or a mixture of experts with grouped routing and a gated shared expert (``parts/moe.py``).
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|dkv|dkv.norm|uk|uv|sink|g|o``, ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router``, ``l<i>.mlp.e<j>.up|down``, ``l<i>.mlp.shared.up|down|sg``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math

from ..config.registry import register_architecture
from ..config.vamadra import VamadraConfig
from ..parts.block import OutputNormBlock
from ..parts.embedding import Embedding, LMHead
from ..parts.model import DecoderModel, LayerCall
from ..parts.registry import build_part
from ..parts.rope import RopeScaling


def _rotation_key(m: dict) -> tuple:
    rot, sc = m["rot"], m["rot"].get("scaling") or {}
    return (m["rot_dim"], rot["dims"], float(rot["base"]), tuple(sorted((k, float(v)) for k, v in sc.items())))


def _rotation(m: dict, max_positions: int):
    rot, sc = m["rot"], m["rot"].get("scaling")
    scaling = None
    if sc:
        # cos and sin are multiplied by 0.1 ln(factor) + 1 whatever the factor
        scaling = RopeScaling("yarn", factor=float(sc["factor"]), original_max_position=sc["original"], beta_fast=float(sc["fast"]),
                              beta_slow=float(sc["slow"]), attention_factor=0.1 * math.log(float(sc["factor"])) + 1.0)
    return build_part("position", "rotary", head_dim=m["rot_dim"], theta=float(rot["base"]), max_positions=max_positions,
                      rotary_dim=rot["dims"], scaling=scaling)


def build_vamadra(cfg: VamadraConfig, max_positions: int) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: build_part("norm", "rmsnorm", width=W, eps=eps, name=name, unit_offset=True)
    rotations = {}
    blocks, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m, mlp = f"l{i}", layer["mixer"], layer["mlp"]
        key = _rotation_key(m)
        if key not in rotations:
            rotations[key] = _rotation(m, max_positions)
        src = m.get("kv_from")
        mixer = build_part("mixer", "latent_attention", hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                           vdim=m["vdim"], q_rank=0, kv_rank=m["kv_rank"], prefix=f"{p}.mix", eps=eps, position=rotations[key],
                           scale=m["scale"], gate="head", sink=True, own_kv=src is None)
        ffn = ffn_norm = None
        if mlp is not None:
            ffn_norm = norm(f"{p}.norm2")
            if mlp["kind"] == "dense":
                ffn = build_part("feed_forward", "gated_mlp", hidden=W, intermediate=mlp["ff"], prefix=f"{p}.mlp",
                                 activation="silu", names=("gate", "up", "down"))
            else:
                r, groups, shared = mlp["router"], mlp["router"].get("groups") or {}, mlp.get("shared") or {}
                ffn = build_part("feed_forward", "routed_experts", hidden=W, experts=r["experts"], top=r["top"],
                                 ff=mlp["expert"]["ff"], prefix=f"{p}.mlp", groups=groups.get("count", 1),
                                 keep_groups=groups.get("keep", 1), scale=r.get("scale", 1.0) if r.get("scale") is not None else 1.0,
                                 activation="relu2", shared_ff=shared.get("ff", 0), shared_gate=True)
        blocks.append(OutputNormBlock(W, mixer, norm(f"{p}.norm1"), ffn, ffn_norm))
        schedule.append(LayerCall(i, i, True) if src is None else LayerCall(i, int(src), False))
    embedding = Embedding(cfg.vocab_size, W, "embed")
    head = LMHead(cfg.vocab_size, W, norm("final.norm"), "head")
    return DecoderModel(cfg, embedding, blocks, head, schedule=schedule)


register_architecture("Vamadra", VamadraConfig.from_dict, build_vamadra, model_types=("vamadra",), replace=True)
