"""Small Vamadra configurations for the tests.

They differ from one another in every size and option: widths and vocabularies that are no powers of two; heads whose
unrotated, rotated and value sizes all differ; the rotated part turned whole or in part, with and without stretched
frequencies (factors above and below what makes the ramp start at the first pair); latents smaller and larger than a head;
which layers project their own rows and which read another's (the first, not the neighbour; several readers of one
writer; a reader between two writers); layers without a feed-forward, dense and mixtures of experts in any order;
mixtures with 1 group, with every group kept, with groups of one expert, with top 1, with and without a shared expert,
a router scale of 1.
"""
from __future__ import annotations

from typing import Dict, Optional

from munizen_cases import Harness, rel_err  # noqa: F401  (the harness steps any architecture's folder)


def rot(dims=4, base=500.0, factor=None, original=32, fast=8.0, slow=1.0):
    r = {"dims": dims, "base": base}
    if factor:
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=12, groups=(3, 2), scale=1.7, shared=20):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        m["router"]["scale"] = scale
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=14, scale=0.25, rotation=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": rotation if rotation is not None else rot(dims=rot_dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(layers, width=40, vocab=97, eps=1e-5, max_positions=1024):
    return {"architecture": "Vamadra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "max_position_embeddings": max_positions}


_yarn = rot(dims=8, base=300.0, factor=3.0, original=24, fast=6.0, slow=0.5)
CASES: Dict[str, dict] = {
    # writer, mixture, two readers of layer 1, part of the rotated part turned
    "A": config([layer(mlp=dense()), layer(rotation=_yarn, mlp=moe()), layer(rotation=_yarn, kv_from=1, heads=2, dim=6, vdim=10, mlp=dense(24)),
                 layer(rotation=_yarn, kv_from=1, mlp=moe(experts=4, top=1, groups=None, scale=None, shared=None))]),
    # a reader of layer 0 between two writers; a layer without a feed-forward; groups of one expert, all groups kept
    "B": config([layer(heads=1, dim=10, rot_dim=6, vdim=7, kv_rank=9, rotation=rot(dims=2, base=77.0), mlp=moe(experts=5, top=3, groups=(5, 4), shared=8)),
                 layer(heads=4, dim=5, rot_dim=2, vdim=3, kv_rank=30, scale=0.5, rotation=rot(dims=2, base=1e4, factor=0.5, original=16), mlp=None),
                 layer(heads=5, dim=4, rot_dim=6, vdim=9, kv_rank=9, rotation=rot(dims=2, base=77.0), kv_from=0, mlp=moe(experts=8, top=4, groups=(2, 2), ff=7, shared=5)),
                 layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=6, mlp=dense(17))], width=36, vocab=61, eps=1e-6),
    # head sizes of the tensor-core kernels (multiples of 16), eight heads so that single tokens pack them into one tile
    "T": config([layer(heads=8, dim=16, rot_dim=16, vdim=32, kv_rank=48, scale=0.18, rotation=rot(dims=16, base=1e4, factor=4.0, original=64, fast=16.0), mlp=dense(96)),
                 layer(heads=8, dim=32, rot_dim=16, vdim=16, kv_rank=48, scale=0.15, rotation=rot(dims=16, base=1e4, factor=4.0, original=64, fast=16.0), kv_from=0,
                       mlp=moe(experts=8, top=2, ff=32, groups=(4, 2), scale=2.0, shared=48))], width=64, vocab=151),
    # wider heads and a latent wider than a head: rows of 192 + 32, values cut into slices by the tensor-core kernel
    "V": config([layer(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=192, scale=0.1, rotation=rot(dims=32, base=1e4, factor=4.0, original=128, fast=16.0),
                       mlp=moe(experts=16, top=4, ff=48, groups=(4, 2), scale=2.0, shared=96)),
                 layer(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=192, scale=0.1, rotation=rot(dims=32, base=1e4, factor=4.0, original=128, fast=16.0), kv_from=0,
                       mlp=dense(272))], width=192, vocab=300),
}
#: one layer alone, for looking at a mechanism by itself
SINGLE = {
    "attention_only": config([layer(mlp=None)]),
    "attention_stretched": config([layer(rotation=_yarn, mlp=None)]),
    "dense": config([layer(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=4, mlp=dense(33))]),
    "experts": config([layer(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=4, mlp=moe())]),
    "experts_plain_router": config([layer(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=4, mlp=moe(experts=7, top=7, groups=None, scale=None, shared=None))]),
}


def write_model(raw: dict, folder: str, seed: int = 3) -> str:
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.vamadra import VamadraConfig
    from carbon_engine_b200.weights.loader import write_random_model
    return write_random_model(VamadraConfig.from_dict(dict(raw)), folder, seed=seed)
