"""Small Pugozen configurations for the tests.

They differ from one another in every size and option: widths and vocabularies that are no powers of two; the order of
the three kinds of layer and which comes first; retention with the rotation over a part of a head, over all of it and
absent, equal and unequal decays, key size against value size; the delta rule with 1 to 5 taps, fewer key heads than value
heads and as many; the pair with one key head for all query heads, one per query head and groups, the rotation whole and in
part, weights of the sum equal, unequal and 1; layers without a feed-forward; layers that run an earlier or a later layer's
weights; an embedding scale of 1.
"""
from __future__ import annotations

from typing import Dict

from munizen_cases import Harness, rel_err  # noqa: F401  (the harness steps any architecture's folder)


def _mlp(ff):
    return {"kind": "dense", "ff": ff} if ff else None


def retention(heads=3, dim=12, vdim=8, decay=(0.9, 0.97, 0.995), rot_dims=8, base=300.0, ff=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "retention", "mixer": m, "mlp": _mlp(ff)}


def delta(heads=4, kv_heads=2, dim=8, vdim=12, conv=4, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": _mlp(ff)}


def pair(heads=4, kv_heads=2, dim=16, rot_dims=6, base=200.0, scale=0.3, r_heads=2, r_kv_heads=1, r_dim=8, r_vdim=12, conv=3,
         a_rank=5, g_rank=3, left_scale=0.7, right_scale=0.6, ff=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot_dims:
        left["rot"] = {"dims": rot_dims, "base": base}
    right = {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": conv, "a_rank": a_rank, "g_rank": g_rank}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": _mlp(ff)}


def shared(layer: dict, owner: int) -> dict:
    """A layer that runs layer ``owner``'s weights: the same entry with ``weights_of``."""
    return {**layer, "weights_of": owner}


def config(layers, width=40, vocab=97, eps=1e-5, scale=3.0, max_positions=1024):
    raw = {"architecture": "Pugozen", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "max_position_embeddings": max_positions}
    if scale is not None:
        raw["embedding"] = {"scale": scale}
    return raw


_A = [delta(ff=44), pair(ff=36), retention(ff=None), pair(heads=2, kv_heads=2, dim=8, rot_dims=8, r_heads=3, r_kv_heads=3, r_dim=4,
                                                           r_vdim=4, conv=2, a_rank=2, g_rank=6, left_scale=1.0, right_scale=0.25, ff=28)]
CASES: Dict[str, dict] = {
    # all three kinds, then the first three once more on the same weights with caches of their own
    "A": config(_A + [shared(_A[0], 0), shared(_A[1], 1), shared(_A[2], 2)]),
    # the pair first, with one key head for all query heads and no rotation; retention without rotation and equal decays;
    # one tap (no convolution state); embedding scale left out; a layer that runs a LATER layer's weights
    "B": config([pair(heads=3, kv_heads=1, dim=20, rot_dims=0, scale=0.2, r_heads=1, r_kv_heads=1, r_dim=12, r_vdim=28, conv=1, a_rank=3,
                      g_rank=3, left_scale=0.5, right_scale=0.5, ff=24),
                 shared(retention(heads=2, dim=6, vdim=20, decay=(0.96, 0.96), rot_dims=0, ff=30), 3),
                 delta(heads=1, kv_heads=1, dim=12, vdim=28, conv=1),
                 retention(heads=2, dim=6, vdim=20, decay=(0.96, 0.96), rot_dims=0, ff=30)],
                width=36, vocab=131, eps=1e-6, scale=None),
    # retention first with the whole head rotated, five taps, as many key heads as heads, odd sizes
    "C": config([retention(heads=2, dim=10, vdim=14, decay=(0.5, 0.999), rot_dims=10, ff=50),
                 delta(heads=3, kv_heads=3, dim=16, vdim=16, conv=5, ff=None),
                 pair(heads=6, kv_heads=3, dim=8, rot_dims=2, scale=0.5, r_heads=2, r_kv_heads=2, r_dim=10, r_vdim=7, conv=4, a_rank=4,
                      g_rank=4, left_scale=0.3, right_scale=1.7),
                 delta(heads=2, kv_heads=1, dim=20, vdim=6, conv=2, ff=30)],
                width=48, vocab=75, scale=1.0),
}
# Head sizes the tensor-core attention kernel takes (multiples of 16) and state heads of the sizes of a mid-sized model
CASES["T"] = config([pair(heads=6, kv_heads=2, dim=64, rot_dims=32, scale=0.11, r_heads=2, r_kv_heads=2, r_dim=64, r_vdim=48, conv=3,
                          a_rank=8, g_rank=8, ff=72),
                     delta(heads=6, kv_heads=3, dim=32, vdim=48, conv=4, ff=96),
                     retention(heads=2, dim=64, vdim=64, decay=(0.97, 0.9995), rot_dims=64, base=5e5),
                     shared(pair(heads=6, kv_heads=2, dim=64, rot_dims=32, scale=0.11, r_heads=2, r_kv_heads=2, r_dim=64, r_vdim=48,
                                 conv=3, a_rank=8, g_rank=8, ff=72), 0)],
                    width=128, vocab=151)
CASES["V"] = config([retention(heads=2, dim=128, vdim=64, decay=(0.99, 0.999), rot_dims=32, ff=256),
                     pair(heads=8, kv_heads=1, dim=32, rot_dims=32, scale=0.15, r_heads=2, r_kv_heads=1, r_dim=136, r_vdim=16, conv=2,
                          a_rank=16, g_rank=16, left_scale=0.9, right_scale=0.6),
                     delta(heads=2, kv_heads=1, dim=64, vdim=128, conv=4)],
                    width=192, vocab=300)
#: one layer of one kind each, for looking at a mechanism alone
SINGLE = {
    "retention": config([retention()]),
    "retention_no_rotation": config([retention(rot_dims=0, heads=1, dim=9, vdim=5, decay=(0.93,))], width=34),
    "retention_wide_keys": config([retention(heads=1, dim=136, vdim=8, decay=(0.98,), rot_dims=136)]),
    "delta": config([delta()]),
    "delta_one_tap": config([delta(conv=1, heads=2, kv_heads=2, dim=36, vdim=5)]),
    "delta_odd_sizes": config([delta(heads=2, kv_heads=1, dim=10, vdim=7, conv=3)], width=34),
    "pair": config([pair()]),
    "pair_left_only_counts": config([pair(left_scale=1.0, right_scale=0.0)]),
    "pair_right_only_counts": config([pair(left_scale=0.0, right_scale=1.0)]),
    "feed_forward": config([delta(heads=1, kv_heads=1, ff=56)]),
}


def write_model(raw: dict, folder: str, seed: int = 3) -> str:
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.pugozen import PugozenConfig
    from carbon_engine_b200.weights.loader import write_random_model
    return write_random_model(PugozenConfig.from_dict(dict(raw)), folder, seed=seed)
