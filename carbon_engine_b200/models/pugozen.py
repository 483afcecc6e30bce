"""The Pugozen decoder, put together from the package's parts.

Every layer normalises once (RMS norm) and both sublayers read that: x += mixer(norm1(x)) + ff(norm1(x))
(``parts/block.py`` ``ParallelBlock``).  The mixer is, as config.json lists them, retention (``parts/retention.py``), the
gated delta rule with one decay per head (``parts/gated_delta.py`` ``HeadGatedDelta``), or two mixers side by side whose
outputs are added with fixed weights (``parts/combine.py``): softmax attention whose values are the projected keys, with a
norm per head, a partial rotation, a temperature and a sink per head (``parts/sink_attention.py``), beside the gated delta
rule with a decay per head and key channel (``ChannelGatedDelta``).  The feed-forward is down(relu(up h)^2), or absent.  A
layer may run another layer's weights with a cache of its own, which the model's schedule expresses as a second call of
that layer's block.  The embedding rows are scaled.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*`` (``.left.*`` and ``.right.*`` for the pair), ``l<i>.mlp.up|down``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.pugozen import DELTA, PARALLEL, RETENTION, PugozenConfig, weight_owner
from ..config.registry import register_architecture
from ..parts.block import ParallelBlock
from ..parts.embedding import Embedding, LMHead
from ..parts.model import DecoderModel, LayerCall
from ..parts.registry import build_part


def build_pugozen(cfg: PugozenConfig, max_positions: int) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: build_part("norm", "rmsnorm", width=W, eps=eps, name=name)
    rotations = {}            # one table per (head size, rotated elements, base)

    def rotation(m: dict):
        rot = m.get("rot")
        if not rot:
            return None
        key = (m["dim"], rot["dims"], float(rot["base"]))
        if key not in rotations:
            rotations[key] = build_part("position", "rotary", head_dim=key[0], theta=key[2], max_positions=max_positions,
                                        rotary_dim=key[1])
        return rotations[key]

    def delta(m: dict, prefix: str, channel: bool):
        if channel:
            return build_part("mixer", "channel_gated_delta", hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"],
                              vdim=m["vdim"], taps=m["conv"], prefix=prefix, eps=eps, decay_rank=m.get("a_rank") or -1,
                              gate_rank=m.get("g_rank") or -1)
        return build_part("mixer", "head_gated_delta", hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"],
                          vdim=m["vdim"], taps=m["conv"], prefix=prefix, eps=eps, gate="silu")

    blocks, block_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}", layer["mixer"]
        if layer["type"] == RETENTION:
            mixer = build_part("mixer", "retention", hidden=W, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], decay=m["decay"],
                               prefix=f"{p}.mix", eps=eps, position=rotation(m), gate="silu")
        elif layer["type"] == DELTA:
            mixer = delta(m, f"{p}.mix", channel=False)
        else:
            assert layer["type"] == PARALLEL
            left = m["left"]
            attention = build_part("mixer", "sink_attention", hidden=W, heads=left["heads"], kv_heads=left["kv_heads"],
                                   dim=left["dim"], prefix=f"{p}.mix.left", eps=eps, position=rotation(left), scale=left["scale"],
                                   qk_norm=True, tied_values=True, head_temperature=True, sink=True)
            mixer = build_part("mixer", "summed_mixers", members=[attention, delta(m["right"], f"{p}.mix.right", channel=True)],
                               weights=[m["left_scale"], m["right_scale"]])
        ffn = None
        if layer["mlp"] is not None:
            ffn = build_part("feed_forward", "dense_mlp", hidden=W, intermediate=layer["mlp"]["ff"], prefix=f"{p}.mlp",
                             activation="relu2", names=("up", "down"))
        block_of[i] = len(blocks)
        blocks.append(ParallelBlock(norm(f"{p}.norm1"), mixer, ffn))
    schedule = [LayerCall(block_of[weight_owner(cfg.layers, i)], i, True) for i in range(len(cfg.layers))]
    embedding = Embedding(cfg.vocab_size, W, "embed", scale=cfg.embedding_scale)
    head = LMHead(cfg.vocab_size, W, norm("final.norm"), "head")
    return DecoderModel(cfg, embedding, blocks, head, schedule=schedule)


register_architecture("Pugozen", PugozenConfig.from_dict, build_pugozen, model_types=("pugozen",), replace=True)
