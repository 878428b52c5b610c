"""Kudazen expressed as parts: a decoder whose sublayers run side by side and whose layers may lend their tensors to later ones.

Every layer is the side-by-side arrangement (h = norm(x); x <- x + (mixer(h) + ff(h)), one norm that both sublayers read) of one
of three mixers: grouped-query attention without rotation that sees its own chunk of positions, with a temperature per head, a
bias that grows with the distance and unit-RMS values (``sloped_attention``); attention over one small latent per token with
a rotated key part shared by all heads and a sink in the softmax (``latent_attention``); time mixing with a matrix state per head
and a decay computed from the token (``wkv``); with a gated feed-forward whose gate and value are clamped (``clamped_glu``), or none.
The norm divides each of ``norm.groups`` equal parts of the row by its own root mean square.  A layer with ``weights_of`` is one more
schedule entry of the layer it names: the same parts, pages or a state of its own.  The head is the embedding table.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``.  The design states no limit on
positions; the engine's own limit of 2^30 stands in.
"""
from __future__ import annotations

from ..config.kudazen import ARCHITECTURE, KudazenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from .registry import Architecture, register_architecture

NO_POSITION_LIMIT = 1 << 30
GATE_SLOPE = 1.702  # the feed-forward's gate is g * sigmoid(1.702 g)
SLOPE_RANGE = 8.0  # head h of H takes the slope 2^(-8 (h + 1) / H)


def build_spec(config: KudazenConfig) -> ModelSpec:
    width, eps, groups = config.width, config.eps, config.norm_groups
    layers, place = [], {}
    for index, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        prefix = f"l{index}."
        m = layer.mixer
        if layer.type == "attention":
            slopes = tuple(2.0 ** (-SLOPE_RANGE * (h + 1) / m.heads) for h in range(m.heads))
            mixer = PartSpec("sloped_attention", prefix + "mix.", {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim,
                                                                   "value_dim": m.vdim, "scale": m.scale, "chunk": m.chunk, "slopes": slopes,
                                                                   "value_unit_rms": True, "head_temperature": True, "eps": eps})
        elif layer.type == "latent_attention":
            position = PartSpec("rope_interleaved", "", {"dims": m.rot_dims, "base": m.rot_base})
            mixer = PartSpec("latent_attention", prefix + "mix.", {"hidden_size": width, "heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                                                                   "value_dim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale,
                                                                   "position": position, "sink": True, "eps": eps})
        else:
            mixer = PartSpec("wkv", prefix + "mix.", {"hidden_size": width, "heads": m.heads, "head_dim": m.dim, "decay_rank": m.decay_rank or 16, "eps": eps})
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec("clamped_glu", prefix + "mlp.", {"hidden_size": width, "intermediate_size": layer.mlp.ff, "limit": layer.mlp.limit,
                                                                     "gate_slope": GATE_SLOPE, "names": {"gate": "gate", "up": "up", "down": "down"}})
        norms = {"input": PartSpec("rmsnorm", prefix, {"hidden_size": width, "eps": eps, "groups": groups, "weight_name": "norm1"})}
        place[index] = len(layers)
        layers.append(LayerSpec(arrangement="side_by_side", mixer=mixer, feed_forward=feed_forward, norms=norms))
    sizes = {"vocab_size": config.vocab, "hidden_size": width}
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", "", {**sizes, "weight_name": "embed"}),
        layers=tuple(layers),
        schedule=tuple(Run(place[config.source_of(index)]) for index in range(len(config.layers))),
        final_norm=PartSpec("rmsnorm", "final.", {"hidden_size": width, "eps": eps, "groups": groups, "weight_name": "norm"}),
        head=PartSpec("linear_head", "", {**sizes, "tied": True}),
    )


register_architecture(Architecture(ARCHITECTURE, KudazenConfig.from_dict, build_spec, KudazenConfig.to_dict))
