"""Tobadra expressed as parts: a decoder whose sublayers are normalised on both sides and gated, whose mixers read their input through a
short convolution, and whose layers may lend their tensors to later ones.

The stream starts as the normalised embedding row.  Every layer is the sandwich arrangement
(x <- x + norm_b(mixer(norm_a(x))); x <- x + norm_d(ff(norm_c(x)))) in which each sublayer's result is first multiplied by
sigmoid(W a + b) of the normalised rows a it was handed (``gated_output``, ``gated_feed_forward``) and the mixer reads a + conv(a), a causal
convolution over time per channel whose last rows are part of a request's state (``input_convolution``).  Mixers: grouped-query
attention inside a sliding window with a rotation of part of every query and key head and values rotated over their whole size
(``rotated_value_attention``); lightning attention, a matrix state per head with a constant decay (``lightning``); the gated delta rule
with a decay per key channel (``channel_delta``).  Feed-forwards: one without a gate (tanh-form GELU), or experts chosen by softmax
scores with a correction inside the best groups, some of them identities, plus a gated shared expert (``scored_experts``, exact GELU);
or none.  A layer with ``weights_of`` is one more schedule entry of the layer it names: the same parts, pages or a state of its own.
The head is the embedding table, the logits times ``logit_scale``.  Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``norm1b``,
``norm2``, ``norm2b``, ``l<i>.canon1``, ``l<i>.rg1``, ``rg1.b``, ``rg2``, ``rg2.b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.  The design states no
limit on positions; the engine's own limit of 2^30 stands in.
"""
from __future__ import annotations

from ..config.tobadra import ARCHITECTURE, DenseFF, TobadraConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from .registry import Architecture, register_architecture

NO_POSITION_LIMIT = 1 << 30


def build_spec(config: TobadraConfig) -> ModelSpec:
    width, eps = config.width, config.eps
    layers, place, tolerated = [], {}, []
    for index, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        prefix = f"l{index}."
        m = layer.mixer
        if layer.type == "attention":
            position = value_position = None
            if m.rot_dims:
                position = PartSpec("rope_half_partial", "", {"dims": m.rot_dims, "base": m.rot_base})
                value_position = PartSpec("rope_half_partial", "", {"dims": m.vdim, "base": m.rot_base})
            mixer = PartSpec("rotated_value_attention", "mix.", {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim,
                                                                 "value_dim": m.vdim, "scale": m.scale, "window": m.window, "bias": True,
                                                                 "position": position, "value_position": value_position})
        elif layer.type == "lightning":
            mixer = PartSpec("lightning", "mix.", {"hidden_size": width, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "decay": tuple(m.decay),
                                                   "eps": eps})
        else:
            mixer = PartSpec("channel_delta", "mix.", {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                                                       "conv": m.conv, "eps": eps, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank})
        if config.taps:
            mixer = PartSpec("input_convolution", "", {"hidden_size": width, "taps": config.taps, "weight_name": "canon1", "inner": mixer})
        mixer = PartSpec("gated_output", prefix, {"hidden_size": width, "weight_name": "rg1", "bias_name": "rg1.b", "inner": mixer})

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", prefix, {"hidden_size": width, "eps": eps, "weight_name": name})

        norms = {"input": norm("norm1"), "mixer_out": norm("norm1b")}
        feed_forward = None
        if layer.mlp is None:  # a checkpoint may carry the feed-forward's norms and gate all the same; nothing reads them
            tolerated += [prefix + name for name in ("norm2", "norm2b", "rg2", "rg2.b")]
        else:
            norms.update({"post_mixer": norm("norm2"), "feed_forward_out": norm("norm2b")})
            if isinstance(layer.mlp, DenseFF):
                inner = PartSpec("activated_mlp", "mlp.", {"hidden_size": width, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh",
                                                           "names": {"up": "up", "down": "down"}})
            else:
                f = layer.mlp
                inner = PartSpec("scored_experts", "mlp.", {"hidden_size": width, "experts": f.experts, "identity": f.identity, "top": f.top,
                                                            "expert_size": f.ff, "activation": "gelu_erf", "scale": f.scale, "group_count": f.group_count,
                                                            "group_keep": f.group_keep, "shared_size": f.shared_ff})
            feed_forward = PartSpec("gated_feed_forward", prefix, {"hidden_size": width, "weight_name": "rg2", "bias_name": "rg2.b", "inner": inner})
        place[index] = len(layers)
        layers.append(LayerSpec(arrangement="sandwich_norm", mixer=mixer, feed_forward=feed_forward, norms=norms))
    sizes = {"vocab_size": config.vocab, "hidden_size": width}
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", "", {**sizes, "weight_name": "embed", "norm_weight_name": "embed.norm", "eps": eps}),
        layers=tuple(layers),
        schedule=tuple(Run(place[config.source_of(index)]) for index in range(len(config.layers))),
        final_norm=PartSpec("rmsnorm", "final.", {"hidden_size": width, "eps": eps, "weight_name": "norm"}),
        head=PartSpec("linear_head", "", {**sizes, "tied": True, "scale": config.logit_scale}),
        tolerated=tuple(tolerated),
    )


register_architecture(Architecture(ARCHITECTURE, TobadraConfig.from_dict, build_spec, TobadraConfig.to_dict))
