"""Typed configuration of the Tobadra decoder.

Its config.json is nested: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (the taps of the convolution every
mixer reads its input through), ``logit_scale`` and ``layers``, a list whose entries give ``type`` (``attention``, ``lightning`` or
``channel_delta``), the mixer's sizes under ``mixer``, the feed-forward under ``mlp`` (``{"kind": "dense", "ff": n}``,
``{"kind": "moe", "expert": {"ff": n}, "router": {...}, "shared": {"ff": n} or absent}`` or null) and optionally ``weights_of``: the index
of the layer whose tensors this layer uses (it then has none of its own, but a cache or state of its own).  Every size and constant is
read from there; nothing is assumed equal between layers.  A key that is missing or of the wrong kind is refused by name.
``decay_rank`` and ``gate_rank`` under a ``channel_delta`` mixer are this package's own keys: the inner sizes of the decay's and the
gate's two small matrices when random weights are made (a checkpoint's tensors decide otherwise).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Optional

from .base import ConfigError
from .nunivik import _get, _positive_int, _positive_number

ARCHITECTURE = "Tobadra"


@dataclass(frozen=True)
class WindowAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int  # 0: every earlier key is seen
    rot_dims: int  # 0: nothing is rotated, values neither
    rot_base: float


@dataclass(frozen=True)
class LightningSizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]


@dataclass(frozen=True)
class ChannelDeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class ExpertsFF:
    ff: int
    experts: int  # the experts with matrices
    identity: int  # router outputs after them that hand their input on as it is
    top: int
    scale: float
    group_count: int  # 0: the choice is made over all outputs at once
    group_keep: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class TobadraLayer:
    type: str
    mixer: Any
    mlp: Any  # DenseFF, ExpertsFF or None
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class TobadraConfig:
    vocab: int
    width: int
    eps: float
    taps: int
    logit_scale: float
    layers: tuple[TobadraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = field(default=ARCHITECTURE)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def source_of(self, index: int) -> int:
        """The layer whose tensors layer ``index`` uses (itself unless it names another)."""
        while self.layers[index].weights_of is not None:
            index = self.layers[index].weights_of
        return index

    @classmethod
    def from_dict(cls, document: dict[str, Any]) -> "TobadraConfig":
        if not isinstance(document, dict):
            raise ConfigError("<root>", "must be a JSON object")
        if document.get("architecture") != ARCHITECTURE:
            raise ConfigError("architecture", f"must be {ARCHITECTURE!r}, got {document.get('architecture')!r}")
        width = _positive_int(document, "", "width")
        norm = _get(document, "", "norm")
        canon = document.get("canon")
        taps = _positive_int(canon, "canon.", "taps") if canon is not None else 0
        entries = _get(document, "", "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers", "must be a non-empty list")
        layers: list[TobadraLayer] = []
        for index, entry in enumerate(entries):
            path = f"layers[{index}]."
            kind = _get(entry, path, "type")
            mixer = _get(entry, path, "mixer")
            if kind == "attention":
                parsed: Any = _attention(mixer, path + "mixer.")
            elif kind == "lightning":
                parsed = _lightning(mixer, path + "mixer.")
            elif kind == "channel_delta":
                parsed = _channel_delta(mixer, path + "mixer.")
            else:
                raise ConfigError(path + "type", f"{kind!r} is not a mixer of this design (attention, lightning, channel_delta)")
            mlp = entry.get("mlp")
            ff: Any = None
            if mlp is not None:
                ff_kind = _get(mlp, path + "mlp.", "kind")
                if ff_kind == "dense":
                    ff = DenseFF(_positive_int(mlp, path + "mlp.", "ff"))
                elif ff_kind == "moe":
                    ff = _experts(mlp, path + "mlp.")
                else:
                    raise ConfigError(path + "mlp.kind", f"{ff_kind!r} is not supported ('dense' or 'moe')")
            source = entry.get("weights_of")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < len(entries) or source == index:
                    raise ConfigError(path + "weights_of", f"must name another layer of the model, got {source!r}")
            layers.append(TobadraLayer(kind, parsed, ff, source))
        for index, layer in enumerate(layers):
            if layer.weights_of is None:
                continue
            seen, at = {index}, layer.weights_of
            while layers[at].weights_of is not None:  # a chain must end at a layer with tensors of its own
                if at in seen:
                    raise ConfigError(f"layers[{index}].weights_of", "the layers named lead back to this one")
                seen.add(at)
                at = layers[at].weights_of
            lender = layers[at]
            if (lender.type, lender.mixer, lender.mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"layers[{index}].weights_of", f"layer {at} has another mixer or feed-forward; a layer can only use the tensors of its like")
        eos = document.get("eos_token_id")
        eos_ids = tuple(eos if isinstance(eos, list) else [eos]) if eos is not None else ()
        scale = _positive_number(document, "", "logit_scale") if document.get("logit_scale") is not None else 1.0
        return cls(vocab=_positive_int(document, "", "vocab"), width=width, eps=_positive_number(norm, "norm.", "eps"), taps=taps, logit_scale=scale,
                   layers=tuple(layers), eos_token_ids=eos_ids)

    def to_dict(self) -> dict[str, Any]:
        """The config.json document this configuration is read back from."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer: dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.window:
                    mixer["mask"] = {"size": m.window}
                if m.rot_dims:
                    mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            elif layer.type == "lightning":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
                if m.decay_rank is not None:
                    mixer["decay_rank"] = m.decay_rank
                if m.gate_rank is not None:
                    mixer["gate_rank"] = m.gate_rank
            ff = layer.mlp
            if ff is None:
                mlp: Any = None
            elif isinstance(ff, DenseFF):
                mlp = {"kind": "dense", "ff": ff.ff}
            else:
                router: dict[str, Any] = {"experts": ff.experts, "top": ff.top, "scale": ff.scale, "identity": ff.identity}
                if ff.group_count:
                    router["groups"] = {"count": ff.group_count, "keep": ff.group_keep}
                mlp = {"kind": "moe", "expert": {"ff": ff.ff}, "router": router}
                if ff.shared_ff is not None:
                    mlp["shared"] = {"ff": ff.shared_ff}
            entry: dict[str, Any] = {"type": layer.type, "mixer": mixer, "mlp": mlp}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        document: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                                    "logit_scale": self.logit_scale, "layers": layers}
        if self.taps:
            document["canon"] = {"taps": self.taps}
        if self.eos_token_ids:
            document["eos_token_id"] = list(self.eos_token_ids)
        return document


def _attention(m: Any, path: str) -> WindowAttentionSizes:
    heads, kv_heads = _positive_int(m, path, "heads"), _positive_int(m, path, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(path + "kv_heads", f"{kv_heads} does not divide heads {heads}")
    dim, vdim = _positive_int(m, path, "dim"), _positive_int(m, path, "vdim")
    mask, rot = m.get("mask"), m.get("rot")
    rot_dims, rot_base = 0, 0.0
    if rot is not None:
        rot_dims, rot_base = _positive_int(rot, path + "rot.", "dims"), _positive_number(rot, path + "rot.", "base")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(path + "rot.dims", f"{rot_dims} must be even and at most dim {dim}")
        if vdim % 2:
            raise ConfigError(path + "vdim", f"values of {vdim} entries cannot be rotated in pairs")
    return WindowAttentionSizes(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_positive_number(m, path, "scale"),
                                window=_positive_int(mask, path + "mask.", "size") if mask is not None else 0, rot_dims=rot_dims, rot_base=rot_base)


def _lightning(m: Any, path: str) -> LightningSizes:
    heads = _positive_int(m, path, "heads")
    decay = _get(m, path, "decay")
    if not isinstance(decay, list) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not 0 <= d <= 1 or math.isnan(d)
                                                                  for d in decay):
        raise ConfigError(path + "decay", f"must list one number between 0 and 1 per head ({heads}), got {decay!r}")
    return LightningSizes(heads=heads, dim=_positive_int(m, path, "dim"), vdim=_positive_int(m, path, "vdim"), decay=tuple(float(d) for d in decay))


def _channel_delta(m: Any, path: str) -> ChannelDeltaSizes:
    heads, kv_heads = _positive_int(m, path, "heads"), _positive_int(m, path, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(path + "kv_heads", f"{kv_heads} does not divide heads {heads}")
    ranks = {key: (_positive_int(m, path, key) if m.get(key) is not None else None) for key in ("decay_rank", "gate_rank")}
    return ChannelDeltaSizes(heads=heads, kv_heads=kv_heads, dim=_positive_int(m, path, "dim"), vdim=_positive_int(m, path, "vdim"),
                             conv=_positive_int(m, path, "conv"), decay_rank=ranks["decay_rank"], gate_rank=ranks["gate_rank"])


def _experts(mlp: Any, path: str) -> ExpertsFF:
    router = _get(mlp, path, "router")
    experts, top = _positive_int(router, path + "router.", "experts"), _positive_int(router, path + "router.", "top")
    identity = router.get("identity") or 0
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise ConfigError(path + "router.identity", f"must be a non-negative integer, got {identity!r}")
    outputs = experts + identity
    groups = router.get("groups")
    count = keep = 0
    if groups is not None:
        count, keep = _positive_int(groups, path + "router.groups.", "count"), _positive_int(groups, path + "router.groups.", "keep")
        if outputs % count:
            raise ConfigError(path + "router.groups.count", f"{count} groups do not divide the router's {outputs} outputs")
        if keep > count:
            raise ConfigError(path + "router.groups.keep", f"{keep} of {count} groups")
    if top > (keep * (outputs // count) if count else outputs):
        raise ConfigError(path + "router.top", f"{top} experts cannot be chosen among those the router may choose from")
    shared = mlp.get("shared")
    return ExpertsFF(ff=_positive_int(_get(mlp, path, "expert"), path + "expert.", "ff"), experts=experts, identity=identity, top=top,
                     scale=_positive_number(router, path + "router.", "scale") if router.get("scale") is not None else 1.0, group_count=count, group_keep=keep,
                     shared_ff=_positive_int(shared, path + "shared.", "ff") if shared is not None else None)
