"""Typed configuration of the Kudazen decoder.

Its config.json is nested: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``norm.groups`` and ``layers``, a list
whose entries give ``type`` (``attention``, ``latent_attention`` or ``wkv``), the mixer's sizes under ``mixer``, the feed-forward
under ``mlp`` (``{"kind": "dense", "ff": n, "limit": c}`` or null) and optionally ``weights_of``: the index of the layer whose
tensors this layer uses (it then has none of its own, but a cache or state of its own).  Every size and constant is read from
there; nothing is assumed equal between layers.  A key that is missing or of the wrong kind is refused by name.
``decay_rank`` under a ``wkv`` mixer is this package's own key: the inner size of the decay's two small matrices when random
weights are made (a checkpoint's tensors decide otherwise).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .base import ConfigError
from .nunivik import _get, _positive_int, _positive_number

ARCHITECTURE = "Kudazen"


@dataclass(frozen=True)
class SlopedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int  # 0: every earlier key is seen


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    kv_heads: Optional[int]  # stated by some documents; the latent's matrices have one block per query head either way
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    rot_dims: int
    rot_base: float
    scale: float


@dataclass(frozen=True)
class WkvSizes:
    heads: int
    dim: int
    decay_rank: Optional[int] = None


@dataclass(frozen=True)
class ClampedFF:
    ff: int
    limit: float


@dataclass(frozen=True)
class KudazenLayer:
    type: str
    mixer: Any
    mlp: Optional[ClampedFF]
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class KudazenConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    layers: tuple[KudazenLayer, ...]
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
    def from_dict(cls, document: dict[str, Any]) -> "KudazenConfig":
        if not isinstance(document, dict):
            raise ConfigError("<root>", "must be a JSON object")
        if document.get("architecture") != ARCHITECTURE:
            raise ConfigError("architecture", f"must be {ARCHITECTURE!r}, got {document.get('architecture')!r}")
        width = _positive_int(document, "", "width")
        norm = _get(document, "", "norm")
        groups = _positive_int(norm, "norm.", "groups")
        if width % groups:
            raise ConfigError("norm.groups", f"{groups} does not divide the width {width}")
        entries = _get(document, "", "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers", "must be a non-empty list")
        layers: list[KudazenLayer] = []
        for index, entry in enumerate(entries):
            path = f"layers[{index}]."
            kind = _get(entry, path, "type")
            mixer = _get(entry, path, "mixer")
            if kind == "attention":
                parsed: Any = _sloped(mixer, path + "mixer.")
            elif kind == "latent_attention":
                parsed = _latent(mixer, path + "mixer.")
            elif kind == "wkv":
                rank = mixer.get("decay_rank") if isinstance(mixer, dict) else None
                parsed = WkvSizes(heads=_positive_int(mixer, path + "mixer.", "heads"), dim=_positive_int(mixer, path + "mixer.", "dim"),
                                  decay_rank=_positive_int(mixer, path + "mixer.", "decay_rank") if rank is not None else None)
            else:
                raise ConfigError(path + "type", f"{kind!r} is not a mixer of this design (attention, latent_attention, wkv)")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if _get(mlp, path + "mlp.", "kind") != "dense":
                    raise ConfigError(path + "mlp.kind", f"{mlp.get('kind')!r} is not supported (only 'dense')")
                ff = ClampedFF(_positive_int(mlp, path + "mlp.", "ff"), _positive_number(mlp, path + "mlp.", "limit"))
            source = entry.get("weights_of")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < len(entries) or source == index:
                    raise ConfigError(path + "weights_of", f"must name another layer of the model, got {source!r}")
            layers.append(KudazenLayer(kind, parsed, ff, source))
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
        return cls(vocab=_positive_int(document, "", "vocab"), width=width, eps=_positive_number(norm, "norm.", "eps"), norm_groups=groups,
                   layers=tuple(layers), eos_token_ids=eos_ids)

    def to_dict(self) -> dict[str, Any]:
        """The config.json document this configuration is read back from."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer: dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.chunk:
                    mixer["mask"] = {"size": m.chunk}
            elif layer.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank,
                         "rot": {"dims": m.rot_dims, "base": m.rot_base}, "scale": m.scale}
                if m.kv_heads is not None:
                    mixer["kv_heads"] = m.kv_heads
            else:
                mixer = {"heads": m.heads, "dim": m.dim}
                if m.decay_rank is not None:
                    mixer["decay_rank"] = m.decay_rank
            entry: dict[str, Any] = {"type": layer.type, "mixer": mixer,
                                     "mlp": {"kind": "dense", "ff": layer.mlp.ff, "limit": layer.mlp.limit} if layer.mlp is not None else None}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        document: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                                    "norm": {"eps": self.eps, "groups": self.norm_groups}, "layers": layers}
        if self.eos_token_ids:
            document["eos_token_id"] = list(self.eos_token_ids)
        return document


def _sloped(m: Any, path: str) -> SlopedAttentionSizes:
    heads, kv_heads = _positive_int(m, path, "heads"), _positive_int(m, path, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(path + "kv_heads", f"{kv_heads} does not divide heads {heads}")
    mask = m.get("mask")
    return SlopedAttentionSizes(heads=heads, kv_heads=kv_heads, dim=_positive_int(m, path, "dim"), vdim=_positive_int(m, path, "vdim"),
                                scale=_positive_number(m, path, "scale"), chunk=_positive_int(mask, path + "mask.", "size") if mask is not None else 0)


def _latent(m: Any, path: str) -> LatentAttentionSizes:
    heads = _positive_int(m, path, "heads")
    kv_heads = None
    if isinstance(m, dict) and m.get("kv_heads") is not None:
        kv_heads = _positive_int(m, path, "kv_heads")  # kept for the write-back only: the tensors' shapes decide
    rot_dim = _positive_int(m, path, "rot_dim")
    rot = _get(m, path, "rot")
    rot_dims = _positive_int(rot, path + "rot.", "dims")
    if rot_dims % 2 or rot_dims > rot_dim:
        raise ConfigError(path + "rot.dims", f"{rot_dims} must be even and at most rot_dim {rot_dim}")
    return LatentAttentionSizes(heads=heads, kv_heads=kv_heads, dim=_positive_int(m, path, "dim"), rot_dim=rot_dim, vdim=_positive_int(m, path, "vdim"),
                                kv_rank=_positive_int(m, path, "kv_rank"), q_rank=_positive_int(m, path, "q_rank"), rot_dims=rot_dims,
                                rot_base=_positive_number(rot, path + "rot.", "base"), scale=_positive_number(m, path, "scale"))
