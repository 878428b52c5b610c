"""RMSNorm with the residual add fused in.

y = x * rsqrt(mean(x^2) + eps) * weight, the weight multiplying after the normalisation
(helios/crates/helios-hal/kernels/rmsnorm.cu:22-58); the fused form first adds the pending delta into
the residual stream (rmsnorm.cu:66-122).  The stream, the sum of squares and the products are float;
the result is rounded once to the activation type.  Parameters: ``hidden_size``, ``eps``, ``weight_name`` (the tensor's
name after the prefix, ``weight`` unless stated), ``one_plus`` (the tensor holds the weight's offset from one, which is added,
in float, when it is loaded), ``groups`` (1 unless stated: the row is cut into that many equal consecutive parts and each is
divided by its own sqrt(mean(part^2) + eps); the weight still has an entry per column).

``add_normed`` is the other placement of the same norm: h <- h + norm(y), for blocks that normalise what a sublayer
returns instead of what it reads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from .. import ops
from .base import BuildContext, Norm, WeightSpec, register_norm
from .spec import PartSpec


@dataclass
class GatedResult:
    """What a sublayer returned together with the pre-activations of a gate on it: ``gate`` [tokens, hidden] float (a tensor, or a product
    still in its split-K pieces) plus the vector ``bias``.  Whoever reads it multiplies ``y``, entry by entry, by sigmoid(gate + bias).  A
    norm that normalises a sublayer's output does so in its own launch (``ops.norm_add_norm``, which also adds up the pieces and the bias);
    any other reader calls :meth:`tensor`."""

    y: object  # a tensor, or a product still in its split-K pieces
    gate: object
    bias: Optional[torch.Tensor] = None

    def tensor(self) -> torch.Tensor:
        y = self.y.tensor() if hasattr(self.y, "tensor") else self.y
        gate = self.gate.tensor() if hasattr(self.gate, "tensor") else self.gate
        if self.bias is not None:
            gate = gate + self.bias
        ops.sigmoid_gate_(y, gate, 0)
        return y


def _ungated(y):
    """(the sublayer's output as a tensor, its gate or None, the gate's bias or None)"""
    if isinstance(y, GatedResult):
        return (y.y.tensor() if hasattr(y.y, "tensor") else y.y), y.gate, y.bias
    return (y.tensor() if hasattr(y, "tensor") else y), None, None


@dataclass
class NormedDelta:
    """What a sublayer returned, still to be normalised by ``norm`` (an :class:`RMSNorm`) before it is added to the stream,
    plus a vector ``offset`` that is added to every row after it.  Either may be absent.  The next norm that reads the stream
    does all of it in its own launch (``ops.norm_add_norm``)."""

    y: Optional[torch.Tensor]
    norm: Optional["RMSNorm"]
    offset: Optional[torch.Tensor] = None

    def apply(self, h: torch.Tensor) -> None:
        """Do it now, for a reader of the stream that is not a norm."""
        y, gate, gate_bias = _ungated(self.y)
        ops.norm_add_norm(h, y, self.norm.weight if y is not None else None, self.norm.eps if y is not None else 0.0, self.offset, None, 0.0, h.dtype, gate=gate,
                          gate_bias=gate_bias)


@dataclass
class SumOfTwo:
    """What two sublayers that read the same rows returned, still to be added to the stream: first to one another, then to the
    stream.  The next norm that reads the stream does it in its own launch (``ops.add_group_rmsnorm``).  Either may be absent."""

    first: Optional[torch.Tensor]
    second: Optional[torch.Tensor]

    def parts(self) -> tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        return tuple(d.tensor() if hasattr(d, "tensor") else d for d in (self.first, self.second))

    def tensor(self) -> Optional[torch.Tensor]:
        """The sum as one tensor, for a reader of the stream that adds a single delta."""
        first, second = self.parts()
        if first is None or second is None:
            return first if second is None else second
        return first.float() + second.float()


def with_offset(h: torch.Tensor, delta, row: torch.Tensor):
    """The pending addition ``delta`` (None, a tensor, split-K pieces or a :class:`NormedDelta`) with ``row`` added after it."""
    if isinstance(delta, NormedDelta):
        if delta.offset is not None:
            row = delta.offset + row
        return NormedDelta(delta.y, delta.norm, row)
    if delta is not None:
        h += (delta.tensor() if hasattr(delta, "tensor") else delta).to(h.dtype)
    return NormedDelta(None, None, row)


class RMSNorm(Norm):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.weight_name = str(spec.params.get("weight_name", "weight"))
        self.one_plus = bool(spec.params.get("one_plus", False))
        self.groups = int(spec.params.get("groups", 1) or 1)
        if self.groups < 1 or self.hidden % self.groups:
            raise ValueError(f"{self.groups} groups do not divide a row of {self.hidden}")
        self.weight: Optional[torch.Tensor] = None

    def weights(self) -> dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden,), init="normal" if self.one_plus else "one_plus_normal")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].to(torch.float32).contiguous()
        if self.one_plus:
            self.weight = (1.0 + self.weight).contiguous()

    def kernel_modules(self):
        return [("elementwise", {})]

    def forward(self, h, delta, rows=None):
        if isinstance(delta, GatedResult):  # a gated result that no norm stands on: multiplied here, added below
            delta = delta.tensor()
        if self.groups > 1 or isinstance(delta, SumOfTwo):
            if isinstance(delta, NormedDelta):
                delta.apply(h)
                delta = None
            first, second = delta.parts() if isinstance(delta, SumOfTwo) else (delta.tensor() if hasattr(delta, "tensor") else delta, None)
            if first is not None and second is not None and first.dtype != second.dtype:
                first, second = first.float(), second.float()
            return ops.add_group_rmsnorm(h, first, second, self.weight, self.groups, self.eps, self.dtype, rows)
        if isinstance(delta, NormedDelta):
            y, gate, gate_bias = _ungated(delta.y)
            return ops.norm_add_norm(h, y, delta.norm.weight if y is not None else None, delta.norm.eps if y is not None else 0.0, delta.offset,
                                     self.weight, self.eps, self.dtype, rows, gate=gate, gate_bias=gate_bias)
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self.dtype, rows)

    def add_normed(self, h, y):
        """h <- h + norm(y) in the float stream; returns the new stream in the activation type (``h`` itself in float32)."""
        if self.groups > 1:
            raise ValueError("a norm in groups stands where a sublayer reads the stream, not on a sublayer's output")
        if hasattr(y, "tensor"):
            y = y.tensor()
        if self.dtype == torch.float32:
            ops.rmsnorm_add(h, y, self.weight, self.eps)
            return h
        return ops.rmsnorm_add(h, y, self.weight, self.eps, copy_dtype=self.dtype)


register_norm("rmsnorm", RMSNorm)
