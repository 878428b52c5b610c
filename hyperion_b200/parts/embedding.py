"""Token embedding and output head.

h[t] = table[ids[t]] (helios/crates/helios-hal/kernels/elementwise.cu:13-19); logits = x head^T kept in
float, where head is ``lm_head.weight`` or, with tied embeddings, the embedding table
(helios/crates/helios-hal/src/backends/hopper_sm90/forward.rs:45-51, session.rs:844-848).
Parameters: ``vocab_size``, ``hidden_size``, ``weight_name`` (the tensor's name after the prefix, ``weight``
unless stated); the embedding also ``scale`` (the looked-up row is multiplied by it in float, 1 unless
stated) and ``norm_weight_name`` with ``eps`` (unless absent: the looked-up row passes an RMS norm with that weight
before it becomes the stream); the head also ``tied`` (then it owns no tensor and is handed the embedding's table)
and ``scale`` (the logits are multiplied by it, 1 unless stated).

``offset_table`` is a learned table [count, hidden] of vectors that the schedule adds to the stream before an entry
runs (a model that passes some layers several times marks each pass this way).  Parameters: ``count``, ``hidden_size``,
``weight_name``.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from .base import BuildContext, Embedding, Head, StreamOffsets, WeightSpec, register_embedding, register_head, register_stream_offsets
from .spec import PartSpec


class TokenEmbedding(Embedding):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.weight_name = str(spec.params.get("weight_name", "weight"))
        self.norm_name = spec.params.get("norm_weight_name")
        self.eps = float(spec.params.get("eps", 0.0))
        self.norm_weight = None

    def weights(self):
        wanted = {self.weight_name: WeightSpec((self.vocab, self.hidden))}
        if self.norm_name is not None:
            wanted[str(self.norm_name)] = WeightSpec((self.hidden,), init="one_plus_normal")
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name].contiguous()
        if self.norm_name is not None:
            self.norm_weight = tensors[str(self.norm_name)].to(torch.float32).contiguous()

    def kernel_modules(self):
        return [("elementwise", {})]

    def forward(self, token_ids):
        h = ops.embedding(self.table, token_ids, scale=self.scale)
        if self.norm_weight is not None:  # the stream starts as the normalised row, in float
            h = ops.add_rmsnorm(h, None, self.norm_weight, self.eps, torch.float32)
        return h

    def shared_table(self):
        return self.table


class LinearHead(Head):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.weight_name = str(spec.params.get("weight_name", "weight"))
        self.scale = float(spec.params.get("scale", 1.0))
        self.weight = None

    def weights(self):
        return {} if self.tied else {self.weight_name: WeightSpec((self.vocab, self.hidden))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors[self.weight_name].contiguous()

    def wants_shared_table(self) -> bool:
        return self.tied

    def use_shared_table(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"the tied head wants a table of {(self.vocab, self.hidden)}, the embedding shares {tuple(table.shape)}")
        self.weight = table

    def kernel_modules(self):
        return [("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})] + ([("elementwise", {})] if self.scale != 1.0 else [])

    def forward(self, x):
        logits = ops.linear(x, self.weight, None, torch.float32)
        return ops.scale_(logits, self.scale) if self.scale != 1.0 else logits


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)


class OffsetTable(StreamOffsets):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.count = int(spec.params["count"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight_name = str(spec.params.get("weight_name", "weight"))

    def weights(self):
        return {self.weight_name: WeightSpec((self.count, self.hidden))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name].to(torch.float32).contiguous()

    def row(self, index: int) -> torch.Tensor:
        return self.table[index]


register_stream_offsets("offset_table", OffsetTable)
