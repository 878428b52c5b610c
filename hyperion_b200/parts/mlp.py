"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases.

gate and up are fused into one [2I, H] matrix at load, as the reference places them back to back for one
matrix product (helios/crates/helios-hal/src/backends/hopper_sm90/backend.rs:95-106, session.rs:779-793);
silu(g) = g / (1 + exp(-g)) in float (kernels/elementwise.cu:28-37).  In bfloat16, when the intermediate size
allows it, the rows alternate in runs of 128 gate rows and their 128 up rows, so that a prompt-sized
product can apply SwiGLU in its epilogue (``ops.gated_linear``); otherwise the gate rows come first.
Parameters: ``hidden_size``, ``intermediate_size``, ``names`` (the three tensors' names after the prefix as
``{"gate": ..., "up": ..., "down": ...}``; the Hugging Face names unless stated).
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import gemm
from .base import BuildContext, FeedForward, WeightSpec, register_feed_forward
from .spec import PartSpec


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        names = dict(spec.params.get("names") or {})
        self.gate_name, self.up_name = names.get("gate", "gate_proj.weight"), names.get("up", "up_proj.weight")
        self.down_name = names.get("down", "down_proj.weight")

    def weights(self) -> dict[str, WeightSpec]:
        return {self.gate_name: WeightSpec((self.inter, self.hidden)), self.up_name: WeightSpec((self.inter, self.hidden)),
                self.down_name: WeightSpec((self.hidden, self.inter))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pair = [tensors[self.gate_name], tensors[self.up_name]]
        dtype = _common_dtype(pair)
        if dtype == torch.bfloat16 and self.inter % gemm.SWIGLU_BLOCK == 0:
            self.block = gemm.SWIGLU_BLOCK
            self.w_gate_up = gemm.interleave_gate_up(pair[0], pair[1])
        else:
            self.block = None
            self.w_gate_up = torch.cat([t.to(dtype) for t in pair], dim=0).contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def kernel_modules(self):
        if self.dtype == torch.float32:
            return [("elementwise", {}), ("sgemm_f32", {})]
        return [("elementwise", {}), ("gemm_tcgen05", {}), ("gemm_pair_tcgen05", {})]

    def forward(self, x, step):
        act = ops.gated_linear(x, self.w_gate_up, self.block, self.dtype)
        return ops.linear(act, self.w_down, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_feed_forward("swiglu", SwiGLU)


class ActivatedMLP(FeedForward):
    """The feed-forward without a gate: down(act(up(x))), no biases, act = the tanh form of GELU or its exact (erf) form.
    Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` (``gelu_tanh`` or ``gelu_erf``), ``names`` (``{"up": ..., "down": ...}``)."""

    ACTIVATIONS = {"gelu_tanh": "gelu_tanh", "gelu_erf": "gelu_erf"}  # the name of the activation -> the operation of ``ops``

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.params.get("activation", "gelu_tanh"))
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"no activation {self.activation!r} (known: {sorted(self.ACTIVATIONS)})")
        names = dict(spec.params.get("names") or {})
        self.up_name, self.down_name = names.get("up", "up_proj.weight"), names.get("down", "down_proj.weight")

    def weights(self) -> dict[str, WeightSpec]:
        return {self.up_name: WeightSpec((self.inter, self.hidden)), self.down_name: WeightSpec((self.hidden, self.inter))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = tensors[self.up_name].contiguous(), tensors[self.down_name].contiguous()

    def kernel_modules(self):
        return [("elementwise", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def forward(self, x, step):
        act = getattr(ops, self.ACTIVATIONS[self.activation])(ops.linear(x, self.w_up, None, self.dtype))
        return ops.linear(act, self.w_down, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_feed_forward("activated_mlp", ActivatedMLP)


class ClampedGLU(FeedForward):
    """A gated feed-forward whose gate and value are clamped: g = min(gate(x), limit), u = clamp(up(x), -limit, limit),
    down(g * sigmoid(slope * g) * (u + 1)), no biases.  gate and up are one [2I, H] matrix, the gate rows first.
    Parameters: ``hidden_size``, ``intermediate_size``, ``limit``, ``gate_slope``, ``names`` (as for ``swiglu``)."""

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.limit = float(spec.params["limit"])
        self.slope = float(spec.params.get("gate_slope", 1.0))
        names = dict(spec.params.get("names") or {})
        self.gate_name, self.up_name = names.get("gate", "gate_proj.weight"), names.get("up", "up_proj.weight")
        self.down_name = names.get("down", "down_proj.weight")

    def weights(self) -> dict[str, WeightSpec]:
        return {self.gate_name: WeightSpec((self.inter, self.hidden)), self.up_name: WeightSpec((self.inter, self.hidden)),
                self.down_name: WeightSpec((self.hidden, self.inter))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pair = [tensors[self.gate_name], tensors[self.up_name]]
        dtype = _common_dtype(pair)
        self.w_gate_up = torch.cat([t.to(dtype) for t in pair], dim=0).contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def kernel_modules(self):
        return [("elementwise", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def forward(self, x, step):
        act = ops.clamped_glu(ops.linear(x, self.w_gate_up, None, self.dtype), self.limit, self.slope)
        return ops.linear(act, self.w_down, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_feed_forward("clamped_glu", ClampedGLU)
