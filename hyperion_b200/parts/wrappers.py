"""Parts that wrap another part of their own kind and change what it reads or what it returns.  A wrapper is registered like any
mixer or feed-forward, builds its inner part from a :class:`PartSpec` among its parameters (the inner part's tensor names follow
the wrapper's own prefix), and hands on whatever the inner part keeps between steps, plans per step and compiles.

``input_convolution`` (mixer): the inner mixer reads ``x + conv(x)`` instead of ``x``: a causal convolution over time on every
channel of the rows, conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j) with zeros before the start of a sequence and no bias.  The
last ``taps - 1`` rows a request has read are its state (one float record per request, zero when the request takes its slot), so
the wrapper asks for that record *and* for whatever the inner mixer asks for.  Parameters: ``hidden_size``, ``taps``,
``weight_name`` (a tensor [hidden_size, taps]), ``inner`` (a PartSpec).

``gated_output`` (mixer) and ``gated_feed_forward``: the inner part's result is multiplied, element by element, by
sigmoid(W x + b) of the rows x that the wrapper itself was handed (the gate's product is kept in float; it travels beside the
result as a ``GatedResult``, so that a norm on the sublayer's output multiplies, normalises and adds in one launch).  Parameters:
``hidden_size``, ``weight_name``, ``bias_name``, ``inner`` (a PartSpec).
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import recurrent
from .base import FEED_FORWARDS, MIXERS, BuildContext, FeedForward, Mixer, RequestState, WeightSpec, make, register_feed_forward, register_mixer
from .norm import GatedResult
from .spec import PartSpec


def _round_up(value: int, step: int) -> int:
    return -(-value // step) * step


class _Wrapper:
    """What the wrappers share: the inner part's tensors under its own prefix, its modules and its step plans."""

    inner: object
    inner_prefix: str

    def _inner_weights(self) -> dict[str, WeightSpec]:
        return {self.inner_prefix + name: wanted for name, wanted in self.inner.weights().items()}

    def _load_inner(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.inner.load({name: tensors[self.inner_prefix + name] for name in self.inner.weights()})

    def step_plans(self):
        return getattr(self.inner, "step_plans", lambda: {})()


class ConvolvedInput(_Wrapper, Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.taps = int(p["hidden_size"]), int(p["taps"])
        if self.taps < 1:
            raise ValueError(f"a convolution of {self.taps} taps")
        self.weight_name = str(p["weight_name"])
        self.inner_prefix = p["inner"].prefix
        self.inner = make(MIXERS, p["inner"], build)
        self.record = _round_up(max(1, (self.taps - 1) * self.hidden), 4)

    def weights(self) -> dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden, self.taps)), **self._inner_weights()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].to(torch.float32).contiguous()
        self._load_inner(tensors)

    def _inner_requests(self) -> tuple:
        need = self.inner.cache_request()
        return need if isinstance(need, tuple) else (() if need is None else (need,))

    def cache_request(self):
        return (RequestState((self.record,), torch.float32), *self._inner_requests())

    def kernel_modules(self):
        return [("recurrent", {})] + self.inner.kernel_modules()

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache or len(cache) != 1 + len(self._inner_requests()):
            raise ValueError("the input convolution keeps a request's last rows; the schedule gave it no record of its own")
        own, rest = cache[0], cache[1:]
        read = recurrent.residual_conv(x, self.weight, own.state, 0, own.slots, step.token_row, step.row_start)
        recurrent.conv_state_keep(x, self.taps, own.state, 0, own.slots, step.row_start, step.n_rows)
        inner_need = self.inner.cache_request()
        view = tuple(rest) if isinstance(inner_need, tuple) else (rest[0] if rest else None)
        return self.inner.forward(read, step, view, own_cache)


def _gate_weights(part) -> dict[str, WeightSpec]:
    return {part.weight_name: WeightSpec((part.hidden, part.hidden)), part.bias_name: WeightSpec((part.hidden,))}


def _gated(part, x: torch.Tensor, y) -> GatedResult:
    """The inner part's result with the gate's pre-activations beside it: the norm that reads the result applies the gate in its own
    launch; any other reader multiplies when it asks for the tensor."""
    return GatedResult(y, ops.linear(x, part.w_gate, None, torch.float32, may_leave_partials=True), part.b_gate)


class GatedMixer(_Wrapper, Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.weight_name, self.bias_name = int(p["hidden_size"]), str(p["weight_name"]), str(p["bias_name"])
        self.inner_prefix = p["inner"].prefix
        self.inner = make(MIXERS, p["inner"], build)

    def weights(self) -> dict[str, WeightSpec]:
        return {**_gate_weights(self), **self._inner_weights()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate, self.b_gate = tensors[self.weight_name].contiguous(), tensors[self.bias_name].to(torch.float32).contiguous()
        self._load_inner(tensors)

    def cache_request(self):
        return self.inner.cache_request()

    def kernel_modules(self):
        return [("elementwise", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})] + self.inner.kernel_modules()

    def forward(self, x, step, cache, own_cache):
        return _gated(self, x, self.inner.forward(x, step, cache, own_cache))


class GatedFeedForward(_Wrapper, FeedForward):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.weight_name, self.bias_name = int(p["hidden_size"]), str(p["weight_name"]), str(p["bias_name"])
        self.inner_prefix = p["inner"].prefix
        self.inner = make(FEED_FORWARDS, p["inner"], build)

    def weights(self) -> dict[str, WeightSpec]:
        return {**_gate_weights(self), **self._inner_weights()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate, self.b_gate = tensors[self.weight_name].contiguous(), tensors[self.bias_name].to(torch.float32).contiguous()
        self._load_inner(tensors)

    def kernel_modules(self):
        return [("elementwise", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})] + self.inner.kernel_modules()

    def forward(self, x, step):
        return _gated(self, x, self.inner.forward(x, step))


register_mixer("input_convolution", ConvolvedInput)
register_mixer("gated_output", GatedMixer)
register_feed_forward("gated_feed_forward", GatedFeedForward)
