"""Mixers that keep a matrix-valued state per request instead of a cache of keys.  The gated delta rule and
the state-space mixer of Mamba-2 are both one in-projection, a short causal convolution with SiLU over some of
its columns, a scan of the recurrence over each request's new tokens (``csrc/recurrent.cu``), a gated RMS norm,
and an out-projection.  The in-projection's result, the convolution, the recurrence with its decays, step
sizes and unit norms, the state and the norm are float32 in both precisions; only the matrix products take
bfloat16 operands in the bfloat16 mode.  A request's state is one float record (``RequestState``): the matrices
of all heads, then the convolution's last taps - 1 inputs; it is zero when the request takes its slot.

Gated delta rule (``delta_rule``), per head with key/query size n and value size e; the q/k head of head h is
h // (heads / kv_heads):
    q, k, v = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x));  q, k <- unit vectors (x / sqrt(|x|^2 + 1e-6)),  q <- q n^(-1/2)
    beta = sigmoid(W_b x);  a = exp(-exp(A_log) softplus(W_a x + dt_bias))
    S <- a S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    y = o / rms(o) * norm * silu(W_g x)  per head, then W_o.
Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``conv`` (taps), ``eps``.  Tensors (after the
prefix): q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o.

State space (``mamba2``), per head with state size n and value size e; the group of head h is h // (heads / groups):
    [z | x | B | C | dt] = W_in x;  x, B, C <- silu(conv([x | B | C]) + conv.b);  dt <- softplus(dt + dt_bias)
    S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
    y <- y silu(z), RMS norm in ``norm_groups`` equal parts, times norm, then W_o.
Parameters: ``hidden_size``, ``heads``, ``value_dim``, ``state``, ``groups``, ``norm_groups``, ``conv`` (taps), ``eps``.
Tensors: in, conv, conv.b, dt_bias, A_log, D, norm, o.

Selective scan (``mamba1``): the state-space mixer whose decay differs per channel and state entry.  With ``inner`` channels,
a state of n entries per channel and step inputs of rank r:
    [x | z] = W_in h;  x <- silu(conv(x) + conv.b);  [d | B | C] = W_x x;  dt = softplus(W_dt d + dt.b), one per channel
    S[c, i] <- exp(dt_c A[c, i]) S[c, i] + dt_c x_c B_i  with A = -exp(A_log);  y_c = sum_i S[c, i] C_i + D_c x_c
    y <- y silu(z), then W_o.
Parameters: ``hidden_size``, ``inner``, ``state``, ``dt_rank``, ``conv`` (taps).  Tensors: in, conv, conv.b, x, dt, dt.b, A_log, D, o.

Time mixing with a decay per key entry (``wkv``), per head with key/query size n and value size n.  Every token is read beside
the one before it: with x' the row of the token before (zeros at the start of a request), each of the five inputs s in (r, k, v, g, w)
is x + (x' - x) * mu_s.
    r, k, v = W_r in_r, W_k in_k, W_v in_v;  gate = silu(W_g in_g);  w = exp(-exp(W_w2 tanh(W_w1 in_w) + w0)), one per head and key entry
    o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T   (the bonus u only ever meets the current token)
    y = o / rms(o) per head, times norm, times gate, then W_o.
The record holds the heads' matrices, then the last token's x.  Mixes, tanh, decays, the recurrence and the norm are float.
Parameters: ``hidden_size``, ``heads``, ``head_dim``, ``decay_rank`` (what random weights get; a checkpoint's tensors decide), ``eps``.
Tensors: mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o.

Gated delta rule with a decay per key channel (``channel_delta``): the delta rule above with
    g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 x) + dt_bias)), one per head and key entry;  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    y = o / rms(o) per head, times norm (one weight of a head's size), times sigmoid(W_g2 (W_g1 x)), then W_o.
The decay and the gate come through two small matrices each; their inner sizes are read off the tensors.
Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``conv`` (taps), ``eps``, ``decay_rank`` and ``gate_rank`` (what
random weights get).  Tensors: q, k, v, q.conv, k.conv, v.conv, b, a1, a2, A_log, dt_bias, g1, g2, norm, o.

Lightning attention (``lightning``): a matrix state per head that fades by a constant of the head, with nothing between the projections and
the recurrence but an activation:
    q, k, v = silu(W_q x), silu(W_k x), silu(W_v x);  S <- decay_h S + k v^T;  o = S^T q
    y = [all heads' o side by side] / its root mean square, times norm, times sigmoid(W_g x), then W_o.
Parameters: ``hidden_size``, ``heads``, ``head_dim``, ``value_dim``, ``decay`` (one per head), ``eps``.  Tensors: q, k, v, g, norm, o.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import recurrent
from .base import BuildContext, Mixer, RequestState, WeightSpec, register_mixer
from .spec import PartSpec


def _round_up(value: int, step: int) -> int:
    return -(-value // step) * step


class _ScanMixer(Mixer):
    """What the two have in common: the record's layout and the sequence of kernels."""

    mode: int
    heads: int
    groups: int
    n: int  # size of keys and queries
    e: int  # size of values
    taps: int
    conv_channels: int

    def _finish_layout(self) -> None:
        if self.n > 256:
            raise ValueError(f"a state of {self.n} per column is above the scan kernel's limit of 256")
        if self.heads % self.groups:
            raise ValueError(f"{self.groups} groups do not divide {self.heads} heads")
        self.n_padded = _round_up(self.n, 4)
        self.conv_off = self.heads * self.e * self.n_padded  # a multiple of 4: the matrices come first
        self.record = _round_up(self.conv_off + (self.taps - 1) * self.conv_channels, 4)

    def cache_request(self):
        return RequestState((self.record,), torch.float32)

    def kernel_modules(self):
        return [("recurrent", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def _float(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor.to(torch.float32).contiguous()


class GatedDeltaRule(_ScanMixer):
    mode = recurrent.MODE_DELTA

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads, self.groups = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.n, self.e, self.taps, self.eps = int(p["head_dim"]), int(p["value_dim"]), int(p["conv"]), float(p["eps"])
        self.qk_width, self.v_width = self.groups * self.n, self.heads * self.e
        self.conv_channels = 2 * self.qk_width + self.v_width
        # columns of the in-projection: [q | k | v | g | b | a]
        self.gate_off = self.conv_channels
        self.beta_off = self.gate_off + self.v_width
        self.decay_off = self.beta_off + self.heads
        self._finish_layout()

    def weights(self) -> dict[str, WeightSpec]:
        h, taps = self.hidden, self.taps
        return {"q": WeightSpec((self.qk_width, h)), "k": WeightSpec((self.qk_width, h)), "v": WeightSpec((self.v_width, h)),
                "q.conv": WeightSpec((self.qk_width, taps)), "k.conv": WeightSpec((self.qk_width, taps)), "v.conv": WeightSpec((self.v_width, taps)),
                "b": WeightSpec((self.heads, h)), "a": WeightSpec((self.heads, h)), "A_log": WeightSpec((self.heads,)),
                "dt_bias": WeightSpec((self.heads,)), "g": WeightSpec((self.v_width, h)), "norm": WeightSpec((self.e,), init="one_plus_normal"),
                "o": WeightSpec((self.hidden, self.v_width))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        mats = [tensors[name] for name in ("q", "k", "v", "g", "b", "a")]
        dtype = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.w_in = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.w_conv = torch.cat([self._float(tensors[name]) for name in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = self._float(tensors["A_log"]), self._float(tensors["dt_bias"])
        self.norm = self._float(tensors["norm"])
        self.w_o = tensors["o"].contiguous()

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("the delta rule keeps a state per request; the schedule gave it none")
        proj = ops.linear(x, self.w_in, None, torch.float32)
        state, slots, rows = cache.state, cache.slots, step.n_rows
        conv = recurrent.causal_conv_silu(proj, 0, self.w_conv, None, state, self.conv_off, slots, step.token_row, step.row_start)
        recurrent.conv_state_update(proj, 0, self.conv_channels, self.taps, state, self.conv_off, slots, step.row_start, rows)
        o = recurrent.state_scan(self.mode, conv, self.qk_width, 0, 2 * self.qk_width, proj, self.decay_off, self.beta_off, self.a_log, self.dt_bias,
                                 None, state, 0, slots, step.row_start, rows, self.heads, self.groups, self.n, self.n_padded, self.e,
                                 q_scale=self.n ** -0.5)
        y = recurrent.gated_group_norm(o, proj, self.gate_off, self.norm, self.e, False, self.eps, self.dtype)
        return ops.linear(y, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


class StateSpaceMixer(_ScanMixer):
    mode = recurrent.MODE_STATE_SPACE

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads, self.groups = int(p["hidden_size"]), int(p["heads"]), int(p["groups"])
        self.n, self.e, self.taps, self.eps = int(p["state"]), int(p["value_dim"]), int(p["conv"]), float(p["eps"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.inner = self.heads * self.e
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.norm_groups} norm groups do not divide the inner width {self.inner}")
        self.conv_channels = self.inner + 2 * self.groups * self.n
        # columns of the in-projection: [z | x | B | C | dt]
        self.conv_col0 = self.inner
        self.dt_off = self.inner + self.conv_channels
        self._finish_layout()

    def weights(self) -> dict[str, WeightSpec]:
        return {"in": WeightSpec((self.dt_off + self.heads, self.hidden)), "conv": WeightSpec((self.conv_channels, self.taps)),
                "conv.b": WeightSpec((self.conv_channels,)), "dt_bias": WeightSpec((self.heads,)), "A_log": WeightSpec((self.heads,)),
                "D": WeightSpec((self.heads,)), "norm": WeightSpec((self.inner,), init="one_plus_normal"), "o": WeightSpec((self.hidden, self.inner))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = tensors["in"].contiguous()
        self.w_conv, self.b_conv = self._float(tensors["conv"]), self._float(tensors["conv.b"])
        self.a_log, self.dt_bias, self.skip = self._float(tensors["A_log"]), self._float(tensors["dt_bias"]), self._float(tensors["D"])
        self.norm = self._float(tensors["norm"])
        self.w_o = tensors["o"].contiguous()

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("the state-space mixer keeps a state per request; the schedule gave it none")
        proj = ops.linear(x, self.w_in, None, torch.float32)
        state, slots, rows = cache.state, cache.slots, step.n_rows
        conv = recurrent.causal_conv_silu(proj, self.conv_col0, self.w_conv, self.b_conv, state, self.conv_off, slots, step.token_row, step.row_start)
        recurrent.conv_state_update(proj, self.conv_col0, self.conv_channels, self.taps, state, self.conv_off, slots, step.row_start, rows)
        bn = self.groups * self.n
        y = recurrent.state_scan(self.mode, conv, self.inner, self.inner + bn, 0, proj, self.dt_off, self.dt_off, self.a_log, self.dt_bias, self.skip,
                                 state, 0, slots, step.row_start, rows, self.heads, self.groups, self.n, self.n_padded, self.e)
        y = recurrent.gated_group_norm(y, proj, 0, self.norm, self.inner // self.norm_groups, True, self.eps, self.dtype)
        return ops.linear(y, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


class SelectiveScanMixer(Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.inner, self.n = int(p["hidden_size"]), int(p["inner"]), int(p["state"])
        self.rank, self.taps = int(p["dt_rank"]), int(p["conv"])
        if self.n > 256:
            raise ValueError(f"a state of {self.n} per channel is above the scan kernel's limit of 256")
        self.n_padded = _round_up(self.n, 4)
        self.conv_off = self.inner * self.n_padded  # a multiple of 4: the channels' states come first
        self.record = _round_up(self.conv_off + (self.taps - 1) * self.inner, 4)

    def weights(self) -> dict[str, WeightSpec]:
        return {"in": WeightSpec((2 * self.inner, self.hidden)), "conv": WeightSpec((self.inner, self.taps)), "conv.b": WeightSpec((self.inner,)),
                "x": WeightSpec((self.rank + 2 * self.n, self.inner)), "dt": WeightSpec((self.inner, self.rank)), "dt.b": WeightSpec((self.inner,)),
                "A_log": WeightSpec((self.inner, self.n)), "D": WeightSpec((self.inner,)), "o": WeightSpec((self.hidden, self.inner))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f = lambda name: tensors[name].to(torch.float32).contiguous()  # noqa: E731
        self.w_in, self.w_x, self.w_o = tensors["in"].contiguous(), tensors["x"].contiguous(), tensors["o"].contiguous()
        self.w_dt, self.b_dt = tensors["dt"].contiguous(), f("dt.b")
        self.w_conv, self.b_conv = f("conv"), f("conv.b")
        self.a = (-torch.exp(f("A_log"))).contiguous()
        self.skip = f("D")

    def cache_request(self):
        return RequestState((self.record,), torch.float32)

    def kernel_modules(self):
        return [("recurrent", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def step_plans(self):
        return recurrent.segment_planner(self.dtype)

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("the selective scan keeps a state per request; the schedule gave it none")
        proj = ops.linear(x, self.w_in, None, torch.float32)  # [x | z]
        state, slots, rows = cache.state, cache.slots, step.n_rows
        conv = recurrent.causal_conv_silu(proj, 0, self.w_conv, self.b_conv, state, self.conv_off, slots, step.token_row, step.row_start)
        recurrent.conv_state_update(proj, 0, self.inner, self.taps, state, self.conv_off, slots, step.row_start, rows)
        dbc = ops.linear(conv, self.w_x, None, torch.float32)  # [d | B | C]
        dt = ops.linear(dbc[:, : self.rank], self.w_dt, self.b_dt, torch.float32)
        # segments pay while one pass leaves the GPU mostly idle (measured on a B200 with a state of 16: 128 blocks 474 -> 298 us for
        # 2,048 tokens, 256 blocks 524 -> 538 us)
        segments = step.host.get("scan_segments", 0) if self.dtype == torch.bfloat16 and -(-self.inner // 32) <= 200 else 0
        if segments:  # a long row: its segments side by side, joined by a second pass
            y = recurrent.selective_in_segments(conv, dt, dbc, self.rank, self.rank + self.n, self.a, self.skip, proj, self.inner, state, slots,
                                                step.extra["scan_seg_start"], step.extra["scan_seg_row"], segments, self.n, self.n_padded, self.dtype)
        else:
            y = recurrent.selective_scan(conv, dt, dbc, self.rank, self.rank + self.n, self.a, self.skip, proj, self.inner, state, 0, slots,
                                         step.row_start, rows, self.n, self.n_padded, self.dtype, precise=self.dtype == torch.float32)
        return ops.linear(y, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


class WkvMixer(Mixer):
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads, self.n = int(p["hidden_size"]), int(p["heads"]), int(p["head_dim"])
        self.decay_rank, self.eps = int(p.get("decay_rank") or 16), float(p["eps"])
        if self.n > 256:
            raise ValueError(f"a state of {self.n} per column is above the scan kernel's limit of 256")
        self.width = self.heads * self.n
        self.n_padded = _round_up(self.n, 4)
        self.shift_off = self.heads * self.n * self.n_padded  # a multiple of 4: the matrices come first, then the last token's input
        self.record = _round_up(self.shift_off + self.hidden, 4)

    def weights(self) -> dict[str, WeightSpec]:
        wanted = {"mu." + s: WeightSpec((self.hidden,)) for s in self.MIXES}
        wanted.update({s: WeightSpec((self.width, self.hidden)) for s in ("r", "k", "v", "g")})
        wanted.update({"w1": WeightSpec((self.decay_rank, self.hidden), any_extent=(0,)), "w2": WeightSpec((self.width, self.decay_rank), any_extent=(1,)),
                       "w0": WeightSpec((self.width,)), "u": WeightSpec((self.heads, self.n)), "norm": WeightSpec((self.width,), init="one_plus_normal"),
                       "o": WeightSpec((self.hidden, self.width))})
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f = lambda name: tensors[name].to(torch.float32).contiguous()  # noqa: E731
        if tensors["w1"].shape[0] != tensors["w2"].shape[1]:
            raise ValueError(f"the decay's two matrices meet in {tensors['w1'].shape[0]} and {tensors['w2'].shape[1]} entries")
        self.mu = torch.stack([f("mu." + s) for s in self.MIXES]).contiguous()
        self.w_in = [tensors[s].contiguous() for s in ("r", "k", "v", "g")]
        self.w_1, self.w_2, self.w_o = tensors["w1"].contiguous(), tensors["w2"].contiguous(), tensors["o"].contiguous()
        self.w0, self.bonus, self.norm = f("w0"), f("u").reshape(-1), f("norm")

    def cache_request(self):
        return RequestState((self.record,), torch.float32)

    def kernel_modules(self):
        return [("recurrent", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("time mixing keeps a state per request; the schedule gave it none")
        state, slots, rows = cache.state, cache.slots, step.n_rows
        mixed = recurrent.token_shift_mix(x, self.mu, state, self.shift_off, slots, step.token_row, step.row_start)
        recurrent.token_shift_keep(x, state, self.shift_off, slots, step.row_start, rows)
        r, k, v, gate = (ops.linear(mixed[i], w, None, torch.float32) for i, w in enumerate(self.w_in))
        inner = recurrent.tanh_rows(ops.linear(mixed[4], self.w_1, None, torch.float32), self.dtype)
        decay_in = ops.linear(inner, self.w_2, None, torch.float32)
        o = recurrent.wkv_scan(k, r, v, decay_in, 0, self.w0, self.bonus, state, 0, slots, step.row_start, rows, self.heads, self.n, self.n_padded, self.n)
        y = recurrent.gated_group_norm(o, gate, 0, self.norm, self.n, False, self.eps, self.dtype)
        return ops.linear(y, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


class ChannelDeltaRule(_ScanMixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads, self.groups = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.n, self.e, self.taps, self.eps = int(p["head_dim"]), int(p["value_dim"]), int(p["conv"]), float(p["eps"])
        self.decay_rank, self.gate_rank = int(p.get("decay_rank") or 16), int(p.get("gate_rank") or 16)
        self.qk_width, self.v_width = self.groups * self.n, self.heads * self.e
        self.conv_channels = 2 * self.qk_width + self.v_width
        self.beta_off = self.conv_channels  # columns of the in-projection: [q | k | v | b | a1 | g1]; the last two as wide as the tensors say
        self._finish_layout()

    def weights(self) -> dict[str, WeightSpec]:
        h, taps = self.hidden, self.taps
        return {"q": WeightSpec((self.qk_width, h)), "k": WeightSpec((self.qk_width, h)), "v": WeightSpec((self.v_width, h)),
                "q.conv": WeightSpec((self.qk_width, taps)), "k.conv": WeightSpec((self.qk_width, taps)), "v.conv": WeightSpec((self.v_width, taps)),
                "b": WeightSpec((self.heads, h)), "A_log": WeightSpec((self.heads,)), "norm": WeightSpec((self.e,), init="one_plus_normal"),
                "a1": WeightSpec((self.decay_rank, h), any_extent=(0,)), "a2": WeightSpec((self.heads * self.n, self.decay_rank), any_extent=(1,)),
                "dt_bias": WeightSpec((self.heads * self.n,)),
                "g1": WeightSpec((self.gate_rank, h), any_extent=(0,)), "g2": WeightSpec((self.v_width, self.gate_rank), any_extent=(1,)),
                "o": WeightSpec((self.hidden, self.v_width))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for first, second in (("a1", "a2"), ("g1", "g2")):
            if tensors[first].shape[0] != tensors[second].shape[1]:
                raise ValueError(f"the matrices {first} and {second} meet in {tensors[first].shape[0]} and {tensors[second].shape[1]} entries")
        mats = [tensors[name] for name in ("q", "k", "v", "b", "a1", "g1")]
        dtype = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.w_in = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.decay_rank, self.gate_rank = int(tensors["a1"].shape[0]), int(tensors["g1"].shape[0])
        self.a1_off = self.beta_off + self.heads
        self.g1_off = self.a1_off + self.decay_rank
        self.w_a2, self.w_g2 = tensors["a2"].contiguous(), tensors["g2"].contiguous()
        self.w_conv = torch.cat([self._float(tensors[name]) for name in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = self._float(tensors["A_log"]), self._float(tensors["dt_bias"])
        self.norm = self._float(tensors["norm"])
        self.w_o = tensors["o"].contiguous()

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("the delta rule keeps a state per request; the schedule gave it none")
        proj = ops.linear(x, self.w_in, None, torch.float32)
        state, slots, rows = cache.state, cache.slots, step.n_rows
        conv = recurrent.causal_conv_silu(proj, 0, self.w_conv, None, state, self.conv_off, slots, step.token_row, step.row_start)
        recurrent.conv_state_update(proj, 0, self.conv_channels, self.taps, state, self.conv_off, slots, step.row_start, rows)
        decay = ops.linear(proj[:, self.a1_off : self.a1_off + self.decay_rank], self.w_a2, None, torch.float32)
        gate = ops.linear(proj[:, self.g1_off : self.g1_off + self.gate_rank], self.w_g2, None, torch.float32)
        o = recurrent.channel_delta_scan(conv, self.qk_width, 0, 2 * self.qk_width, decay, proj, self.beta_off, self.a_log, self.dt_bias, state, 0, slots,
                                         step.row_start, rows, self.heads, self.groups, self.n, self.n_padded, self.e, q_scale=self.n ** -0.5)
        y = recurrent.gated_group_norm(o, gate, 0, self.norm, self.e, False, self.eps, self.dtype, sigmoid_gate=True)
        return ops.linear(y, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


class LightningAttention(Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.n, self.e, self.eps = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"]), float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        if self.n > 256:
            raise ValueError(f"a state of {self.n} per column is above the scan kernel's limit of 256")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(build.device)
        self.qk_width, self.v_width = self.heads * self.n, self.heads * self.e
        self.n_padded = _round_up(self.n, 4)
        self.record = self.heads * self.e * self.n_padded

    def weights(self) -> dict[str, WeightSpec]:
        h = self.hidden
        return {"q": WeightSpec((self.qk_width, h)), "k": WeightSpec((self.qk_width, h)), "v": WeightSpec((self.v_width, h)), "g": WeightSpec((self.v_width, h)),
                "norm": WeightSpec((self.v_width,), init="one_plus_normal"), "o": WeightSpec((h, self.v_width))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        mats = [tensors[name] for name in ("q", "k", "v", "g")]
        dtype = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.w_in = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()  # columns of the in-projection: [q | k | v | g]
        self.norm = tensors["norm"].to(torch.float32).contiguous()
        self.w_o = tensors["o"].contiguous()

    def cache_request(self):
        return RequestState((self.record,), torch.float32)

    def kernel_modules(self):
        return [("recurrent", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def step_plans(self):
        return recurrent.segment_planner(self.dtype)

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("lightning attention keeps a state per request; the schedule gave it none")
        proj = ops.linear(x, self.w_in, None, torch.float32)
        k_off, v_off = self.qk_width, 2 * self.qk_width
        recurrent.silu_columns_(proj, 0, v_off + self.v_width)
        # long rows in segments while one pass leaves the GPU mostly idle, as for the package's other constant-decay recurrence
        blocks = self.heads * -(-self.e // 32)
        segments = step.host.get("scan_segments", 0) if self.dtype == torch.bfloat16 and blocks <= 100 else 0
        if segments:
            o = recurrent.retention_in_segments(proj, k_off, 0, v_off, self.decay, cache.state, cache.slots, step.extra["scan_seg_start"],
                                                step.extra["scan_seg_row"], segments, self.heads, self.n, self.n_padded, self.e)
        else:
            o = recurrent.state_scan(recurrent.MODE_RETENTION, proj, k_off, 0, v_off, proj, 0, 0, self.decay, self.decay, None, cache.state, 0, cache.slots,
                                     step.row_start, step.n_rows, self.heads, self.heads, self.n, self.n_padded, self.e)
        y = recurrent.gated_group_norm(o, proj, v_off + self.v_width, self.norm, self.v_width, False, self.eps, self.dtype, sigmoid_gate=True)
        return ops.linear(y, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_mixer("channel_delta", ChannelDeltaRule)
register_mixer("lightning", LightningAttention)
register_mixer("delta_rule", GatedDeltaRule)
register_mixer("mamba1", SelectiveScanMixer)
register_mixer("mamba2", StateSpaceMixer)
register_mixer("wkv", WkvMixer)
