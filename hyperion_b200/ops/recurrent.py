"""The operations of mixers that carry a state per request (``csrc/recurrent.cu``): the short causal convolution with its
activation, the scan of a matrix-valued linear recurrence in its two modes, and the gated group norm.  All of them work in
float32; a request's state is its slot of a float record [slots, floats] (the matrices first, the convolution's last
inputs after them)."""
from __future__ import annotations

import ctypes

import torch

from .native import KernelError, check, f32, i32, is_bf16, library, ptr, require_cuda, stream_ptr

MODE_DELTA, MODE_STATE_SPACE, MODE_RETENTION = 0, 1, 2


def _floats(*tensors) -> None:
    for t in tensors:
        if t is not None and (t.dtype != torch.float32 or t.stride(-1) != 1):
            raise KernelError("the recurrent operations take float32 tensors with unit inner stride")


def causal_conv_silu(x: torch.Tensor, col0: int, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor, state_off: int,
                     slots: torch.Tensor, token_row: torch.Tensor, row_start: torch.Tensor) -> torch.Tensor:
    """silu(causal convolution) of the columns ``col0 .. col0 + C`` of ``x`` [tokens, *] with ``weight`` [C, taps] (the last
    column multiplies the current token); a row's earlier inputs come from its slot of ``state``."""
    require_cuda(x, weight, bias, state, slots, token_row, row_start)
    _floats(x, weight, bias, state)
    channels, taps = weight.shape
    out = torch.empty((x.shape[0], channels), dtype=torch.float32, device=x.device)
    check(library("recurrent").hb_causal_conv_silu(ptr(x), i32(x.stride(0)), i32(col0), i32(channels), ptr(weight), ptr(bias), i32(taps), ptr(state),
                                                   ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(token_row), ptr(row_start),
                                                   ptr(out), i32(x.shape[0]), stream_ptr()), "causal_conv_silu")
    return out


def conv_state_update(x: torch.Tensor, col0: int, channels: int, taps: int, state: torch.Tensor, state_off: int, slots: torch.Tensor,
                      row_start: torch.Tensor, rows: int) -> None:
    """Every row's slot keeps its last ``taps - 1`` inputs (call after :func:`causal_conv_silu` of the same step)."""
    require_cuda(x, state, slots, row_start)
    _floats(x, state)
    check(library("recurrent").hb_conv_state_update(ptr(x), i32(x.stride(0)), i32(col0), i32(channels), i32(taps), ptr(state),
                                                    ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(row_start), i32(rows),
                                                    stream_ptr()), "conv_state_update")


def residual_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, state_off: int, slots: torch.Tensor, token_row: torch.Tensor,
                  row_start: torch.Tensor) -> torch.Tensor:
    """``x + conv(x)``: a causal convolution over time per column of ``x`` [tokens, C] with ``weight`` [C, taps] (the last column
    multiplies the current token), added to its own input; a row's earlier inputs come from its slot of ``state`` (floats).  The
    result has ``x``'s element type; the sum is float."""
    require_cuda(x, weight, state, slots, token_row, row_start)
    _floats(weight, state)
    if x.dim() != 2 or x.stride(1) != 1 or weight.shape[0] != x.shape[1] or not weight.is_contiguous():
        raise KernelError("residual_conv: rows with unit inner stride and a dense [columns, taps] weight")
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    check(library("recurrent").hb_residual_conv(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), i32(x.shape[1]), ptr(weight), i32(weight.shape[1]), ptr(state),
                                                ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(token_row), ptr(row_start), ptr(out),
                                                i32(out.stride(0)), i32(x.shape[0]), stream_ptr()), "residual_conv")
    return out


def conv_state_keep(x: torch.Tensor, taps: int, state: torch.Tensor, state_off: int, slots: torch.Tensor, row_start: torch.Tensor, rows: int) -> None:
    """Every row's slot keeps the last ``taps - 1`` rows of ``x`` (any element type, kept as floats) for the next step (call after
    :func:`residual_conv` of the same step)."""
    require_cuda(x, state, slots, row_start)
    _floats(state)
    check(library("recurrent").hb_conv_state_keep(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), i32(x.shape[1]), i32(taps), ptr(state),
                                                  ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(row_start), i32(rows), stream_ptr()),
          "conv_state_keep")


def silu_columns_(x: torch.Tensor, col0: int, columns: int) -> None:
    """silu in place over the columns ``col0 .. col0 + columns`` of float rows."""
    require_cuda(x)
    _floats(x)
    if x.dim() != 2 or col0 < 0 or col0 + columns > x.shape[1]:
        raise KernelError("silu_columns: columns of a float matrix")
    check(library("recurrent").hb_silu_columns(ptr(x), i32(x.stride(0)), i32(col0), i32(columns), i32(x.shape[0]), stream_ptr()), "silu_columns")


def state_scan(mode: int, conv: torch.Tensor, k_off: int, q_off: int, v_off: int, proj: torch.Tensor, decay_off: int, step_off: int,
               a_log: torch.Tensor, dt_bias: torch.Tensor, skip: torch.Tensor | None, state: torch.Tensor, state_off: int, slots: torch.Tensor,
               row_start: torch.Tensor, rows: int, heads: int, groups: int, n: int, n_padded: int, e: int, q_scale: float = 1.0,
               states_only: bool = False) -> torch.Tensor | None:
    """Walk every row's tokens through the recurrence of ``mode`` from and into its slot of ``state``; returns [tokens, heads * e]
    (nothing with ``states_only``: the walk then only leaves the rows' states)."""
    require_cuda(conv, proj, a_log, dt_bias, skip, state, slots, row_start)
    _floats(conv, proj, a_log, dt_bias, skip, state)
    out = None if states_only else torch.empty((conv.shape[0], heads * e), dtype=torch.float32, device=conv.device)
    check(library("recurrent").hb_state_scan(i32(mode), ptr(conv), i32(conv.stride(0)), i32(k_off), i32(q_off), i32(v_off), ptr(proj), i32(proj.stride(0)),
                                             i32(decay_off), i32(step_off), ptr(a_log), ptr(dt_bias), ptr(skip), ptr(state),
                                             ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(row_start), ptr(out), i32(rows),
                                             i32(heads), i32(groups), i32(n), i32(n_padded), i32(e), f32(q_scale), stream_ptr()), "state_scan")
    return out


def channel_delta_scan(conv: torch.Tensor, k_off: int, q_off: int, v_off: int, decay: torch.Tensor, step: torch.Tensor, step_off: int, a_log: torch.Tensor,
                       dt_bias: torch.Tensor, state: torch.Tensor, state_off: int, slots: torch.Tensor, row_start: torch.Tensor, rows: int, heads: int, groups: int,
                       n: int, n_padded: int, e: int, q_scale: float = 1.0) -> torch.Tensor:
    """The gated delta rule with a decay per head and key entry, per head:  S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q  with
    g_i = exp(-exp(a_log) softplus(decay_i + dt_bias_i)), b = sigmoid(step), k and q made unit vectors and q times ``q_scale``.  ``conv``
    [tokens, *] holds keys, queries and values at their offsets, ``decay`` [tokens, heads * n] the decays' pre-activations, ``step`` [tokens, *]
    the steps' at ``step_off``; ``a_log`` has one entry per head, ``dt_bias`` one per head and key entry.  Every row's tokens walk from
    and into its slot of ``state``.  Returns [tokens, heads * e]."""
    require_cuda(conv, decay, step, a_log, dt_bias, state, slots, row_start)
    _floats(conv, decay, step, a_log, dt_bias, state)
    if a_log.numel() != heads or dt_bias.numel() != heads * n or decay.shape[1] != heads * n or not a_log.is_contiguous() or not dt_bias.is_contiguous():
        raise KernelError("channel_delta_scan: a rate per head, a bias and a pre-activation per head and key entry")
    out = torch.empty((conv.shape[0], heads * e), dtype=torch.float32, device=conv.device)
    check(library("recurrent").hb_channel_delta_scan(ptr(conv), i32(conv.stride(0)), i32(k_off), i32(q_off), i32(v_off), ptr(decay), i32(decay.stride(0)), i32(0),
                                                     ptr(step), i32(step.stride(0)), i32(step_off), ptr(a_log), ptr(dt_bias), ptr(state),
                                                     ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(row_start), ptr(out), i32(rows), i32(heads),
                                                     i32(groups), i32(n), i32(n_padded), i32(e), f32(q_scale), stream_ptr()), "channel_delta_scan")
    return out


def wkv_scan(k: torch.Tensor, q: torch.Tensor, v: torch.Tensor, x: torch.Tensor, x_off: int, w0: torch.Tensor, bonus: torch.Tensor, state: torch.Tensor,
             state_off: int, slots: torch.Tensor, row_start: torch.Tensor, rows: int, heads: int, n: int, n_padded: int, e: int) -> torch.Tensor:
    """The recurrence with a decay per key entry computed from the token and a bonus for the current token, per head:
    o = S^T q + (sum_i u_i k_i q_i) v;  S <- diag(w) S + k v^T  with w = exp(-exp(x + w0)).  ``k``, ``q`` [tokens, heads * n] and ``v``
    [tokens, heads * e] are float matrices of their own, ``x`` [tokens, *] holds the decays' pre-activations at column ``x_off``,
    ``w0`` and ``bonus`` have heads * n entries.  Every row's tokens walk from and into its slot of ``state``.  Returns [tokens, heads * e]."""
    require_cuda(k, q, v, x, w0, bonus, state, slots, row_start)
    _floats(k, q, v, x, w0, bonus, state)
    if w0.numel() != heads * n or bonus.numel() != heads * n or not w0.is_contiguous() or not bonus.is_contiguous():
        raise KernelError("wkv_scan: the decay offset and the bonus have an entry per head and key entry")
    out = torch.empty((k.shape[0], heads * e), dtype=torch.float32, device=k.device)
    check(library("recurrent").hb_wkv_scan(ptr(k), i32(k.stride(0)), ptr(q), i32(q.stride(0)), ptr(v), i32(v.stride(0)), ptr(x), i32(x.stride(0)), i32(x_off),
                                           ptr(w0), ptr(bonus), ptr(state), ctypes.c_longlong(state.stride(0)), i32(state_off), ptr(slots), ptr(row_start),
                                           ptr(out), i32(rows), i32(heads), i32(n), i32(n_padded), i32(e), stream_ptr()), "wkv_scan")
    return out


def token_shift_mix(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, state_off: int, slots: torch.Tensor, token_row: torch.Tensor,
                    row_start: torch.Tensor) -> torch.Tensor:
    """[n_mix, tokens, hidden] in ``x``'s type: input s is ``x + (x' - x) * mu[s]``, x' the row of the token before of the same request
    (from the request's slot of ``state`` at ``state_off`` for the first token of a step)."""
    require_cuda(x, mu, state, slots, token_row, row_start)
    _floats(mu, state)
    tokens, hidden = x.shape
    if x.stride(1) != 1 or mu.dim() != 2 or mu.shape[1] != hidden or not mu.is_contiguous():
        raise KernelError("token_shift_mix: rows with unit inner stride and a dense [n_mix, hidden] table of mixing weights")
    out = torch.empty((mu.shape[0], tokens, hidden), dtype=x.dtype, device=x.device)
    check(library("recurrent").hb_token_shift_mix(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), ptr(mu), i32(mu.shape[0]), ptr(state), ctypes.c_longlong(state.stride(0)),
                                                  i32(state_off), ptr(slots), ptr(token_row), ptr(row_start), ptr(out), i32(tokens), i32(hidden), stream_ptr()),
          "token_shift_mix")
    return out


def token_shift_keep(x: torch.Tensor, state: torch.Tensor, state_off: int, slots: torch.Tensor, row_start: torch.Tensor, rows: int) -> None:
    """Every row's slot keeps the row's last token of ``x`` (as floats) for the next step (call after :func:`token_shift_mix`)."""
    require_cuda(x, state, slots, row_start)
    _floats(state)
    check(library("recurrent").hb_token_shift_keep(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), ptr(state), ctypes.c_longlong(state.stride(0)), i32(state_off),
                                                   ptr(slots), ptr(row_start), i32(rows), i32(x.shape[1]), stream_ptr()), "token_shift_keep")


def tanh_rows(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """tanh of a dense float tensor, rounded once to ``out_dtype``."""
    require_cuda(x)
    _floats(x)
    if not x.is_contiguous():
        raise KernelError("tanh_rows: a dense tensor")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(library("recurrent").hb_tanh_rows(ptr(x), ptr(out), i32(is_bf16(out)), ctypes.c_longlong(x.numel()), stream_ptr()), "tanh_rows")
    return out


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, gate_off: int, weight: torch.Tensor | None, group: int, gate_first: bool, eps: float,
                     out_dtype: torch.dtype, scale: float = 1.0, out: torch.Tensor | None = None, sigmoid_gate: bool = False) -> torch.Tensor:
    """RMS norm of ``y`` [tokens, width] in groups of ``group`` columns, times ``weight`` (indexed by column modulo its length;
    None: no weight), gated by silu (``sigmoid_gate``: by the sigmoid) of the columns ``gate_off ..`` of ``gate``: before the norm
    (``gate_first``) or after it, times ``scale``.  ``out``: a [tokens, >= width] view the result is written to."""
    require_cuda(y, gate, weight, out)
    _floats(y, gate, weight)
    tokens, width = y.shape
    if width % group:
        raise KernelError(f"gated_group_norm: groups of {group} do not divide {width} columns")
    if out is None:
        out = torch.empty((tokens, width), dtype=out_dtype, device=y.device)
    elif out.dtype != out_dtype or out.shape[0] != tokens or out.shape[1] < width or out.stride(1) != 1:
        raise KernelError("gated_group_norm: the output is a [tokens, >= width] view of the stated type")
    check(library("recurrent").hb_gated_group_norm(ptr(y), i32(y.stride(0)), ptr(gate), i32(gate.stride(0)), i32(gate_off), ptr(weight),
                                                   i32(weight.numel() if weight is not None else 0), i32(group), i32(width // group),
                                                   i32(1 if gate_first else 0), f32(eps), f32(scale), ptr(out), i32(is_bf16(out)), i32(out.stride(0)),
                                                   i32(tokens), i32(1 if sigmoid_gate else 0), stream_ptr()), "gated_group_norm")
    return out


def selective_scan(x: torch.Tensor, dt: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, a: torch.Tensor, skip: torch.Tensor, gate: torch.Tensor,
                   gate_off: int, state: torch.Tensor, state_off: int, slots: torch.Tensor, row_start: torch.Tensor, rows: int, n: int, n_padded: int,
                   out_dtype: torch.dtype, states_only: bool = False, dt_sums: torch.Tensor | None = None, precise: bool = False) -> torch.Tensor | None:
    """The recurrence with a decay per channel and state entry: per channel c, S[c] <- exp(dt_c A[c]) S[c] + dt_c x_c B,
    y_c = (S[c] . C + D_c x_c) silu(z_c), with dt = softplus(``dt``), B and C the columns ``b_off ..`` and ``c_off ..`` of ``bc``,
    A = ``a`` [inner, n] (negative), D = ``skip``, z the columns ``gate_off ..`` of ``gate``; every row's tokens walk from and
    into its slot of ``state``.  Returns [tokens, inner] in ``out_dtype`` (nothing with ``states_only``).  ``dt_sums`` [rows, inner] float
    receives the sum of every row's steps per channel.  ``precise``: a token's arithmetic in double precision, rounded to float once
    (the float32 mode; the state stays float from token to token, so results do not depend on how the rows were cut)."""
    require_cuda(x, dt, bc, a, skip, gate, state, slots, row_start, dt_sums)
    _floats(x, dt, bc, a, skip, gate, state, dt_sums)
    tokens, inner = x.shape
    if a.shape != (inner, n) or not a.is_contiguous() or skip.numel() != inner or dt.shape != x.shape:
        raise KernelError("selective_scan: A is [inner, n], D [inner], the steps [tokens, inner]")
    out = None if states_only else torch.empty((tokens, inner), dtype=out_dtype, device=x.device)
    check(library("recurrent").hb_selective_scan(ptr(x), i32(x.stride(0)), ptr(dt), i32(dt.stride(0)), ptr(bc), i32(bc.stride(0)), i32(b_off), i32(c_off),
                                                 ptr(a), ptr(skip), ptr(gate), i32(gate.stride(0)), i32(gate_off), ptr(state), ctypes.c_longlong(state.stride(0)),
                                                 i32(state_off), ptr(slots), ptr(row_start), ptr(out), i32(is_bf16(out) if out is not None else 0),
                                                 i32(out.stride(0) if out is not None else 0), i32(rows), i32(inner), i32(n), i32(n_padded), ptr(dt_sums),
                                                 i32(1 if precise else 0), stream_ptr()), "selective_scan")
    return out


SEGMENT = 256  # tokens per segment when a long row's scan is cut into segments that run side by side


def plan_segments(counts) -> tuple[list[int], list[int]] | None:
    """Rows of at least two segments' length are cut into segments of ``SEGMENT`` tokens, every other row is one segment:
    (first token of every segment plus the end, the row of every segment), or None when no row is that long."""
    if max(counts) < 2 * SEGMENT:
        return None
    starts, rows, at = [], [], 0
    for row, count in enumerate(counts):
        count = int(count)
        pieces = max(1, count // SEGMENT) if count >= 2 * SEGMENT else 1
        for piece in range(pieces):
            starts.append(at + piece * SEGMENT)
            rows.append(row)
        at += count
    return starts + [at], rows


def retention_in_segments(proj: torch.Tensor, k_off: int, q_off: int, v_off: int, decay: torch.Tensor, state: torch.Tensor, slots: torch.Tensor,
                          seg_start: torch.Tensor, seg_row: torch.Tensor, segments: int, heads: int, n: int, n_padded: int, e: int) -> torch.Tensor:
    """The retention scan of :func:`state_scan` with long rows cut into segments that are walked side by side: every segment from a
    zero state, the segments' states joined (``csrc/recurrent.cu``: ``join_segments_kernel``), every segment again from its true
    start.  Twice the arithmetic for as many times the blocks; the result differs from the one-pass scan by rounding."""
    require_cuda(proj, decay, state, slots, seg_start, seg_row)
    per_head = e * n_padded
    ends = torch.zeros((segments, heads * per_head), dtype=torch.float32, device=proj.device)
    own = torch.arange(segments, dtype=torch.int32, device=proj.device)
    state_scan(MODE_RETENTION, proj, k_off, q_off, v_off, proj, 0, 0, decay, decay, None, ends, 0, own, seg_start, segments, heads, heads, n, n_padded, e,
               states_only=True)
    check(library("recurrent").hb_join_segments(ptr(ends), ctypes.c_longlong(ends.stride(0)), ptr(state), ctypes.c_longlong(state.stride(0)), i32(0), ptr(slots),
                                                ptr(seg_start), ptr(seg_row), i32(segments), ptr(decay), i32(heads), i32(per_head), stream_ptr()), "join_segments")
    return state_scan(MODE_RETENTION, proj, k_off, q_off, v_off, proj, 0, 0, decay, decay, None, ends, 0, own, seg_start, segments, heads, heads, n, n_padded, e)


def selective_in_segments(x: torch.Tensor, dt: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, a: torch.Tensor, skip: torch.Tensor,
                          gate: torch.Tensor, gate_off: int, state: torch.Tensor, slots: torch.Tensor, seg_start: torch.Tensor, seg_row: torch.Tensor,
                          segments: int, n: int, n_padded: int, out_dtype: torch.dtype) -> torch.Tensor:
    """:func:`selective_scan` with long rows cut into segments that are walked side by side (see :func:`retention_in_segments`); a
    segment's decay per channel and state entry is exp(A times the sum of the channel's steps over the segment)."""
    inner = x.shape[1]
    ends = torch.zeros((segments, inner * n_padded), dtype=torch.float32, device=x.device)
    sums = torch.empty((segments, inner), dtype=torch.float32, device=x.device)
    own = torch.arange(segments, dtype=torch.int32, device=x.device)
    selective_scan(x, dt, bc, b_off, c_off, a, skip, gate, gate_off, ends, 0, own, seg_start, segments, n, n_padded, out_dtype, states_only=True, dt_sums=sums)
    check(library("recurrent").hb_join_selective_segments(ptr(ends), ctypes.c_longlong(ends.stride(0)), ptr(state), ctypes.c_longlong(state.stride(0)), i32(0),
                                                          ptr(slots), ptr(seg_row), i32(segments), ptr(a), ptr(sums), i32(inner), i32(n), i32(n_padded),
                                                          stream_ptr()), "join_selective_segments")
    return selective_scan(x, dt, bc, b_off, c_off, a, skip, gate, gate_off, ends, 0, own, seg_start, segments, n, n_padded, out_dtype)


def segment_planner(dtype: torch.dtype) -> dict:
    """The step planner of mixers that scan long rows in segments: in bfloat16, where bits need not repeat across cuts of the work, a
    step with a row of at least two segments' length gets ``scan_seg_start`` and ``scan_seg_row`` among its arrays and their number in
    ``step.host["scan_segments"]`` (0 otherwise)."""
    if dtype != torch.bfloat16:
        return {}

    def plan(rows, packer, host):
        if "scan_segments" in host:
            return
        counts = rows.counts if hasattr(rows, "counts") else [row.count for row in rows]
        cut = plan_segments([int(c) for c in counts])
        host["scan_segments"] = 0 if cut is None else len(cut[1])
        if cut is not None:
            packer.add("scan_seg_start", cut[0])
            packer.add("scan_seg_row", cut[1])

    return {("scan_segments", SEGMENT): plan}
