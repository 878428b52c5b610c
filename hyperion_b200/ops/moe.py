"""The operations of a feed-forward made of many small experts (``csrc/moe.cu``): the router, the plan that sorts
(token, choice) pairs by expert, the gather of the sorted rows, the grouped matrix product and the sum of a token's experts.
The host learns nothing about which expert got how many rows: every buffer has its worst-case size, which follows from the
step's shape alone, so a step of a shape seen before replays the same launches."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .basic import status_word
from .native import KernelError, check, f32, i32, is_bf16, library, ptr, require_cuda, stream_ptr

PAD = 128  # an expert's rows are padded to whole tiles of this many rows
FEW_PAIRS = 128  # steps of at most this many (token, choice) pairs stream the matrices of the experts they use instead of taking tensor-core tiles


@dataclass
class Plan:
    """Where the rows of a step lie once they are sorted by expert."""

    capacity: int  # rows of the sorted buffers: every (token, choice) pair plus each expert's padding
    top: int
    slot_of: torch.Tensor  # [tokens * top] int32: the row of a pair
    slot_token: torch.Tensor  # [capacity] int32: the token of a row, -1 for padding
    slot_weight: torch.Tensor  # [capacity] float: what the row's input is multiplied by
    tile_expert: torch.Tensor  # [capacity / PAD] int32: the expert of a tile of rows, -1 beyond the last used tile
    tile_rows: torch.Tensor  # [capacity / PAD] int32: how many rows of a tile are taken (they come first)
    pairs: int = 0


def route(x: torch.Tensor, router: torch.Tensor, top: int, weighted: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Router logits ``x router^T`` in float, the ``top`` largest per token (lowest index first among equals) and their
    weights sigmoid(logit), not renormalised (1 when not ``weighted``): ([tokens, top] int32, [tokens, top] float)."""
    require_cuda(x, router)
    if router.dtype != torch.float32 or not router.is_contiguous() or x.stride(-1) != 1 or x.shape[1] != router.shape[1]:
        raise KernelError("moe.route: a dense float32 router matrix [experts, hidden] and rows with unit inner stride")
    tokens, hidden = x.shape
    experts = router.shape[0]
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    check(library("moe").hb_moe_route(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), ptr(router), i32(tokens), i32(hidden), i32(experts), i32(top),
                                      i32(1 if weighted else 0), ptr(chosen), ptr(weights), stream_ptr()), "moe_route")
    return chosen, weights


def route_scored(x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, top: int, group_count: int, group_keep: int,
                 scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """Router logits ``x router^T`` in float, scores = softmax over all outputs, choice scores = scores + ``correction``; only outputs of
    the ``group_keep`` groups (of ``group_count`` equal groups of neighbours; at most 1: no groups) whose largest choice score is
    largest can be chosen; the ``top`` largest choice scores (lowest index first among equals); weights = the plain scores of the
    chosen times ``scale``, not renormalised: ([tokens, top] int32, [tokens, top] float)."""
    require_cuda(x, router, correction)
    if router.dtype != torch.float32 or not router.is_contiguous() or x.stride(-1) != 1 or x.shape[1] != router.shape[1]:
        raise KernelError("moe.route_scored: a dense float32 router matrix [outputs, hidden] and rows with unit inner stride")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != router.shape[0] or not correction.is_contiguous()):
        raise KernelError("moe.route_scored: the correction is a dense float32 vector with one entry per router output")
    tokens, hidden = x.shape
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    check(library("moe").hb_moe_route_scored(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), ptr(router), ptr(correction), i32(tokens), i32(hidden),
                                             i32(router.shape[0]), i32(top), i32(group_count), i32(group_keep), f32(scale), ptr(chosen), ptr(weights),
                                             stream_ptr()), "moe_route_scored")
    return chosen, weights


def capacity_for(pairs: int, experts: int, pad: int = PAD) -> int:
    """Rows the sorted buffers need whatever the routing: all pairs, each expert's run padded to whole tiles."""
    return -(-(pairs + experts * (pad - 1)) // pad) * pad


def plan(chosen: torch.Tensor, weights: torch.Tensor | None, experts: int) -> Plan:
    """``weights`` None: every row's weight is 1 (the weights then multiply what the experts return: :func:`combine_weighted`).  A choice
    of ``experts`` or above (a router output without matrices) takes no row; its ``slot_of`` is -1."""
    require_cuda(chosen, weights)
    tokens, top = chosen.shape
    pairs = tokens * top
    capacity = capacity_for(pairs, experts)
    device = chosen.device
    out = Plan(capacity, top, torch.empty(pairs, dtype=torch.int32, device=device), torch.empty(capacity, dtype=torch.int32, device=device),
               torch.empty(capacity, dtype=torch.float32, device=device), torch.empty(capacity // PAD, dtype=torch.int32, device=device),
               torch.empty(capacity // PAD, dtype=torch.int32, device=device), pairs)
    check(library("moe").hb_moe_plan(ptr(chosen), ptr(weights), i32(pairs), i32(top), i32(experts), i32(PAD), i32(capacity), ptr(out.slot_of),
                                     ptr(out.slot_token), ptr(out.slot_weight), ptr(out.tile_expert), ptr(out.tile_rows), stream_ptr()), "moe_plan")
    return out


def gather(x: torch.Tensor, where: Plan) -> torch.Tensor:
    """[capacity, hidden]: row s = slot_weight[s] * x[slot_token[s]] in the element type of ``x``; padding rows are not written
    (rows never meet in a product and no one reads what comes of them)."""
    require_cuda(x)
    if x.stride(-1) != 1:
        raise KernelError("moe.gather: rows with unit inner stride")
    out = torch.empty((where.capacity, x.shape[1]), dtype=x.dtype, device=x.device)
    check(library("moe").hb_moe_gather(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), ptr(where.slot_token), ptr(where.slot_weight), ptr(out),
                                       i32(where.capacity), i32(x.shape[1]), stream_ptr()), "moe_gather")
    return out


def takes_tensor_cores(a: torch.Tensor, w: torch.Tensor) -> bool:
    """bfloat16 operands whose rows are multiples of 16 bytes go to ``csrc/moe_gemm_tcgen05.cu``; everything else (float32, where
    every output is one chain of fused multiply-adds whatever the step's size, and odd sizes) to the plain kernel."""
    return a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def grouped_linear(a: torch.Tensor, w: torch.Tensor, where: Plan) -> torch.Tensor:
    """``a`` [capacity, k] times the matrix of each tile's expert: ``w`` [experts, n, k] -> [capacity, n], float accumulation."""
    require_cuda(a, w)
    if a.dtype != w.dtype or not a.is_contiguous() or not w.is_contiguous() or w.dim() != 3 or w.shape[2] != a.shape[1] or a.shape[0] != where.capacity:
        raise KernelError("moe.grouped_linear: dense operands of one element type, rows [capacity, k] and matrices [experts, n, k]")
    out = torch.empty((where.capacity, w.shape[1]), dtype=a.dtype, device=a.device)
    if takes_tensor_cores(a, w):
        lib = library("moe_gemm_tcgen05")
        if where.pairs <= FEW_PAIRS:
            check(lib.hb_moe_gemm_rows(ptr(a), ptr(w), ptr(out), ptr(where.tile_expert), ptr(where.tile_rows), i32(PAD), i32(where.capacity), i32(w.shape[1]),
                                       i32(w.shape[2]), stream_ptr()), "moe_gemm_rows")
        else:
            check(lib.hb_moe_gemm_tiles(ptr(a), ptr(w), ptr(out), ptr(where.tile_expert), i32(where.capacity), i32(w.shape[0]), i32(w.shape[1]),
                                        i32(w.shape[2]), ptr(status_word(a.device)), stream_ptr()), "moe_gemm_tiles")
        return out
    check(library("moe").hb_moe_gemm(ptr(a), ptr(w), ptr(out), i32(is_bf16(a)), ptr(where.tile_expert), i32(PAD), i32(where.capacity), i32(w.shape[1]),
                                     i32(w.shape[2]), stream_ptr()), "moe_gemm")
    return out


def combine(y: torch.Tensor, where: Plan, base: torch.Tensor | None, tokens: int) -> torch.Tensor:
    """out[t] = base[t] + the rows of token t's choices, added in the order of the choices, in float; rounded once."""
    require_cuda(y, base)
    if not y.is_contiguous() or (base is not None and (base.dtype != y.dtype or not base.is_contiguous() or base.shape != (tokens, y.shape[1]))):
        raise KernelError("moe.combine: dense rows, and a base of the same element type and width")
    out = torch.empty((tokens, y.shape[1]), dtype=y.dtype, device=y.device)
    check(library("moe").hb_moe_combine(ptr(y), ptr(where.slot_of), i32(where.top), ptr(base), ptr(out), i32(is_bf16(y)), i32(tokens), i32(y.shape[1]),
                                        stream_ptr()), "moe_combine")
    return out


def combine_weighted(y: torch.Tensor, where: Plan, weights: torch.Tensor, x: torch.Tensor, base: torch.Tensor | None, base_gate: torch.Tensor | None) -> torch.Tensor:
    """out[t] = sigmoid(base_gate[t]) * base[t] + sum over t's choices of weight * (the choice's row of ``y``, or ``x[t]`` itself where the
    choice took no row), added in the order of the choices, in float; rounded once.  ``base_gate`` [tokens] float (None: the base is
    added as it is)."""
    require_cuda(y, weights, x, base, base_gate)
    tokens, hidden = x.shape
    if (not y.is_contiguous() or y.shape[1] != hidden or x.dtype != y.dtype or x.stride(1) != 1 or weights.dtype != torch.float32 or not weights.is_contiguous()
            or weights.shape != (tokens, where.top)):
        raise KernelError("moe.combine_weighted: dense rows of one element type and float32 weights [tokens, top]")
    if base is not None and (base.dtype != y.dtype or not base.is_contiguous() or base.shape != (tokens, hidden)):
        raise KernelError("moe.combine_weighted: a base of the same element type and width")
    if base_gate is not None and (base_gate.dtype != torch.float32 or base_gate.numel() != tokens or not base_gate.is_contiguous()):
        raise KernelError("moe.combine_weighted: the base's gate is a dense float32 vector with one entry per token")
    out = torch.empty((tokens, hidden), dtype=y.dtype, device=y.device)
    check(library("moe").hb_moe_combine_weighted(ptr(y), ptr(where.slot_of), ptr(weights), i32(where.top), ptr(x), i32(x.stride(0)), ptr(base), ptr(base_gate),
                                                 ptr(out), i32(is_bf16(y)), i32(tokens), i32(hidden), stream_ptr()), "moe_combine_weighted")
    return out
