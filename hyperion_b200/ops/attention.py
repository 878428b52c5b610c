"""Tensor-core attention over the paged bfloat16 cache: planning on the host and the two launches.

A step's rows are divided by length: rows of more than ``TOKEN_SHAPE_MAX`` tokens are cut into tiles
of ``tile_tokens`` tokens (times the heads of one key/value group = the virtual rows of a block: up to
256 for the tcgen05 kernel, 64 for the others); the tokens of shorter rows (decoded tokens, very short
portions) each get blocks of their own, with the keys split over several blocks when the batch alone
would not fill the GPU.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import host as host_runtime
from .basic import status_word
from .native import KernelError, check, f32, i32, library, ptr, require_cuda, sm_count, stream_ptr

TOKEN_SHAPE_MAX = 4  # at most csrc/attention_tma.cu's FRESH_TOKENS: its producer fetches older keys before the kernel ahead has finished
TILE_ROWS = 64
TC_TILE_ROWS = 256  # csrc/attention_tcgen05.cu: two halves of 128 rows per block
KEY_TILE = 64
BLOCKS_PER_SM = 2  # two blocks of the token shape fit one SM


def supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def uses_tma(head_dim: int, page_size: int) -> bool:
    """Head sizes that are multiples of 64 with pages of 8 to 64 tokens take the TMA-fed kernels."""
    return head_dim % 64 == 0 and 8 <= page_size <= 64


def _entry(head_dim: int, page_size: int, shape: str):
    if uses_tma(head_dim, page_size):
        return getattr(library("attention_tma", HB_HEAD_DIM=head_dim), f"hb_attention_tma_{shape}_capped")
    return getattr(library("attention_bf16", HB_HEAD_DIM=head_dim), f"hb_attention_{shape}_capped")


def takes_distance_bias(head_dim: int, page_size: int) -> bool:
    """A bias per head and distance on the scores is an argument of the TMA-fed kernels and of the tcgen05 kernel."""
    return uses_tma(head_dim, page_size)


def _bias_arguments(bias, heads: int, head_dim: int, page_size: int):
    if bias.dtype != torch.float32 or bias.dim() != 2 or bias.shape[0] != heads or not bias.is_contiguous():
        raise KernelError("attention: the distance bias is a dense float32 table [heads, span] (times log2(e))")
    if not takes_distance_bias(head_dim, page_size):
        raise KernelError(f"attention: no tensor-core kernel takes a distance bias with heads of {head_dim} and pages of {page_size}")
    return ptr(bias), i32(bias.shape[1])


def uses_tcgen05(head_dim: int, page_size: int) -> bool:
    """Head sizes 64 and 128 with pages of 8 to 64 tokens: prompt portions take the tcgen05 kernel (256-row tiles)."""
    return head_dim in (64, 128) and 8 <= page_size <= 64


def tile_rows(head_dim: int, page_size) -> int:
    """Virtual rows (tokens x heads of a group) per tile of the kernel that will run."""
    return TC_TILE_ROWS if page_size is not None and uses_tcgen05(head_dim, page_size) else TILE_ROWS


def tile_tokens(heads: int, kv_heads: int, rows: int = TILE_ROWS) -> int:
    return rows // min(heads // kv_heads, rows)


def plan(rows, tokens_per_tile: int) -> tuple[np.ndarray, np.ndarray]:
    """(tiles as flat triples [first token, count, batch row], items = flat token indices), int32 arrays, made by the
    host runtime from the rows' token counts (rows follow one another in the flat batch)."""
    counts = host_runtime.ints(rows.counts if hasattr(rows, "counts") else [row.count for row in rows])
    tiles = np.empty(3 * int((-(-counts // tokens_per_tile)).sum()), dtype=np.int32)
    items = np.empty(int(counts.sum()), dtype=np.int32)
    n_tiles, n_items = ctypes.c_int(), ctypes.c_int()
    host_runtime.check(host_runtime.library().hb_plan_attention(len(counts), host_runtime.address(counts), tokens_per_tile, TOKEN_SHAPE_MAX,
                                                                host_runtime.address(tiles), ctypes.byref(n_tiles), host_runtime.address(items),
                                                                ctypes.byref(n_items)))
    return tiles[: 3 * n_tiles.value], items[: n_items.value]


def choose_splits(n_items: int, heads: int, kv_heads: int, longest_context: int, sms: int | None = None) -> int:
    """Splits of the keys for the token shape: about two blocks per SM of the device (``sms``, asked from the current
    device when absent) in all, at least 3 key tiles each."""
    group = heads // kv_heads
    blocks = n_items * kv_heads * ((group + 15) // 16)
    key_tiles = -(-longest_context // KEY_TILE)
    target = BLOCKS_PER_SM * (sms or sm_count())
    return max(1, min(target // max(1, blocks), key_tiles // 3, 64))


_WORK: dict[int, torch.Tensor] = {}


def work_counters(device: torch.device) -> torch.Tensor:
    """Two int32 words per device from which the persistent blocks of the tcgen05 prompt attention take their work items:
    zero between launches (the kernel's last block sets them back).  Launches on one device follow one another in one
    stream; two streams launching that kernel at once would share the counter."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _WORK:
        _WORK[index] = torch.zeros(2, dtype=torch.int32, device=torch.device("cuda", index))
    return _WORK[index]


def _common(q, out, cache, block_table, token_row, positions):
    require_cuda(q, out, cache, block_table, token_row, positions)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or q.stride(-1) != 1 or not cache.is_contiguous():
        raise KernelError("attention (bfloat16): queries and cache must be dense bfloat16")


def attention_tiles(q, heads, cache, block_table, token_row, positions, tiles, n_tiles, scale, window, out, tile_size: int = TILE_ROWS,
                    softcap: float = 0.0, bias=None, bias_per_position=None):
    """``tile_size``: the virtual rows per tile the tiles were planned for (64, or 256 for the tcgen05 kernel).
    ``softcap`` > 0: scores become cap * tanh(score / cap) before the softmax.  ``bias`` [heads, span] float, times log2(e):
    the score of a key n positions back takes ``bias[head, min(n, span - 1)]``.  ``bias_per_position`` [heads] float, times log2(e):
    where the bias is n times a number per head, the tcgen05 kernel computes it instead of looking it up (the others take ``bias``)."""
    _common(q, out, cache, block_table, token_row, positions)
    pages, _, kv_heads, page_size, head_dim = cache.shape
    if bias_per_position is not None and uses_tcgen05(head_dim, page_size) and tile_size == TC_TILE_ROWS:
        require_cuda(bias_per_position)
        if bias_per_position.dtype != torch.float32 or bias_per_position.numel() != heads or not bias_per_position.is_contiguous():
            raise KernelError("attention: the bias per position is a dense float32 vector with one entry per head")
        check(library("attention_tcgen05", HB_HEAD_DIM=head_dim).hb_attention_tc_tiles_biased(
            ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row),
            ptr(positions), ptr(tiles), i32(n_tiles), i32(q.shape[0]), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages),
            f32(scale), f32(softcap or 0.0), i32(window or 0), ptr(bias_per_position), i32(-1), ptr(status_word(q.device)), ptr(work_counters(q.device)),
            stream_ptr()), "attention_tiles")
        return
    if bias is not None:
        require_cuda(bias)
        bias_ptr, span = _bias_arguments(bias, heads, head_dim, page_size)
        if uses_tcgen05(head_dim, page_size) and tile_size == TC_TILE_ROWS:
            check(library("attention_tcgen05", HB_HEAD_DIM=head_dim).hb_attention_tc_tiles_biased(
                ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row),
                ptr(positions), ptr(tiles), i32(n_tiles), i32(q.shape[0]), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages),
                f32(scale), f32(softcap or 0.0), i32(window or 0), bias_ptr, span, ptr(status_word(q.device)), ptr(work_counters(q.device)),
                stream_ptr()), "attention_tiles")
            return
        check(library("attention_tma", HB_HEAD_DIM=head_dim).hb_attention_tma_tiles_biased(
            ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row),
            ptr(positions), ptr(tiles), i32(n_tiles), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale),
            f32(softcap or 0.0), i32(window or 0), bias_ptr, span, ptr(status_word(q.device)), stream_ptr()), "attention_tiles")
        return
    if uses_tcgen05(head_dim, page_size) and tile_size == TC_TILE_ROWS:
        check(library("attention_tcgen05", HB_HEAD_DIM=head_dim).hb_attention_tc_tiles_capped(
            ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row),
            ptr(positions), ptr(tiles), i32(n_tiles), i32(q.shape[0]), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages),
            f32(scale), f32(softcap or 0.0), i32(window or 0), ptr(status_word(q.device)), ptr(work_counters(q.device)), stream_ptr()), "attention_tiles")
        return
    entry = _entry(head_dim, page_size, "tiles")
    check(entry(ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table),
                                 i32(block_table.shape[1]), ptr(token_row), ptr(positions), ptr(tiles), i32(n_tiles), i32(heads),
                                 i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale), f32(softcap or 0.0), i32(window or 0),
                                 ptr(status_word(q.device)), stream_ptr()), "attention_tiles")


def attention_tokens(q, heads, cache, block_table, token_row, positions, items, n_items, splits, scale, window, out, workspace=None,
                     softcap: float = 0.0, bias=None):
    _common(q, out, cache, block_table, token_row, positions)
    pages, _, kv_heads, page_size, head_dim = cache.shape
    if splits > 1:
        need = n_items * heads * splits * (head_dim + 2)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.float32, device=q.device)
        elif workspace.numel() < need or workspace.dtype != torch.float32:
            raise KernelError(f"attention_tokens: workspace of {need} floats needed")
    if bias is not None:
        require_cuda(bias)
        bias_ptr, span = _bias_arguments(bias, heads, head_dim, page_size)
        check(library("attention_tma", HB_HEAD_DIM=head_dim).hb_attention_tma_tokens_biased(
            ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row),
            ptr(positions), ptr(items), i32(n_items), i32(splits), ptr(workspace), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages),
            f32(scale), f32(softcap or 0.0), i32(window or 0), bias_ptr, span, ptr(status_word(q.device)), stream_ptr()), "attention_tokens")
    else:
        check(_entry(head_dim, page_size, "tokens")(ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table),
                                      i32(block_table.shape[1]), ptr(token_row), ptr(positions), ptr(items), i32(n_items), i32(splits),
                                      ptr(workspace), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale),
                                      f32(softcap or 0.0), i32(window or 0), ptr(status_word(q.device)), stream_ptr()), "attention_tokens")
    if splits > 1:
        from . import native

        native.LAUNCHES[0] += 1  # the merge kernel


# ------------------------------------------------------------------ attention over latent records (csrc/attention_latent.cu)
LATENT_LARGEST_RECORD = 640


def latent_supported(record: int, value: int) -> bool:
    """Records whose size is a multiple of 16 (up to 640) with values, their first entries, a multiple of 8."""
    return record % 16 == 0 and value % 8 == 0 and 0 < value <= record <= LATENT_LARGEST_RECORD


def choose_latent_shape(rows: int, longest_count: int, heads: int, longest_context: int, sms: int | None = None) -> tuple[bool, int]:
    """(blocks of 32 rows instead of 16, splits of the keys): 32 rows as soon as one request brings more than 16 (token, head) pairs;
    the keys are split only when the blocks would leave most of the device idle, into shares of at least two key tiles."""
    wide = longest_count * heads > 16
    blocks = rows * -(-longest_count * heads // (32 if wide else 16))
    key_tiles = -(-longest_context // KEY_TILE)
    sms = sms or sm_count()
    if 2 * blocks > sms:
        return wide, 1
    return wide, max(1, min(sms // blocks, key_tiles // 2, 64))


def attention_latent(query: torch.Tensor, heads: int, record: int, value: int, cache: torch.Tensor, block_table: torch.Tensor, row_start: torch.Tensor,
                     positions: torch.Tensor, n_rows: int, longest_count: int, longest_context: int, scale: float, sinks: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, workspace: torch.Tensor | None = None, shape: tuple[bool, int] | None = None) -> torch.Tensor:
    """Causal attention of ``heads`` query heads over one shared key/value head: ``query`` [tokens, heads * record] bfloat16 meets the
    records of ``cache`` [pages, 1, page_size, record]; a record's first ``value`` entries are its value.  ``row_start`` [rows + 1] int32:
    the tokens of each request row (consecutive positions); ``longest_count`` the most tokens of a row and ``longest_context`` the
    largest position plus one (they size the launch).  ``sinks`` [heads] float: one more term exp(sink) in each softmax's denominator.
    Returns [tokens, heads * value]."""
    require_cuda(query, cache, block_table, row_start, positions, sinks, out, workspace)
    tokens = query.shape[0]
    if query.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or query.stride(-1) != 1 or query.shape[1] != heads * record:
        raise KernelError("attention_latent: bfloat16 queries of [tokens, heads * record]")
    if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != record or not cache.is_contiguous() or not latent_supported(record, value):
        raise KernelError("attention_latent: a dense cache of [pages, 1, page_size, record], records a multiple of 16 up to 640, values a multiple of 8")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != heads or not sinks.is_contiguous()):
        raise KernelError("attention_latent: sinks are a dense float32 vector with one entry per head")
    if out is None:
        out = torch.empty((tokens, heads * value), dtype=torch.bfloat16, device=query.device)
    elif out.dtype != torch.bfloat16 or out.shape[0] != tokens or out.shape[1] < heads * value or out.stride(1) != 1:
        raise KernelError("attention_latent: the output is a bfloat16 [tokens, >= heads * value] view")
    wide, splits = shape if shape is not None else choose_latent_shape(n_rows, longest_count, heads, longest_context)
    if splits > 1:
        need = tokens * heads * splits * (value + 2)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.float32, device=query.device)
        elif workspace.numel() < need or workspace.dtype != torch.float32:
            raise KernelError(f"attention_latent: workspace of {need} floats needed")
    pages, _, page_size, _ = cache.shape
    check(library("attention_latent", HB_RECORD=record, HB_VALUE=value).hb_attention_latent(
        ptr(query), i32(query.stride(0)), ptr(out), i32(out.stride(0)), ptr(workspace if splits > 1 else None), ptr(cache), ptr(block_table),
        i32(block_table.shape[1]), ptr(row_start), ptr(positions), ptr(sinks), i32(tokens), i32(n_rows), i32(longest_count), i32(heads), i32(page_size),
        i32(pages), i32(splits), i32(1 if wide else 0), f32(scale), ptr(status_word(query.device)), stream_ptr()), "attention_latent")
    if splits > 1:
        from . import native

        native.LAUNCHES[0] += 1  # the merge kernel
    return out
