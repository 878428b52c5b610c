"""The row-wise operations and the 32-bit matrix product, as functions over torch tensors."""
from __future__ import annotations

import ctypes

import torch

from .native import KernelError, check, f32, i32, is_bf16, library, ptr, require_cuda, stream_ptr

_STATUS: dict[int, torch.Tensor] = {}
STATUS_BITS = {1: "a block-table entry that had to be valid was missing", 2: "a token id outside the vocabulary",
               4: "a position beyond the position table", 8: "a bounded wait inside a kernel ran out",
               0x100: "(in the tile-shaped GEMM)", 0x200: "(in the swapped GEMM)", 0x400: "(in the TMA attention, tile shape)",
               0x800: "(in the TMA attention, token shape)", 0x1000: "(in the tcgen05 attention)"}


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word kernels set bits in instead of faulting; one per device."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _STATUS:
        _STATUS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return _STATUS[index]


def raise_on_status(device: torch.device) -> None:
    """Read the status word (this waits for the device) and raise if a kernel reported a problem."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise KernelError(f"a kernel reported (status word {value:#x}): " + "; ".join(reasons))


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """out[t] = float(table[ids[t]]) * scale; ids int32 on the device."""
    require_cuda(table, ids)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    lib = library("elementwise")
    check(lib.hb_embedding(ptr(table), i32(is_bf16(table)), ptr(ids), ptr(out), i32(tokens), i32(hidden), i32(vocab),
                           f32(scale), ptr(status_word(table.device)), stream_ptr()), "embedding")
    return out


def place_tokens(ids: torch.Tensor, source: torch.Tensor, pairs: torch.Tensor) -> None:
    """ids[pairs[i, 0]] = source[pairs[i, 1]] on the device (all int32); the caller has checked the pairs."""
    require_cuda(ids, source, pairs)
    check(library("elementwise").hb_place_tokens(ptr(ids), ptr(source), ptr(pairs), i32(pairs.numel() // 2), stream_ptr()), "place_tokens")


def add_rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                rows: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of ``h (+ delta)`` times ``weight``.

    Without ``rows`` the sum is written back into ``h`` (float residual stream) and every row is
    normalised; with ``rows`` (int32 indices) only those rows are read and ``h`` is left alone.
    ``delta`` is a tensor, None, or a ``SplitSum`` (a product whose split-K pieces this kernel adds up itself).
    """
    from .gemm import SplitSum

    pieces = delta if isinstance(delta, SplitSum) else None
    hidden = h.shape[-1]
    if pieces is not None:
        fits = (out_dtype == torch.bfloat16 and pieces.dtype == torch.bfloat16 and hidden % 8 == 0 and hidden <= 16384
                and pieces.shape == tuple(h.shape) and pieces.partials.is_contiguous())
        delta = None if fits else pieces.tensor()
        pieces = pieces if fits else None
    require_cuda(h, delta, weight, rows)
    if h.dtype != torch.float32 or weight.dtype != torch.float32 or not h.is_contiguous():
        raise KernelError("add_rmsnorm: the residual stream and the norm weight are float32")
    n_rows = rows.numel() if rows is not None else h.shape[0]
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=out_dtype, device=h.device)
    if delta is not None and (delta.shape != h.shape or not delta.is_contiguous()):
        raise KernelError("add_rmsnorm: delta must have the shape of h")
    lib = library("elementwise")
    write_h = i32(0 if rows is not None else 1)
    if pieces is not None:
        bias = pieces.bias
        bias_f = bias if bias is not None and bias.dtype == torch.float32 else None
        bias_h = bias if bias is not None and bias.dtype == torch.bfloat16 else None
        check(lib.hb_add_rmsnorm_splits(ptr(h), ptr(pieces.partials), i32(pieces.partials.shape[0]), i32(h.shape[0]), ptr(bias_f), ptr(bias_h),
                                        ptr(weight), ptr(out), ptr(rows), i32(n_rows), i32(hidden), f32(eps), write_h, stream_ptr()), "add_rmsnorm")
        return out
    check(lib.hb_add_rmsnorm(ptr(h), ptr(delta), i32(is_bf16(delta) if delta is not None else 0), ptr(weight), ptr(out),
                             i32(is_bf16(out)), ptr(rows), i32(n_rows), i32(hidden), f32(eps), write_h,
                             stream_ptr()), "add_rmsnorm")
    return out


def rmsnorm_add(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, copy_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """h += y / sqrt(mean(y^2) + eps) * weight, row by row, in the float residual stream ``h``.  With ``copy_dtype``
    bfloat16 the new rows are also returned in that type (the next sublayer's input); otherwise None."""
    require_cuda(h, y, weight)
    if h.dtype != torch.float32 or weight.dtype != torch.float32 or not h.is_contiguous() or not y.is_contiguous() or y.shape != h.shape:
        raise KernelError("rmsnorm_add: a dense float32 stream, a float32 weight and a dense sublayer output of the stream's shape")
    copy = None
    if copy_dtype == torch.bfloat16:
        if y.dtype != torch.bfloat16:
            raise KernelError("rmsnorm_add: a bfloat16 copy is made beside a bfloat16 sublayer output")
        copy = torch.empty_like(y)
    check(library("elementwise").hb_rmsnorm_add(ptr(h), ptr(y), i32(is_bf16(y)), ptr(weight), ptr(copy), i32(h.shape[0]), i32(h.shape[1]),
                                                f32(eps), stream_ptr()), "rmsnorm_add")
    return copy


def stream_copy(h: torch.Tensor) -> torch.Tensor:
    """The float stream rounded to bfloat16."""
    require_cuda(h)
    if h.dtype != torch.float32 or not h.is_contiguous():
        raise KernelError("stream_copy: a dense float32 stream")
    out = torch.empty(h.shape, dtype=torch.bfloat16, device=h.device)
    check(library("elementwise").hb_stream_copy(ptr(h), ptr(out), ctypes.c_longlong(h.numel()), stream_ptr()), "stream_copy")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int | None = None) -> torch.Tensor:
    """[tokens, 2I] -> silu(gate) * up, [tokens, I].  ``block``: gate and up columns alternate in runs of that many columns
    (``block`` gate columns, then their up columns); None: all gate columns first."""
    require_cuda(gate_up)
    tokens, twice = gate_up.shape
    inter = twice // 2
    block = inter if block is None else block
    if block <= 0 or inter % block:
        raise KernelError(f"swiglu: runs of {block} columns do not divide {inter}")
    if out is None:
        out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    lib = library("elementwise")
    for start in range(0, tokens, 65535):
        count = min(65535, tokens - start)
        check(lib.hb_swiglu(ptr(gate_up[start:]), ptr(out[start:]), i32(is_bf16(gate_up)), i32(count), i32(inter), i32(block), stream_ptr()), "swiglu")
    return out


def rope_(x: torch.Tensor, heads: int, head_dim: int, positions: torch.Tensor, table: torch.Tensor) -> None:
    """Rotate the first ``heads`` heads of every row of ``x`` in place; table [max_pos, head_dim/2, 2] float."""
    require_cuda(x, positions, table)
    if x.stride(-1) != 1 or table.dtype != torch.float32 or table.shape[1] * 2 != head_dim:
        raise KernelError("rope: bad layout")
    lib = library("elementwise")
    check(lib.hb_rope(ptr(x), i32(is_bf16(x)), ptr(positions), ptr(table), i32(x.shape[0]), i32(x.stride(0)), i32(heads),
                      i32(head_dim), i32(table.shape[0]), ptr(status_word(x.device)), stream_ptr()), "rope")


def kv_store(src: torch.Tensor, k_offset: int, v_offset: int, cache: torch.Tensor, block_table: torch.Tensor,
             token_row: torch.Tensor, positions: torch.Tensor) -> None:
    """Write each token's keys and values (columns of ``src``) into ``cache`` [pages, 2, kv_heads, page, d]."""
    require_cuda(src, cache, block_table, token_row, positions)
    pages, two, kv_heads, page_size, head_dim = cache.shape
    if src.dtype != cache.dtype or two != 2 or not cache.is_contiguous() or src.stride(-1) != 1:
        raise KernelError("kv_store: source and cache must share their element type and be dense")
    lib = library("elementwise")
    check(lib.hb_kv_store(ptr(src), i32(is_bf16(src)), i32(src.shape[0]), i32(src.stride(0)), i32(k_offset), i32(v_offset),
                          ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row), ptr(positions), i32(kv_heads),
                          i32(head_dim), i32(page_size), i32(pages), ptr(status_word(src.device)), stream_ptr()), "kv_store")


def rope_kv_store_(x: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, positions: torch.Tensor, table: torch.Tensor,
                   cache: torch.Tensor, block_table: torch.Tensor, token_row: torch.Tensor) -> None:
    """RoPE on the q heads of ``x`` = [q | k | v] in place, rotated keys and the values written to ``cache``."""
    require_cuda(x, positions, table, cache, block_table, token_row)
    pages, two, cache_heads, page_size, cache_dim = cache.shape
    if (x.dtype != cache.dtype or x.stride(-1) != 1 or table.dtype != torch.float32 or table.shape[1] * 2 != head_dim
            or cache_heads != kv_heads or cache_dim != head_dim or not cache.is_contiguous()):
        raise KernelError("rope_kv_store: bad layout")
    lib = library("elementwise")
    check(lib.hb_rope_kv_store(ptr(x), i32(is_bf16(x)), i32(x.shape[0]), i32(x.stride(0)), i32(q_heads), i32(kv_heads), i32(head_dim),
                               ptr(positions), ptr(table), i32(table.shape[0]), ptr(cache), ptr(block_table), i32(block_table.shape[1]),
                               ptr(token_row), i32(page_size), i32(pages), ptr(status_word(x.device)), stream_ptr()), "rope_kv_store")


def attention_generic(q: torch.Tensor, heads: int, cache: torch.Tensor, block_table: torch.Tensor, token_row: torch.Tensor,
                      positions: torch.Tensor, scale: float, window: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of every token over its request's pages; q is [tokens, >= heads*d] (a view is fine)."""
    require_cuda(q, cache, block_table, token_row, positions)
    pages, two, kv_heads, page_size, head_dim = cache.shape
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, heads * head_dim), dtype=q.dtype, device=q.device)
    if q.dtype != cache.dtype or q.stride(-1) != 1:
        raise KernelError("attention: queries and cache must share their element type")
    lib = library("attention_generic")
    check(lib.hb_attention_generic(ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), i32(is_bf16(q)), ptr(cache),
                                   ptr(block_table), i32(block_table.shape[1]), ptr(token_row), ptr(positions), i32(tokens),
                                   i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale), i32(window or 0),
                                   ptr(status_word(q.device)), stream_ptr()), "attention_generic")
    return out


def paged_strides(cache: torch.Tensor, head_dim: int, v_dim: int) -> tuple[int, int, int, int]:
    """(offset of the values, page stride, head stride, token stride), in elements, of a cache of keys and values in
    either arrangement: [pages, 2, kv_heads, page, d] (keys and values of one size) or [pages, kv_heads, page, d + e]."""
    if cache.dim() == 5:
        pages, two, kv_heads, page_size, d = cache.shape
        if two != 2 or d != head_dim or v_dim != head_dim or not cache.is_contiguous():
            raise KernelError("a cache of [pages, 2, kv_heads, page, d] holds keys and values of one size d")
        return kv_heads * page_size * d, 2 * kv_heads * page_size * d, page_size * d, d
    pages, kv_heads, page_size, both = cache.shape
    if both != head_dim + v_dim or not cache.is_contiguous():
        raise KernelError("a cache of [pages, kv_heads, page, d + e] holds a key of d and a value of e per token")
    return head_dim, kv_heads * page_size * both, page_size * both, both


def heads_prepare_(x: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, v_dim: int, positions: torch.Tensor, *,
                   q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None, eps: float = 0.0,
                   inv_freq: torch.Tensor | None = None, rot_dims: int = 0, v_first: torch.Tensor | None = None,
                   mix: torch.Tensor | None = None, cache: torch.Tensor | None = None, block_table: torch.Tensor | None = None,
                   token_row: torch.Tensor | None = None, page_size: int = 0) -> None:
    """Rows ``x`` = [q | k | v]: query/key norm per head, rotation of interleaved pairs, value mixing with ``v_first``
    (a view of another layer's value columns) by the scalar ``mix``, queries back in place, keys and values into
    ``cache`` (either arrangement of :func:`paged_strides`); every step is optional."""
    require_cuda(x, positions, q_norm, k_norm, inv_freq, v_first, mix, cache, block_table, token_row)
    if x.stride(-1) != 1 or (v_first is not None and (v_first.stride(-1) != 1 or v_first.dtype != x.dtype)):
        raise KernelError("heads_prepare: rows with unit inner stride")
    for t in (q_norm, k_norm, inv_freq, mix):
        if t is not None and t.dtype != torch.float32:
            raise KernelError("heads_prepare: norm weights, frequencies and the mixing scalar are float32")
    v_off = page_stride = head_stride = token_stride = pages = 0
    if cache is not None:
        if cache.dtype != x.dtype:
            raise KernelError("heads_prepare: rows and cache must share their element type")
        v_off, page_stride, head_stride, token_stride = paged_strides(cache, head_dim, v_dim)
        pages = cache.shape[0]
    element = x.element_size()
    v_cache = ctypes.c_void_p(cache.data_ptr() + v_off * element) if cache is not None else ctypes.c_void_p(0)
    check(library("heads_prepare").hb_heads_prepare(
        ptr(x), i32(is_bf16(x)), i32(x.shape[0]), i32(x.stride(0)), i32(q_heads), i32(kv_heads), i32(head_dim), i32(v_dim), ptr(q_norm), ptr(k_norm),
        f32(eps), ptr(inv_freq), i32(rot_dims if inv_freq is not None else 0), ptr(positions), ptr(v_first), i32(v_first.stride(0) if v_first is not None else 0),
        ptr(mix), ptr(cache), v_cache, ctypes.c_longlong(page_stride), ctypes.c_longlong(head_stride), i32(token_stride), ptr(block_table),
        i32(block_table.shape[1] if block_table is not None else 0), ptr(token_row), i32(page_size), i32(pages),
        i32(1 if (cache is not None or v_first is not None) else 0), ptr(status_word(x.device)), stream_ptr()), "heads_prepare")


def attention_general(q: torch.Tensor, heads: int, kv_heads: int, head_dim: int, v_dim: int, cache: torch.Tensor, block_table: torch.Tensor,
                      token_row: torch.Tensor, positions: torch.Tensor, page_size: int, scale: float, softcap: float = 0.0, window: int = 0, *,
                      distance_bias: torch.Tensor | None = None, gate: torch.Tensor | None = None, gate_off: int = 0, out_scale: float = 1.0,
                      out: torch.Tensor | None = None, head_scale: torch.Tensor | None = None, slopes: torch.Tensor | None = None,
                      sinks: torch.Tensor | None = None, chunk: int = 0, value_prefix: bool = False) -> torch.Tensor:
    """Causal attention of every token over its request's pages with keys of ``head_dim`` and values of ``v_dim``, a smooth
    cap on the scores (0 = none) and a window (0 = all keys); the cache in either arrangement of :func:`paged_strides`.
    ``distance_bias`` [heads, span] float: the score of a key ``n`` positions back takes ``distance_bias[head, min(n, span - 1)]``
    (after scale and cap).  ``gate`` [tokens, *] float: the result is multiplied by ``out_scale * sigmoid(gate[:, gate_off:][token, head * v_dim + i])``.
    ``out``: a [tokens, >= heads * v_dim] view the result is written to.  ``head_scale`` [heads] float: a factor on the scaled score;
    ``slopes`` [heads] float: ``slopes[head] * (query position - key position)`` is taken off the score; ``sinks`` [heads] float: one more
    term ``exp(sinks[head])`` in the softmax's denominator, with no key and no value; ``chunk`` > 0: a query sees only the keys of its own
    chunk of ``chunk`` positions (counted from position 0).  ``value_prefix``: the cache is [pages, kv_heads, page, head_dim] and a
    token's value is the first ``v_dim`` entries of its key (attention over a latent)."""
    require_cuda(q, cache, block_table, token_row, positions, distance_bias, gate, out, head_scale, slopes, sinks)
    for t in (head_scale, slopes, sinks):
        if t is not None and (t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous()):
            raise KernelError("attention: factors, slopes and sinks are dense float32 vectors with one entry per head")
    for t in (distance_bias, gate):
        if t is not None and (t.dtype != torch.float32 or t.stride(-1) != 1 or t.dim() != 2):
            raise KernelError("attention: the distance bias and the gate are float32 matrices with unit inner stride")
    if distance_bias is not None and (distance_bias.shape[0] != heads or not distance_bias.is_contiguous()):
        raise KernelError("attention: the distance bias is a dense [heads, span] table")
    if q.dtype != cache.dtype or q.stride(-1) != 1:
        raise KernelError("attention: queries and cache must share their element type")
    if value_prefix:
        if cache.dim() != 4 or cache.shape[1] != kv_heads or cache.shape[3] != head_dim or v_dim > head_dim or not cache.is_contiguous():
            raise KernelError("attention: a cache of [pages, kv_heads, page, head_dim] whose values are the keys' first v_dim entries")
        v_off, page_stride, head_stride, token_stride = 0, kv_heads * cache.shape[2] * head_dim, cache.shape[2] * head_dim, head_dim
    else:
        v_off, page_stride, head_stride, token_stride = paged_strides(cache, head_dim, v_dim)
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, heads * v_dim), dtype=q.dtype, device=q.device)
    elif out.dtype != q.dtype or out.shape[0] != tokens or out.shape[1] < heads * v_dim or out.stride(1) != 1:
        raise KernelError("attention: the output is a [tokens, >= heads * v_dim] view of the queries' element type")
    v_cache = ctypes.c_void_p(cache.data_ptr() + v_off * cache.element_size())
    check(library("attention_generic").hb_attention_extended(
        ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), i32(is_bf16(q)), ptr(cache), v_cache, ctypes.c_longlong(page_stride),
        ctypes.c_longlong(head_stride), i32(token_stride), ptr(block_table), i32(block_table.shape[1]), ptr(token_row), ptr(positions), i32(tokens),
        i32(heads), i32(kv_heads), i32(head_dim), i32(v_dim), i32(page_size), i32(cache.shape[0]), f32(scale), f32(softcap or 0.0), i32(window or 0),
        ptr(distance_bias), i32(distance_bias.shape[1] if distance_bias is not None else 0), ptr(gate), i32(gate.stride(0) if gate is not None else 0),
        i32(gate_off), f32(out_scale), ptr(head_scale), ptr(slopes), ptr(sinks), i32(chunk or 0), ptr(status_word(q.device)), stream_ptr()),
        "attention_general")
    return out


def heads_prepare_wide(x: torch.Tensor, q_off: int, k_off: int, v_off: int, q_heads: int, kv_heads: int, head_dim: int, v_dim: int,
                       positions: torch.Tensor, *, q_out: torch.Tensor, k_out: torch.Tensor | None = None, q_norm: torch.Tensor | None = None,
                       k_norm: torch.Tensor | None = None, norm_whole: bool = False, eps: float = 0.0, inv_freq: torch.Tensor | None = None,
                       rot_dims: int = 0, rot_half: bool = False, k_scale: float = 1.0, cache: torch.Tensor | None = None,
                       block_table: torch.Tensor | None = None, token_row: torch.Tensor | None = None, page_size: int = 0,
                       v_unit_eps: float | None = None, q_head_scale: torch.Tensor | None = None, v_inv_freq: torch.Tensor | None = None,
                       v_rot_dims: int = 0, v_rot_half: bool = False) -> None:
    """Float projections ``x`` [tokens, *] with queries at column ``q_off``, keys at ``k_off``, values at ``v_off``: query/key
    norm (per head with one weight, or over the whole projection with a weight per column), rotation (adjacent pairs, or
    dimension i with i + rot_dims / 2), keys times ``k_scale``; queries to ``q_out`` [tokens, >= q_heads * head_dim], keys and
    values into ``cache`` (either arrangement of :func:`paged_strides`) or keys to ``k_out`` (values then stay where they are).
    ``q_out`` and ``k_out`` may be float views of ``x`` itself.  ``v_unit_eps`` (with a cache): every value head is divided by
    sqrt(mean(v^2) + v_unit_eps) before it is stored.  ``q_head_scale`` [q_heads] float: a factor on every query head, after norm and rotation.
    ``v_inv_freq`` (with a cache): every value head is stored turned by its token's position over its first ``v_rot_dims`` entries (pairs as
    ``v_rot_half`` says, pair i by position * v_inv_freq[i])."""
    require_cuda(x, positions, q_out, k_out, q_norm, k_norm, inv_freq, cache, block_table, token_row, q_head_scale, v_inv_freq)
    if v_inv_freq is not None and (v_inv_freq.dtype != torch.float32 or not v_inv_freq.is_contiguous() or v_inv_freq.numel() < v_rot_dims // 2 or cache is None):
        raise KernelError("heads_prepare_wide: the values' frequencies are dense float32, one per rotated pair, and go with a cache")
    if q_head_scale is not None and (q_head_scale.dtype != torch.float32 or q_head_scale.numel() != q_heads or not q_head_scale.is_contiguous()):
        raise KernelError("heads_prepare_wide: the queries' factors are a dense float32 vector with one entry per head")
    if x.dtype != torch.float32 or x.stride(-1) != 1 or q_out.stride(-1) != 1 or (k_out is not None and (k_out.stride(-1) != 1 or k_out.dtype != q_out.dtype)):
        raise KernelError("heads_prepare_wide: float32 projections and outputs with unit inner stride")
    for t in (q_norm, k_norm, inv_freq):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError("heads_prepare_wide: norm weights and frequencies are dense float32")
    if (cache is None) == (k_out is None):
        raise KernelError("heads_prepare_wide: keys go either to a cache or to k_out")
    v_cache_off = page_stride = head_stride = token_stride = pages = 0
    if cache is not None:
        if cache.dtype != q_out.dtype:
            raise KernelError("heads_prepare_wide: queries and cache must share their element type")
        v_cache_off, page_stride, head_stride, token_stride = paged_strides(cache, head_dim, v_dim)
        pages = cache.shape[0]
    v_cache = ctypes.c_void_p(cache.data_ptr() + v_cache_off * cache.element_size()) if cache is not None else ctypes.c_void_p(0)
    check(library("heads_prepare").hb_heads_prepare_wide(
        ptr(x), i32(x.shape[0]), i32(x.stride(0)), i32(q_off), i32(k_off), i32(v_off), i32(q_heads), i32(kv_heads), i32(head_dim), i32(v_dim),
        ptr(q_norm), ptr(k_norm), i32(1 if norm_whole else 0), f32(eps), ptr(inv_freq), i32(rot_dims if inv_freq is not None else 0),
        i32(1 if rot_half else 0), ptr(positions), f32(k_scale), ptr(q_out), i32(q_out.stride(0)), ptr(k_out),
        i32(k_out.stride(0) if k_out is not None else 0), i32(is_bf16(q_out)), ptr(cache), v_cache, ctypes.c_longlong(page_stride),
        ctypes.c_longlong(head_stride), i32(token_stride), ptr(block_table), i32(block_table.shape[1] if block_table is not None else 0),
        ptr(token_row), i32(page_size), i32(pages), f32(-1.0 if v_unit_eps is None else v_unit_eps), ptr(q_head_scale), ptr(v_inv_freq),
        i32(v_rot_dims if v_inv_freq is not None else 0), i32(1 if v_rot_half else 0), ptr(status_word(x.device)), stream_ptr()),
        "heads_prepare_wide")


def latent_prepare(x: torch.Tensor, q_off: int, q_rank: int, kv_off: int, kv_rank: int, rot_dim: int, q_norm: torch.Tensor, kv_norm: torch.Tensor, eps: float,
                   inv_freq: torch.Tensor | None, rot_dims: int, positions: torch.Tensor, out_dtype: torch.dtype, cache: torch.Tensor, block_table: torch.Tensor,
                   token_row: torch.Tensor, page_size: int) -> torch.Tensor:
    """Float down-projections ``x`` [tokens, *]: the query latent (``q_rank`` columns at ``q_off``) and the key/value latent (``kv_rank``
    columns at ``kv_off``) followed by the shared key part of ``rot_dim`` columns.  Both latents pass an RMS norm with a weight per
    entry; the key part's first ``rot_dims`` entries are rotated in adjacent pairs.  Returns the normed query latent [tokens, q_rank]
    in ``out_dtype``; latent and key part go to ``cache`` [pages, 1, page, kv_rank + rot_dim]."""
    require_cuda(x, q_norm, kv_norm, inv_freq, positions, cache, block_table, token_row)
    if x.dtype != torch.float32 or x.stride(-1) != 1 or q_norm.dtype != torch.float32 or kv_norm.dtype != torch.float32:
        raise KernelError("latent_prepare: float32 projections and norm weights")
    if q_norm.numel() != q_rank or kv_norm.numel() != kv_rank or (rot_dims and (inv_freq is None or inv_freq.numel() < rot_dims // 2)):
        raise KernelError("latent_prepare: a weight per latent entry and a frequency per rotated pair")
    if cache.dtype != out_dtype or cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != kv_rank + rot_dim or not cache.is_contiguous():
        raise KernelError("latent_prepare: a cache of [pages, 1, page, kv_rank + rot_dim] in the output's element type")
    cq = torch.empty((x.shape[0], q_rank), dtype=out_dtype, device=x.device)
    record = kv_rank + rot_dim
    check(library("heads_prepare").hb_latent_prepare(
        ptr(x), i32(x.shape[0]), i32(x.stride(0)), i32(q_off), i32(q_rank), i32(kv_off), i32(kv_rank), i32(rot_dim), i32(rot_dims), ptr(q_norm), ptr(kv_norm),
        f32(eps), ptr(inv_freq), ptr(positions), ptr(cq), i32(cq.stride(0)), i32(is_bf16(cq)), ptr(cache), ctypes.c_longlong(cache.shape[2] * record),
        i32(record), ptr(block_table), i32(block_table.shape[1]), ptr(token_row), i32(page_size), i32(cache.shape[0]), ptr(status_word(x.device)),
        stream_ptr()), "latent_prepare")
    return cq


def latent_query(q: torch.Tensor, q_lat: torch.Tensor, heads: int, dim: int, rot_dim: int, inv_freq: torch.Tensor | None, rot_dims: int,
                 positions: torch.Tensor) -> torch.Tensor:
    """The queries that meet cached latent records: per head, ``q_lat`` [heads, tokens, kv_rank] float (the head's unrotated query part
    carried into the latent's space) followed by the head's rotated part, taken from ``q`` [tokens, heads * (dim + rot_dim)] and
    rotated in adjacent pairs over its first ``rot_dims`` entries.  Returns [tokens, heads * (kv_rank + rot_dim)] in ``q``'s type."""
    require_cuda(q, q_lat, inv_freq, positions)
    tokens = q.shape[0]
    if q_lat.dtype != torch.float32 or q_lat.dim() != 3 or q_lat.shape[0] != heads or q_lat.shape[1] != tokens or q_lat.stride(2) != 1 or q.stride(-1) != 1:
        raise KernelError("latent_query: q_lat is float32 [heads, tokens, kv_rank] with unit inner stride")
    kv_rank = q_lat.shape[2]
    out = torch.empty((tokens, heads * (kv_rank + rot_dim)), dtype=q.dtype, device=q.device)
    check(library("heads_prepare").hb_latent_query(ptr(q), i32(is_bf16(q)), i32(tokens), i32(q.stride(0)), i32(heads), i32(dim), i32(rot_dim), i32(rot_dims),
                                                   ptr(q_lat), ctypes.c_longlong(q_lat.stride(0)), i32(q_lat.stride(1)), i32(kv_rank), ptr(inv_freq),
                                                   ptr(positions), ptr(out), i32(out.stride(0)), stream_ptr()), "latent_query")
    return out


def add_group_rmsnorm(h: torch.Tensor, first: torch.Tensor | None, second: torch.Tensor | None, weight: torch.Tensor, groups: int, eps: float,
                      out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
    """``h + (first + second)`` (either may be absent; the two are added to one another first), then the row is cut into ``groups``
    equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps), the whole times ``weight``.  Without ``rows`` the sum is
    written back into the float stream ``h``; with ``rows`` (int32 indices) only those rows are read and ``h`` is left alone."""
    require_cuda(h, first, second, weight, rows)
    if h.dtype != torch.float32 or weight.dtype != torch.float32 or not h.is_contiguous() or h.dim() != 2:
        raise KernelError("add_group_rmsnorm: the residual stream and the norm weight are float32")
    hidden = h.shape[1]
    deltas = [d for d in (first, second) if d is not None]
    for d in deltas:
        if d.shape != h.shape or not d.is_contiguous() or d.dtype != deltas[0].dtype:
            raise KernelError("add_group_rmsnorm: sublayer outputs are dense, of the stream's shape and of one element type")
    if groups <= 0 or groups > 64 or hidden % groups:
        raise KernelError(f"add_group_rmsnorm: {groups} groups do not divide {hidden} columns (at most 64 groups)")
    n_rows = rows.numel() if rows is not None else h.shape[0]
    out = torch.empty((n_rows, hidden), dtype=out_dtype, device=h.device)
    check(library("elementwise").hb_add_group_rmsnorm(ptr(h), ptr(first), ptr(second), i32(is_bf16(deltas[0]) if deltas else 0), ptr(weight), ptr(out),
                                                      i32(is_bf16(out)), ptr(rows), i32(n_rows), i32(hidden), i32(groups), f32(eps),
                                                      i32(0 if rows is not None else 1), stream_ptr()), "add_group_rmsnorm")
    return out


def clamped_glu(gate_up: torch.Tensor, limit: float, slope: float) -> torch.Tensor:
    """[tokens, 2I] (all gate columns first) -> g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    require_cuda(gate_up)
    if gate_up.dim() != 2 or not gate_up.is_contiguous() or gate_up.shape[1] % 2:
        raise KernelError("clamped_glu: a dense [tokens, 2I] matrix")
    tokens, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    check(library("elementwise").hb_clamped_glu(ptr(gate_up), ptr(out), i32(is_bf16(gate_up)), i32(tokens), i32(inter), f32(limit), f32(slope), stream_ptr()),
          "clamped_glu")
    return out


def norm_add_norm(h: torch.Tensor, y: torch.Tensor | None, w_post: torch.Tensor | None, eps_post: float, offset: torch.Tensor | None,
                  w_next: torch.Tensor | None, eps_next: float, out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                  gate=None, gate_bias: torch.Tensor | None = None) -> torch.Tensor | None:
    """One launch per sublayer boundary of a block that normalises what a sublayer reads *and* what it returns:
    ``h += y / rms(y) * w_post (+ offset)`` in the float stream, then ``h / rms(h) * w_next`` returned in ``out_dtype``.
    Without ``y`` only the offset is added; without ``w_next`` nothing is returned; with ``rows`` (int32 indices) only
    those rows are worked on and ``h`` stays as it was.  ``gate`` [tokens, hidden] float, or a product still in its split-K pieces
    (``ops.gemm.SplitSum`` without a bias of its own), and ``gate_bias`` [hidden] float: ``y`` is first multiplied, entry by entry, by
    sigmoid(gate + gate_bias)."""
    from .gemm import SplitSum

    gate_splits, gate_split_stride = 1, 0
    if isinstance(gate, SplitSum):
        if gate.bias is not None or not gate.partials.is_contiguous():
            raise KernelError("norm_add_norm: a gate in split-K pieces comes dense and without a bias of its own")
        pieces = gate.partials
        gate_splits, gate_split_stride, gate = pieces.shape[0], pieces.shape[1] * pieces.shape[2], pieces[0]
    require_cuda(h, y, w_post, offset, w_next, rows, gate, gate_bias)
    if gate is not None and (y is None or gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape != h.shape or gate.stride(1) != 1):
        raise KernelError("norm_add_norm: the gate is a float32 matrix of the stream's shape beside a sublayer output")
    if gate_bias is not None and (gate is None or gate_bias.dtype != torch.float32 or gate_bias.numel() != h.shape[1] or not gate_bias.is_contiguous()):
        raise KernelError("norm_add_norm: the gate's bias is a dense float32 vector of the stream's width beside a gate")
    if h.dtype != torch.float32 or not h.is_contiguous() or h.dim() != 2:
        raise KernelError("norm_add_norm: a dense float32 stream")
    tokens, hidden = h.shape
    if y is not None and (y.shape != h.shape or not y.is_contiguous() or w_post is None):
        raise KernelError("norm_add_norm: a dense sublayer output of the stream's shape with its norm weight")
    for t in (w_post, offset, w_next):
        if t is not None and (t.dtype != torch.float32 or t.numel() != hidden or not t.is_contiguous()):
            raise KernelError("norm_add_norm: weights and the offset are dense float32 vectors of the stream's width")
    n_rows = rows.numel() if rows is not None else tokens
    out = torch.empty((n_rows, hidden), dtype=out_dtype, device=h.device) if w_next is not None else None
    check(library("elementwise").hb_norm_add_norm(ptr(h), ptr(y), i32(is_bf16(y) if y is not None else 0), ptr(w_post), ptr(offset), ptr(w_next), ptr(out),
                                                  i32(is_bf16(out) if out is not None else 0), ptr(rows), i32(n_rows), i32(hidden), f32(eps_post),
                                                  f32(eps_next), ptr(gate), i32(gate.stride(0) if gate is not None else 0), i32(gate_splits),
                                                  ctypes.c_longlong(gate_split_stride), ptr(gate_bias), stream_ptr()), "norm_add_norm")
    return out


def sigmoid_gate_(x: torch.Tensor, gate: torch.Tensor, gate_off: int, scale: float = 1.0) -> None:
    """x[t, c] <- x[t, c] * scale * sigmoid(gate[t, gate_off + c]) in place; ``x`` may be a view of some columns, ``gate`` is float."""
    require_cuda(x, gate)
    if x.dim() != 2 or x.stride(1) != 1 or gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[0] != x.shape[0]:
        raise KernelError("sigmoid_gate: rows with unit inner stride and a float32 gate of as many rows")
    check(library("elementwise").hb_sigmoid_gate(ptr(x), i32(is_bf16(x)), i32(x.stride(0)), ptr(gate), i32(gate.stride(0)), i32(gate_off), f32(scale),
                                                 i32(x.shape[0]), i32(x.shape[1]), stream_ptr()), "sigmoid_gate")


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), computed in float, in the element type of ``x``."""
    require_cuda(x)
    if not x.is_contiguous():
        raise KernelError("gelu_tanh: a dense tensor")
    out = torch.empty_like(x)
    check(library("elementwise").hb_gelu_tanh(ptr(x), ptr(out), i32(is_bf16(x)), ctypes.c_longlong(x.numel()), stream_ptr()), "gelu_tanh")
    return out


def sgemm_f32(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] (rows may be strided) times weight [N, K] transposed, plus bias, in plain float."""
    require_cuda(x, weight, bias)
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or x.stride(-1) != 1 or not weight.is_contiguous():
        raise KernelError("sgemm_f32: float32 operands with unit inner stride")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"sgemm_f32: x has {k} columns, weight {weight.shape[1]}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    lib = library("sgemm_f32")
    step = 65535 * 64
    for start in range(0, m, step):
        count = min(step, m - start)
        check(lib.hb_sgemm_f32(ptr(x[start:]), ptr(weight), ptr(bias), ptr(out[start:]), i32(count), i32(n), i32(k),
                               i32(x.stride(0)), i32(out.stride(0)), stream_ptr()), "sgemm_f32")
    return out


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    """0.5 z (1 + erf(z / sqrt(2))), computed in float, in the element type of ``x``."""
    require_cuda(x)
    if not x.is_contiguous():
        raise KernelError("gelu_erf: a dense tensor")
    out = torch.empty_like(x)
    check(library("elementwise").hb_gelu_erf(ptr(x), ptr(out), i32(is_bf16(x)), ctypes.c_longlong(x.numel()), stream_ptr()), "gelu_erf")
    return out


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x <- x * scale in place over a dense float32 tensor."""
    require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_: a dense float32 tensor")
    check(library("elementwise").hb_scale_rows(ptr(x), f32(scale), ctypes.c_longlong(x.numel()), stream_ptr()), "scale_rows")
    return x


def rotate_heads_(x: torch.Tensor, col0: int, heads: int, head_dim: int, positions: torch.Tensor, inv_freq: torch.Tensor, rot_dims: int, rot_half: bool,
                  sign: float = 1.0) -> None:
    """Every head of the columns ``col0 .. col0 + heads * head_dim`` of ``x`` turns in place by ``sign`` times its token's position: within a
    head's first ``rot_dims`` entries pair i (entry i with i + rot_dims / 2 when ``rot_half``, else 2i with 2i + 1) by the angle
    sign * position * inv_freq[i].  Float arithmetic, one rounding at the store."""
    require_cuda(x, positions, inv_freq)
    if x.dim() != 2 or x.stride(1) != 1 or inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous() or inv_freq.numel() < rot_dims // 2:
        raise KernelError("rotate_heads: rows with unit inner stride and a dense float32 frequency per pair")
    if col0 < 0 or col0 + heads * head_dim > x.shape[1]:
        raise KernelError("rotate_heads: the heads lie outside the rows")
    check(library("heads_prepare").hb_rotate_heads(ptr(x), i32(is_bf16(x)), i32(x.shape[0]), i32(x.stride(0)), i32(col0), i32(heads), i32(head_dim), i32(rot_dims),
                                                   i32(1 if rot_half else 0), ptr(inv_freq), ptr(positions), f32(sign), stream_ptr()), "rotate_heads")
