"""Grouped-query attention inside a sliding window whose *values* are rotated too.

    q, k, v = W_q x + b_q, W_k x + b_k, W_v x + b_v
    q, k:  the first ``dims`` entries of every head turn by the token's position (``position``: any registered position part that
           offers frequencies; the rest of the head passes unchanged)
    v:     every head turns by its own token's position j over ``value_position``'s entries, and is cached so
    o_i = sum_j softmax_j((q_i . k_j) * scale) v_j  over the keys with 0 <= i - j < window (window 0: every earlier key)
    o_i:   every head is turned back by the query's position i (the same pairs and frequencies, the angle negated)
    y = W_o [o heads side by side] + b_o

Because a rotation by j followed by one by -i is a rotation by j - i, what a head adds up are values turned by their distance from
the query; turning after the sum instead of every term is what lets the cache hold one rotated value per token.  The projections
stay float from the product to the rotation (angles, sines and cosines are float), queries, keys and values are rounded once where
they are stored, scores and softmax are float.  Query head h reads key/value head h // (heads / kv_heads).

Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim`` (``head_dim`` unless stated), ``scale``, ``window``
(0 = all keys), ``bias`` (bool: biases on q, k, v and o), ``position`` and ``value_position`` (PartSpecs or None), ``names`` (tensor names
after the prefix: q, k, v, o; a bias is its matrix's name with ``.b`` added).  Keys and values of one size lie in pages of
[2, kv_heads, page, d] and, in bfloat16 with head sizes the tensor-core kernels take, are read by those kernels (tcgen05 tiles for
prompt portions, the TMA-fed split-key kernel for decoded tokens) with the window as an argument; of two sizes they lie in pages of
[kv_heads, page, d + e] and are read by the general kernel, as is everything in float32.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import attention as fast_attention
from .attention import GroupedQueryAttention
from .base import POSITIONS, BuildContext, Mixer, PagedKV, PagedTokens, WeightSpec, make, register_mixer
from .spec import PartSpec

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o"}
LARGEST_HEAD = 640  # csrc/attention_generic.cu


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class RotatedValueAttention(GroupedQueryAttention):
    """Shares the planning and the launches of the tensor-core path with its base; everything else is its own."""

    def __init__(self, spec: PartSpec, build: BuildContext):
        Mixer.__init__(self, spec, build)
        p = spec.params
        self.shares_kv, self.softcap = False, 0.0
        self.hidden, self.heads, self.kv_heads = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.window = int(p.get("window") or 0)
        self.bias = bool(p.get("bias", False))
        self.names = {**DEFAULT_NAMES, **dict(p.get("names") or {})}
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.kv_heads} key/value heads do not divide {self.heads} heads")
        if max(self.head_dim, self.value_dim) > LARGEST_HEAD:
            raise ValueError(f"heads of {self.head_dim} / {self.value_dim} are above the kernel's limit of {LARGEST_HEAD}")
        self.position = make(POSITIONS, p["position"], build) if p.get("position") is not None else None
        self.value_position = make(POSITIONS, p["value_position"], build) if p.get("value_position") is not None else None
        for part, size in ((self.position, self.head_dim), (self.value_position, self.value_dim)):
            if part is not None and not hasattr(part, "inv_freq"):
                raise ValueError("this attention's rotations take frequencies: 'rope_half_partial' or 'rope_interleaved'")
            if part is not None and part.dims > size:
                raise ValueError(f"a rotation of {part.dims} entries in heads of {size}")
        self.q_width, self.k_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_width, self.core_width = self.kv_heads * self.value_dim, self.heads * self.value_dim
        self.fast = self.dtype == torch.bfloat16 and self.value_dim == self.head_dim and fast_attention.supported(self.head_dim)

    def weights(self) -> dict[str, WeightSpec]:
        n = self.names
        wanted = {n["q"]: WeightSpec((self.q_width, self.hidden)), n["k"]: WeightSpec((self.k_width, self.hidden)),
                  n["v"]: WeightSpec((self.v_width, self.hidden)), n["o"]: WeightSpec((self.hidden, self.core_width))}
        if self.bias:
            wanted.update({n["q"] + ".b": WeightSpec((self.q_width,)), n["k"] + ".b": WeightSpec((self.k_width,)),
                           n["v"] + ".b": WeightSpec((self.v_width,)), n["o"] + ".b": WeightSpec((self.hidden,))})
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        mats = [tensors[n[s]] for s in ("q", "k", "v")]
        dtype = _common_dtype(mats)
        self.w_qkv = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.b_qkv = torch.cat([tensors[n[s] + ".b"].to(torch.float32) for s in ("q", "k", "v")], dim=0).contiguous() if self.bias else None
        self.b_o = tensors[n["o"] + ".b"].contiguous() if self.bias else None

    def cache_request(self):
        if self.value_dim == self.head_dim:
            return PagedKV(self.kv_heads, self.head_dim, self.window)
        return PagedTokens((self.kv_heads,), (self.head_dim + self.value_dim,), self.window)

    def kernel_modules(self):
        modules = [("heads_prepare", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]
        if not self.fast:
            return modules + [("attention_generic", {})]
        modules += [("elementwise", {}), ("attention_bf16", {"HB_HEAD_DIM": self.head_dim})]  # which is launched depends on the page size of the cache
        if self.head_dim % 64 == 0:
            modules.append(("attention_tma", {"HB_HEAD_DIM": self.head_dim}))
        if self.head_dim in (64, 128):
            modules.append(("attention_tcgen05", {"HB_HEAD_DIM": self.head_dim}))
        return modules

    def _turn_values(self, rows: torch.Tensor, col0: int, heads: int, positions: torch.Tensor, sign: float) -> None:
        part = self.value_position
        ops.rotate_heads_(rows, col0, heads, self.value_dim, positions, part.inv_freq, part.dims, bool(getattr(part, "half", False)), sign)

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("this attention writes a paged cache of its own; the schedule gave it none")
        proj = ops.linear(x, self.w_qkv, self.b_qkv, torch.float32)
        k_off, v_off = self.q_width, self.q_width + self.k_width
        q = torch.empty((x.shape[0], self.q_width), dtype=self.dtype, device=x.device)
        part, turned = self.position, self.value_position
        ops.heads_prepare_wide(proj, 0, k_off, v_off, self.heads, self.kv_heads, self.head_dim, self.value_dim, step.positions, q_out=q,
                               inv_freq=part.inv_freq if part is not None else None, rot_dims=part.dims if part is not None else 0,
                               rot_half=bool(getattr(part, "half", False)), cache=cache.kv, block_table=cache.block_table, token_row=step.token_row,
                               page_size=cache.page_size, v_inv_freq=turned.inv_freq if turned is not None else None,  # a value is cached turned by its own position
                               v_rot_dims=turned.dims if turned is not None else 0, v_rot_half=bool(getattr(turned, "half", False)))
        if self.fast:
            attn = self._attend_fast(q, step, cache)
        else:
            attn = ops.attention_general(q, self.heads, self.kv_heads, self.head_dim, self.value_dim, cache.kv, cache.block_table, step.token_row,
                                         step.positions, cache.page_size, self.scale, 0.0, self.window)
        if self.value_position is not None:  # the sum of a head's values is turned back by the query's position
            self._turn_values(attn, 0, self.heads, step.positions, -1.0)
        return ops.linear(attn, self.w_o, self.b_o, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_mixer("rotated_value_attention", RotatedValueAttention)
