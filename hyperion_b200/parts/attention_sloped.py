"""Grouped-query attention that knows positions only through a bias that grows with the distance, and sees only the query's
own chunk of positions.

    score(i, j) = (q_i . k_j) * scale * temp_h - slope_h * (i - j),   softmax over the keys j <= i of i's chunk,

with one slope per head given by the model (a constant of the design, not a tensor), an optional learned factor per head
(``temp``), and chunks of ``chunk`` positions counted from position 0 of the sequence (0: every earlier key is seen).  Nothing is
rotated.  Values may be divided by their root mean square per head before they are cached (``value_unit_rms``, no weight).
Keys of ``head_dim`` and values of ``value_dim`` lie in pages like every other attention's of the package.

Per step: one product to [q | k | v] kept in float; one kernel (``csrc/heads_prepare.cu``) that norms the values and writes keys
and values to their pages and the queries to a dense buffer; attention of every token over its request's pages; the output
projection.  In bfloat16, with keys and values of one size that is a multiple of 64 and chunks of at most ``LONGEST_TABLE``
positions, attention runs in the tensor-core kernels of the package's other attentions (tcgen05 tiles for prompt portions, split
keys for decoded tokens): inside a chunk no distance exceeds the chunk, so the slopes become a table by distance (the tcgen05
kernel computes slope times distance itself), the chunk is
those kernels' window argument with a negative sign, and the head's factor multiplies its query (in float, before the query's one
rounding).  Everything else, and float32, runs in ``csrc/attention_generic.cu`` (scores, factor, slope and softmax in float).

Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim`` (``head_dim`` unless stated), ``scale``, ``chunk``,
``slopes`` (one per head, or None), ``head_temperature`` (bool: the tensor ``temp`` [heads]), ``value_unit_rms`` (bool), ``eps``.
Tensors: q, k, v, temp, o.
"""
from __future__ import annotations

from typing import Mapping

import math

import torch

from .. import ops
from ..ops import attention as fast_attention
from .attention import GroupedQueryAttention
from .base import BuildContext, Mixer, PagedKV, PagedTokens, WeightSpec, register_mixer
from .spec import PartSpec

LARGEST_HEAD = 640  # csrc/attention_generic.cu
LONGEST_TABLE = 16384  # chunks up to this many positions get their slopes as a table by distance


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class SlopedAttention(Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.chunk = int(p.get("chunk") or 0)
        self.eps = float(p.get("eps", 0.0))
        self.value_unit_rms = bool(p.get("value_unit_rms", False))
        self.head_temperature = bool(p.get("head_temperature", False))
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.kv_heads} key/value heads do not divide {self.heads} heads")
        if max(self.head_dim, self.value_dim) > LARGEST_HEAD:
            raise ValueError(f"heads of {self.head_dim} / {self.value_dim} are above the kernel's limit of {LARGEST_HEAD}")
        slopes = p.get("slopes")
        if slopes is not None and len(slopes) != self.heads:
            raise ValueError(f"{len(slopes)} slopes for {self.heads} heads")
        self.slopes = torch.tensor([float(v) for v in slopes], dtype=torch.float64).to(torch.float32).to(build.device) if slopes is not None else None
        self.q_width, self.k_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_width, self.core_width = self.kv_heads * self.value_dim, self.heads * self.value_dim
        self.temp = None
        self.window, self.softcap = -self.chunk, 0.0  # as the tensor-core kernels take them: a negative window is a chunk
        self.fast = (self.dtype == torch.bfloat16 and self.value_dim == self.head_dim and self.head_dim % 64 == 0 and fast_attention.supported(self.head_dim)
                     and (self.slopes is None or 0 < self.chunk <= LONGEST_TABLE))
        self.by_distance_log2 = self.per_position_log2 = None
        if self.fast and self.slopes is not None:  # [heads, chunk]: minus slope times distance, in the base-2 units of those kernels' softmax
            distance = torch.arange(self.chunk, dtype=torch.float32, device=build.device)
            self.by_distance_log2 = (-(self.slopes[:, None] * distance[None, :]) * math.log2(math.e)).contiguous()
            self.per_position_log2 = (-self.slopes * math.log2(math.e)).contiguous()  # [heads]: kernels that compute the bias take this

    def weights(self) -> dict[str, WeightSpec]:
        wanted = {"q": WeightSpec((self.q_width, self.hidden)), "k": WeightSpec((self.k_width, self.hidden)), "v": WeightSpec((self.v_width, self.hidden)),
                  "o": WeightSpec((self.hidden, self.core_width))}
        if self.head_temperature:
            wanted["temp"] = WeightSpec((self.heads,), init="one_plus_normal")
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        mats = [tensors["q"], tensors["k"], tensors["v"]]
        dtype = _common_dtype(mats)
        self.w_qkv = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.temp = tensors["temp"].to(torch.float32).contiguous() if self.head_temperature else None

    def cache_request(self):
        if self.value_dim == self.head_dim:
            return PagedKV(self.kv_heads, self.head_dim, 0)
        return PagedTokens((self.kv_heads,), (self.head_dim + self.value_dim,), 0)

    def kernel_modules(self):
        modules = [("heads_prepare", {}), ("attention_generic", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]
        if self.fast:  # which is launched depends on the page size of the cache
            modules += [("elementwise", {}), ("attention_tma", {"HB_HEAD_DIM": self.head_dim})]
            if self.head_dim in (64, 128):
                modules.append(("attention_tcgen05", {"HB_HEAD_DIM": self.head_dim}))
        return modules

    def step_plans(self):
        return GroupedQueryAttention.step_plans(self)

    _attend_fast = GroupedQueryAttention._attend_fast
    _longest_short_row = staticmethod(GroupedQueryAttention._longest_short_row)

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("this attention writes a paged cache of its own; the schedule gave it none")
        proj = ops.linear(x, self.w_qkv, None, torch.float32)
        q = torch.empty((x.shape[0], self.q_width), dtype=self.dtype, device=x.device)
        fast = self.fast and fast_attention.takes_distance_bias(self.head_dim, cache.page_size)
        ops.heads_prepare_wide(proj, 0, self.q_width, self.q_width + self.k_width, self.heads, self.kv_heads, self.head_dim, self.value_dim, step.positions,
                               q_out=q, cache=cache.kv, block_table=cache.block_table, token_row=step.token_row, page_size=cache.page_size,
                               v_unit_eps=self.eps if self.value_unit_rms else None, q_head_scale=self.temp if fast else None)
        if fast:
            attn = self._attend_fast(q, step, cache, bias=self.by_distance_log2, bias_per_position=self.per_position_log2)
            return ops.linear(attn, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta
        attn = ops.attention_general(q, self.heads, self.kv_heads, self.head_dim, self.value_dim, cache.kv, cache.block_table, step.token_row, step.positions,
                                     cache.page_size, self.scale, head_scale=self.temp, slopes=self.slopes, chunk=self.chunk)
        return ops.linear(attn, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_mixer("sloped_attention", SlopedAttention)
