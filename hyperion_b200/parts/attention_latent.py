"""Attention whose keys and values are made from one small latent per token.

A token leaves one record in the cache: its latent c (``kv_rank`` entries, RMS-normed with a weight per entry) and one rotated
key part (``rot_dim`` entries) that all heads share.  Per head h, key = [K_h c | rotated part], value = V_h c, and queries come
through a latent of their own: c_q = norm(D_q x), q = U_q c_q, laid out head by head as [``head_dim`` unrotated | ``rot_dim`` rotated].

    score_h(i, j) = (q_h,plain(i) . K_h c_j + q_h,rot(i) . k_rot(j)) * scale,  causal softmax (optionally with a sink per head:
    one more term exp(sink_h) in the denominator), out_h = sum_j p_ij V_h c_j, then the output projection.

Nothing per head is ever cached or rebuilt from the cache.  Since q . (K_h c) = (K_h^T q) . c, the query is carried into the
latent's space once per token and head (a batched product with K_h), attention then runs as if there were ONE key/value head
whose keys are the cached records and whose values are the records' first ``kv_rank`` entries, and the result is carried out of
the latent's space by a batched product with V_h.  Norms, angles, scores and softmax are float.

Per step: one product for both down-projections (kept in float); one kernel that norms the latents, rotates the shared key part
and writes the record to its page (``csrc/heads_prepare.cu``); the queries' up-projection; the batched product with K_h; one
kernel that puts the query of every head together (rotating its rotated part); attention; the batched product with V_h; the
output projection.  In bfloat16, with records of a multiple of 16 entries and latents of a multiple of 8, attention runs on the
tensor cores (``csrc/attention_latent.cu``: blocks of 16 or 32 (token, head) pairs over key tiles of 64 records, the keys split over
several blocks when a step brings few tokens).  Everything else, and float32, runs in ``csrc/attention_generic.cu``.

Parameters: ``hidden_size``, ``heads``, ``head_dim``, ``rot_dim``, ``value_dim``, ``kv_rank``, ``q_rank``, ``scale``, ``position`` (a PartSpec
of kind ``rope_interleaved``, or None), ``sink`` (bool), ``eps``.  Tensors: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, o.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import attention as fast_attention
from .attention_sloped import LARGEST_HEAD
from .base import POSITIONS, BuildContext, Mixer, PagedTokens, WeightSpec, make, register_mixer
from .spec import PartSpec


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class LatentAttention(Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.head_dim, self.rot_dim, self.value_dim = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"])
        self.kv_rank, self.q_rank = int(p["kv_rank"]), int(p["q_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.has_sink = bool(p.get("sink", False))
        self.position = make(POSITIONS, p["position"], build) if p.get("position") is not None else None
        if self.position is not None and not hasattr(self.position, "inv_freq"):
            raise ValueError("this attention rotates adjacent pairs: its position encoding must offer frequencies ('rope_interleaved')")
        self.rot_dims = self.position.dims if self.position is not None else 0
        if self.rot_dims > self.rot_dim:
            raise ValueError(f"a rotation of {self.rot_dims} dimensions in a part of {self.rot_dim}")
        self.record = self.kv_rank + self.rot_dim
        if self.record > LARGEST_HEAD:
            raise ValueError(f"a record of {self.record} entries per token is above the kernel's limit of {LARGEST_HEAD}")
        self.q_head = self.head_dim + self.rot_dim
        self.fast = self.dtype == torch.bfloat16 and fast_attention.latent_supported(self.record, self.kv_rank)

    def weights(self) -> dict[str, WeightSpec]:
        wanted = {"dq": WeightSpec((self.q_rank, self.hidden)), "dq.norm": WeightSpec((self.q_rank,), init="one_plus_normal"),
                  "uq": WeightSpec((self.heads * self.q_head, self.q_rank)), "dkv": WeightSpec((self.record, self.hidden)),
                  "dkv.norm": WeightSpec((self.kv_rank,), init="one_plus_normal"), "uk": WeightSpec((self.heads * self.head_dim, self.kv_rank)),
                  "uv": WeightSpec((self.heads * self.value_dim, self.kv_rank)), "o": WeightSpec((self.hidden, self.heads * self.value_dim))}
        if self.has_sink:
            wanted["sink"] = WeightSpec((self.heads,))
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        down = [tensors["dq"], tensors["dkv"]]
        dtype = _common_dtype(down)
        self.w_down = torch.cat([m.to(dtype) for m in down], dim=0).contiguous()
        self.w_uq, self.w_o = tensors["uq"].contiguous(), tensors["o"].contiguous()
        self.q_norm = tensors["dq.norm"].to(torch.float32).contiguous()
        self.kv_norm = tensors["dkv.norm"].to(torch.float32).contiguous()
        self.k_heads = tensors["uk"].reshape(self.heads, self.head_dim, self.kv_rank).contiguous()  # q_plain [H, T, d] x this = the query in the latent's space
        self.v_heads = tensors["uv"].reshape(self.heads, self.value_dim, self.kv_rank).transpose(1, 2).contiguous()  # [H, R, e]
        self.sink = tensors["sink"].to(torch.float32).contiguous() if self.has_sink else None

    def cache_request(self):
        return PagedTokens((1,), (self.record,), 0)

    def kernel_modules(self):
        modules = [("heads_prepare", {}), ("attention_generic", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]
        if self.fast:
            modules.append(("attention_latent", {"HB_RECORD": self.record, "HB_VALUE": self.kv_rank}))
        return modules

    @staticmethod
    def _batched(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        if a.dtype == torch.float32 or out_dtype == a.dtype:
            return torch.bmm(a, b)
        return torch.bmm(a, b, out_dtype=out_dtype)

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("this attention writes a paged cache of its own; the schedule gave it none")
        tokens = x.shape[0]
        inv_freq = self.position.inv_freq if self.position is not None else None
        proj = ops.linear(x, self.w_down, None, torch.float32)
        cq = ops.latent_prepare(proj, 0, self.q_rank, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm, self.eps, inv_freq, self.rot_dims,
                                step.positions, self.dtype, cache.kv, cache.block_table, step.token_row, cache.page_size)
        q = ops.linear(cq, self.w_uq, None, self.dtype)
        plain = q.view(tokens, self.heads, self.q_head)[:, :, : self.head_dim].transpose(0, 1)
        q_lat = self._batched(plain, self.k_heads.to(q.dtype) if self.k_heads.dtype != q.dtype else self.k_heads, torch.float32)
        query = ops.latent_query(q, q_lat, self.heads, self.head_dim, self.rot_dim, inv_freq, self.rot_dims, step.positions)
        if self.fast:
            # a step replayed from a CUDA graph fixes its launch shape for every context its tables can hold
            longest = step.host.get("context_cap") or step.rows.longest_context
            attn = fast_attention.attention_latent(query, self.heads, self.record, self.kv_rank, cache.kv, cache.block_table, step.row_start, step.positions,
                                                   len(step.rows), int(step.rows.counts.max()), int(longest), self.scale, sinks=self.sink)
        else:
            attn = ops.attention_general(query, self.heads, 1, self.record, self.kv_rank, cache.kv, cache.block_table, step.token_row, step.positions,
                                         cache.page_size, self.scale, sinks=self.sink, value_prefix=True)
        core = torch.empty((tokens, self.heads, self.value_dim), dtype=self.dtype, device=x.device)
        v_heads = self.v_heads.to(attn.dtype) if self.v_heads.dtype != attn.dtype else self.v_heads
        torch.bmm(attn.view(tokens, self.heads, self.kv_rank).transpose(0, 1), v_heads, out=core.transpose(0, 1))
        return ops.linear(core.view(tokens, self.heads * self.value_dim), self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_mixer("latent_attention", LatentAttention)
