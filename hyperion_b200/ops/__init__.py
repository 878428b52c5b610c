from .basic import (gelu_erf, rotate_heads_, scale_, add_group_rmsnorm, clamped_glu, latent_prepare, latent_query, add_rmsnorm, gelu_tanh, sigmoid_gate_, heads_prepare_wide, norm_add_norm, attention_general, attention_generic, embedding, heads_prepare_, kv_store, place_tokens, raise_on_status, rmsnorm_add, rope_, rope_kv_store_, sgemm_f32,
                    status_word, stream_copy, swiglu)
from .linear import gated_linear, linear
from .native import KernelError

__all__ = ["gelu_erf", "rotate_heads_", "scale_", "add_group_rmsnorm", "clamped_glu", "latent_prepare", "latent_query", "add_rmsnorm", "gelu_tanh", "sigmoid_gate_", "heads_prepare_wide", "norm_add_norm", "attention_general", "heads_prepare_", "rmsnorm_add", "stream_copy", "attention_generic", "embedding", "kv_store", "raise_on_status", "rope_", "rope_kv_store_", "sgemm_f32",
           "status_word", "swiglu", "linear", "gated_linear", "KernelError"]
