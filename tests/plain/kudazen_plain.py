"""A plain, slow implementation of the Kudazen decoder: whole sequences, no cache, no batching, one
function per mechanism, torch on the CPU in float64 (or the dtype asked for).

It shares no code with the package: it reads the model folder with its own safetensors reader and
walks the recurrence token by token.  Notation: T tokens, W the model width, H heads, G key/value
heads, d the query/key size of a head, e the value size of a head, R the size of a latent.
Weights are stored [out, in].

A layer reads the stream through one norm and adds both sublayers' results at once:
    h = norm1(x);  x <- x + (mixer(h) + ff(h))
with norm(y) = y split into equal consecutive groups, each divided by its own sqrt(mean(part^2) + eps),
the whole times w.  A layer may use another layer's tensors (``weights_of``) and still be a layer of
its own in the order of layers.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: Path) -> dict[str, torch.Tensor]:
    blob = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + length])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        begin, end = meta["data_offsets"]
        raw = bytearray(blob[8 + length + begin : 8 + length + end])
        out[name] = torch.frombuffer(raw, dtype=DTYPES[meta["dtype"]]).reshape(meta["shape"]).clone() if raw else torch.zeros(meta["shape"], dtype=DTYPES[meta["dtype"]])
    return out


def read_model_folder(folder: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ------------------------------------------------------------------------------------------ small pieces
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The stream's norm: ``groups`` equal consecutive parts, each with a root mean square of its own."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    return unit_rms(parts, eps).reshape(x.shape) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., n]: within the first ``dims`` entries, (x[2i], x[2i+1]) turns by positions * base^(-2i/dims)."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = torch.tensor(base, dtype=x.dtype) ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    cos, sin = angle.cos(), angle.sin()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------------------ feed-forward
def clamped_glu(h: torch.Tensor, w: dict, prefix: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ w[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


# ------------------------------------------------------------------------------------------ mixers
def chunked_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention without rotation: unit-RMS values, a temperature per head, a bias that grows with the
    distance, and sight only inside the query's own chunk of positions."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, d)
    k = (h @ w[prefix + "k"].T).reshape(T, G, d)
    v = unit_rms((h @ w[prefix + "v"].T).reshape(T, G, e), eps)
    temp = w[prefix + "temp"]
    pos = torch.arange(T)
    distance = (pos[:, None] - pos[None, :]).to(h.dtype)
    seen = pos[None, :] <= pos[:, None]
    if m.get("mask") is not None:
        size = int(m["mask"]["size"])
        seen = seen & ((pos[:, None] // size) == (pos[None, :] // size))
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        score = (q[:, head] @ k[:, kv].T) * m["scale"] * temp[head] - slope * distance
        score = score.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, kv]
    return out.reshape(T, H * e) @ w[prefix + "o"].T


def latent_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are made from one small latent per token, with one rotated key part for all heads
    and a softmax whose denominator holds one more term per head (the sink)."""
    T = h.shape[0]
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot_dims, base = int(m["rot"]["dims"]), float(m["rot"]["base"])
    pos = torch.arange(T)
    cq = unit_rms(h @ w[prefix + "dq"].T, eps) * w[prefix + "dq.norm"]
    q = (cq @ w[prefix + "uq"].T).reshape(T, H, d + r)
    q_plain, q_turned = q[..., :d], rotate_pairs(q[..., d:], pos, rot_dims, base)
    down = h @ w[prefix + "dkv"].T
    c = unit_rms(down[:, :R], eps) * w[prefix + "dkv.norm"]
    k_turned = rotate_pairs(down[:, R:], pos, rot_dims, base)  # [T, r], one for all heads
    k_plain = (c @ w[prefix + "uk"].T).reshape(T, H, d)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, e)
    sink = w[prefix + "sink"]
    seen = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        score = (q_plain[:, head] @ k_plain[:, head].T + q_turned[:, head] @ k_turned.T) * m["scale"]
        score = score.masked_fill(~seen, -math.inf)
        top = torch.maximum(score.max(dim=-1, keepdim=True).values, sink[head])
        weights = torch.exp(score - top)
        out[:, head] = (weights / (weights.sum(dim=-1, keepdim=True) + torch.exp(sink[head] - top))) @ v[:, head]
    return out.reshape(T, H * e) @ w[prefix + "o"].T


def wkv(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    """Time mixing with a matrix state per head whose rows fade by a decay computed from the token."""
    T = h.shape[0]
    H, n = m["heads"], m["dim"]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mixed(which: str) -> torch.Tensor:
        return h + (before - h) * w[prefix + "mu." + which]

    r = (mixed("r") @ w[prefix + "r"].T).reshape(T, H, n)
    k = (mixed("k") @ w[prefix + "k"].T).reshape(T, H, n)
    v = (mixed("v") @ w[prefix + "v"].T).reshape(T, H, n)
    gate = silu(mixed("g") @ w[prefix + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed("w") @ w[prefix + "w1"].T) @ w[prefix + "w2"].T + w[prefix + "w0"])).reshape(T, H, n)
    bonus = w[prefix + "u"]  # [H, n]
    state = torch.zeros(H, n, n, dtype=h.dtype)  # [head, key entry, value entry]
    out = torch.zeros(T, H, n, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hij,hi->hj", state + bonus[:, :, None] * kv, r[t])
        state = decay[t][:, :, None] * state + kv
    y = unit_rms(out, eps).reshape(T, H * n) * w[prefix + "norm"] * gate
    return y @ w[prefix + "o"].T


MIXERS = {"attention": chunked_attention, "latent_attention": latent_attention, "wkv": wkv}


# ------------------------------------------------------------------------------------------ the model
def source_of(layers: list, index: int) -> int:
    """The layer whose tensors layer ``index`` uses."""
    while layers[index].get("weights_of") is not None:
        index = int(layers[index]["weights_of"])
    return index


def forward(config: dict, weights: dict[str, torch.Tensor], tokens, dtype=torch.float64, layer_outputs: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs`` receives the stream after every layer."""
    w = {name: t.to(dtype) if t.is_floating_point() else t for name, t in weights.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{source_of(config['layers'], index)}."
        h = group_norm(x, w[prefix + "norm1"], groups, eps)
        delta = MIXERS[layer["type"]](h, w, prefix + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            delta = delta + clamped_glu(h, w, prefix + "mlp.", float(layer["mlp"]["limit"]))
        x = x + delta
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return group_norm(x, w["final.norm"], groups, eps) @ w["embed"].T
