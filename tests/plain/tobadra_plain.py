"""A plain, slow implementation of the Tobadra decoder: whole sequences, no cache, no batching, one
function per mechanism, torch on the CPU in float64 (or the dtype asked for).

It shares no code with the package: it reads the model folder with its own safetensors reader and
walks every recurrence token by token.  Notation: T tokens, W the model width, H heads, G key/value
heads, d the query/key size of a head, e the value size of a head.  Weights are stored [out, in].

The stream starts as norm(embed[token]).  A layer normalises what each sublayer reads and what it returns:
    a = norm1(x);  x <- x + norm1b(mixer(a + conv(a)) * sigmoid(R1 a + r1))
    b = norm2(x);  x <- x + norm2b(ff(b) * sigmoid(R2 b + r2))
with conv a short causal convolution over time per channel.  A layer may use another layer's tensors
(``weights_of``) and still be a layer of its own in the order of layers.  The logits are
embed . norm(x) * logit_scale.
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


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def causal_conv(h: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """h [T, C], weight [C, taps]: out_t = sum_j weight[:, j] * h_(t - taps + 1 + j), zeros before the first token."""
    taps = weight.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < h.shape[0]:
            out[back:] += h[: h.shape[0] - back] * weight[:, j]
    return out


def turn_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, sign: float = 1.0) -> torch.Tensor:
    """x [T, heads, n]: within the first ``dims`` entries, entry i turns together with entry i + dims/2 by
    sign * position * base^(-2i/dims); the rest passes unchanged."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.tensor(base, dtype=x.dtype) ** (-2.0 * i / dims)
    angle = sign * positions.to(x.dtype)[:, None, None] * freq[None, None, :]
    cos, sin = angle.cos(), angle.sin()
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------------------ mixers
def window_attention(h: torch.Tensor, w: dict, p: str, m: dict) -> torch.Tensor:
    """Grouped-query softmax attention inside a sliding window, with biases on all four projections, a rotation of part of
    every query and key head, and values that are rotated by their own position over their whole size when they are
    stored and turned back by the query's position after the weighted sum."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, e)
    rot = m.get("rot")
    if rot is not None:
        q = turn_halves(q, positions, rot["dims"], rot["base"])
        k = turn_halves(k, positions, rot["dims"], rot["base"])
        v = turn_halves(v, positions, e, rot["base"])
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    distance = positions[:, None] - positions[None, :]
    seen = distance >= 0
    if m.get("mask") is not None:
        seen &= distance < m["mask"]["size"]
    scores = scores.masked_fill(~seen[None], float("-inf"))
    o = torch.einsum("hij,jhe->ihe", torch.softmax(scores, dim=-1), v)
    if rot is not None:
        o = turn_halves(o, positions, e, rot["base"], sign=-1.0)
    return o.reshape(T, H * e) @ w[p + "o"].T + w[p + "o.b"]


def lightning(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """A matrix state per head that fades by a constant of the head: S <- decay_h S + k v^T, o = S^T q, with q, k, v
    passed through silu; all heads' outputs are normalised together, gated by sigmoid(W_g h), and projected."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, e)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, e, dtype=h.dtype)
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    y = rms_norm(out.reshape(T, H * e), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def channel_delta(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel:
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, e)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)  # [T, H]
    pre = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(pre).reshape(T, H, d))  # [T, H, d]
    S = torch.zeros(H, d, e, dtype=h.dtype)
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, e)
    y = unit_rms(out, eps) * w[p + "norm"] * gate
    return y.reshape(T, H * e) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def route(h: torch.Tensor, w: dict, p: str, r: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """([T, top] chosen router outputs, [T, top] their weights).  Scores are a softmax over every router output (identity
    experts included); the choice is made on score + correction, inside the best ``keep`` of ``count`` groups of neighbours (a
    group's rank is its best choice score); the weight is the plain score times ``scale``."""
    z = h @ w[p + "router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups is not None:
        T, n = choice.shape
        best = choice.reshape(T, groups["count"], n // groups["count"]).max(dim=-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(groups["keep"], dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(n // groups["count"], dim=1), float("-inf"))
    chosen = choice.topk(r["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * r["scale"]


def expert_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def experts_ff(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    real = r["experts"]
    chosen, weight = route(h, w, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(r["top"]):
            which = int(chosen[t, c])
            y = expert_ff(h[t : t + 1], w, f"{p}e{which}.")[0] if which < real else h[t]  # the last outputs are identity experts
            out[t] += weight[t, c] * y
    if mlp.get("shared") is not None:
        out = out + expert_ff(h, w, p + "shared.") * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------------------ the model
def forward(config: dict, weights: dict[str, torch.Tensor], token_ids, dtype=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every layer."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    x = rms_norm(w["embed"][ids], w["embed.norm"], eps)
    for index, layer in enumerate(config["layers"]):
        source = index
        while config["layers"][source].get("weights_of") is not None:
            source = config["layers"][source]["weights_of"]
        p = f"l{source}."
        m = layer["mixer"]
        a = rms_norm(x, w[p + "norm1"], eps)
        read = a + causal_conv(a, w[p + "canon1"]) if config.get("canon") is not None else a
        if layer["type"] == "attention":
            y = window_attention(read, w, p + "mix.", m)
        elif layer["type"] == "lightning":
            y = lightning(read, w, p + "mix.", m, eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(read, w, p + "mix.", m, eps)
        else:
            raise ValueError(f"no mixer {layer['type']!r}")
        y = y * torch.sigmoid(a @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            b = rms_norm(x, w[p + "norm2"], eps)
            f = dense_ff(b, w, p + "mlp.") if mlp["kind"] == "dense" else experts_ff(b, w, p + "mlp.", mlp)
            f = f * torch.sigmoid(b @ w[p + "rg2"].T + w[p + "rg2.b"])
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_norm(x, w["final.norm"], eps) @ w["embed"].T) * config["logit_scale"]
