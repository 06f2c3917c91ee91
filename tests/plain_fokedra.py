"""A plain, slow implementation of the Fokedra decoder on the CPU, one function per mechanism.

Written from the design's equations alone, in double precision, over a whole sequence at a
time (no cache, no batching).  It shares no code with the package: the tests compare the
engine's logits against it.

Notation: ``x`` is [tokens, width]; a head's vector has ``dim`` (queries, keys) or ``vdim``
(values) elements; ``p`` is a token's position in its sequence, counted from 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Per-pair frequencies f_i (i < dims / 2) and the factor on every cosine and sine."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x: [tokens, heads, dim].  Neighbouring elements (2i, 2i+1) of the first ``dims`` are a pair."""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    angle = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(angle) * m)[:, None, :], (torch.sin(angle) * m)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def visible(n: int, mask: dict | None) -> torch.Tensor:
    """[n, n] bool: query i (rows) sees key j."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if mask and mask.get("size"):
        size = int(mask["size"])
        ok = ok & (i // size == j // size)
    return ok


def keys_and_values(h: torch.Tensor, w: dict, mixer: dict, eps: float,
                    positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Keys as a cache would hold them (rotated, then divided by their root mean square) and values."""
    n, G, dim, vdim = h.shape[0], int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    k = (h @ w["k"].T).reshape(n, G, dim)
    v = (h @ w["v"].T).reshape(n, G, vdim)
    if mixer.get("rot"):
        k = rotate_pairs(k, positions, mixer["rot"])
    return rms_unit(k, eps), v


def attention(h: torch.Tensor, w: dict, mixer: dict, eps: float, positions: torch.Tensor,
              kv: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """The attention mixer over one whole sequence; ``kv`` are this layer's or another layer's keys and values."""
    n, H, G = h.shape[0], int(mixer["heads"]), int(mixer["kv_heads"])
    dim, vdim = int(mixer["dim"]), int(mixer["vdim"])
    q = (h @ w["q"].T).reshape(n, H, dim)
    if mixer.get("rot"):
        q = rotate_pairs(q, positions, mixer["rot"])
    q = rms_unit(q, eps)
    k, v = kv
    see = visible(n, mixer.get("mask"))
    heads = []
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head, :] @ k[:, g, :].T) * float(mixer["scale"])
        score = score.masked_fill(~see, float("-inf"))
        heads.append(torch.softmax(score, dim=-1) @ v[:, g, :])
    out = torch.cat(heads, dim=-1)
    out = out * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def dense_ff(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = (h @ w["gate"].T).clamp(max=limit)
    u = (h @ w["up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def hyper_read(streams: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """streams: [s, tokens, width] -> the sublayer's input before its norm."""
    return torch.einsum("s,snw->nw", w_in, streams)


def hyper_write(streams: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """New stream t = sum_s mix[s, t] * old stream s + out[t] * y."""
    return torch.einsum("st,snw->tnw", mix, streams) + w_out[:, None, None] * y[None]


def layer_tensors(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F64) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: dict, tokens: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """Logits [tokens, vocab] and the stream after every layer [layers, tokens, width] (streams summed)."""
    eps = float(config["norm"]["eps"])
    n = len(tokens)
    positions = torch.arange(n)
    x = weights["embed"].to(F64)[torch.tensor(tokens)] * float(config["embedding"]["scale"])
    s = config.get("streams")
    streams = torch.stack([x] * int(s)) if s else None
    cache: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        w = layer_tensors(weights, f"l{i}.")
        mixer = layer["mixer"]
        if layer["type"] != "attention":
            raise ValueError(f"unknown mixer {layer['type']!r}")
        subs = [(1, "mix."), (2, "mlp.")] if layer.get("mlp") else [(1, "mix.")]
        for q, sub in subs:
            u = hyper_read(streams, w[f"hc{q}.in"]) if streams is not None else x
            h = rms_norm(u, w[f"norm{q}"], eps)
            part = {k[len(sub):]: v for k, v in w.items() if k.startswith(sub)}
            if q == 1:
                if mixer.get("kv_from") is None:
                    cache[i] = keys_and_values(h, part, mixer, eps, positions)
                    kv = cache[i]
                else:
                    kv = cache[int(mixer["kv_from"])]
                y = attention(h, part, mixer, eps, positions, kv)
            else:
                y = dense_ff(h, part, layer["mlp"])
            if streams is not None:
                streams = hyper_write(streams, y, w[f"hc{q}.mix"], w[f"hc{q}.out"])
            else:
                x = x + y
        after.append(streams.sum(dim=0) if streams is not None else x)
    x = streams.sum(dim=0) if streams is not None else x
    logits = rms_norm(x, weights["final.norm"].to(F64), eps) @ weights["head"].to(F64).T
    return logits, torch.stack(after)
