"""A plain, slow implementation of the Sarudra decoder on the CPU, one function per mechanism.

Written from the design's equations alone, in double precision, over a whole sequence at a
time (no cache, no batching, no chunking: the state-space layer is the literal recurrence).
It shares no code with the package: the tests compare the engine's logits against it.

Notation: ``x`` is [tokens, width]; ``p`` is a token's position in its sequence, from 0.
Weights come as a dict name -> tensor; a mixer's tensor ``foo`` is ``<layer>.mix.foo``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.minimum(z, torch.full_like(z, 30.0)))))


def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis in ``groups`` equal consecutive parts, each over its own root mean square, times weight."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * weight


def soft_cap(z: torch.Tensor, cap: float | None) -> torch.Tensor:
    return z if not cap else cap * torch.tanh(z / cap)


def turn_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, sign: float = 1.0) -> torch.Tensor:
    """x: [tokens, heads, size].  Element i < dims/2 pairs with i + dims/2; pair i turns by sign * p * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    angle = sign * positions.to(F64)[:, None] * f[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def window_visible(n: int, size: int | None) -> torch.Tensor:
    """[n, n] bool: query i (rows) sees key j when 0 <= i - j < size (no size: every j <= i)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i - j < size)
    return ok


def attention_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, dim, vdim = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"]))
    pos = torch.arange(n)
    q = (h @ w[f"{p}.q"].T).reshape(n, H, dim)
    k = (h @ w[f"{p}.k"].T).reshape(n, G, dim)
    v = (h @ w[f"{p}.v"].T).reshape(n, G, vdim)
    q = grouped_rms_norm(q, w[f"{p}.q.norm"], 1, eps)
    k = grouped_rms_norm(k, w[f"{p}.k.norm"], 1, eps)
    rot = m.get("rot")
    if rot:
        q = turn_halves(q, pos, int(rot["dims"]), float(rot["base"]))
        k = turn_halves(k, pos, int(rot["dims"]), float(rot["base"]))
        v = turn_halves(v, pos, vdim, float(rot["base"]))
    see = window_visible(n, (m.get("mask") or {}).get("size"))
    out = torch.zeros(n, H, vdim, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        s = soft_cap((q[:, head] @ k[:, g].T) * float(m["scale"]), m.get("softcap"))
        s = s.masked_fill(~see, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    if rot:
        out = turn_halves(out, pos, vdim, float(rot["base"]), sign=-1.0)
    return out.reshape(n, H * vdim) @ w[f"{p}.o"].T


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u: [tokens, channels]; taps: [channels, T], the last column multiplies the current token; zeros in front."""
    n, t = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(t - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    out = bias.expand(n, -1).clone()
    for j in range(t):
        out = out + padded[j: j + n] * taps[:, j]
    return out


def state_space_scan(x: torch.Tensor, B: torch.Tensor, C: torch.Tensor, dt: torch.Tensor, a_log: torch.Tensor,
                     D: torch.Tensor) -> torch.Tensor:
    """x [n, heads, vdim], B and C [n, groups, N], dt [n, heads] (already positive).  Per head the state S [N, vdim]
    follows S <- exp(-exp(a_log) dt) S + dt B x^T; the output is S^T C + D x."""
    n, heads, vdim = x.shape
    groups, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for head in range(heads):
        g = head // (heads // groups)
        S = torch.zeros(N, vdim, dtype=F64)
        rate = torch.exp(a_log[head])
        for t in range(n):
            S = torch.exp(-rate * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + D[head] * x[t, head]
    return y


def mamba2_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    heads, vdim, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = heads * vdim
    proj = h @ w[f"{p}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"]))
    x = xbc[:, :inner].reshape(n, heads, vdim)
    B = xbc[:, inner: inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + w[f"{p}.dt_bias"])
    y = state_space_scan(x, B, C, dt, w[f"{p}.A_log"], w[f"{p}.D"]).reshape(n, inner)
    y = grouped_rms_norm(y * silu(z), w[f"{p}.norm"], int(m["norm_groups"]), eps)
    return y @ w[f"{p}.o"].T


def gated_unit(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def routed_experts(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert fed score * h; a shared expert for everyone."""
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    scores = torch.sigmoid(h @ w[f"{p}.router"].T)
    chosen = torch.topk(scores, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            assert 0 <= e < experts
            out[t] += gated_unit((scores[t, e] * h[t])[None], w, f"{p}.e{e}")[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, w, f"{p}.shared")
    return out


def feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_unit(h, w, p)
    return routed_experts(h, w, p, mlp)


def layer_streams(config: dict, weights: dict, tokens: list[int]) -> tuple[list[torch.Tensor], torch.Tensor]:
    """The stream after every layer, and the logits [tokens, vocab]."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"].get("groups", 1))
    x = w["embed"][torch.tensor(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    after = []
    for i, layer in enumerate(config["layers"]):
        mixer = attention_mixer if layer["type"] == "attention" else mamba2_mixer
        x = x + grouped_rms_norm(mixer(x, w, f"l{i}.mix", layer["mixer"], eps), w[f"l{i}.norm1"], groups, eps)
        if layer.get("mlp"):
            x = x + grouped_rms_norm(feed_forward(x, w, f"l{i}.mlp", layer["mlp"]), w[f"l{i}.norm2"], groups, eps)
        after.append(x)
    logits = grouped_rms_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    return after, soft_cap(logits, config.get("logit_softcap"))


def logits(config: dict, weights: dict, tokens: list[int]) -> torch.Tensor:
    return layer_streams(config, weights, tokens)[1]
