"""A plain, slow statement of the Darusun design in 64-bit torch on the CPU: one function per mechanism,
whole sequences only, no cache.  The tests compare the library with it; it shares no code with the library.

Notation: h [T, W] is a sublayer's input (the residual stream itself: this design norms what a sublayer
returns, not what it reads), ``w`` a dict from tensor name (as the model file spells it) to a 64-bit tensor,
``cfg`` the config.json dict, ``m`` a mixer's entry of it, ``pre`` the prefix of a sublayer's tensor names.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_number_norm(x, g, eps):
    """RMS norm whose weight is a single number for all coordinates."""
    return unit_rms(x, eps) * g


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def xielu(z, p, q):
    """Above zero a parabola through the origin with slope 1/2, below it an exponential branch with the same slope
    at zero: softplus(p) z^2 + z/2  |  (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    up = softplus(p) * z * z + 0.5 * z
    down = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, up, down)


def _angles(T, n, base, first_position=0):
    half = n // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / n) for i in range(half)], dtype=F64)
    a = torch.arange(first_position, first_position + T, dtype=F64)[:, None] * freq[None, :]
    return torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]


def rotate_halves(x, rot):
    """x [T, heads, dim]: the first rot.dims dims of every head turned by position * base^(-2i/dims), dim i paired
    with dim i + dims/2; the rest stays."""
    n = int(rot["dims"]) if rot else 0
    if n == 0:
        return x
    c, s = _angles(x.shape[0], n, rot["base"])
    half = n // 2
    a, b = x[..., :half], x[..., half:n]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., n:]], -1)


def rotate_neighbours(x, rot):
    """The same turn with dim 2i paired with dim 2i + 1."""
    n = int(rot["dims"]) if rot else 0
    if n == 0:
        return x
    c, s = _angles(x.shape[0], n, rot["base"])
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    turned = torch.stack([a * c - b * s, b * c + a * s], -1).reshape(*x.shape[:-1], n)
    return torch.cat([turned, x[..., n:]], -1)


def attention_keys_values(h, w, pre, m, eps):
    """Keys (rotated, then every head to unit root mean square) and values of a layer that has projections."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = unit_rms(rotate_halves((h @ w[pre + "k"].T).view(T, G, D), m.get("rot")), eps)
    v = (h @ w[pre + "v"].T).view(T, G, V)
    return k, v


def talking_attention(h, w, pre, m, eps, k, v):
    """Grouped causal softmax attention whose heads' scores are mixed by a table before the softmax."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(rotate_halves((h @ w[pre + "q"].T).view(T, H, D), m.get("rot")), eps)
    raw = torch.stack([(q[:, g] @ k[:, g // (H // G)].T) * m["scale"] for g in range(H)])        # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", w[pre + "talk"], raw)
    pos = torch.arange(T)
    hidden = pos[None, :] > pos[:, None]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        p = torch.softmax(mixed[head].masked_fill(hidden, -math.inf), -1)
        out[:, head] = p @ v[:, head // (H // G)]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def latent_attention(h, w, pre, m, eps):
    """Attention whose keys and values are read out of a small latent per position, with a rotated key part all heads
    share, a window, a sink per head in the denominator and a gate per head on the output."""
    T = h.shape[0]
    H, D, R, V, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = {"dims": R, "base": m["rot"]["base"]} if R else None
    cq = unit_rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, D + R)
    q_flat, q_turn = q[..., :D], rotate_neighbours(q[..., D:], rot)
    down = h @ w[pre + "dkv"].T
    c = unit_rms(down[:, :L], eps) * w[pre + "dkv.norm"]
    k_turn = rotate_neighbours(down[:, None, L:], rot)[:, 0]                  # [T, R], one for all heads
    k_flat = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, V)
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    visible = (dist >= 0) & (dist < int(m["mask"]["size"])) if m.get("mask") else dist >= 0
    gate = torch.sigmoid(h @ w[pre + "g"].T)                                   # [T, H]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        s = (q_flat[:, head] @ k_flat[:, head].T + q_turn[:, head] @ k_turn.T) * m["scale"]
        s = s.masked_fill(~visible, -math.inf)
        sink = w[pre + "sink"][head]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        out[:, head] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))) @ v[:, head] * gate[:, head, None]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    act = w[pre + "act"]
    return xielu(h @ w[pre + "up"].T, act[0], act[1]) @ w[pre + "down"].T


def gated_expert(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, top):
    """(experts [T, top], weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    best = torch.topk(z, top, dim=-1)
    return best.indices, torch.softmax(best.values, -1)


def moe_ff(h, w, pre, mlp):
    ids, weights = route(h, w, pre, int(mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), weights[t]):
            out[t] += a * gated_expert(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[pre + "shared.sg"].T) * gated_expert(h, w, pre + "shared.")
    return out


def forward(cfg, w, tokens, layer_outputs=None):
    """Logits [T, vocab] of one sequence; ``layer_outputs``: a list that receives the stream after every layer."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F64)
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        m, pre = L["mixer"], f"l{i}.mix."
        if L["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(x, w, pre, m, eps)
            k, v = kept[m["kv_from"] if m.get("kv_from") is not None else i]
            y = talking_attention(x, w, pre, m, eps, k, v)
        elif L["type"] == "latent_attention":
            y = latent_attention(x, w, pre, m, eps)
        else:
            raise ValueError(f"unknown layer type {L['type']!r}")
        x = x + mult * one_number_norm(y, w[f"l{i}.norm1"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, f"l{i}.mlp.", mlp)
            x = x + mult * one_number_norm(y, w[f"l{i}.norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return one_number_norm(x, w["final.norm"], eps) @ w["head"].T
