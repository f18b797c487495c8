"""A plain, slow statement of the Lilupel design in 64-bit torch on the CPU: one function per mechanism,
whole sequences only, no cache.  The tests compare the library with it; it shares no code with the library.

Notation: h [T, W] is a sublayer's input (the residual stream itself: this design norms what a sublayer
returns, not what it reads), ``w`` a dict from tensor name (as the model file spells it) to a 64-bit tensor,
``cfg`` the config.json dict, ``m`` a mixer's entry of it.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, rot, first_position=0):
    """x [T, heads, dim]: the first rot.dims dims of every head turned by position * base^(-2i/dims), dim i
    paired with dim i + dims/2; the other dims stay.  No ``rot`` entry, or zero dims: nothing is turned."""
    n = int(rot["dims"]) if rot else 0
    if n == 0:
        return x
    T = x.shape[0]
    half = n // 2
    freq = torch.tensor([float(rot["base"]) ** (-2.0 * i / n) for i in range(half)], dtype=F64)
    angle = torch.arange(first_position, first_position + T, dtype=F64)[:, None] * freq[None, :]       # [T, half]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:n]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., n:]], -1)


def window_attention(h, w, pre, m, eps):
    """Grouped softmax attention over the last mask.size positions with a sink in the denominator."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, V)
    q = unit_rms(rotate(q, m.get("rot")), eps)
    k = unit_rms(rotate(k, m.get("rot")), eps)
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    visible = (dist >= 0) & (dist < int(m["mask"]["size"]))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~visible, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, w[pre + "sink"][head])
        e = torch.exp(s - top)
        out[:, head] = (e / (e.sum(-1, keepdim=True) + torch.exp(w[pre + "sink"][head] - top))) @ v[:, g]
    return out.reshape(T, H * V) @ w[pre + "o"].T + w[pre + "o.b"]


def retention(h, w, pre, m, eps):
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q; no softmax."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[pre + "q"].T).view(T, H, D), m.get("rot"))
    k = rotate((h @ w[pre + "k"].T).view(T, H, D), m.get("rot")) * D ** -0.5
    v = (h @ w[pre + "v"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][head]) * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = unit_rms(out, eps).reshape(T, H * V) * silu(h @ w[pre + "g"].T)
    return out @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    return (m["left_scale"] * window_attention(h, w, pre + "left.", m["left"], eps)
            + m["right_scale"] * retention(h, w, pre + "right.", m["right"], eps))


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = bias.expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y


def mamba2_mixer(h, w, pre, m, eps):
    """State-space duality: per head a state S [state, vdim] with a scalar decay a token,
    S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; gated by silu(z), normed in parts, projected."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ w[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[pre + "dt_bias"], beta=1.0, threshold=1e9)     # [T, H]
    rate = torch.exp(w[pre + "A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[pre + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def expert_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def table_moe(h, tokens, w, pre, mlp):
    """Every token id has its experts in a table; each counts 1 / top."""
    top = int(mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens.tolist()):
        for e in w[pre + "table"][tok].tolist():
            out[t] += expert_ff(h[t:t + 1], w, f"{pre}e{int(e)}.")[0] / top
    return out


MIXERS = {"parallel": parallel_mixer, "mamba2": mamba2_mixer}


def forward(tokens, w, cfg, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{int(layer.get('weights_of', i))}."
        x = x + offset_norm(MIXERS[layer["type"]](x, w, pre + "mix.", layer["mixer"], eps), w[pre + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + offset_norm(table_moe(x, tokens, w, pre + "mlp.", layer["mlp"]), w[pre + "norm2"], eps)
        if keep_layers:
            layers.append(x.clone())
    logits = offset_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, layers) if keep_layers else logits
