"""Kilurax, plainly: whole sequences, no cache, no batching, one function per mechanism, in the precision of the tensors it is
given (the tests use 64-bit).  It shares no code with the engine.

Notation: a sequence's hidden states are rows ``x [T, width]``; ``P`` maps tensor names to tensors; ``cfg`` is the
configuration as config.json holds it (a dictionary).
"""
from __future__ import annotations

import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def grouped_rms_norm(x, weight, groups: int, eps: float):
    """Every row is cut into ``groups`` equal consecutive parts; each part is divided by sqrt(mean(part^2) + eps); then times weight."""
    rows, width = x.shape
    parts = x.reshape(rows, groups, width // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(rows, width) * weight


def causal_conv(x, taps, bias=None):
    """out[t, c] = sum_j taps[c, j] x[t - n + 1 + j, c] (+ bias[c]) with zeros before the first row; the last column is the current row's."""
    rows, channels = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, channels, dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(n):
        out = out + padded[j : j + rows] * taps[:, j]
    return out if bias is None else out + bias


def embed(tokens, P, cfg):
    """Token row times a constant, plus a row of the bigram table chosen by (previous token, token), then the model's norm."""
    bigram = cfg["embedding"].get("bigram")
    rows = []
    for t, token in enumerate(tokens):
        row = P["embed"][int(token)] * cfg["embedding"]["scale"]
        if bigram is not None:
            buckets = int(bigram["buckets"])
            index = buckets if t == 0 else (int(tokens[t - 1]) * int(bigram["mul_prev"]) + int(token) * int(bigram["mul_cur"])) % buckets
            row = row + P["bigram"][index]
        rows.append(row)
    x = torch.stack(rows)
    return grouped_rms_norm(x, P["embed.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"])


def rotate(x, dims: int, base: float, angle_dtype=None):
    """x [T, heads, dim]: of each head's first ``dims`` columns, column i pairs with column i + dims / 2; the pair turns by t * base^(-2i/dims)."""
    rows = x.shape[0]
    half = dims // 2
    angle_dtype = angle_dtype or x.dtype
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64).to(angle_dtype)
    angle = (torch.arange(rows, dtype=angle_dtype)[:, None] * freq[None, :]).to(x.dtype)
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def softmax_attention(h, P, prefix, m, angle_dtype=None):
    """Causal grouped-query attention with biased projections and a partial rotation."""
    rows = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ P[f"{prefix}.q"].T + P[f"{prefix}.q.b"]).reshape(rows, heads, dim)
    k = (h @ P[f"{prefix}.k"].T + P[f"{prefix}.k.b"]).reshape(rows, kv, dim)
    v = (h @ P[f"{prefix}.v"].T + P[f"{prefix}.v.b"]).reshape(rows, kv, vdim)
    q = rotate(q, m["rot"]["dims"], m["rot"]["base"], angle_dtype)
    k = rotate(k, m["rot"]["dims"], m["rot"]["base"], angle_dtype)
    out = torch.zeros(rows, heads, vdim, dtype=h.dtype)
    visible = torch.tril(torch.ones(rows, rows, dtype=torch.bool))
    for head in range(heads):
        g = head // (heads // kv)
        score = (q[:, head] @ k[:, g].T) * m["scale"]
        score = score.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, g]
    return out.reshape(rows, heads * vdim) @ P[f"{prefix}.o"].T + P[f"{prefix}.o.b"]


def mamba2(h, P, prefix, m, eps: float):
    """State-space duality: per head a state [N, vdim] with a scalar decay exp(-exp(A_log) dt) and the write dt B x^T."""
    rows = h.shape[0]
    heads, vdim, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * vdim
    u = h @ P[f"{prefix}.in"].T
    z, xbc, dt = u[:, :inner], u[:, inner : 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N :]
    xbc = silu(causal_conv(xbc, P[f"{prefix}.conv"], P[f"{prefix}.conv.b"]))
    x = xbc[:, :inner].reshape(rows, heads, vdim)
    B = xbc[:, inner : inner + G * N].reshape(rows, G, N)
    C = xbc[:, inner + G * N :].reshape(rows, G, N)
    dt = softplus(dt + P[f"{prefix}.dt_bias"])
    rate = torch.exp(P[f"{prefix}.A_log"])
    y = torch.zeros(rows, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        g = head // (heads // G)
        S = torch.zeros(N, vdim, dtype=h.dtype)
        for t in range(rows):
            S = torch.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + P[f"{prefix}.D"][head] * x[t, head]
    y = y.reshape(rows, inner) * silu(z)
    y = grouped_rms_norm(y, P[f"{prefix}.norm"], m["norm_groups"], eps)
    return y @ P[f"{prefix}.o"].T


def hgrn2(h, P, prefix, m, eps: float):
    """Linear attention whose forget gate f also writes: S = diag(f) S + (1 - f) v^T, o = S^T q."""
    rows = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ P[f"{prefix}.q"].T).reshape(rows, heads, dim)
    v = (h @ P[f"{prefix}.v"].T).reshape(rows, heads, vdim)
    lower = P[f"{prefix}.lower"]
    f = (lower + (1.0 - lower) * torch.sigmoid(h @ P[f"{prefix}.f"].T + P[f"{prefix}.f.b"])).reshape(rows, heads, dim)
    o = torch.zeros(rows, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(rows):
            S = f[t, head][:, None] * S + torch.outer(1.0 - f[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * P[f"{prefix}.norm"]
    return o.reshape(rows, heads * vdim) @ P[f"{prefix}.o"].T


def gated_delta(h, P, prefix, m, eps: float):
    """The gated delta rule with one decay per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    rows = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ P[f"{prefix}.q"].T, P[f"{prefix}.q.conv"])).reshape(rows, kv, dim)
    k = silu(causal_conv(h @ P[f"{prefix}.k"].T, P[f"{prefix}.k.conv"])).reshape(rows, kv, dim)
    v = silu(causal_conv(h @ P[f"{prefix}.v"].T, P[f"{prefix}.v.conv"])).reshape(rows, heads, vdim)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P[f"{prefix}.b"].T)
    g = torch.exp(-torch.exp(P[f"{prefix}.A_log"]) * softplus(h @ P[f"{prefix}.a"].T + P[f"{prefix}.dt_bias"]))
    o = torch.zeros(rows, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        j = head // (heads // kv)
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(rows):
            S = g[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            o[t, head] = S.T @ q[t, j]
    o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * P[f"{prefix}.norm"]
    o = o.reshape(rows, heads * vdim) * silu(h @ P[f"{prefix}.g"].T)
    return o @ P[f"{prefix}.o"].T


def expert(h, P, prefix):
    return (silu(h @ P[f"{prefix}.gate"].T) * (h @ P[f"{prefix}.up"].T)) @ P[f"{prefix}.down"].T


def routed_experts(h, P, prefix, mlp):
    """Every row goes, multiplied by its score, through the ``top`` experts with the largest sigmoid scores, and through the shared one."""
    scores = torch.sigmoid(h @ P[f"{prefix}.router"].T)
    top = int(mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(scores.shape[1]), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in order:
            out[t] = out[t] + expert(scores[t, e] * h[t : t + 1], P, f"{prefix}.e{e}")[0]
    if mlp.get("shared"):
        out = out + expert(h, P, f"{prefix}.shared")
    return out


def mixer(h, P, prefix, layer, eps: float, angle_dtype=None):
    kind, m = layer["type"], layer["mixer"]
    if kind == "parallel":
        left = softmax_attention(h, P, f"{prefix}.left", m["left"], angle_dtype)
        right = mamba2(h, P, f"{prefix}.right", m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    if kind == "hgrn2":
        return hgrn2(h, P, prefix, m, eps)
    if kind == "delta":
        return gated_delta(h, P, prefix, m, eps)
    raise ValueError(kind)


def layer_forward(x, P, index: int, layer, cfg, angle_dtype=None):
    groups, eps, mult = cfg["norm"]["groups"], cfg["norm"]["eps"], cfg["residual_mult"]
    name = f"l{index}"
    h = grouped_rms_norm(x, P[f"{name}.norm1"], groups, eps)
    if cfg.get("canon"):
        h = h + causal_conv(h, P[f"{name}.canon1"])
    x = x + mult * grouped_rms_norm(mixer(h, P, f"{name}.mix", layer, eps, angle_dtype), P[f"{name}.norm1b"], groups, eps)
    if layer.get("mlp") is not None:
        h = grouped_rms_norm(x, P[f"{name}.norm2"], groups, eps)
        if cfg.get("canon"):
            h = h + causal_conv(h, P[f"{name}.canon2"])
        x = x + mult * grouped_rms_norm(routed_experts(h, P, f"{name}.mlp", layer["mlp"]), P[f"{name}.norm2b"], groups, eps)
    return x


def forward(tokens, P, cfg, angle_dtype=None):
    """Logits [T, vocab] of a whole sequence, and the stream after every layer."""
    x = embed(tokens, P, cfg)
    layers = []
    for index, layer in enumerate(cfg["layers"]):
        x = layer_forward(x, P, index, layer, cfg, angle_dtype)
        layers.append(x)
    x = grouped_rms_norm(x, P["final.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"])
    return x @ P["head"].T, layers
