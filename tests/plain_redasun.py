"""A plain, slow implementation of Redasun: whole sequences, no cache, scores materialised, one function per mechanism.

It shares nothing with the engine.  ``config`` is the dictionary of a config.json; ``tensors`` maps tensor names to torch tensors
(any floating dtype; everything is computed in ``dtype``, 32-bit unless said otherwise).
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, weight, eps):
    mean = x.mean(-1, keepdim=True)
    centred = x - mean
    return centred / torch.sqrt((centred * centred).mean(-1, keepdim=True) + eps) * weight


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_front(x, positions, dims, base):
    """x [T, n, d]: the first ``dims`` columns turn, column i with column i + dims / 2, by position * base^(-2 i / dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).to(x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def differential_lambda(tensors, prefix, diff):
    t = {name: tensors[f"{prefix}.{name}"].double() for name in ("lq1", "lk1", "lq2", "lk2")}
    return float(torch.exp((t["lq1"] * t["lk1"]).sum()) - torch.exp((t["lq2"] * t["lk2"]).sum()) + diff)


def two_map_heads(q, k, v, positions, sizes, eps, lam, w_q_norm, w_k_norm):
    """q [T, 2 H, d], k [T, 2 G, d], v [T, G, dv] as projected -> the heads' outputs [T, H, dv]: norm and rotation of q and k, two causal
    softmax maps per head over the same values, map 1 minus lam times map 2, divided by its root mean square, times (1 - diff)."""
    T = q.shape[0]
    H, G, dv = sizes["heads"], sizes["kv_heads"], sizes["vdim"]
    diff = float(sizes["diff"])
    q = rms(q, eps) * w_q_norm
    k = rms(k, eps) * w_k_norm
    rot = sizes.get("rot") or {"dims": 0, "base": 1.0}
    if rot["dims"]:
        q = rotate_front(q, positions, rot["dims"], rot["base"])
        k = rotate_front(k, positions, rot["dims"], rot["base"])
    visible = positions[:, None] >= positions[None, :]
    out = torch.empty(T, H, dv, dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        maps = []
        for m in range(2):
            score = (q[:, head * 2 + m] @ k[:, g * 2 + m].T) * float(sizes["scale"])
            score = score.masked_fill(~visible, float("-inf"))
            maps.append(torch.softmax(score, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, head] = rms(o, eps) * (1.0 - diff)
    return out


def differential_attention(h, tensors, prefix, sizes, eps, positions=None):
    """h [T, width] -> [T, width]."""
    dtype = h.dtype
    T = h.shape[0]
    H, G, d, dv = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    w = lambda name: tensors[f"{prefix}.{name}"].to(dtype)
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w("q").T).view(T, H * 2, d)
    k = (h @ w("k").T).view(T, G * 2, d)
    v = (h @ w("v").T).view(T, G, dv)
    lam = differential_lambda(tensors, prefix, float(sizes["diff"]))
    heads = two_map_heads(q, k, v, positions, sizes, eps, lam, w("q.norm"), w("k.norm"))
    return heads.reshape(T, H * dv) @ w("o").T


def gated_ff(h, tensors, prefix, act):
    w = lambda name: tensors[f"{prefix}.{name}"].to(h.dtype)
    return (act(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


def route(h, tensors, prefix, router):
    """Per token: the chosen experts (a list of indices) and their weights."""
    z = h.float() @ tensors[f"{prefix}.router"].float().T
    s = torch.sigmoid(z)
    choice = s + tensors[f"{prefix}.correction"].float()
    experts, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    per = experts // groups["count"]
    chosen, weights = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        group_scores = []
        for g in range(groups["count"]):
            members = sorted((float(x) for x in c[g * per:(g + 1) * per]), reverse=True)
            group_scores.append(sum(members[:2]))
        kept = sorted(range(groups["count"]), key=lambda g: -group_scores[g])[: groups["keep"]]
        for g in range(groups["count"]):
            if g not in kept:
                c[g * per:(g + 1) * per] = float("-inf")
        picks = sorted(range(experts), key=lambda e: -float(c[e]))[:top]
        total = sum(float(s[t, e]) for e in picks) + 1e-20
        chosen.append(picks)
        weights.append([float(s[t, e]) / total * float(router["scale"]) for e in picks])
    return chosen, weights


def moe_ff(h, tensors, prefix, mlp):
    silu = lambda z: z * torch.sigmoid(z)
    chosen, weights = route(h, tensors, prefix, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * gated_ff(h[t:t + 1], tensors, f"{prefix}.e{e}", silu)[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, tensors, f"{prefix}.shared", silu)
    return out


def feed_forward(h, tensors, prefix, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, tensors, prefix, gelu_tanh)
    return moe_ff(h, tensors, prefix, mlp)


def layer(x, tensors, index, spec, eps):
    p = f"l{index}"
    n = lambda name: tensors[f"{p}.{name}"].to(x.dtype)
    x = x + layer_norm(differential_attention(layer_norm(x, n("norm1"), eps), tensors, f"{p}.mix", spec["mixer"], eps), n("norm1b"), eps)
    if spec.get("mlp") is not None:
        x = x + layer_norm(feed_forward(layer_norm(x, n("norm2"), eps), tensors, f"{p}.mlp", spec["mlp"]), n("norm2b"), eps)
    return x


def runs_of(config):
    """The order in which layers run: (layer index, whether a pass of the repeated run starts here)."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], count)]


def forward(config, tensors, tokens, dtype=torch.float32):
    """Logits [T, vocab] and the stream after every run of a layer [runs, T, width]."""
    eps = float(config["norm"]["eps"])
    table = tensors["embed"].to(dtype)
    x0 = table[torch.as_tensor(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    x = x0
    trace = []
    for index, starts_pass in runs_of(config):
        if starts_pass:
            x = torch.cat([x, x0], dim=-1) @ tensors["loop.in"].to(dtype).T
        x = layer(x, tensors, index, config["layers"][index], eps)
        trace.append(x)
    logits = layer_norm(x, tensors["final.norm"].to(dtype), eps) @ table.T
    return logits, torch.stack(trace)
