"""The Tutizen decoder written out plainly in float64, one function per mechanism, key by key and token by token.
Slow on purpose; shares no code with the package. Weights are a dict name -> float64 tensor, the configuration is the
config.json dictionary.

Notation: x is the residual stream [T, width] of one sequence that starts at position 0; a sublayer reads x itself and
its output is normed before it joins the stream: x <- x + m * g * unit_rms(sublayer(x)), g one number.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return unit_rms(x, eps) * g


def position_vectors(positions, width):
    """[T, width]: entry 2i is sin(p * 10000^(-2i / width)), entry 2i + 1 the cosine of the same angle."""
    out = torch.zeros(len(positions), width, dtype=F64)
    for row, p in enumerate(positions):
        for e in range(width):
            angle = float(p) * 10000.0 ** (-2.0 * (e // 2) / width)
            out[row, e] = math.cos(angle) if e % 2 else math.sin(angle)
    return out


def embed(tokens, table, width):
    return table[torch.as_tensor(tokens, dtype=torch.long)] + position_vectors(range(len(tokens)), width)


def head_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def keys_and_values(x, w, prefix, m, eps):
    """What a layer with projections of its own keeps per token: keys divided by their root mean square over a head,
    values likewise. [T, kv_heads, dim] and [T, kv_heads, vdim]."""
    T = x.shape[0]
    k = (x @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, m["kv_heads"], m["dim"])
    v = (x @ w[prefix + "v"].T + w[prefix + "v.b"]).view(T, m["kv_heads"], m["vdim"])
    return unit_rms(k, eps), unit_rms(v, eps)


def attention(x, w, prefix, m, eps, k, v):
    """Causal attention with a distance penalty per head and a gate per head; ``k``, ``v`` as ``keys_and_values`` gives
    them (this layer's, or those of the layer it borrows from)."""
    T = x.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((x @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, D), eps)
    gate = torch.sigmoid(x @ w[prefix + "g"].T)                      # [T, H]
    slopes = head_slopes(H)
    heads = torch.zeros(T, H, DV, dtype=F64)
    for h in range(H):
        kh = h // (H // G)
        for i in range(T):
            scores = torch.stack([(q[i, h] * k[j, kh]).sum() * m["scale"] - slopes[h] * (i - j) for j in range(i + 1)])
            p = torch.softmax(scores, 0)
            heads[i, h] = (p[:, None] * v[:i + 1, kh]).sum(0) * gate[i, h]
    return heads.reshape(T, H * DV) @ w[prefix + "o"].T + w[prefix + "o.b"]


def clamped_unit(x, gate, up, down, limit):
    """down((g * sigmoid(1.702 g)) * (u + 1)), g = min(gate x, limit), u = clamp(up x, -limit, limit)."""
    g = torch.clamp(x @ gate.T, max=limit)
    u = torch.clamp(x @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def dense_ff(x, w, prefix, mlp):
    return clamped_unit(x, w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"], mlp["limit"])


def route(x, w, prefix, router):
    """Per token: the chosen experts and their weights. [T, top] each."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(x @ w[prefix + "router"].T)                     # [T, E]
    choice = s + w[prefix + "correction"]
    size = E // groups["count"]
    ids, weights = [], []
    for t in range(x.shape[0]):
        totals = []
        for g in range(groups["count"]):
            members = sorted((float(choice[t, e]) for e in range(g * size, (g + 1) * size)), reverse=True)
            totals.append(sum(members[:2]))
        kept = sorted(range(groups["count"]), key=lambda g: (-totals[g], g))[:groups["keep"]]
        allowed = [e for e in range(E) if e // size in kept]
        chosen = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:top]
        total = sum(s[t, e] for e in chosen) + 1e-20
        ids.append(chosen)
        weights.append([s[t, e] / total * router["scale"] for e in chosen])
    return ids, weights


def moe_ff(x, w, prefix, mlp):
    ids, weights = route(x, w, prefix, mlp["router"])
    out = torch.zeros(x.shape[0], w[prefix + "e0.down"].shape[0], dtype=F64)
    for t in range(x.shape[0]):
        for e, a in zip(ids[t], weights[t]):
            p = f"{prefix}e{e}."
            out[t] += a * clamped_unit(x[t:t + 1], w[p + "gate"], w[p + "up"], w[p + "down"], mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        p = prefix + "shared."
        out = out + torch.sigmoid(x @ w[p + "sg"].T) * clamped_unit(x, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["shared"]["limit"])
    return out


def forward(cfg: dict, w: dict, tokens, capture=None):
    """float64 logits [T, vocab] of one sequence. ``capture``: a list that receives the stream after every layer."""
    eps, mult, width = cfg["norm"]["eps"], cfg["residual_mult"], cfg["width"]
    x = embed(tokens, w["embed"], width)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        source = m.get("kv_from")
        if source is None:
            kept[i] = keys_and_values(x, w, p + "mix.", m, eps)
        k, v = kept[i if source is None else source]
        x = x + mult * scalar_norm(attention(x, w, p + "mix.", m, eps, k, v), w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe_ff(x, w, p + "mlp.", mlp)
            x = x + mult * scalar_norm(y, w[p + "norm2"], eps)
        if capture is not None:
            capture.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T
