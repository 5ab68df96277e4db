"""The Netusun decoder written out plainly in float64, one function per mechanism, token by token where a mechanism has
a memory. Slow on purpose; shares no code with the package. Weights are a dict name -> float64 tensor, the configuration
is the config.json dictionary.

Notation: x is the residual stream [T, width] of one sequence that starts at position 0. A layer is
x <- x + s1 * norm(mixer(norm(x))), x <- x + s2 * norm(ff(norm(x))) with a norm on either side of a sublayer and a
learned vector s on what it adds. A block of layers may run several times over; before every pass the stream is mixed
with the embedding output again and a vector of the pass is added.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


# ---------------------------------------------------------------------------------------------------------- rotation
def rotation_frequencies(rot: dict):
    """Frequencies of the dims / 2 pairs and the factor on cos and sin (1 without rescaling)."""
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot: dict):
    """x [T, ..., n]: entry i of the first ``dims`` turns with entry i + dims / 2 by the angle position * f_i."""
    dims = rot["dims"]
    f, magnitude = rotation_frequencies(rot)
    out = x.clone()
    half = dims // 2
    for t, p in enumerate(positions):
        for i in range(half):
            a = float(p) * f[i]
            c, s = math.cos(a) * magnitude, math.sin(a) * magnitude
            u, v = x[t, ..., i], x[t, ..., i + half]
            out[t, ..., i] = u * c - v * s
            out[t, ..., i + half] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------------------ mixers
def latent_attention(h, w, p, m, eps):
    """Causal attention whose keys and values are expanded from one latent vector per token; queries come through a
    latent of their own; one rotated key part for all heads; exp(sink_h) in the denominator; gate on the heads' output."""
    T = h.shape[0]
    H, D, R, DV, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = list(range(T))
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], positions, m["rot"])
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, rank:], positions, m["rot"])                 # [T, R], shared by the heads
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, DV)
    heads = torch.zeros(T, H, DV, dtype=F64)
    for a in range(H):
        for i in range(T):
            s = ((k_plain[:i + 1, a] * q_plain[i, a]).sum(-1) + (k_rot[:i + 1] * q_rot[i, a]).sum(-1)) * m["scale"]
            top = max(float(s.max()), float(w[p + "sink"][a]))
            e = torch.exp(s - top)
            heads[i, a] = (e[:, None] * v[:i + 1, a]).sum(0) / (e.sum() + math.exp(float(w[p + "sink"][a]) - top))
    gated = heads.reshape(T, H * DV) * torch.sigmoid(h @ w[p + "g"].T)
    return gated @ w[p + "o"].T


def short_convolution(u, taps):
    """u [T, C], taps [C, n]: y_t = sum_j taps[:, j] * u_(t - n + 1 + j), zeros before the first token."""
    T, n = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(n):
            s = t - n + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * u[s]
    return y


def window_attention(h, w, p, m, eps):
    """Grouped attention without positions: a short convolution on q, k and v, a norm on every query and key head, capped
    scores, a window, and one added to the softmax's denominator."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = (short_convolution(u, w[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_norm(q.view(T, H, D), w[p + "q.norm"], eps)
    k = rms_norm(k.view(T, G, D), w[p + "k.norm"], eps)
    v = v.view(T, G, DV)
    window = m["mask"]["size"] if m.get("mask") else None
    cap = m.get("softcap")
    heads = torch.zeros(T, H, DV, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            first = 0 if window is None else max(0, i - window + 1)
            s = (k[first:i + 1, g] * q[i, a]).sum(-1) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s)                                            # capped or normed: no overflow to guard against
            heads[i, a] = (e[:, None] * v[first:i + 1, g]).sum(0) / (1.0 + e.sum())
    return heads.reshape(T, H * DV) @ w[p + "o"].T


def log_sigmoid(z):
    return -math.log1p(math.exp(-z)) if z >= 0 else z - math.log1p(math.exp(z))


def matrix_lstm(h, w, p, m, eps):
    """A matrix memory per head with exponential input gates, kept in range by a running maximum that starts at zero."""
    T = h.shape[0]
    H, D, DV, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, DV)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)       # [T, H] log input gate
    gf = cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap)
    out = torch.zeros(T, H, DV, dtype=F64)
    for a in range(H):
        S, n, top = torch.zeros(D, DV, dtype=F64), torch.zeros(D, dtype=F64), 0.0
        for t in range(T):
            li, lf = float(gi[t, a]), log_sigmoid(float(gf[t, a]))
            new_top = max(lf + top, li)
            keep, take = math.exp(lf + top - new_top), math.exp(li - new_top)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            top = new_top
            out[t, a] = (S.T @ q[t, a]) / (max(abs(float(n @ q[t, a])), math.exp(-top)) + 1e-6)
    out = rms_unit(out, eps).reshape(T, H * DV) * w[p + "norm"]
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "mlstm": matrix_lstm}


# ------------------------------------------------------------------------------------------------------ feed-forward
def gated_unit(x, gate, up, down):
    g = x @ gate.T
    return (g * torch.sigmoid(g) * (x @ up.T)) @ down.T


def route(x, w, p, router):
    """Per token the chosen experts and their weights: softmax over all experts, the best groups by their best member,
    the ``top`` largest scores inside them, weights = scores * scale."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    size = E // groups["count"]
    s = torch.softmax(x @ w[p + "router"].T, -1)
    ids, weights = [], []
    for t in range(x.shape[0]):
        best = [max(float(s[t, e]) for e in range(g * size, (g + 1) * size)) for g in range(groups["count"])]
        kept = sorted(range(groups["count"]), key=lambda g: (-best[g], g))[:groups["keep"]]
        chosen = sorted((e for e in range(E) if e // size in kept), key=lambda e: (-float(s[t, e]), e))[:top]
        ids.append(chosen)
        weights.append([s[t, e] * router["scale"] for e in chosen])
    return ids, weights


def feed_forward(x, w, p, mlp):
    if mlp["kind"] == "dense":
        return gated_unit(x, w[p + "gate"], w[p + "up"], w[p + "down"])
    ids, weights = route(x, w, p, mlp["router"])
    out = torch.zeros(x.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(x.shape[0]):
        for e, a in zip(ids[t], weights[t]):
            q = f"{p}e{e}."
            out[t] += a * gated_unit(x[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"])[0]
    if mlp.get("shared"):
        q = p + "shared."
        out = out + torch.sigmoid(x @ w[q + "sg"].T) * gated_unit(x, w[q + "gate"], w[q + "up"], w[q + "down"])
    return out


# -------------------------------------------------------------------------------------------------------------- model
def layer(x, w, i, spec, eps):
    p = f"l{i}."
    y = MIXERS[spec["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    x = x + rms_norm(y, w[p + "norm1b"], eps) * w[p + "ls1"]
    if spec.get("mlp") is not None:
        y = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", spec["mlp"])
        x = x + rms_norm(y, w[p + "norm2b"], eps) * w[p + "ls2"]
    return x


def run_order(cfg: dict):
    """(layer, pass number or None): a pass number marks the first layer of a pass over the repeated block."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, w: dict, tokens, capture=None):
    """float64 logits [T, vocab] of one sequence. ``capture``: a list that receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, enters in run_order(cfg):
        if enters is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][enters]
        x = layer(x, w, i, cfg["layers"][i], eps)
        if capture is not None:
            capture.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
