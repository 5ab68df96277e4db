"""Small Netusun configurations and seeded weights for the tests. Nothing here imports the product package."""

from __future__ import annotations

import copy
import math

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale=None, base=10000.0, scaling=None, dims=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                                "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": rot}


def windowed(heads, kv, dim, vdim=None, conv=None, window=None, softcap=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim if vdim is not None else dim,
         "scale": scale if scale is not None else dim ** -0.5}
    if conv is not None:
        m["conv"] = conv
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    return "attention", m


def lstm(heads, dim, vdim=None, cap=8.0):
    return "mlstm", {"heads": heads, "dim": dim, "vdim": vdim if vdim is not None else dim, "gate_cap": cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    """``groups``: (count, keep) or None; ``shared``: the shared expert's width or None."""
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(width, vocab, layers, eps=1e-6, loop=None):
    """``layers``: list of ((type, mixer sizes), mlp or None); ``loop``: (start, stop, times) or None."""
    d = {"architecture": "Netusun", "width": width, "vocab": vocab, "norm": {"eps": eps},
         "layers": [{"type": kind, "mixer": m, "mlp": mlp} for (kind, m), mlp in layers]}
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# A: a block in the middle that runs three times, a matrix LSTM in front of it without a feed-forward; three query heads
# on latents of other widths than the heads'; four taps; a window shorter than the prompts; two of four groups kept.
CASE_A = config(96, 211, [
    (lstm(2, 24, 16, cap=6.0), None),
    (latent(3, 16, 8, 24, 40, 24, scale=0.3), dense(72)),
    (windowed(4, 2, 16, 24, conv=4, window=20, softcap=5.0, scale=0.6), moe(8, 2, 24, groups=(4, 2), scale=2.0, shared=40)),
    (windowed(3, 3, 8, 8, conv=2, window=7, softcap=50.0), moe(6, 3, 20, scale=0.7)),
], eps=1e-6, loop=(1, 3, 3))

# B: nothing runs twice (no pass input at all); as many key heads as query heads; one tap; no window, no cap; one choice
# out of four with every group kept; a single head everywhere; values narrower than keys.
CASE_B = config(80, 157, [
    (windowed(2, 2, 24, 8, conv=1, scale=0.3), dense(56)),
    (latent(1, 8, 4, 12, 16, 8, base=500.0), moe(4, 1, 32, groups=(2, 2), scale=0.5, shared=16)),
    (lstm(1, 8, 40, cap=20.0), dense(24)),
    (windowed(1, 1, 32, window=300), None),
], eps=1e-5)

# C: the sizes the tensor-core kernels take in bfloat16 (attention heads of 64 and 128 with values as wide as keys, a latent
# of 64 + 16, pages of 16); every layer inside a block that runs twice; YaRN whose ramp lies inside the rotated pairs;
# sixteen experts of which four are chosen in two of four groups.
CASE_C = config(128, 263, [
    (latent(6, 32, 16, 32, 64, 48, scale=0.2, scaling=(4.0, 64, 8.0, 1.0)), dense(96)),
    (windowed(4, 2, 64, conv=3, window=48, softcap=10.0, scale=0.4), moe(16, 4, 32, groups=(4, 2), scale=1.5, shared=64)),
    (lstm(2, 64, 128, cap=12.0), moe(8, 2, 48, groups=(2, 1), scale=1.7)),
    (windowed(2, 1, 128, conv=3, window=33, scale=0.3), dense(64)),
], eps=2e-6, loop=(0, 4, 2))

# D: sizes that are multiples of 2 only, so rows of 16-bit numbers start off a 16-byte boundary and every packed path has
# to step aside; a block of one layer that "repeats" once; nine experts in three groups of which one stays; fewer rotated
# entries than the rotated part has.
CASE_D = config(100, 103, [
    (latent(2, 10, 6, 14, 18, 10, scale=0.4, dims=4), moe(9, 2, 14, groups=(3, 1), scale=1.2, shared=22)),
    (windowed(6, 3, 10, 6, conv=2, window=11, softcap=3.0), dense(36)),
    (lstm(3, 10, 14, cap=4.0), None),
], eps=1e-6, loop=(0, 1, 1))

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D}


def run_count(cfg: dict) -> int:
    loop = cfg.get("loop")
    return len(cfg["layers"]) + ((loop["stop"] - loop["start"]) * (loop["times"] - 1) if loop else 0)


def seeded_state(cfg: dict, seed: int, forget_bias: float = 2.0) -> dict:
    """float32 weights by checkpoint name. Matrices N(0, gain^2 / in); norm weights and scales away from one, sinks and
    gate biases of a size that shows."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(n, mean=0.0, std=0.3):
        return mean + std * torch.randn(n, generator=g)

    def unit(p, ff):
        s[p + "gate"], s[p + "up"], s[p + "down"] = mat(ff, width, 1.5), mat(ff, width, 1.5), mat(width, ff)

    s = {"embed": torch.randn(vocab, width, generator=g), "final.norm": vec(width, 1.0, 0.2)}
    if cfg.get("loop"):
        s["loop.in"] = mat(width, 2 * width, 1.4)
        s["loop.step"] = torch.randn(cfg["loop"]["times"], width, generator=g) * 0.5
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        x = p + "mix."
        s[p + "norm1"], s[p + "norm1b"], s[p + "ls1"] = vec(width, 1.0), vec(width, 1.0), vec(width, 0.6, 0.3)
        h, d, dv = m["heads"], m["dim"], m["vdim"]
        if kind == "latent_attention":
            r, rank, qr = m["rot_dim"], m["kv_rank"], m["q_rank"]
            s[x + "dq"], s[x + "dq.norm"], s[x + "uq"] = mat(qr, width), vec(qr, 1.0), mat(h * (d + r), qr, 1.5)
            s[x + "dkv"], s[x + "dkv.norm"] = mat(rank + r, width, 1.5), vec(rank, 1.0)
            s[x + "uk"], s[x + "uv"] = mat(h * d, rank, 1.5), mat(h * dv, rank)
            s[x + "sink"], s[x + "g"], s[x + "o"] = vec(h, 0.5, 1.0), mat(h * dv, width, 2.0), mat(width, h * dv)
        elif kind == "attention":
            kv = m["kv_heads"]
            s[x + "q"], s[x + "k"], s[x + "v"] = mat(h * d, width), mat(kv * d, width), mat(kv * dv, width)
            s[x + "q.norm"], s[x + "k.norm"] = vec(d, 1.0), vec(d, 1.0)
            if m.get("conv"):
                for n, rows in (("q", h * d), ("k", kv * d), ("v", kv * dv)):
                    s[f"{x}{n}.conv"] = torch.randn(rows, m["conv"], generator=g) * 0.6
            s[x + "o"] = mat(width, h * dv)
        else:
            s[x + "q"], s[x + "k"], s[x + "v"] = mat(h * d, width, 1.5), mat(h * d, width, 1.5), mat(h * dv, width)
            s[x + "g"], s[x + "o"], s[x + "norm"] = mat(h * dv, width, 2.0), mat(width, h * dv), vec(h * dv, 1.0)
            s[x + "i"], s[x + "i.b"] = mat(h, width, 2.0), vec(h, 0.0, 1.0)
            s[x + "f"], s[x + "f.b"] = mat(h, width, 2.0), vec(h, forget_bias, 1.0)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        s[p + "norm2"], s[p + "norm2b"], s[p + "ls2"] = vec(width, 1.0), vec(width, 1.0), vec(width, 0.6, 0.3)
        if mlp["kind"] == "dense":
            unit(p + "mlp.", mlp["ff"])
            continue
        experts = mlp["router"]["experts"]
        for e in range(experts):
            unit(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
        s[p + "mlp.router"] = mat(experts, width, 2.0)
        if mlp.get("shared"):
            unit(p + "mlp.shared.", mlp["shared"]["ff"])
            s[p + "mlp.shared.sg"] = mat(1, width, 2.0)
    return s


def sharpened(cfg: dict, factor: float) -> dict:
    """The same configuration with every attention scale multiplied."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if "scale" in layer["mixer"]:
            layer["mixer"]["scale"] *= factor
    return out
