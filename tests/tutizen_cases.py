"""Small Tutizen configurations and seeded weights for the tests. Nothing here imports the product package."""

from __future__ import annotations

import math

import torch


def attn(heads, kv, dim, vdim=None, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim if vdim is not None else dim,
         "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit=2.0, groups=None, scale=2.5, shared=None):
    """``groups``: (count, keep) or None; ``shared``: (ff, limit) or None."""
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def config(width, vocab, layers, eps=1e-6, mult=0.7):
    """``layers``: list of (mixer sizes, mlp or None)."""
    return {"architecture": "Tutizen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": [{"type": "attention", "mixer": m, "mlp": mlp} for m, mlp in layers]}


# A: three query heads on one key head, a mixture behind borrowed pages, values wider than keys, a layer without a
# feed-forward, a mixture without groups and without a shared expert.
CASE_A = config(96, 211, [
    (attn(3, 1, 32, scale=0.2), dense(72, 1.0)),
    (attn(3, 1, 32, scale=0.3, kv_from=0), moe(8, 2, 24, 1.2, groups=(4, 2), shared=(40, 0.8))),
    (attn(4, 4, 16, 24), None),
    (attn(4, 4, 16, 24, kv_from=2), moe(6, 3, 20, 2.0, scale=1.0)),
], eps=1e-6, mult=0.7)

# B: no multiplier on the sums, as many key heads as query heads, values narrower than keys, one choice out of four with
# every group kept, two layers that borrow from one, a single query head.
CASE_B = config(80, 157, [
    (attn(2, 2, 48, 16), dense(56, 2.5)),
    (attn(1, 1, 8), moe(4, 1, 32, 0.7, groups=(2, 2), scale=0.5, shared=(16, 3.0))),
    (attn(2, 2, 48, 16, scale=0.1, kv_from=0), dense(24, 0.5)),
    (attn(2, 2, 48, 16, kv_from=0), None),
], eps=1e-5, mult=1.0)

# C: head sizes of 64 and 128 with pages of 16: the sizes the tensor-core attention kernels take in bfloat16; six heads, so
# the gates' columns are padded; sixteen experts of which four are chosen in two of four groups.
CASE_C = config(128, 263, [
    (attn(4, 2, 64, scale=0.15), dense(96, 1.5)),
    (attn(4, 2, 64, scale=0.15, kv_from=0), moe(16, 4, 32, 1.5, groups=(4, 2), shared=(64, 1.5))),
    (attn(6, 2, 128, scale=0.1), moe(8, 2, 48, 2.0, groups=(2, 1), scale=1.7)),
    (attn(6, 2, 128, scale=0.08, kv_from=2), dense(64, 1.0)),
], eps=2e-6, mult=0.5)

# D: sizes that are multiples of 2 only, so rows of 16-bit numbers start off a 16-byte boundary and every vector path has
# to step aside; nine experts in three groups of which one stays.
CASE_D = config(100, 103, [
    (attn(3, 3, 20, 18), moe(9, 2, 14, 1.1, groups=(3, 1), shared=(22, 1.3))),
    (attn(6, 3, 10, 6, kv_from=None), dense(36, 0.9)),
    (attn(3, 3, 20, 18, kv_from=0), None),
], eps=1e-6, mult=1.3)

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D}


def seeded_state(cfg: dict, seed: int) -> dict:
    """float32 weights by checkpoint name. Matrices N(0, gain^2 / in)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(n, mean=0.0, std=0.3):
        return mean + std * torch.randn(n, generator=g)

    def number(mean, std):
        return (mean + std * torch.randn((), generator=g)).reshape(())

    def unit(p, ff):
        s[p + "gate"], s[p + "up"], s[p + "down"] = mat(ff, width, 1.5), mat(ff, width, 1.5), mat(width, ff)

    s = {"embed": torch.randn(vocab, width, generator=g), "final.norm": number(1.0, 0.2), "head": mat(vocab, width, 2.5)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h, kv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[p + "norm1"] = number(1.0, 0.3)
        s[p + "mix.q"], s[p + "mix.q.b"] = mat(h * d, width), vec(h * d)
        if m.get("kv_from") is None:
            s[p + "mix.k"], s[p + "mix.k.b"] = mat(kv * d, width), vec(kv * d)
            s[p + "mix.v"], s[p + "mix.v.b"] = mat(kv * dv, width), vec(kv * dv)
        s[p + "mix.g"], s[p + "mix.o"], s[p + "mix.o.b"] = mat(h, width, 2.0), mat(width, h * dv), vec(width)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        s[p + "norm2"] = number(1.0, 0.3)
        if mlp["kind"] == "dense":
            unit(p + "mlp.", mlp["ff"])
            continue
        experts = mlp["router"]["experts"]
        for e in range(experts):
            unit(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
        # corrections larger than the scores' spread, some of them below -1: choice scores change the order and go negative
        s[p + "mlp.router"], s[p + "mlp.correction"] = mat(experts, width, 2.0), vec(experts, -0.4, 0.6)
        if mlp.get("shared"):
            unit(p + "mlp.shared.", mlp["shared"]["ff"])
            s[p + "mlp.shared.sg"] = mat(1, width, 2.0)
    return s


def sharpened(cfg: dict, factor: float) -> dict:
    """The same configuration with every attention scale multiplied: queries and keys are unit vectors, so the scale alone
    decides how sharply a softmax settles on few keys."""
    import copy
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        layer["mixer"]["scale"] *= factor
    return out
