"""Named shapes, as config.json dictionaries (Llama 3, and two of the Nidilix design): the tiny shapes used
for correctness runs (tiny-d has the head size and widths that the tensor-core
kernels take) and the 8B / 3B / 70B shapes used for measurements. The
reference keeps such presets in crates/stride-model/src/presets.rs:73-91."""

from __future__ import annotations

import copy


def _llama3_scaling(factor: float, original: int) -> dict:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": original}


def _llama(layers, hidden, heads, kv_heads, head_dim, inter, vocab, theta, scaling, eps, tied, max_pos) -> dict:
    d = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "hidden_size": hidden,
         "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter,
         "vocab_size": vocab, "rope_theta": theta, "rms_norm_eps": eps, "tie_word_embeddings": tied,
         "max_position_embeddings": max_pos, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False}
    if scaling:
        d["rope_scaling"] = scaling
    return d


def _nidilix(width, vocab, pattern, recurrent, attention, mlp, side, mult=0.5, eps=1e-6) -> dict:
    """``pattern``: a string of ``r`` (recurrent layer), ``a`` (latent attention with a cache of its own) and ``b`` (latent
    attention that reads the cache of the nearest ``a`` before it)."""
    layers, last = [], None
    for i, kind in enumerate(pattern):
        if kind == "r":
            layers.append({"type": "rglru", "mixer": dict(recurrent), "mlp": copy.deepcopy(mlp)})
            continue
        mixer = copy.deepcopy(attention)
        if kind == "b":
            mixer["kv_from"] = last
        else:
            last = i
        layers.append({"type": "latent_attention", "mixer": mixer, "mlp": copy.deepcopy(mlp)})
    d = {"architecture": "Nidilix", "width": width, "vocab": vocab, "residual_mult": mult, "norm": {"eps": eps}, "layers": layers}
    if side:
        d["token_side"] = {"dim": side}
    return d


def _netusun_tiny() -> dict:
    """Four layers of which the first two run twice: latent attention, windowed attention behind a convolution, a matrix
    LSTM, windowed attention; a dense feed-forward and small mixtures."""
    latent = {"heads": 2, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 64, "q_rank": 48, "scale": 48 ** -0.5,
              "rot": {"base": 10000.0, "dims": 16, "scaling": {"factor": 2.0, "original": 128, "fast": 16.0, "slow": 1.0}}}
    windowed = {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 32 ** -0.5, "conv": 3, "mask": {"size": 64}, "softcap": 20.0}
    moe = {"kind": "moe", "expert": {"ff": 64}, "shared": {"ff": 32},
           "router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    layers = [{"type": "latent_attention", "mixer": latent, "mlp": {"kind": "dense", "ff": 192}},
              {"type": "attention", "mixer": windowed, "mlp": copy.deepcopy(moe)},
              {"type": "mlstm", "mixer": {"heads": 2, "dim": 32, "vdim": 32, "gate_cap": 10.0}, "mlp": copy.deepcopy(moe)},
              {"type": "attention", "mixer": copy.deepcopy(windowed), "mlp": None}]
    return {"architecture": "Netusun", "width": 128, "vocab": 384, "norm": {"eps": 1e-6}, "layers": layers,
            "loop": {"start": 0, "stop": 2, "times": 2}}


PRESETS = {
    "netusun-tiny": _netusun_tiny(),
    "nidilix-tiny": _nidilix(128, 512, "rarb", {"width": 160, "blocks": 5, "conv": 3},
                             {"heads": 4, "dim": 16, "rot_dim": 16, "vdim": 24, "kv_rank": 48, "rot": {"base": 10000.0, "dims": 16},
                              "scale": 32 ** -0.5},
                             {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": 64}, "shared": {"ff": 32}}, 8),
    "nidilix-2048": _nidilix(2048, 32000, "rrarrb", {"width": 2560, "blocks": 10, "conv": 4},
                             {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "rot": {"base": 10000.0, "dims": 64},
                              "scale": 192 ** -0.5},
                             {"kind": "moe", "router": {"experts": 32, "top": 4}, "expert": {"ff": 768}, "shared": {"ff": 1024}}, 128),
    "tiny-a": _llama(2, 64, 4, 2, 16, 192, 256, 10000.0, None, 1e-5, False, 256),
    "tiny-b": _llama(3, 96, 3, 1, 32, 256, 384, 500000.0, _llama3_scaling(8.0, 64), 1e-6, True, 512),
    "tiny-d": _llama(2, 192, 4, 2, 128, 384, 515, 500000.0, _llama3_scaling(8.0, 128), 1e-5, False, 2048),
    "llama3.1-8b": _llama(32, 4096, 32, 8, 128, 14336, 128256, 500000.0, _llama3_scaling(8.0, 8192), 1e-5, False, 131072),
    "llama3.2-3b": _llama(28, 3072, 24, 8, 128, 8192, 128256, 500000.0, _llama3_scaling(32.0, 8192), 1e-5, True, 131072),
    "llama3.1-70b": _llama(80, 8192, 64, 8, 128, 28672, 128256, 500000.0, _llama3_scaling(8.0, 8192), 1e-5, False, 131072),
}


def preset(name: str) -> dict:
    try:
        return copy.deepcopy(PRESETS[name])
    except KeyError:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}") from None
