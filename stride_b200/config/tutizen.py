"""Typed configuration of the Tutizen decoder.

config.json gives ``vocab``, ``width``, ``residual_mult``, ``norm.eps`` and a list ``layers``; each entry has ``type``
(``attention``), the mixer's sizes and constants (``mixer``: ``heads, kv_heads, dim, vdim, scale`` and optionally
``kv_from``) and its feed-forward (``mlp``: ``kind`` ``dense`` with ``ff, limit``; ``kind`` ``moe`` with ``expert``
(``ff, limit``), ``router`` (``experts, top, scale`` and optionally ``groups`` with ``count, keep``) and optionally
``shared`` (``ff, limit``); or null). Nothing else is read, and no size stands in code. The architecture is laid out
from the package's parts:

* the embedding is the ``lookup`` kind with the sinusoidal position vector added (base 10000);
* a layer is the ``output_norm`` arrangement, ``x += m * norm(sublayer(x))``, with ``residual_mult`` as m; its norms are
  ``rmsnorm`` whose weight is one number;
* ``attention`` is the paged attention part without rotation: biases on all four projections, queries, keys and values
  divided by their root mean square per head, a penalty on the key's distance with slopes ``2^(-8 (h + 1) / heads)``, one
  output gate per head. ``kv_from: j`` makes the layer read the pages that layer j writes (no key and value
  projections of its own): its run names j's cache slot and writes nothing;
* the dense feed-forward is ``swiglu`` with the clamped activation (``alpha`` 1.702); the mixture is ``routed_experts``
  with the same activation, the ``sigmoid_groups`` router and a gated shared expert;
* final norm ``final.norm`` (one number), head ``head``.

The design names no longest sequence: ``max_positions`` only bounds what the engine accepts and is raised on demand
(``with_max_positions``); no table depends on it.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field

from .registry import ConfigError, register_architecture
from .specs import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                    ScheduleEntry)

DEFAULT_MAX_POSITIONS = 32768
SINUSOID_BASE = 10000.0         # of the position vector
SLOPE_EXPONENT = 8.0            # slopes 2^(-8 (h + 1) / heads)
SWISH_ALPHA = 1.702             # g sigmoid(1.702 g)
_KNOWN = ("architecture", "architectures", "vocab", "width", "layers", "norm", "residual_mult", "max_positions")


def _int(d, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"{where}: `{key}` must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


def _check_unit(u, where: str) -> None:
    if not isinstance(u, dict):
        raise ConfigError(f"{where} must be an object with `ff` and `limit`")
    _int(u, "ff", where)
    if not _num(u, "limit", where) > 0:
        raise ConfigError(f"{where}: `limit` must be positive")


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}: `mlp` must be null or have `kind` 'dense' or 'moe'")
    if mlp["kind"] == "dense":
        return _check_unit(mlp, where)
    _check_unit(mlp.get("expert"), where + ".expert")
    r = mlp.get("router")
    if not isinstance(r, dict):
        raise ConfigError(f"{where}: a mixture needs `router`")
    experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
    _num(r, "scale", where + ".router")
    groups = r.get("groups")
    count, keep = 1, 1
    if groups is not None:
        count, keep = _int(groups, "count", where + ".router.groups"), _int(groups, "keep", where + ".router.groups")
    if experts % count or keep > count or top > keep * (experts // count):
        raise ConfigError(f"{where}.router: {experts} experts in {count} groups of which {keep} stay cannot give {top} choices")
    if experts > 256 or top > 32:
        raise ConfigError(f"{where}.router: up to 32 of up to 256 experts are supported")
    if mlp.get("shared") is not None:
        _check_unit(mlp["shared"], where + ".shared")


@dataclass(frozen=True)
class TutizenConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers_json: str                        # the ``layers`` list as canonical JSON (keeps the record hashable)
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "TutizenConfig":
        for key in ("vocab", "width", "layers", "norm", "residual_mult"):
            if key not in d:
                raise ConfigError(f"config.json is missing `{key}`")
        if not isinstance(d["norm"], dict):
            raise ConfigError("`norm` must be an object with `eps`")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        cfg = cls(vocab=_int(d, "vocab", "config.json"), width=_int(d, "width", "config.json"), norm_eps=_num(d["norm"], "eps", "norm"),
                  residual_mult=_num(d, "residual_mult", "config.json"), layers_json=json.dumps(d["layers"], sort_keys=True),
                  max_position_embeddings=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  extra={k: v for k, v in d.items() if k not in _KNOWN})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        layers = self.layers
        if not self.norm_eps >= 0:
            raise ConfigError("norm.eps must not be negative")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") != "attention":
                raise ConfigError(f"{where}: `type` must be 'attention', got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"{where}: `mixer` must be an object")
            heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
            dim, vdim = _int(m, "dim", where), _int(m, "vdim", where)
            _num(m, "scale", where)
            if heads % kv:
                raise ConfigError(f"{where}: {heads} heads do not group into {kv} kv_heads")
            if dim > 256 or vdim > 256:
                raise ConfigError(f"{where}: head sizes up to 256 are supported, got dim {dim} and vdim {vdim}")
            source = m.get("kv_from")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                    raise ConfigError(f"{where}: kv_from must name an earlier layer, got {source!r}")
                other = layers[source]["mixer"]
                if other.get("kv_from") is not None:
                    raise ConfigError(f"{where}: kv_from {source} names a layer that has no keys and values of its own")
                if any(other.get(k) != m.get(k) for k in ("heads", "kv_heads", "dim", "vdim")):
                    raise ConfigError(f"{where}: head counts and sizes must equal those of layer {source}")
            _check_mlp(layer.get("mlp"), where + ".mlp")

    def to_dict(self) -> dict:
        d = {"architecture": "Tutizen", "layers": self.layers, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "vocab": self.vocab, "width": self.width}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        d.update(copy.deepcopy(self.extra))
        return d

    def with_max_positions(self, count: int) -> "TutizenConfig":
        import dataclasses
        return dataclasses.replace(self, max_position_embeddings=int(count))

    # ------------------------------------------------------------------- layout
    def _norm(self, name: str) -> NormSpec:
        return NormSpec(kind="rmsnorm", width=self.width, eps=self.norm_eps, prefix=name, params=(("tensor", name), ("shape", "scalar")))

    def _mixer(self, m: dict, prefix: str) -> MixerSpec:
        params = [("names", "short"), ("value_dim", int(m["vdim"])), ("qk_norm", "unit"), ("v_norm", "unit"), ("norm_eps", self.norm_eps),
                  ("distance_slopes", SLOPE_EXPONENT), ("output_gate", "head"), ("output_bias", True)]
        if m.get("kv_from") is not None:
            params.append(("borrowed_kv", True))
        return MixerSpec(kind="attention", hidden=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                         scale=float(m["scale"]), window=None, bias=True, position=PositionSpec(kind="none"), prefix=prefix,
                         params=tuple(params))

    def _feed_forward(self, mlp: dict, prefix: str) -> FeedForwardSpec:
        if mlp["kind"] == "dense":
            return FeedForwardSpec(kind="swiglu", hidden=self.width, intermediate=mlp["ff"], activation="swish_clamped", prefix=prefix,
                                   params=(("names", "short"), ("limit", float(mlp["limit"])), ("alpha", SWISH_ALPHA)))
        r, groups, shared = mlp["router"], mlp["router"].get("groups") or {"count": 1, "keep": 1}, mlp.get("shared")
        params = [("experts", r["experts"]), ("top", r["top"]), ("router", "sigmoid_groups"), ("groups", groups["count"]),
                  ("keep", groups["keep"]), ("route_scale", float(r["scale"])), ("limit", float(mlp["expert"]["limit"])), ("alpha", SWISH_ALPHA)]
        if shared is not None:
            params += [("shared", shared["ff"]), ("shared_limit", float(shared["limit"])), ("shared_gate", True)]
        return FeedForwardSpec(kind="routed_experts", hidden=self.width, intermediate=mlp["expert"]["ff"], activation="swish_clamped",
                               prefix=prefix, params=tuple(params))

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            p, mlp = f"l{i}.", layer.get("mlp")
            ffn = self._feed_forward(mlp, p + "mlp.") if mlp is not None else None
            layers.append(LayerSpec(kind="output_norm", mixer=self._mixer(layer["mixer"], p + "mix."), feed_forward=ffn,
                                    mixer_norm=self._norm(p + "norm1"), ffn_norm=self._norm(p + "norm2") if ffn is not None else None,
                                    residual_mult=self.residual_mult))
            source = layer["mixer"].get("kv_from")
            schedule.append(ScheduleEntry(layer=i, cache=i) if source is None else ScheduleEntry(layer=i, cache=source, writes_cache=False))
        embedding = EmbeddingSpec("lookup", self.vocab, self.width, "embed", params=(("sinusoid", SINUSOID_BASE),))
        return ModelSpec(architecture="Tutizen", hidden=self.width, vocab=self.vocab, layers=tuple(layers), schedule=tuple(schedule),
                         final_norm=self._norm("final.norm"), embed_name="embed", head_name="head",
                         max_positions=self.max_position_embeddings, extra=self, embedding=embedding,
                         head=HeadSpec("linear", self.vocab, self.width, "head"))


register_architecture("Tutizen", TutizenConfig)
