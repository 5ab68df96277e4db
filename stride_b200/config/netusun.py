"""Typed configuration of the Netusun decoder.

config.json gives ``vocab``, ``width``, ``norm.eps``, a list ``layers`` and optionally ``loop``. A layer entry has ``type``
(``latent_attention``, ``attention`` or ``mlstm``), the mixer's sizes and constants (``mixer``) and its feed-forward
(``mlp``: ``kind`` ``dense`` with ``ff``; ``kind`` ``moe`` with ``expert.ff``, ``router`` (``experts, top, scale`` and optionally
``groups`` with ``count, keep``) and optionally ``shared.ff``; or null). ``loop`` (``start, stop, times``) makes the layers
``start .. stop - 1`` run ``times`` times in a row on the same tensors, every pass with a cache and a state of its own. Nothing
else is read, and no size stands in code. The architecture is laid out from the package's parts:

* a layer is the ``sandwich`` arrangement: a norm before and a norm after either sublayer, ``x += s * norm_b(sublayer(norm(x)))``;
  the learned vectors s (``ls1``, ``ls2``) are params of the output norms;
* ``latent_attention`` is the latent attention part with queries through a latent of their own, the rotated part turned
  in halves (entry i with entry i + dims / 2) with optional YaRN rescaling, a sink per head and a gate on every output entry;
* ``attention`` is the paged attention part without rotation: a short convolution over time on q, k and v, weighted head
  norms on queries and keys, capped scores, a window, and one added to the softmax's denominator;
* ``mlstm`` is the matrix LSTM mixer;
* the dense feed-forward is ``swiglu`` with SiLU; the mixture is ``routed_experts`` with SiLU units, the ``softmax_groups``
  router and a gated shared expert;
* before every pass over the repeated block (the first too) the stream goes through the ``mix_embedding`` pass input
  (tensors ``loop.in``, ``loop.step``);
* final norm ``final.norm``; the head shares the embedding table.

The design names no longest sequence: ``max_positions`` only sizes the rotation tables and is raised on demand
(``with_max_positions``).
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field

from .registry import ConfigError, register_architecture
from .specs import (FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PassInputSpec, PositionSpec, RopeScaling,
                    ScheduleEntry)

MIXERS = ("latent_attention", "attention", "mlstm")
DEFAULT_MAX_POSITIONS = 32768
_KNOWN = ("architecture", "architectures", "vocab", "width", "layers", "norm", "loop", "max_positions")


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


def _check_rotation(rot, limit: int, where: str) -> None:
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}: `rot` must be an object with `base` and `dims`")
    dims = _int(rot, "dims", where, minimum=0)
    if dims % 2 or dims > limit or not _num(rot, "base", where) > 0:
        raise ConfigError(f"{where}: rot.dims must be even and at most {limit}, rot.base positive")
    sc = rot.get("scaling")
    if sc is not None:
        for key in ("factor", "original", "fast", "slow"):
            if not _num(sc, key, where + ".scaling") > 0:
                raise ConfigError(f"{where}.scaling: `{key}` must be positive")


def _check_mixer(kind: str, m, where: str) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"{where}: `mixer` must be an object")
    heads, dim, vdim = _int(m, "heads", where), _int(m, "dim", where), _int(m, "vdim", where)
    if kind == "latent_attention":
        _int(m, "kv_rank", where), _int(m, "q_rank", where)
        rot_dim = _int(m, "rot_dim", where)
        _num(m, "scale", where)
        _check_rotation(m.get("rot"), rot_dim, where + ".rot")
        if m["kv_rank"] > 512:
            raise ConfigError(f"{where}: kv_rank up to 512 is supported, got {m['kv_rank']}")
    elif kind == "attention":
        kv = _int(m, "kv_heads", where)
        _num(m, "scale", where)
        if heads % kv:
            raise ConfigError(f"{where}: {heads} heads do not group into {kv} kv_heads")
        if dim > 256 or vdim > 256:
            raise ConfigError(f"{where}: head sizes up to 256 are supported, got dim {dim} and vdim {vdim}")
        if m.get("conv") is not None and _int(m, "conv", where) > 16:
            raise ConfigError(f"{where}: up to 16 taps are supported")
        if m.get("softcap") is not None and not _num(m, "softcap", where) > 0:
            raise ConfigError(f"{where}: softcap must be positive")
        if m.get("mask") is not None:
            _int(m["mask"], "size", where + ".mask")
    else:
        if not _num(m, "gate_cap", where) > 0:
            raise ConfigError(f"{where}: gate_cap must be positive")
        if dim > 256:
            raise ConfigError(f"{where}: dim up to 256 is supported, got {dim}")


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}: `mlp` must be null or have `kind` 'dense' or 'moe'")
    if mlp["kind"] == "dense":
        _int(mlp, "ff", where)
        return
    _int(mlp.get("expert"), "ff", where + ".expert")
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
        _int(mlp["shared"], "ff", where + ".shared")


@dataclass(frozen=True)
class NetusunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers_json: str                        # the ``layers`` list as canonical JSON (keeps the record hashable)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0                     # 0: no block of layers runs more than once and there is no pass input
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "NetusunConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in d:
                raise ConfigError(f"config.json is missing `{key}`")
        if not isinstance(d["norm"], dict):
            raise ConfigError("`norm` must be an object with `eps`")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        loop = d.get("loop")
        start = stop = times = 0
        if loop is not None:
            start, stop = _int(loop, "start", "loop", minimum=0), _int(loop, "stop", "loop", minimum=0)
            times = _int(loop, "times", "loop")
        cfg = cls(vocab=_int(d, "vocab", "config.json"), width=_int(d, "width", "config.json"), norm_eps=_num(d["norm"], "eps", "norm"),
                  layers_json=json.dumps(d["layers"], sort_keys=True), loop_start=start, loop_stop=stop, loop_times=times,
                  max_position_embeddings=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  extra={k: v for k, v in d.items() if k not in _KNOWN})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        layers = self.layers
        if not self.norm_eps >= 0:
            raise ConfigError("norm.eps must not be negative")
        if self.loop_times and not 0 <= self.loop_start < self.loop_stop <= len(layers):
            raise ConfigError(f"loop: start {self.loop_start} and stop {self.loop_stop} must enclose at least one of the {len(layers)} layers")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"{where}: `type` must be one of {MIXERS}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            _check_mixer(layer["type"], layer.get("mixer"), where)
            _check_mlp(layer.get("mlp"), where + ".mlp")

    def to_dict(self) -> dict:
        d = {"architecture": "Netusun", "layers": self.layers, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        d.update(copy.deepcopy(self.extra))
        return d

    def with_max_positions(self, count: int) -> "NetusunConfig":
        import dataclasses
        return dataclasses.replace(self, max_position_embeddings=int(count))

    # ------------------------------------------------------------------- layout
    def _norm(self, name: str, scale: str | None = None) -> NormSpec:
        params = (("tensor", name),) + ((("scale_tensor", scale),) if scale else ())
        return NormSpec(kind="rmsnorm", width=self.width, eps=self.norm_eps, prefix=name, params=params)

    def _mixer(self, layer: dict, prefix: str) -> MixerSpec:
        m, kind = layer["mixer"], layer["type"]
        if kind == "latent_attention":
            rot = m["rot"]
            sc = rot.get("scaling")
            scaling = None
            if sc:
                # YaRN: `fast` and `slow` are the numbers of turns over the original length between which the
                # frequencies go over from kept to divided by `factor`
                scaling = RopeScaling(rope_type="yarn", factor=float(sc["factor"]), low_freq_factor=float(sc["slow"]),
                                      high_freq_factor=float(sc["fast"]), original_max_position_embeddings=int(sc["original"]))
            position = PositionSpec(kind="rope", head_dim=int(rot["dims"]), theta=float(rot["base"]),
                                    max_positions=self.max_position_embeddings, scaling=scaling, params=(("angles", "float64"),))
            return MixerSpec(kind="latent_attention", hidden=self.width, num_heads=m["heads"], head_dim=m["dim"], scale=float(m["scale"]),
                             position=position, prefix=prefix,
                             params=(("rot_dim", m["rot_dim"]), ("value_dim", m["vdim"]), ("kv_rank", m["kv_rank"]), ("q_rank", m["q_rank"]),
                                     ("latent_eps", self.norm_eps), ("output_gate", "full"), ("sinks", True), ("pairing", "halves")))
        if kind == "attention":
            params = [("names", "short"), ("value_dim", int(m["vdim"])), ("qk_norm", "weighted"), ("norm_eps", self.norm_eps), ("sinks", "zero")]
            if m.get("conv"):
                params.append(("conv", int(m["conv"])))
            if m.get("softcap"):
                params.append(("softcap", float(m["softcap"])))
            return MixerSpec(kind="attention", hidden=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                             scale=float(m["scale"]), window=int(m["mask"]["size"]) if m.get("mask") else None, bias=False,
                             position=PositionSpec(kind="none"), prefix=prefix, params=tuple(params))
        return MixerSpec(kind="mlstm", hidden=self.width, num_heads=m["heads"], head_dim=m["dim"], prefix=prefix,
                         params=(("value_dim", m["vdim"]), ("gate_cap", float(m["gate_cap"])), ("norm_eps", self.norm_eps)))

    def _feed_forward(self, mlp: dict, prefix: str) -> FeedForwardSpec:
        if mlp["kind"] == "dense":
            return FeedForwardSpec(kind="swiglu", hidden=self.width, intermediate=mlp["ff"], activation="silu", prefix=prefix,
                                   params=(("names", "short"),))
        r, groups, shared = mlp["router"], mlp["router"].get("groups") or {"count": 1, "keep": 1}, mlp.get("shared")
        params = [("experts", r["experts"]), ("top", r["top"]), ("router", "softmax_groups"), ("groups", groups["count"]),
                  ("keep", groups["keep"]), ("route_scale", float(r["scale"]))]
        if shared is not None:
            params += [("shared", shared["ff"]), ("shared_gate", True)]
        return FeedForwardSpec(kind="routed_experts", hidden=self.width, intermediate=mlp["expert"]["ff"], activation="silu", prefix=prefix,
                               params=tuple(params))

    def run_order(self) -> list:
        """(layer, pass number or None) in the order the layers run; a pass number marks the first layer of a pass."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        order = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            order += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, n)]

    def to_model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p, mlp = f"l{i}.", layer.get("mlp")
            ffn = self._feed_forward(mlp, p + "mlp.") if mlp is not None else None
            layers.append(LayerSpec(kind="sandwich", mixer=self._mixer(layer, p + "mix."), feed_forward=ffn,
                                    mixer_norm=self._norm(p + "norm1"), ffn_norm=self._norm(p + "norm2") if ffn is not None else None,
                                    mixer_out_norm=self._norm(p + "norm1b", p + "ls1"),
                                    ffn_out_norm=self._norm(p + "norm2b", p + "ls2") if ffn is not None else None))
        # every run has a cache slot and a state slot of its own, a second pass over a layer too
        schedule = tuple(ScheduleEntry(layer=i, cache=run, enters_pass=t) for run, (i, t) in enumerate(self.run_order()))
        pass_input = PassInputSpec("mix_embedding", self.width, self.loop_times, "loop.in", "loop.step") if self.loop_times else None
        return ModelSpec(architecture="Netusun", hidden=self.width, vocab=self.vocab, layers=tuple(layers), schedule=schedule,
                         final_norm=self._norm("final.norm"), embed_name="embed", head_name=None,
                         max_positions=self.max_position_embeddings, extra=self, pass_input=pass_input)


register_architecture("Netusun", NetusunConfig)
