"""What a model is made of, as data.

A model is a list of layers and a list that says in which order they run. A
layer is an arrangement of four parts: a mixer (attention here), a feed-forward,
and the norms before them. Each part is described by a small frozen record that
carries every size and constant the part needs; the record's ``kind`` selects
the implementation from the part registry (``stride_b200.parts``). No part knows
which architecture it serves, and layers of one model may use different kinds.

The records also carry the checkpoint prefix under which a part finds its
tensors, so that tensor naming stays with the architecture that defines it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of rotary embeddings (``rope_scaling`` in config.json)."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer. kind ``rope`` | ``none``."""
    kind: str
    head_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: Optional[RopeScaling] = None
    params: tuple = ()          # free-form (key, value) pairs for other kinds


@dataclass(frozen=True)
class NormSpec:
    """kind ``rmsnorm``: y = x * rsqrt(mean(x^2) + eps) * weight."""
    kind: str
    width: int
    eps: float
    prefix: str                 # e.g. "model.layers.0.input_layernorm."
    params: tuple = ()


@dataclass(frozen=True)
class MixerSpec:
    """kind ``attention``: grouped-query attention over the paged cache.

    ``window`` of None keeps every key; an integer W lets a token read only its
    last W keys (its own included).
    """
    kind: str
    hidden: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    bias: bool = False
    position: Optional[PositionSpec] = None
    prefix: str = ""            # e.g. "model.layers.0.self_attn."
    params: tuple = ()


@dataclass(frozen=True)
class FeedForwardSpec:
    """kind ``swiglu``: down(act(gate(x)) * up(x))."""
    kind: str
    hidden: int
    intermediate: int = 0
    activation: str = "silu"
    prefix: str = ""            # e.g. "model.layers.0.mlp."
    params: tuple = ()


@dataclass(frozen=True)
class StreamInputSpec:
    """Something a layer adds to the residual stream from the token ids and the stream itself, after its
    feed-forward. kind ``token_side``: a slice [offset, offset + dim) of row ``id`` of a second embedding table
    (``table_name`` [vocab, table_width]) gated by a projection of the stream, projected back to ``hidden`` and
    normed to unit root mean square with a plain weight."""
    kind: str
    hidden: int
    vocab: int = 0
    dim: int = 0
    offset: int = 0
    table_width: int = 0
    table_name: str = ""
    eps: float = 0.0
    prefix: str = ""
    params: tuple = ()


@dataclass(frozen=True)
class LayerSpec:
    """kind ``pre_norm``: x += m * mixer(norm(x)); x += m * ffn(norm(x)); then every part of ``after`` adds
    m * part(x, tokens). ``residual_mult`` is m (1 where an architecture has none); ``feed_forward`` and
    ``ffn_norm`` may be None for a layer without a feed-forward. kind ``sandwich`` has a second norm on either
    sublayer's output (``mixer_out_norm``, ``ffn_out_norm``): x += m * out_norm(mixer(norm(x)))."""
    kind: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    residual_mult: float = 1.0
    after: tuple = ()           # of StreamInputSpec
    mixer_out_norm: Optional[NormSpec] = None
    ffn_out_norm: Optional[NormSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache`` names the cache slot (and state slot) that the
    run's mixer uses; two runs with the same slot share keys and values, and
    ``writes_cache=False`` makes a run read what another run wrote. ``enters_pass`` t: the run is the first of pass t
    over a block of layers that runs several times, and the model's ``pass_input`` part works on the stream before it."""
    layer: int
    cache: int
    writes_cache: bool = True
    enters_pass: Optional[int] = None


@dataclass(frozen=True)
class PassInputSpec:
    """What happens to the residual stream before every pass over a repeated block of layers. kind ``mix_embedding``:
    ``x <- W [x; x0] + s[t]`` with x0 the embedding's output, ``W`` the tensor ``mix_name`` [hidden, 2 * hidden] (the
    stream's columns first) and ``s`` the tensor ``step_name`` [passes, hidden], t the number of the pass."""
    kind: str
    hidden: int
    passes: int
    mix_name: str
    step_name: str
    params: tuple = ()


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the first residual stream. kind ``lookup``: row ``id`` of the table ``name``
    [vocab, hidden], no scaling (python/stride_worker/model.py:250-252)."""
    kind: str
    vocab: int
    hidden: int
    name: str                   # checkpoint name of the table
    params: tuple = ()          # free-form (key, value) pairs for other kinds (a multiplier, say)


@dataclass(frozen=True)
class HeadSpec:
    """How the normed last hidden states become logits. kind ``linear``: ``x @ W.T`` in the compute dtype with a
    float32 result; ``name`` None ties W to the embedding table (python/stride_worker/model.py:127-130,322-341)."""
    kind: str
    vocab: int
    hidden: int
    name: Optional[str]
    params: tuple = ()          # free-form (key, value) pairs for other kinds (a bias, a cap on the logits)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    layers: tuple               # of LayerSpec
    schedule: tuple             # of ScheduleEntry
    final_norm: NormSpec
    embed_name: str             # checkpoint name of the embedding table
    head_name: Optional[str]    # checkpoint name of the output head; None: tied to the embedding
    max_positions: int
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    ignorable_tensors: tuple = ()   # glob patterns of checkpoint tensors that may be present and are not read
    extra: Any = field(default=None, compare=False)
    # The two ends of the model are parts like the rest. Left out, they are the plain kinds built from the two
    # names above: a table lookup and a linear head.
    embedding: Optional[EmbeddingSpec] = None
    head: Optional[HeadSpec] = None
    pass_input: Optional[PassInputSpec] = None      # for schedules whose entries name ``enters_pass``

    def embedding_spec(self) -> EmbeddingSpec:
        return self.embedding or EmbeddingSpec("lookup", self.vocab, self.hidden, self.embed_name)

    def head_spec(self) -> HeadSpec:
        return self.head or HeadSpec("linear", self.vocab, self.hidden, self.head_name)

    @property
    def num_cache_slots(self) -> int:
        return 1 + max(e.cache for e in self.schedule) if self.schedule else 0


def default_schedule(num_layers: int) -> tuple:
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(num_layers))
