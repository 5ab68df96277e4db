"""The two ends of a decoder as parts: token ids in, logits out.

``lookup``: the residual stream starts as row ``id`` of the embedding table, widened to float32, no multiplier
(python/stride_worker/model.py:250-252). ``linear``: logits are the normed rows times the head matrix, computed in
the compute dtype and returned in float32; a head whose spec names no tensor shares the embedding table
(python/stride_worker/model.py:127-130, 322-341). An architecture that scales its embedding, adds a bias to its
head registers another kind; the model itself does not change. ``lookup`` with the param ``sinusoid`` b adds the fixed
position vector of Vaswani et al., "Attention Is All You Need", in neighbouring pairs: entry 2i gets sin(p b^(-2i / hidden)),
entry 2i + 1 the cosine of the same angle, formed in float64 on the device. A ``linear`` head whose spec gives the param
``softcap`` c caps its logits at c tanh(logits / c).
"""

from __future__ import annotations

from ..csrc import ops
from .base import Embedding, Head, TensorDecl, register_part


class LookupEmbedding(Embedding):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.weight = None
        base = dict(spec.params).get("sinusoid")
        self.freq = None
        if base:
            import torch
            pairs = torch.arange((spec.hidden + 1) // 2, dtype=torch.float64)
            self.freq = (float(base) ** (-2.0 * pairs / spec.hidden)).to(runtime.device)

    def declare(self):
        return {self.spec.name: TensorDecl((self.spec.vocab, self.spec.hidden))}

    def bind(self, weights):
        self.weight = weights[self.spec.name]

    def named_tensors(self):
        return {self.spec.name: self.weight}

    def table(self):
        return self.weight

    def forward(self, ctx, out):
        tokens = out.shape[0]
        ops.embed_gather(ctx.token_ids[:tokens], ctx.seq_of_token[:tokens], self.weight, out)
        if self.freq is not None:
            ops.add_sinusoid(out, None, ctx.positions[:tokens], ctx.seq_of_token[:tokens], self.freq)


class LinearHead(Head):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.weight = None

    def declare(self):
        return {} if self.spec.name is None else {self.spec.name: TensorDecl((self.spec.vocab, self.spec.hidden))}

    def bind(self, weights, tied=None):
        if self.spec.name is not None:
            self.weight = weights[self.spec.name]
        elif tied is None:
            raise ValueError("the head names no tensor and the embedding offers no table to share")
        else:
            self.weight = tied

    def named_tensors(self):
        return {} if self.spec.name is None else {self.spec.name: self.weight}

    def forward(self, x, out):
        ops.linear(x, self.weight, out)
        cap = dict(self.spec.params).get("softcap")
        if cap:         # logits <- cap * tanh(logits / cap), in float32
            ops.softcap_(out, float(cap))


register_part("embedding", "lookup", LookupEmbedding)
register_part("head", "linear", LinearHead)
