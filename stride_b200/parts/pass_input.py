"""What a model does to its residual stream before every pass over a block of layers that runs several times.

``mix_embedding``: ``x <- W [x; x0] + s[t]``: the stream beside the embedding's output x0 through one matrix ``W``
[hidden, 2 * hidden] (the stream's columns first), then the vector of pass t added. The product reads the stream rounded to
the compute dtype and leaves float32 sums, which become the new stream; the vector is added in float32. Three launches: the
two inputs side by side, the product, the vector.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import PassInput, TensorDecl, register_part


class MixEmbedding(PassInput):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.passes = int(spec.hidden), int(spec.passes)
        if self.passes < 1:
            raise ValueError("a repeated block runs at least once")
        self.weight = self.steps = None

    def declare(self):
        return {self.spec.mix_name: TensorDecl((self.hidden, 2 * self.hidden)),
                self.spec.step_name: TensorDecl((self.passes, self.hidden), "vector")}

    def bind(self, weights):
        self.weight, self.steps = weights[self.spec.mix_name], weights[self.spec.step_name]

    def named_tensors(self):
        return {self.spec.mix_name: self.weight, self.spec.step_name: self.steps}

    def forward(self, stream, first, number, ctx):
        if not 0 <= number < self.passes:
            raise ValueError(f"pass {number} of {self.passes}")
        residual = stream.materialize()
        tokens = residual.shape[0]
        both = self.rt.buffer("pass_inputs", tokens, 2 * self.hidden)
        ops.stream_concat(residual, first, both)
        ops.linear(both, self.weight, residual)             # float32 sums straight into the stream
        ops.add_row_vector(residual, self.steps[number], ctx.seq_of_token[:tokens])


register_part("pass_input", "mix_embedding", MixEmbedding)
