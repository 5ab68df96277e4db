"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * weight`` in float32, the weight
multiplying after the normalisation (python/stride_worker/layers.py:24-35).

Spec params: ``tensor`` names the weight (default: the prefix + ``weight``); ``weight_offset`` c makes the factor
``c + w`` for checkpoints that keep w = factor - c (the sum is formed once, in float32, when the weight is bound);
``shape`` ``scalar``: the checkpoint keeps one number for all coordinates (a tensor without dimensions), which is spread
over the width when it is bound, so every kernel sees a vector; ``scale_tensor`` names a second vector [width] (a learned scale
on what a sublayer adds to the stream) that multiplies the norm's output element by element: the two are one float32 factor
from load on.

Besides the pre-norm use (``apply``) the norm can sit on a sublayer's output: ``add_normed`` adds ``mult * norm(delta)``
to the residual stream."""

from __future__ import annotations

from ..csrc import ops
from .base import Norm, TensorDecl, register_part


class RMSNorm(Norm):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.eps = float(spec.eps)
        self.width = int(spec.width)
        self.weight = None
        p = dict(spec.params)
        self._name = p.get("tensor", spec.prefix + "weight")
        self.offset = float(p.get("weight_offset", 0.0))
        self.scalar = p.get("shape") == "scalar"
        self._scale_name = p.get("scale_tensor")
        self.stored = self.stored_scale = None

    def declare(self):
        d = {self._name: TensorDecl(() if self.scalar else (self.width,), "vector")}
        if self._scale_name:
            d[self._scale_name] = TensorDecl((self.width,), "vector")
        return d

    def bind(self, weights):
        self.stored = weights[self._name]
        weight = self.stored.reshape(1).expand(self.width).contiguous() if self.scalar else self.stored
        self.weight = weight + self.offset if self.offset else weight
        if self._scale_name:
            self.stored_scale = weights[self._scale_name]
            self.weight = (self.weight * self.stored_scale).contiguous()

    def named_tensors(self):
        out = {self._name: self.stored}
        if self._scale_name:
            out[self._scale_name] = self.stored_scale
        return out

    def fold_inputs(self):
        return self.weight, self.eps

    def apply(self, residual, pending, out, rows=None):
        ops.add_rmsnorm(residual, pending, self.weight, out, self.eps, rows=rows)      # sum, write-back and norm in one kernel

    def add_normed(self, residual, delta, bias, mult, copy):
        ops.norm_add(residual, delta, bias, self.weight, copy, self.eps, mult)         # norm, sum, write-back and copy in one kernel

    def add_normed_then(self, residual, delta, bias, mult, following, out) -> bool:
        """``add_normed`` and, from the row while it is at hand, the norm ``following`` of the new rows into ``out``: one
        kernel for the norm behind a sublayer and the norm in front of the next one. False: not done (another kind of norm)."""
        if not isinstance(following, RMSNorm):
            return False
        ops.norm_add(residual, delta, bias, self.weight, None, self.eps, mult, following.weight, following.eps, out)
        return True


register_part("norm", "rmsnorm", RMSNorm)
