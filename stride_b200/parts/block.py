"""Arrangement of parts in a layer. ``pre_norm``: the mixer and the feed-forward
each read a normed copy of the residual stream and add their output back
(python/stride_worker/model.py:254-310). The spec may put a multiplier on every
sum into the stream, leave the feed-forward out, and name parts that add a
token-dependent input to the stream after the feed-forward.

``output_norm``: the sublayers read the stream itself and the norm sits on what they give back,
``x += m * norm(mixer(x)); x += m * norm(ffn(x))``. A sublayer's last bias (``output_bias``) is added inside the
norm's kernel.

``sandwich``: a norm on either side of a sublayer, ``x += m * out_norm(mixer(norm(x))); x += m * out_norm(ffn(norm(x)))``
(the spec's ``mixer_out_norm`` and ``ffn_out_norm``; a learned scale on the sum is a param of those norms)."""

from __future__ import annotations

from .base import Layer, build_part, register_part


class PreNormLayer(Layer):
    adds_output_bias = False

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        has_ffn = spec.feed_forward is not None
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime) if has_ffn else None
        self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime) if has_ffn else None
        self.after = tuple(build_part("stream_input", s, runtime) for s in getattr(spec, "after", ()))
        self.mult = float(getattr(spec, "residual_mult", 1.0))
        if not self.adds_output_bias and any(getattr(p, "has_output_bias", False) for p in (self.mixer, self.feed_forward)):
            raise ValueError(f"the arrangement {spec.kind!r} does not add a sublayer's output bias")

    def parts(self):
        own = (self.mixer_norm, self.mixer) + ((self.ffn_norm, self.feed_forward) if self.feed_forward is not None else ())
        return own + self.after

    def declare(self):
        d = {}
        for p in self.parts():
            d.update(p.declare())
        return d

    def bind(self, weights):
        for p in self.parts():
            p.bind(weights)

    def named_tensors(self):
        d = {}
        for p in self.parts():
            d.update(p.named_tensors())
        return d

    def forward(self, stream, ctx, cache):
        # A part that can, gets the norm folded into its first product and leaves its last product to the stream,
        # which folds it into the next norm (decode steps in bfloat16; everything else runs part by part).
        mixer, ffn, mult = self.mixer, self.feed_forward, self.mult
        h = stream.normed(self.mixer_norm, fold_ok=mixer.accepts_folded)
        stream.add(mixer.forward(h, ctx, cache, lazy_output=True) if mixer.lazy_output else mixer.forward(h, ctx, cache), mult)
        if ffn is not None:
            h = stream.normed(self.ffn_norm, fold_ok=ffn.accepts_folded)
            stream.add(ffn.forward(h, ctx, lazy_output=True) if ffn.lazy_output else ffn.forward(h, ctx), mult)
        for part in self.after:
            part.forward(stream, ctx, mult)


class OutputNormLayer(PreNormLayer):
    """The same parts in the other arrangement: no norm before a sublayer, one on its output."""
    adds_output_bias = True

    def forward(self, stream, ctx, cache):
        mixer, ffn, mult = self.mixer, self.feed_forward, self.mult
        stream.add_normed(mixer.forward(stream.values(), ctx, cache), self.mixer_norm, mult, getattr(mixer, "output_bias", None))
        if ffn is not None:
            stream.add_normed(ffn.forward(stream.values(), ctx), self.ffn_norm, mult, getattr(ffn, "output_bias", None))
        for part in self.after:
            part.forward(stream, ctx, mult)


class SandwichLayer(PreNormLayer):
    """Norm, sublayer, norm, sum: the pre-norm kernel in front (the stream is settled, so it only norms), the output norm's
    kernel behind (norm, multiplier and residual sum in one)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.mixer_out_norm is None or (self.feed_forward is not None and spec.ffn_out_norm is None):
            raise ValueError("the sandwich arrangement needs a norm on every sublayer's output")
        self.mixer_out_norm = build_part("norm", spec.mixer_out_norm, runtime)
        self.ffn_out_norm = build_part("norm", spec.ffn_out_norm, runtime) if self.feed_forward is not None else None

    def parts(self):
        return super().parts() + (self.mixer_out_norm,) + ((self.ffn_out_norm,) if self.ffn_out_norm is not None else ())

    def forward(self, stream, ctx, cache):
        mixer, ffn, mult = self.mixer, self.feed_forward, self.mult
        stream.add_normed(mixer.forward(stream.normed(self.mixer_norm), ctx, cache), self.mixer_out_norm, mult, keep_copy=False)
        if ffn is not None:
            stream.add_normed(ffn.forward(stream.normed(self.ffn_norm), ctx), self.ffn_out_norm, mult, keep_copy=False)
        for part in self.after:
            part.forward(stream, ctx, mult)


register_part("layer", "pre_norm", PreNormLayer)
register_part("layer", "sandwich", SandwichLayer)
register_part("layer", "output_norm", OutputNormLayer)
