"""Routed feed-forward (a mixture of experts) with an optional shared expert.

Router logits ``z = W_r h + b`` in float32; a token uses the ``top`` experts with the largest logits, weighted with
the softmax over those logits only; an expert is ``W_down act(W_up h)`` without biases, ``act`` the square of relu;
a shared expert of the same form runs for every token and is added.

On the device: the router's product leaves float32 logits, a kernel chooses, a one-CTA plan lays the (token, choice) pairs out expert by expert, two
grouped products run all experts' rows in one launch each (the first gathers its rows through the plan and applies
the activation, the second leaves float32 rows), and one kernel sums a token's rows with its weights and the
shared expert's output. Nothing returns to the host, so a step can be captured in a graph.

Spec: ``hidden``, ``intermediate`` (an expert's width), ``activation`` (``relu_squared``), params ``experts``, ``top``,
``shared`` (the shared expert's width, 0 for none), ``router_bias``. Tensors under the prefix: ``router``, ``router.b``,
``e<k>.up``, ``e<k>.down``, ``shared.up``, ``shared.down``.

Another family of the same part, chosen by the spec:

* ``activation`` ``swish_clamped`` makes every expert a gated unit ``W_down (g' sigmoid(alpha g') (u' + 1))`` with
  ``g' = min(W_gate h, limit)``, ``u' = clamp(W_up h, -limit, limit)`` (params ``limit``, ``alpha``; the shared expert's
  own ``shared_limit``). Tensors ``e<k>.gate`` and ``shared.gate`` join the others. Gate and up rows of an expert are
  laid out in neighbouring pairs at load, so the first grouped product applies the activation in its epilogue.
* param ``router`` ``sigmoid_groups``: scores are ``sigmoid(z)``; the choice is made on ``score + correction`` (tensor
  ``correction`` [experts]); the experts form ``groups`` equal groups of neighbours, a group counts as the sum of its two
  largest choice scores, and only experts of the ``keep`` best groups can be chosen; the weights are the chosen scores
  (without the correction) over their sum, times ``route_scale``.
* ``activation`` ``silu`` makes every expert the plain gated unit ``W_down (silu(W_gate h) * (W_up h))``, laid out and run
  the same way.
* param ``router`` ``softmax_groups``: scores are the softmax of z over all experts; a group counts as its largest
  score; the ``top`` largest scores inside the ``keep`` best groups win; the weights are those scores times
  ``route_scale``, not divided by their sum. No ``correction`` tensor.
* param ``shared_gate``: the shared expert's output is multiplied by ``sigmoid(W_sg h)``, one number per token (tensor
  ``shared.sg`` [1, hidden]); its row rides in the router's product.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, TensorDecl, register_part
from .swiglu import interleave_gate_up


class RoutedExperts(FeedForward):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = dict(spec.params)
        self.hidden, self.ff = int(spec.hidden), int(spec.intermediate)
        self.experts, self.top, self.shared_ff = int(p["experts"]), int(p["top"]), int(p.get("shared", 0))
        self.router_bias = bool(p.get("router_bias", False))
        if spec.activation not in ("relu_squared", "swish_clamped", "silu"):
            raise ValueError(f"activation {spec.activation!r} is not supported by the routed experts (relu_squared, swish_clamped and silu are)")
        if not 1 <= self.top <= min(self.experts, 32) or self.experts > 256:
            raise ValueError(f"top {self.top} of {self.experts} experts is not supported (up to 32 of up to 256 are)")
        self.gated = spec.activation in ("swish_clamped", "silu")
        self.clamped = spec.activation == "swish_clamped"
        self.limit, self.alpha = float(p.get("limit", 0.0)), float(p.get("alpha", 1.0))
        self.shared_limit = float(p.get("shared_limit", self.limit))
        self.router_kind = p.get("router", "softmax_top")
        self.groups, self.keep, self.route_scale = int(p.get("groups", 1)), int(p.get("keep", 1)), float(p.get("route_scale", 1.0))
        self.shared_gate = bool(p.get("shared_gate", False))
        if self.router_kind not in ("softmax_top", "sigmoid_groups", "softmax_groups"):
            raise ValueError(f"router {self.router_kind!r} is not known (softmax_top, sigmoid_groups and softmax_groups are)")
        if self.router_kind != "softmax_top" and (self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups
                                                     or self.top > self.keep * (self.experts // self.groups)):
            raise ValueError(f"{self.experts} experts in {self.groups} groups of which {self.keep} stay cannot give {self.top} choices")
        if self.clamped and not (self.limit > 0 and self.shared_limit > 0):
            raise ValueError("the clamped activation needs a positive `limit`")
        if self.shared_gate and not self.shared_ff:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.shared_block = self.shared_ff
        self.w_router = self.bias = self.w_up = self.w_down = self.shared_up = self.shared_down = self.correction = None

    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        d = {self._n("router"): TensorDecl((self.experts, self.hidden))}
        if self.router_bias:
            d[self._n("router.b")] = TensorDecl((self.experts,), "vector")
        if self.router_kind == "sigmoid_groups":
            d[self._n("correction")] = TensorDecl((self.experts,), "vector")
        for e in range(self.experts):
            if self.gated:
                d[self._n(f"e{e}.gate")] = TensorDecl((self.ff, self.hidden))
            d[self._n(f"e{e}.up")] = TensorDecl((self.ff, self.hidden))
            d[self._n(f"e{e}.down")] = TensorDecl((self.hidden, self.ff))
        if self.shared_ff:
            if self.gated:
                d[self._n("shared.gate")] = TensorDecl((self.shared_ff, self.hidden))
            d[self._n("shared.up")] = TensorDecl((self.shared_ff, self.hidden))
            d[self._n("shared.down")] = TensorDecl((self.hidden, self.shared_ff))
        if self.shared_gate:
            d[self._n("shared.sg")] = TensorDecl((1, self.hidden))
        return d

    @staticmethod
    def _pairs(gate, up):
        """[2 * ff, hidden]: row 2i is gate row i, row 2i + 1 up row i."""
        return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1])

    def bind(self, weights):
        router = weights[self._n("router")]
        # the shared expert's gate is one more row of the router's product
        self.w_router = torch.cat([router, weights[self._n("shared.sg")]], dim=0).contiguous() if self.shared_gate else router
        self.bias = weights[self._n("router.b")] if self.router_bias else None
        self.correction = weights[self._n("correction")] if self.router_kind == "sigmoid_groups" else None
        ups = [weights[self._n(f"e{e}.up")] for e in range(self.experts)]
        if self.gated:
            ups = [self._pairs(weights[self._n(f"e{e}.gate")], up) for e, up in enumerate(ups)]
        self.w_up = torch.stack(ups).contiguous()
        self.w_down = torch.stack([weights[self._n(f"e{e}.down")] for e in range(self.experts)]).contiguous()
        if self.shared_ff:
            self.shared_up, self.shared_down = weights[self._n("shared.up")], weights[self._n("shared.down")]
            if self.gated:
                # gate and up rows alternate in blocks, as in the dense gated feed-forward: 64 rows where the tcgen05
                # product can apply the activation in its epilogue, else all gate rows before all up rows
                gate = weights[self._n("shared.gate")]
                self.shared_block = ops.GATED_BLOCK if gate.dtype == torch.bfloat16 and self.shared_ff % ops.GATED_BLOCK == 0 else self.shared_ff
                self.shared_up = interleave_gate_up(gate, self.shared_up, self.shared_block)

    def named_tensors(self):
        out = {self._n("router"): self.w_router[:self.experts]}
        if self.router_bias:
            out[self._n("router.b")] = self.bias
        if self.correction is not None:
            out[self._n("correction")] = self.correction
        for e in range(self.experts):
            if self.gated:
                out[self._n(f"e{e}.gate")], out[self._n(f"e{e}.up")] = self.w_up[e, 0::2], self.w_up[e, 1::2]
            else:
                out[self._n(f"e{e}.up")] = self.w_up[e]
            out[self._n(f"e{e}.down")] = self.w_down[e]
        if self.shared_ff:
            if self.gated:
                blocks = self.shared_up.view(self.shared_ff // self.shared_block, 2, self.shared_block, self.hidden)
                out[self._n("shared.gate")] = blocks[:, 0].reshape(self.shared_ff, self.hidden)
                out[self._n("shared.up")] = blocks[:, 1].reshape(self.shared_ff, self.hidden)
            else:
                out[self._n("shared.up")] = self.shared_up
            out[self._n("shared.down")] = self.shared_down
        if self.shared_gate:
            out[self._n("shared.sg")] = self.w_router[self.experts:]
        return out

    def forward(self, x, ctx):
        tokens, top = x.shape[0], self.top
        pairs = tokens * top
        i32 = torch.int32
        ids = self.rt.buffer("moe_ids", tokens, top, i32)
        weights = self.rt.buffer("moe_weights", tokens, top, torch.float32)
        logits = self.rt.buffer("moe_logits", tokens, self.w_router.shape[0], torch.float32)
        ops.linear(x, self.w_router, logits)            # float32 sums of exact products, float32 logits
        if self.router_kind == "sigmoid_groups":
            ops.moe_select_sigmoid(logits, self.correction, ctx.seq_of_token[:tokens], ids, weights, self.experts, self.groups, self.keep,
                                   self.route_scale)
        elif self.router_kind == "softmax_groups":
            ops.moe_select_groups(logits, None, ctx.seq_of_token[:tokens], ids, weights, self.experts, self.groups, self.keep,
                                  self.route_scale, softmax=True, group_max=True, keep_scores=True)
        else:
            ops.moe_select(logits if not self.shared_gate else logits[:, :self.experts].contiguous(), self.bias,
                           ctx.seq_of_token[:tokens], ids, weights)
        row_of = self.rt.buffer("moe_row_of", tokens, top, i32)
        perm = self.rt.buffer("moe_perm", tokens, top, i32).view(-1)
        rank = self.rt.buffer("moe_rank", tokens, top, i32).view(-1)
        offsets = self.rt.scratch(f"moe_offsets_{self.experts}", self.experts + 1, i32)
        ops.moe_plan(ids, self.experts, offsets, perm, row_of, rank)
        hidden_rows = self.rt.buffer("moe_hidden", tokens, top * self.ff).view(pairs, self.ff)
        y = self.rt.buffer("moe_y", tokens, top * self.hidden, torch.float32).view(pairs, self.hidden)
        act = (2 if self.clamped else 3) if self.gated else 1
        if not self._products_tc(x, perm, offsets, hidden_rows, y, tokens, pairs, act):
            ops.grouped_gemm(x, perm, self.w_up, offsets, hidden_rows, pairs, act=act, limit=self.limit, alpha=self.alpha)
            ops.grouped_gemm(hidden_rows, None, self.w_down, offsets, y, pairs, act=0)
        shared = None
        if self.shared_ff:
            mid = self.rt.buffer("moe_shared_mid", tokens, self.shared_ff)
            if self.gated:
                kind = self.spec.activation
                if not (self.shared_block == ops.GATED_BLOCK
                        and ops.linear_gated_tc(x, self.shared_up, mid, None, kind, self.shared_limit, self.alpha)):
                    both = self.rt.buffer("moe_shared_gate_up", tokens, 2 * self.shared_ff)
                    ops.linear(x, self.shared_up, both)
                    if self.clamped:
                        ops.gated_act(both, mid, self.shared_block, kind, self.shared_limit, self.alpha)
                    else:
                        ops.silu_mul(both, mid, self.shared_block)
            else:
                ops.linear(x, self.shared_up, mid)
                ops.relu_squared(mid)
            shared = self.rt.buffer("moe_shared_out", tokens, self.hidden)
            ops.linear(mid, self.shared_down, shared)
        out = self.rt.buffer("ffn_out", tokens, self.hidden)
        ops.moe_combine(y, row_of, weights, shared, out, logits[:, self.experts] if self.shared_gate else None)
        return out


    def _products_tc(self, x, perm, offsets, hidden_rows, y, tokens, pairs, act) -> bool:
        """Both products of all experts on the tcgen05 kernel, for steps of many rows: the tokens' rows are laid out
        expert by expert first, so that every expert's rows are one block of a matrix. False: nothing was done."""
        if not ops.grouped_tc_wanted(x.dtype, pairs):
            return False
        rows = self.rt.buffer("moe_rows", tokens, self.top * self.hidden).view(pairs, self.hidden)
        if not ops.gather_rows(x, perm, offsets, self.experts, rows, pairs):
            return False
        if not ops.grouped_gemm_tc(rows, self.w_up, offsets, hidden_rows, pairs, act, self.limit, self.alpha):
            return False
        if not ops.grouped_gemm_tc(hidden_rows, self.w_down, offsets, y, pairs, 0):
            ops.grouped_gemm(hidden_rows, None, self.w_down, offsets, y, pairs, act=0)
        return True


register_part("feed_forward", "routed_experts", RoutedExperts)
