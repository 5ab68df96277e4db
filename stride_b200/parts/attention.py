"""Grouped-query attention over the paged cache.

q/k/v projections (fused into one matrix product at load time), position
encoding and cache write, attention of every token over its request's pages,
output projection: python/stride_worker/model.py:258-299 with the attention rule
of python/stride_worker/layers.py:109-149. Biases are used when the spec says so.
A window (not used by Llama 3) limits each token to its last W keys.

Spec params, all optional:

* ``values`` ``keys``: there is no value projection; a token's value is its key as projected (bias included),
  before the rotation. The key rows are used twice in the fused projection, so keys and values go through the same
  kernels and pages as ever.
* ``softcap`` c: scaled scores become c tanh(s / c).
* ``sinks``: a tensor ``sink`` [heads]; exp(sink_h) joins the denominator of head h's softmax.
* ``output_gate``: a matrix ``g`` [heads * head_dim, hidden]; the concatenated heads are multiplied by
  sigmoid(g x) before the output projection.
  ``output_gate`` ``head``: ``g`` is [heads, hidden] and gives one gate per head; its rows join the fused projection.
* ``names`` ``short``: tensors are ``q, k, v, o`` with biases ``q.b, k.b, v.b`` under the prefix (default:
  ``q_proj.weight`` and so on).
* ``value_dim``: the width of a value head where it is not the keys' (keys and values then lie in pages of their own width).
* ``qk_norm`` / ``v_norm`` ``unit``: every query and key head / every value head is divided by its root mean square
  (``norm_eps`` inside the root, no weight) after the bias and before any rotation; keys and values are kept so.
* ``distance_slopes`` c: head h of H takes ``2^(-c (h + 1) / H) * (i - j)`` off the score of query i and key j (Press et
  al., "Train Short, Test Long: Attention with Linear Biases Enables Input Length Extrapolation", with c = 8).
* ``output_bias``: a bias ``o.b`` on the output projection. The mixer hands it out as ``output_bias`` and the layer's
  arrangement adds it (the ``output_norm`` arrangement inside its norm's kernel).
* ``conv`` n: a causal convolution of n taps over time on every channel of the q, k and v projections, directly after the
  projection (tensors ``q.conv``, ``k.conv``, ``v.conv`` [channels, n], no bias): ``y_t = sum_j w[:, j] u_(t - n + 1 + j)``, zeros
  before a request's start. The last n - 1 projected rows of a request are its state (one float32 row in a state slot).
* ``qk_norm`` ``weighted``: every query and key head goes through an RMS norm with a weight of the head's size shared by the
  heads (tensors ``q.norm``, ``k.norm``; ``norm_eps`` inside the root), after the convolution. One kernel does the
  convolution, the norms and the write into the pages; a second one moves the tails on.
* ``sinks`` ``zero``: no tensor; every head's denominator gains exp(0) = 1.
* ``borrowed_kv``: the mixer has no key and value projections and reads the pages of the cache slot it is given, which
  another layer's mixer of the same shape writes.

When the position part asks for another order of a head's entries (``head_permutation``), the rows of the query and
key projections (and of whatever else must follow them: values taken from keys, the gate, the columns of the output
projection) are laid out in that order at load; scores and outputs are the same, and ``named_tensors`` gives the
stored order back.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .runtime import sequence_slots
from .base import CacheRequest, Mixer, Projection, StateRequest, TensorDecl, build_part, register_part


class PagedAttention(Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads do not group into {s.num_kv_heads} KV heads")
        if s.head_dim <= 0 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim} is not supported by the attention kernels (up to 256 is)")
        if s.window is not None and s.window <= 0:
            raise ValueError("an attention window must be positive")
        self.hidden = s.hidden
        self.nq, self.nkv, self.hd = s.num_heads, s.num_kv_heads, s.head_dim
        self.q_dim, self.kv_dim = self.nq * self.hd, self.nkv * self.hd
        self.qkv_dim = self.q_dim + 2 * self.kv_dim
        self.scale = float(s.scale)
        self.window = 0 if s.window is None else int(s.window)
        self.position = build_part("position", s.position, runtime)
        p = dict(s.params)
        self.values_are_keys = p.get("values") == "keys"
        self.softcap = float(p.get("softcap", 0.0))
        self.zero_sinks = p.get("sinks") == "zero"
        self.has_sinks, self.gated = bool(p.get("sinks", False)) and not self.zero_sinks, bool(p.get("output_gate", False))
        self.taps, self.weighted_qk = int(p.get("conv", 0)), p.get("qk_norm") == "weighted"
        self.short_names = p.get("names") == "short"
        self.vd = int(p.get("value_dim", self.hd))
        self.unit_qk, self.unit_v = p.get("qk_norm") == "unit", p.get("v_norm") == "unit"
        self.norm_eps = float(p.get("norm_eps", 0.0))
        self.head_gate = p.get("output_gate") == "head"
        self.has_output_bias, self.borrows = bool(p.get("output_bias", False)), bool(p.get("borrowed_kv", False))
        self.output_bias = None
        if not 0 < self.vd <= 256:
            raise ValueError(f"value_dim {self.vd} is not supported by the attention kernels (up to 256 is)")
        if self.values_are_keys and (self.vd != self.hd or self.borrows or self.unit_qk or self.unit_v):
            raise ValueError("values taken from keys go with neither a value width of their own, borrowed pages nor head norms")
        # what the plain path (projection, then the position part's rotation and cache write) cannot do goes through
        # the head-norm kernel, which adds the bias, norms and writes the pages itself when there is no rotation
        self.plain_position = s.position is None or s.position.kind == "none"
        self.conv_path = self.taps > 0 or self.weighted_qk
        if self.conv_path and (self.unit_qk or self.unit_v or self.borrows or s.bias or self.head_gate or not self.plain_position
                               or not self.short_names or self.taps > 16):
            raise ValueError("a convolution or weighted head norms go with no rotation, no biases, no unit norms, no borrowed pages, "
                             "no per-head gate, short tensor names and at most 16 taps")
        self.own_prepare = self.unit_qk or self.unit_v or self.vd != self.hd or self.borrows or self.conv_path
        if self.own_prepare and not self.plain_position and (self.vd != self.hd or self.borrows):
            raise ValueError("a rotation with borrowed pages or a value width of its own is not supported")
        self.fused_gate = self.head_gate and self.own_prepare and self.plain_position
        slope_c = p.get("distance_slopes")
        self.slopes = None if slope_c is None else torch.tensor(
            [2.0 ** (-float(slope_c) * (h + 1) / self.nq) for h in range(self.nq)], dtype=torch.float32, device=runtime.device)
        self.v_dim, self.o_in = self.nkv * self.vd, self.nq * self.vd
        self.kv_cols = 0 if self.borrows else self.kv_dim + self.v_dim
        # gate columns are padded so that every row of the fused buffer starts on a 16-byte boundary
        self.gate_cols = -(-self.nq // 8) * 8 if self.fused_gate else 0
        self.qkv_dim = self.q_dim + self.kv_cols + self.gate_cols
        permutation = getattr(self.position, "head_permutation", lambda: None)()
        self.perm = None if permutation is None else torch.tensor(permutation, dtype=torch.long)
        self.w_qkv = self.w_o = self.bias = self.w_gate = self.sinks = self.conv_w = self.wq_norm = self.wk_norm = None
        if self.zero_sinks:
            self.sinks = torch.zeros(self.nq, dtype=torch.float32, device=runtime.device)
        self._fast = ops.fast_attention_supported(runtime.dtype, self.nq, self.nkv, self.hd) and self.vd == self.hd
        self.accepts_folded = not self.gated          # the gate reads the normed input as a tensor

    # ----------------------------------------------------------------- weights
    def _names(self):
        p = self.spec.prefix
        if self.short_names:
            w, b = {k: p + k for k in "qkvo"}, {k: f"{p}{k}.b" for k in "qkv"}
        else:
            w, b = {k: f"{p}{k}_proj.weight" for k in "qkvo"}, {k: f"{p}{k}_proj.bias" for k in "qkv"}
        w["g"], w["sink"] = p + "g", p + "sink"
        b["o"] = f"{p}o.b" if self.short_names else f"{p}o_proj.bias"
        return w, b

    def declare(self):
        w, b = self._names()
        d = {w["q"]: TensorDecl((self.q_dim, self.hidden)), w["o"]: TensorDecl((self.hidden, self.o_in))}
        if not self.borrows:
            d[w["k"]] = TensorDecl((self.kv_dim, self.hidden))
            if not self.values_are_keys:
                d[w["v"]] = TensorDecl((self.v_dim, self.hidden))
        if self.spec.bias:
            d[b["q"]] = TensorDecl((self.q_dim,), "vector")
            if not self.borrows:
                d[b["k"]] = TensorDecl((self.kv_dim,), "vector")
                if not self.values_are_keys:
                    d[b["v"]] = TensorDecl((self.v_dim,), "vector")
        if self.has_output_bias:
            d[b["o"]] = TensorDecl((self.hidden,), "vector")
        if self.gated:
            d[w["g"]] = TensorDecl((self.nq if self.head_gate else self.q_dim, self.hidden))
        if self.has_sinks:
            d[w["sink"]] = TensorDecl((self.nq,), "vector")
        p = self.spec.prefix
        if self.taps:
            d.update({f"{p}{n}.conv": TensorDecl((rows, self.taps), "vector") for n, rows in (("q", self.q_dim), ("k", self.kv_dim), ("v", self.v_dim))})
        if self.weighted_qk:
            d.update({f"{p}{n}.norm": TensorDecl((self.hd,), "vector") for n in "qk"})
        d.update(self.position.declare())          # a position encoding may have tensors of its own
        return d

    def _reorder(self, t, inverse: bool = False, dim: int = 0):
        """The heads' entries of ``t`` along ``dim`` (length heads * head_dim) in the position part's order."""
        if self.perm is None:
            return t
        perm = torch.argsort(self.perm) if inverse else self.perm
        heads = t.shape[dim] // self.hd
        index = (torch.arange(heads)[:, None] * self.hd + perm[None, :]).reshape(-1).to(t.device)
        return t.index_select(dim, index).contiguous()

    def bind(self, weights):
        w, b = self._names()
        if self.own_prepare:
            return self._bind_own(weights, w, b)
        q, k = self._reorder(weights[w["q"]]), self._reorder(weights[w["k"]])
        v = k if self.values_are_keys else weights[w["v"]]
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        if self.has_output_bias:
            self.output_bias = weights[b["o"]]
        # values taken from keys come in the keys' order, and so do the heads' outputs
        self.w_o = self._reorder(weights[w["o"]], dim=1) if self.values_are_keys else weights[w["o"]]
        if self.spec.bias:
            bq, bk = self._reorder(weights[b["q"]]), self._reorder(weights[b["k"]])
            self.bias = torch.cat([bq, bk, bk if self.values_are_keys else weights[b["v"]]]).contiguous()
        if self.gated:
            self.w_gate = self._reorder(weights[w["g"]]) if self.values_are_keys else weights[w["g"]]
        if self.has_sinks:
            self.sinks = weights[w["sink"]]
        self.position.bind(weights)

    def _bind_own(self, weights, w, b):
        """The fused projection of the head-norm path: query rows, then key and value rows unless they are borrowed,
        then the rows of a per-head gate. No reordering: a rotation that wants one is not combined with this path."""
        if self.perm is not None:
            raise ValueError("head norms are not combined with a rotation that reorders the heads' entries")
        order = ["q"] + ([] if self.borrows else ["k", "v"])
        rows = [weights[w[n]] for n in order] + ([weights[w["g"]]] if self.fused_gate else [])
        if self.gate_cols > self.nq:
            rows.append(torch.zeros((self.gate_cols - self.nq, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = weights[w["o"]]
        if self.spec.bias:
            self.bias = torch.cat([weights[b[n]] for n in order]).contiguous()
        if self.gated and not self.fused_gate:
            self.w_gate = weights[w["g"]]
        if self.has_sinks:
            self.sinks = weights[w["sink"]]
        if self.has_output_bias:
            self.output_bias = weights[b["o"]]
        p = self.spec.prefix
        if self.taps:
            # [taps, channels]: a tap's weights of neighbouring channels side by side, as the kernel reads them
            self.conv_w = torch.cat([weights[f"{p}{n}.conv"] for n in "qkv"], dim=0).t().contiguous()
        if self.weighted_qk:
            self.wq_norm, self.wk_norm = weights[p + "q.norm"], weights[p + "k.norm"]
        self.position.bind(weights)

    def _named_own(self):
        w, b = self._names()
        out, at = {w["o"]: self.w_o}, 0
        for n, rows in [("q", self.q_dim)] + ([] if self.borrows else [("k", self.kv_dim), ("v", self.v_dim)]):
            out[w[n]] = self.w_qkv[at:at + rows]
            if self.bias is not None:
                out[b[n]] = self.bias[at:at + rows]
            at += rows
        if self.gated:
            out[w["g"]] = self.w_qkv[at:at + self.nq] if self.fused_gate else self.w_gate
        if self.has_sinks:
            out[w["sink"]] = self.sinks
        if self.has_output_bias:
            out[b["o"]] = self.output_bias
        p = self.spec.prefix
        if self.taps:
            q, k = self.q_dim, self.q_dim + self.kv_dim
            stored = self.conv_w.t()
            out.update({p + "q.conv": stored[:q], p + "k.conv": stored[q:k], p + "v.conv": stored[k:]})
        if self.weighted_qk:
            out.update({p + "q.norm": self.wq_norm, p + "k.norm": self.wk_norm})
        out.update(self.position.named_tensors())
        return out

    def named_tensors(self):
        if self.own_prepare:
            return self._named_own()
        w, b = self._names()
        q, k = self.q_dim, self.q_dim + self.kv_dim
        back = lambda t, dim=0: self._reorder(t, inverse=True, dim=dim)
        out = {w["q"]: back(self.w_qkv[:q]), w["k"]: back(self.w_qkv[q:k]),
               w["o"]: back(self.w_o, 1) if self.values_are_keys else self.w_o}
        if not self.values_are_keys:
            out[w["v"]] = self.w_qkv[k:]
        if self.bias is not None:
            out.update({b["q"]: back(self.bias[:q]), b["k"]: back(self.bias[q:k])})
            if not self.values_are_keys:
                out[b["v"]] = self.bias[k:]
        if self.gated:
            out[w["g"]] = back(self.w_gate) if self.values_are_keys else self.w_gate
        if self.has_sinks:
            out[w["sink"]] = self.sinks
        if self.has_output_bias:
            out[b["o"]] = self.output_bias
        out.update(self.position.named_tensors())
        return out

    # ------------------------------------------------------------------- cache
    def cache_request(self):
        if self.vd != self.hd:
            return CacheRequest(window=self.spec.window, tensors=(("k", self.nkv, self.hd), ("v", self.nkv, self.vd)))
        return CacheRequest(self.nkv, self.hd, self.spec.window)

    def state_request(self):
        """The convolution's tail: the last taps - 1 projected rows of a request, float32."""
        if self.taps > 1:
            return StateRequest(((self.taps - 1) * (self.q_dim + self.kv_dim + self.v_dim),), torch.float32)
        return None

    # ----------------------------------------------------------------- forward
    lazy_output = True
    accepts_folded = True       # an instance with an output gate says False

    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens = x.shape[0]
        qkv = self.rt.buffer("qkv", tokens, self.qkv_dim)
        folded = x if isinstance(x, ops.FoldedNorm) else None
        if self.conv_path:
            if folded:
                x = folded.tensor()
            raw = self.rt.buffer("qkv_raw", tokens, self.qkv_dim)
            ops.linear(x, self.w_qkv, raw)
            self._convolve_and_store(raw, qkv, ctx, cache, tokens)
        elif self.own_prepare:
            if folded:
                x = folded.tensor()
            ops.linear(x, self.w_qkv, qkv)
            self._norm_and_store(qkv, ctx, cache, tokens)
        elif not self._project_and_rotate(folded.xt if folded else x, qkv, ctx, cache, tokens, folded):
            if folded:
                x = folded.tensor()
            ops.linear(x, self.w_qkv, qkv)
            self.position.encode_and_store(qkv, self.bias, ctx, cache, self.nq, self.nkv, self.hd)
        attn = self.rt.buffer("attn", tokens, self.o_in)
        ungated = self._attend(qkv, attn, ctx, cache, tokens)
        if self.fused_gate:
            if ungated:         # the decode kernel applies the gates of its rows itself
                ops.head_gate(attn[:ungated], qkv[:ungated, self.q_dim + self.kv_cols:], self.qkv_dim, self.nq, self.vd)
        elif self.head_gate:
            gate = self.rt.buffer("attn_gate", tokens, self.nq)
            ops.linear(x, self.w_gate, gate)
            ops.head_gate(attn, gate, self.nq, self.nq, self.vd)
        elif self.gated:
            gate = self.rt.buffer("attn_gate", tokens, self.q_dim)
            ops.linear(x, self.w_gate, gate)
            ops.sigmoid_gate(attn, gate)
        if lazy_output:
            return Projection(attn, self.w_o)          # the residual stream runs it, with the sum and norm that follow if it can
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(attn, self.w_o, out)
        return out


    def _convolve_and_store(self, raw, qkv, ctx, cache, tokens):
        """Convolution over time, weighted head norms and the pages in one kernel; then the tails of the step's requests move on."""
        slots = ctx.slot_mapping[cache.group][:tokens] if cache.writes else None
        state = cache.state if self.taps > 1 else None
        ops.conv_head_norm(raw, qkv, self.conv_w, state, 0, ctx.seq_of_token[:tokens], ctx.q_start, ctx.state_slot, self.wq_norm, self.wk_norm,
                           self.norm_eps, slots, cache.k_pages if cache.writes else None, cache.v_pages if cache.writes else None, self.nq,
                           self.nkv, self.hd, self.vd, cache.page_size)
        if state is not None:
            ops.conv_tail(raw, state, 0, ctx.q_start, ctx.q_len, ctx.state_slot, sequence_slots(ctx), self.qkv_dim, self.taps)

    def _norm_and_store(self, qkv, ctx, cache, tokens):
        """Bias, head norms and the pages: in one kernel when there is no rotation, else the norms here and rotation and
        pages through the position part."""
        writes = cache.writes and not self.borrows
        nkv = 0 if self.borrows else self.nkv
        if self.plain_position:
            slots = ctx.slot_mapping[cache.group][:tokens] if writes else None
            ops.qkv_unit_norm(qkv, self.bias, slots, cache.k_pages if writes else None, cache.v_pages if writes else None, self.nq, nkv,
                              self.hd, self.vd, cache.page_size, self.norm_eps, self.unit_qk, self.unit_v)
        else:
            ops.qkv_unit_norm(qkv, self.bias, None, None, None, self.nq, nkv, self.hd, self.vd, cache.page_size, self.norm_eps,
                              self.unit_qk, self.unit_v)
            self.position.encode_and_store(qkv, None, ctx, cache, self.nq, self.nkv, self.hd)

    def _project_and_rotate(self, x, qkv, ctx, cache, tokens, folded=None) -> bool:
        """A decode step's projection with the position encoding and the cache write in its epilogue, when the
        position part says that what it does is the standard rotation. False: nothing was done."""
        if tokens > max(ops.TC_GEMM_MAX_TOKENS, ops.ROWS_GEMM_MAX_TOKENS) or x.dtype != torch.bfloat16:
            return False
        tables = self.position.rotation_tables()
        if tables is None:
            return False
        cos, sin, rotate = tables
        slots = ctx.slot_mapping[cache.group][:tokens] if cache.writes else None
        if tokens > ops.TC_GEMM_MAX_TOKENS:         # the tokens-as-rows kernel, where the policy sends steps of this size to it
            return ops.rows_wanted(tokens) and ops.linear_rows_qkv_rope(
                x, self.w_qkv, qkv, self.bias, ctx.positions[:tokens], slots, cos, sin, cache.k_pages, cache.v_pages, self.nq, self.nkv,
                self.hd, cache.page_size, rotate, folded)
        return ops.linear_qkv_rope(x, self.w_qkv, qkv, self.bias, ctx.positions[:tokens], slots, cos, sin, cache.k_pages,
                                   cache.v_pages, self.nq, self.nkv, self.hd, cache.page_size, rotate, folded)

    def _attend(self, qkv, attn, ctx, cache, tokens) -> int:
        """Attention of the step's rows. Returns how many leading rows still lack the per-head gate (all of them unless the
        gates' logits stand in the rows of ``qkv`` and the decode kernel took the rows after the portions)."""
        table = ctx.block_table[cache.group]
        geometry = (self.nq, self.nkv, self.hd, cache.page_size, self.scale, self.window)
        if not self._fast:
            # the exact kernel: the whole 32-bit path, and bfloat16 sizes the tensor-core kernels refuse
            ops.paged_attention(qkv, self.qkv_dim, attn, cache.k_pages, cache.v_pages, table, ctx.seq_of_token[:tokens],
                                ctx.positions[:tokens], *geometry, self.softcap, self.sinks, self.slopes, self.vd)
            return tokens
        split = min(ctx.decode_tail_start, tokens)          # portions before, single decoded tokens after
        if split > 0:
            args = (qkv[:split], self.qkv_dim, attn[:split], cache.k_pages, cache.v_pages, table, ctx.q_start, ctx.q_len,
                    ctx.ctx_len, ctx.decode_tail_seq, *geometry, self.softcap, self.sinks, self.slopes)
            # tcgen05 kernel first; the mma.sync kernel takes what it refuses (odd page sizes)
            if not (ops.TC_ATTENTION and ops.paged_attention_prefill_tc(*args)):
                ops.paged_attention_prefill(*args)
        if tokens > split:
            n = tokens - split
            scratch = self.rt.scratch("attention_splits", ops.decode_scratch_floats(n, self.nq, self.nkv, self.hd, ctx.context_bound))
            ops.paged_attention_decode(qkv[split:tokens], self.qkv_dim, attn[split:tokens], cache.k_pages, cache.v_pages, table,
                                       ctx.seq_of_token[split:tokens], ctx.positions[split:tokens], scratch, *geometry,
                                       ctx.context_bound, self.softcap, self.sinks, self.slopes,
                                       self.q_dim + self.kv_cols if self.fused_gate else -1)
            return split if self.fused_gate else tokens
        return tokens


register_part("mixer", "attention", PagedAttention)
