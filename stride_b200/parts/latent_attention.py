"""Attention over a compressed cache (latent attention).

Per token the layer keeps one latent vector ``c`` [kv_rank] (an RMS-normed projection of its input) and one rotated
key part ``k_r`` [rot_dim] that all heads share. Head a has the query ``[q_a | q_rot_a]`` ([dim | rot_dim], the
second part rotated by position), the key ``[W_uk_a c | k_r]`` and the value ``W_uv_a c``; scores are causal,
softmaxed, and the head's output may be gated by ``sigmoid(W_g h)_a`` before the output projection.

The keys and values are never formed. With ``q~_a = W_uk_a^T q_a`` the score is ``(q~_a . c + q_rot_a . k_r) * scale``
and the output ``W_uv_a (sum_j p_j c_j)``: attention runs on the cached vectors themselves, with one key/value
"head" of width kv_rank + rot_dim for all query heads, in prompts and in decoding alike. Steps:

    one product     [W_q ; W_dkv ; W_g] h                          (``ops.linear``)
    latent_prepare  norm of the latent, rotations, cache write     (one kernel)
    head_gemm       q~ = W_uk^T q per head                         (one kernel)
    attention       over the latent pages                          (tensor cores in bfloat16 where rank and rot_dim
                                                                    are multiples of 16; the exact kernel otherwise
                                                                    and for the whole 32-bit path)
    head_gemm       W_uv per head, times the gate                  (one kernel)
    output product  W_o                                            (left to the residual stream)

Other forms, chosen by spec params: ``q_rank`` r > 0 sends the queries through a latent of their own,
``q = W_uq rms_norm(W_dq h)`` (tensors ``dq`` [r, hidden], ``dq.norm`` [r], ``uq`` in place of ``q``; the norm uses
``latent_eps``): W_dq joins the fused product, one kernel norms its columns and a second product makes the queries.
``sinks``: a tensor ``sink`` [heads]; exp(sink_a) joins the denominator of head a's softmax (no key, no value).
``output_gate`` ``full``: ``g`` is [heads * value_dim, hidden] and gates every output entry (the default form is one gate a
head). ``pairing`` ``halves``: rotated entry i turns with entry i + dims / 2 (the kernels turn neighbours (2i, 2i + 1)): the
rotated rows of the query and key projections are laid out pair by pair at load, which leaves every score as it is, and
``named_tensors`` gives the stored order back.

A layer with ``own_latent`` False has no W_dkv: its run is scheduled on another layer's cache slot without writing
it, and reads what that layer stored (latent after the norm, key part after the rotation).

Spec: ``num_heads``, ``head_dim`` (the unrotated query/key width), ``scale``, ``position`` (a rotary table; its
``head_dim`` is the number of rotated entries, pairs (2i, 2i+1)), params ``rot_dim``, ``value_dim``, ``kv_rank``,
``latent_eps``, ``own_latent``, ``output_gate``, ``q_rank``, ``sinks``, ``pairing``. Tensors under the prefix: ``q`` (or ``dq``,
``dq.norm``, ``uq``), ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``g``, ``sink``, ``o``.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheRequest, Mixer, Projection, TensorDecl, build_part, register_part


class LatentAttention(Mixer):
    lazy_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s, p = spec, dict(spec.params)
        self.hidden, self.heads, self.dim = int(s.hidden), int(s.num_heads), int(s.head_dim)
        self.rot, self.vdim, self.rank = int(p["rot_dim"]), int(p["value_dim"]), int(p["kv_rank"])
        self.eps = float(p.get("latent_eps", 0.0))
        self.own_latent = bool(p.get("own_latent", True))
        self.gated = bool(p.get("output_gate", False))
        self.full_gate = p.get("output_gate") == "full"
        self.q_rank = int(p.get("q_rank", 0))
        self.has_sinks = bool(p.get("sinks", False))
        self.halves = p.get("pairing", "neighbours") == "halves"
        if p.get("pairing", "neighbours") not in ("neighbours", "halves") or self.q_rank < 0:
            raise ValueError("latent attention: `pairing` is neighbours or halves, `q_rank` not negative")
        self.scale = float(s.scale)
        if min(self.heads, self.dim, self.vdim, self.rank) <= 0 or self.rot <= 0:
            raise ValueError("latent attention needs positive heads, dim, rot_dim, value_dim and kv_rank")
        if self.rank > 512:
            raise ValueError(f"kv_rank {self.rank} is not supported by the latent attention kernel (up to 512 is)")
        self.position = build_part("position", s.position, runtime)
        self.rot_dims = int(s.position.head_dim)
        if self.rot_dims > self.rot or self.rot_dims % 2:
            raise ValueError(f"{self.rot_dims} rotated entries do not fit a rotated part of {self.rot}")
        self.q_dim = self.heads * (self.dim + self.rot)
        self.q_cols = self.q_rank if self.q_rank else self.q_dim        # what the fused product makes of the queries
        self.kv_dim = self.rank + self.rot if self.own_latent else 0
        self.g_dim = (self.heads * self.vdim if self.full_gate else self.heads) if self.gated else 0
        # columns of the fused product, each block starting at a multiple of 8 so that rows of 16-bit numbers stay
        # 16-byte aligned inside it
        self.q_off = 0
        self.kv_off = -(-self.q_cols // 8) * 8
        self.g_off = self.kv_off + -(-self.kv_dim // 8) * 8
        self.proj_dim = -(-(self.g_off + self.g_dim) // 8) * 8
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.latent_w = self.w_uq = self.q_norm_w = self.sinks = None
        # rotated entries in the order the kernels pair them: new entry 2i is old entry i, new entry 2i + 1 old entry i + dims / 2
        half = self.rot_dims // 2
        order = [j for i in range(half) for j in (i, i + half)] + list(range(self.rot_dims, self.rot))
        self.rot_order = torch.tensor(order, dtype=torch.long) if self.halves else None
        self._fast = ops.latent_tc_supported(runtime.dtype, self.heads, self.rank, self.rot)

    # ----------------------------------------------------------------- weights
    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        d = {self._n("uk"): TensorDecl((self.heads * self.dim, self.rank)),
             self._n("uv"): TensorDecl((self.heads * self.vdim, self.rank)), self._n("o"): TensorDecl((self.hidden, self.heads * self.vdim))}
        if self.q_rank:
            d[self._n("dq")] = TensorDecl((self.q_rank, self.hidden))
            d[self._n("dq.norm")] = TensorDecl((self.q_rank,), "vector")
            d[self._n("uq")] = TensorDecl((self.q_dim, self.q_rank))
        else:
            d[self._n("q")] = TensorDecl((self.q_dim, self.hidden))
        if self.own_latent:
            d[self._n("dkv")] = TensorDecl((self.rank + self.rot, self.hidden))
            d[self._n("dkv.norm")] = TensorDecl((self.rank,), "vector")
        if self.gated:
            d[self._n("g")] = TensorDecl((self.g_dim, self.hidden))
        if self.has_sinks:
            d[self._n("sink")] = TensorDecl((self.heads,), "vector")
        d.update(self.position.declare())
        return d

    def _pair_rows(self, t, first: int, blocks: int, stride: int, inverse: bool = False):
        """Rows ``first + b * stride .. + rot`` of ``t`` for b < blocks (the rotated parts) in the kernels' order of pairs."""
        if self.rot_order is None:
            return t
        order = torch.argsort(self.rot_order) if inverse else self.rot_order
        t = t.clone()
        for b in range(blocks):
            at = first + b * stride
            t[at:at + self.rot] = t[at:at + self.rot].index_select(0, order.to(t.device))
        return t

    def bind(self, weights):
        q = self._pair_rows(weights[self._n("uq" if self.q_rank else "q")], self.dim, self.heads, self.dim + self.rot)
        w = torch.zeros((self.proj_dim, self.hidden), dtype=q.dtype, device=q.device)
        if self.q_rank:
            w[:self.q_rank] = weights[self._n("dq")]
            self.w_uq, self.q_norm_w = q.contiguous(), weights[self._n("dq.norm")]
        else:
            w[:self.q_dim] = q
        if self.own_latent:
            w[self.kv_off:self.kv_off + self.kv_dim] = self._pair_rows(weights[self._n("dkv")], self.rank, 1, 0)
            self.latent_w = weights[self._n("dkv.norm")]
        if self.gated:
            w[self.g_off:self.g_off + self.g_dim] = weights[self._n("g")]
        if self.has_sinks:
            self.sinks = weights[self._n("sink")]
        self.w_in = w
        self.w_uk, self.w_uv, self.w_o = weights[self._n("uk")], weights[self._n("uv")], weights[self._n("o")]
        self.position.bind(weights)

    def named_tensors(self):
        out = {self._n("uk"): self.w_uk, self._n("uv"): self.w_uv, self._n("o"): self.w_o}
        if self.q_rank:
            out[self._n("dq")], out[self._n("dq.norm")] = self.w_in[:self.q_rank], self.q_norm_w
            out[self._n("uq")] = self._pair_rows(self.w_uq, self.dim, self.heads, self.dim + self.rot, inverse=True)
        else:
            out[self._n("q")] = self._pair_rows(self.w_in[:self.q_dim], self.dim, self.heads, self.dim + self.rot, inverse=True)
        if self.own_latent:
            out[self._n("dkv")] = self._pair_rows(self.w_in[self.kv_off:self.kv_off + self.kv_dim], self.rank, 1, 0, inverse=True)
            out[self._n("dkv.norm")] = self.latent_w
        if self.gated:
            out[self._n("g")] = self.w_in[self.g_off:self.g_off + self.g_dim]
        if self.has_sinks:
            out[self._n("sink")] = self.sinks
        out.update(self.position.named_tensors())
        return out

    # ------------------------------------------------------------------- cache
    def cache_request(self):
        return CacheRequest(tensors=(("latent", 1, self.rank), ("key_rot", 1, self.rot)))

    # ----------------------------------------------------------------- forward
    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens = x.shape[0]
        if self.own_latent != bool(cache.writes):
            raise ValueError("a latent attention layer writes the cache exactly when it has a latent projection of its own")
        proj = self.rt.buffer("latent_proj", tokens, self.proj_dim)
        ops.linear(x, self.w_in, proj)
        width = self.rank + self.rot
        qa = self.rt.buffer("latent_q", tokens, self.heads * width)
        latent, key_rot = cache.tensors["latent"], cache.tensors["key_rot"]
        cos, sin = self.position.tables()
        seq, pos = ctx.seq_of_token[:tokens], ctx.positions[:tokens]
        q, q_ld, q_off = proj, self.proj_dim, self.q_off
        if self.q_rank:         # queries through their own latent: norm of its columns, then the second product
            q_latent = self.rt.buffer("latent_q_latent", tokens, self.q_rank)
            ops.rms_norm_cols(proj, 0, self.q_rank, self.q_norm_w, q_latent, self.eps)
            q, q_ld, q_off = self.rt.buffer("latent_q_full", tokens, self.q_dim), self.q_dim, 0
            ops.linear(q_latent, self.w_uq, q)
        ops.latent_prepare(proj, self.q_off, self.kv_off if self.own_latent else -1, qa, pos, seq,
                           ctx.slot_mapping[cache.group][:tokens] if cache.writes else None, cos, sin, self.latent_w, self.eps,
                           latent, key_rot, self.heads, self.dim, self.rot, self.rot_dims, self.rank, q=q if self.q_rank else None)
        # q~[t, a, :] = q[t, a, :dim] @ W_uk[a]          W_uk [heads * dim, rank]: B_a[k, n] = W_uk[a * dim + k, n]
        ops.head_gemm(q, q_ld, self.dim + self.rot, self.w_uk, self.dim * self.rank, self.rank, 1, qa, self.heads * width, width,
                      tokens, self.heads, self.rank, self.dim, a_off=q_off)
        mixed = self.rt.buffer("latent_mixed", tokens, self.heads * self.rank)
        self._attend(qa, mixed, latent, key_rot, ctx, cache, tokens)
        # o[t, a, :] = W_uv[a] mixed[t, a, :]            W_uv [heads * vdim, rank]: B_a[k, n] = W_uv[a * vdim + n, k]
        attn = self.rt.buffer("latent_out", tokens, self.heads * self.vdim)
        gate = proj if self.gated else None
        ops.head_gemm(mixed, self.heads * self.rank, self.rank, self.w_uv, self.vdim * self.rank, 1, self.rank, attn, self.heads * self.vdim,
                      self.vdim, tokens, self.heads, self.vdim, self.rank, gate=gate, ldg=self.proj_dim, gate_off=self.g_off,
                      gate_per_output=self.full_gate)
        if lazy_output:
            return Projection(attn, self.w_o)
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(attn, self.w_o, out)
        return out


    def _attend(self, qa, mixed, latent, key_rot, ctx, cache, tokens):
        table = ctx.block_table[cache.group]
        if not self._fast:
            # the exact kernel: the whole 32-bit path, and sizes the tensor-core kernel refuses
            ops.latent_attention(qa, mixed, latent, key_rot, table, ctx.seq_of_token[:tokens], ctx.positions[:tokens], self.heads, self.rank,
                                 self.rot, cache.page_size, self.scale, sinks=self.sinks)
            return
        geometry = (self.heads, self.rank, self.rot, cache.page_size, self.scale)
        split = min(ctx.decode_tail_start, tokens)          # portions before, single tokens after
        if split > 0:
            ops.latent_attention_tc(qa, mixed, None, latent, key_rot, table, ctx.q_start, ctx.q_len, ctx.ctx_len, ctx.seq_of_token, 0,
                                    ctx.decode_tail_seq, 0, split, max(ctx.max_q_len, 2), *geometry, sinks=self.sinks)
        if tokens > split:
            n = tokens - split
            # enough CTAs to fill the device, no split shorter than 128 keys
            tiles = n * -(-self.heads // 16)
            splits = max(1, min(-(-ctx.context_bound // 128), -(-296 // tiles), 64))
            per_split = -(-(-(-ctx.context_bound // splits)) // 64) * 64
            splits = max(1, -(-ctx.context_bound // per_split))
            partial = None
            if splits > 1:
                partial = self.rt.scratch("latent_splits", tokens * self.heads * splits * (self.rank + 2))
            ops.latent_attention_tc(qa, mixed, partial, latent, key_rot, table, ctx.q_start, ctx.q_len, ctx.ctx_len, ctx.seq_of_token,
                                    ctx.decode_tail_seq, n, split, n, 1, *geometry, splits=splits, keys_per_split=per_split, sinks=self.sinks)


register_part("mixer", "latent_attention", LatentAttention)
