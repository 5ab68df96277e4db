"""The matrix memory of xLSTM (mLSTM; Beck et al., "xLSTM: Extended Long Short-Term Memory") as a mixer
(``csrc/kernels/mlstm.cu``).

From the layer's input h: ``q = W_q h * dim^-1/2``, ``k = W_k h`` ([heads, dim]) and ``v = W_v h`` ([heads, vdim]); per head a
log input gate ``li = c tanh((W_i h + b_i) / c)`` and a log forget gate ``lf = logsigmoid(c tanh((W_f h + b_f) / c))`` with the
cap ``c`` (``gate_cap``). Per head, with S [dim, vdim], n [dim] and a running maximum m, all from zero:

    m' = max(lf + m, li);  S' = exp(lf + m - m') S + exp(li - m') k v^T;  n' likewise with k alone
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

Each head's o is divided by its root mean square (``norm_eps``); the heads side by side are multiplied by a weight
(``norm`` [heads * vdim]) and by ``sigmoid(W_g h)``, then projected out. Everything after the projections is float32; the
gates' projections leave their product as float32 sums.

Steps: one product for ``[W_q; W_k; W_v; W_g] h``, one for the gates with float32 output, the scan (S, n and m live in the
request's state row, which the cache manager hands out and the model clears when a request starts), ``head_norm_gate``, and
the output product (left to the residual stream where it can fold it). Tensors under the prefix: ``q, k, v, g, o, norm, i,
i.b, f, f.b``.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .runtime import sequence_slots
from .base import Mixer, Projection, StateRequest, TensorDecl, register_part


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class MatrixLstmMixer(Mixer):
    lazy_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = dict(spec.params)
        self.hidden, self.H, self.D = int(spec.hidden), int(spec.num_heads), int(spec.head_dim)
        self.DV, self.cap = int(p["value_dim"]), float(p["gate_cap"])
        self.norm_eps = float(p.get("norm_eps", 0.0))
        if min(self.H, self.D, self.DV) <= 0 or not self.cap > 0:
            raise ValueError("the matrix LSTM needs positive heads, dim and vdim and a positive gate_cap")
        if self.D > 256:
            raise ValueError(f"dim {self.D} is not supported by the recurrence kernel (up to 256 is)")
        self.HD, self.HV = self.H * self.D, self.H * self.DV
        # columns of the first product, every block on a multiple of 8: q, k, v, the output gate
        self.k_off = _pad8(self.HD)
        self.v_off = self.k_off + _pad8(self.HD)
        self.g_off = self.v_off + _pad8(self.HV)
        self.c_in = self.g_off + _pad8(self.HV)
        self.gate_cols = _pad8(2 * self.H)
        self.w_in = self.w_gates = self.w_o = self.norm_w = self.bias_i = self.bias_f = None

    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        h = self.hidden
        return {self._n("q"): TensorDecl((self.HD, h)), self._n("k"): TensorDecl((self.HD, h)), self._n("v"): TensorDecl((self.HV, h)),
                self._n("g"): TensorDecl((self.HV, h)), self._n("o"): TensorDecl((h, self.HV)), self._n("norm"): TensorDecl((self.HV,), "vector"),
                self._n("i"): TensorDecl((self.H, h)), self._n("i.b"): TensorDecl((self.H,), "vector"),
                self._n("f"): TensorDecl((self.H, h)), self._n("f.b"): TensorDecl((self.H,), "vector")}

    def bind(self, weights):
        g = lambda short: weights[self._n(short)]
        q = g("q")
        w = torch.zeros((self.c_in, self.hidden), dtype=q.dtype, device=q.device)
        w[:self.HD], w[self.k_off:self.k_off + self.HD] = q, g("k")
        w[self.v_off:self.v_off + self.HV], w[self.g_off:self.g_off + self.HV] = g("v"), g("g")
        self.w_in = w
        gates = torch.zeros((self.gate_cols, self.hidden), dtype=q.dtype, device=q.device)
        gates[:self.H], gates[self.H:2 * self.H] = g("i"), g("f")
        self.w_gates = gates
        self.bias_i, self.bias_f, self.norm_w, self.w_o = g("i.b"), g("f.b"), g("norm"), g("o")

    def named_tensors(self):
        HD, HV, H = self.HD, self.HV, self.H
        return {self._n("q"): self.w_in[:HD], self._n("k"): self.w_in[self.k_off:self.k_off + HD],
                self._n("v"): self.w_in[self.v_off:self.v_off + HV], self._n("g"): self.w_in[self.g_off:self.g_off + HV],
                self._n("o"): self.w_o, self._n("norm"): self.norm_w, self._n("i"): self.w_gates[:H], self._n("i.b"): self.bias_i,
                self._n("f"): self.w_gates[H:2 * H], self._n("f.b"): self.bias_f}

    def state_request(self):
        return StateRequest((ops.mlstm_state_floats(self.H, self.D, self.DV),), torch.float32)

    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens, f32 = x.shape[0], torch.float32
        proj = self.rt.buffer("mlstm_proj", tokens, self.c_in)
        ops.linear(x, self.w_in, proj)
        gates = self.rt.buffer("mlstm_gates", tokens, self.gate_cols, f32)
        ops.linear(x, self.w_gates, gates)                  # float32 sums: what enters the recurrence is never rounded to 16 bits
        o = self.rt.buffer("mlstm_o", tokens, self.HV, f32)
        ops.mlstm_scan(proj, 0, self.k_off, self.v_off, gates, self.bias_i, self.bias_f, self.cap, self.D ** -0.5, o, cache.state,
                       ctx.q_start, ctx.q_len, ctx.state_slot, sequence_slots(ctx), self.H, self.D, self.DV)
        mixed = self.rt.buffer("mlstm_mixed", tokens, self.HV)
        ops.head_norm_gate(o, self.norm_w, True, proj, "sigmoid_compute", mixed, self.H, self.DV, self.norm_eps, gate_off=self.g_off)
        if lazy_output:
            return Projection(mixed, self.w_o)
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(mixed, self.w_o, out)
        return out


register_part("mixer", "mlstm", MatrixLstmMixer)
