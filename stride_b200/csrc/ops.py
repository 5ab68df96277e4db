"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, contiguity, sizes) and calls
one ``extern "C"`` launcher through ctypes on the current torch stream. There is
no CPU path and no fallback: a tensor that is not on a CUDA device, a missing
compiler or a size that a kernel refuses raises an error.
"""

from __future__ import annotations

import ctypes
import os as _os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-1: "bad argument", -2: "size not supported by this kernel"}


class KernelError(RuntimeError):
    pass


_bound: dict[str, ctypes._CFuncPtr] = {}

_SIGNATURES = {
    # name: (library, argtypes)
    "stride_embed_gather": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_add_rmsnorm": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "stride_add_residual": ("elementwise", [c_void_p, c_void_p, c_longlong, c_int, c_void_p]),
    "stride_zero_fresh_state": ("elementwise", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "stride_rope_kv_write": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_silu_mul": ("elementwise", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_gemm_tc_gated": ("gemm_bf16_tc", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
                                              c_int, c_float, c_float, c_void_p]),
    "stride_gemm_nt_f32": ("gemm_f32", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_paged_attention_generic": ("attention_generic", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                             c_int, c_float, c_void_p, c_void_p, c_int, c_void_p]),
    "stride_gemm_tc_skinny": ("gemm_bf16_tc", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_longlong,
                                               c_void_p, c_int, c_void_p, c_void_p]),
    "stride_gemm_tc_clustered": ("gemm_bf16_tc", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_rows": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_rows_add": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_rows_gated": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float,
                                                  c_void_p, c_void_p]),
    "stride_gemm_rows_qkv_rope": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                     c_int, c_float, c_void_p, c_void_p]),
    "stride_gemm_rows_add_norm": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                                                     c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "stride_gemm_stream_bf16": ("gemm_bf16_stream", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_stream_qkv_rope": ("gemm_bf16_stream", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                         c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "stride_gemm_stream_add_norm": ("gemm_bf16_stream", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                                                         c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "stride_scale_rows": ("elementwise", [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p]),
    "stride_paged_decode_attention": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                           c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int,
                                                           c_float, c_int, c_int, c_void_p]),
    "stride_paged_decode_attention_tma": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                               c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                                               c_int, c_float, c_int, c_int, c_void_p, c_void_p]),
    "stride_paged_decode_attention_rules": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                                 c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                                                 c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "stride_paged_decode_attention_gated": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                                 c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                                                 c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "stride_paged_prefill_attention": ("attention_prefill", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                             c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "stride_paged_prefill_attention_tc": ("attention_prefill_tc", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                                   c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                                   c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "stride_sample_ranked": ("sampling_ranked", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_longlong, c_void_p]),
    "stride_sample_rows": ("sampling", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_longlong, c_void_p]),
    "stride_add_dyt": ("dynamic_tanh", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_void_p]),
    "stride_add_scaled": ("dynamic_tanh", [c_void_p, c_void_p, c_float, c_longlong, c_int, c_void_p]),
    "stride_token_side": ("token_side", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "stride_latent_prepare": ("latent_attention", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_void_p]),
    "stride_head_gemm": ("latent_attention", [c_void_p, c_int, c_int, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_latent_attention": ("latent_attention", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                                     c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "stride_latent_attention_tc": ("latent_attention_tc", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                           c_float, c_int, c_int, c_void_p, c_void_p]),
    "stride_side_gate": ("token_side", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "stride_side_norm_add": ("token_side", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "stride_cast_rows": ("token_side", [c_void_p, c_void_p, c_longlong, c_int, c_void_p]),
    "stride_moe_select": ("moe", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "stride_rglru_conv": ("rglru", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_void_p]),
    "stride_rglru_gates": ("rglru", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                     c_int, c_int, c_void_p]),
    "stride_rglru_scan": ("rglru", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_rglru_scan_pieces": ("rglru", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_moe_route": ("moe", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_moe_plan": ("moe", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "stride_grouped_gemm": ("moe", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                    c_float, c_int, c_void_p]),
    "stride_grouped_gemm_tc5": ("moe_tc", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                           c_float, c_int, c_void_p, c_void_p]),
    "stride_gather_rows": ("moe_tc", [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p]),
    "stride_moe_combine": ("moe", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_relu_squared": ("moe", [c_void_p, c_longlong, c_int, c_void_p]),
    "stride_gated_act": ("pointwise", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "stride_head_gate": ("pointwise", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_add_sinusoid": ("pointwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "stride_norm_add": ("unit_norm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p, c_float,
                                      c_void_p, c_int, c_void_p]),
    "stride_qkv_unit_norm": ("unit_norm", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_float, c_int, c_int, c_int, c_void_p]),
    "stride_moe_select_sigmoid": ("moe", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                          c_void_p]),
    "stride_moe_select_groups": ("moe", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                         c_int, c_void_p]),
    "stride_stream_concat": ("pointwise", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "stride_add_row_vector": ("pointwise", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "stride_rms_norm_cols": ("unit_norm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "stride_conv_head_norm": ("short_conv", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_conv_tail": ("short_conv", [c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_void_p]),
    "stride_mlstm_scan": ("mlstm", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p,
                                    c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_pointwise": ("pointwise", [c_void_p, c_void_p, c_int, c_float, c_longlong, c_int, c_void_p]),
    "stride_weighted_sum": ("pointwise", [c_void_p, c_void_p, c_float, c_void_p, c_float, c_longlong, c_int, c_void_p]),
    "stride_delta_prepare": ("linear_recurrence", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong,
                                                   c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "stride_delta_scan": ("linear_recurrence", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p,
                                                c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_int, c_int, c_void_p, c_void_p]),
    "stride_bonus_scan": ("linear_recurrence", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_shift_mix": ("linear_recurrence", [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_head_norm_gate": ("linear_recurrence", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                                                    c_float, c_int, c_void_p]),
}


def _fn(name: str, what: str | None = None):
    f = _bound.get(name)
    if f is None:
        library, argtypes = _SIGNATURES[name]
        f = getattr(build.load_kernel_library(library), name)
        f.argtypes = argtypes
        f.restype = c_int
        _bound[name] = f
    if _timer is not None:
        return _timer.timed(what or _CLASS_OF.get(name, name), f)
    return f


# ---------------------------------------------------------------- time per class of kernel
# What a launcher counts as when the time of a step is split up. Matrix products say more (their shape) at the call.
_CLASS_OF = {
    "stride_embed_gather": "embedding", "stride_add_rmsnorm": "norm", "stride_add_residual": "residual sum",
    "stride_scale_rows": "norm", "stride_zero_fresh_state": "state slots", "stride_rope_kv_write": "rotation + cache write",
    "stride_silu_mul": "silu * up", "stride_paged_attention_generic": "attention (exact kernel)",
    "stride_paged_decode_attention_tma": "attention (decode)", "stride_paged_decode_attention_rules": "attention (decode)", "stride_paged_decode_attention_gated": "attention (decode)", "stride_paged_prefill_attention": "attention (prefill, mma.sync)",
    "stride_paged_prefill_attention_tc": "attention (prefill, tcgen05)", "stride_sample_rows": "sampling", "stride_sample_ranked": "sampling",
    "stride_add_dyt": "norm", "stride_add_scaled": "residual sum", "stride_token_side": "token side input",
    "stride_latent_prepare": "latent norm + rotation + cache write", "stride_head_gemm": "per-head product",
    "stride_latent_attention": "attention (latent, exact kernel)", "stride_latent_attention_tc": "attention (latent, tensor cores)",
    "stride_side_gate": "token side input", "stride_side_norm_add": "token side input", "stride_cast_rows": "token side input",
    "stride_moe_select": "router", "stride_moe_select_sigmoid": "router", "stride_moe_select_groups": "router", "stride_head_gate": "gates and caps",
    "stride_add_sinusoid": "embedding", "stride_norm_add": "norm", "stride_qkv_unit_norm": "head norms + cache write",
    "stride_rglru_conv": "recurrent block: convolution",
    "stride_rglru_gates": "recurrent block: gates", "stride_rglru_scan": "recurrent block: recurrence", "stride_rglru_scan_pieces": "recurrent block: recurrence", "stride_moe_route": "router",
    "stride_moe_plan": "router", "stride_grouped_gemm": "expert products", "stride_moe_combine": "expert sum",
    "stride_grouped_gemm_tc5": "expert products (tcgen05)", "stride_gather_rows": "expert rows gathered",
    "stride_relu_squared": "relu^2", "stride_gated_act": "act * up", "stride_pointwise": "gates and caps", "stride_weighted_sum": "sum of branches",
    "stride_delta_prepare": "delta rule: convolution, unit vectors, decay", "stride_delta_scan": "delta rule: recurrence",
    "stride_bonus_scan": "decayed memory: recurrence", "stride_shift_mix": "decayed memory: token shift",
    "stride_head_norm_gate": "per-head norm and gate",
    "stride_stream_concat": "repeated block: input", "stride_add_row_vector": "repeated block: input",
    "stride_rms_norm_cols": "latent norm", "stride_conv_head_norm": "convolution + head norms + cache write",
    "stride_conv_tail": "convolution + head norms + cache write", "stride_mlstm_scan": "matrix LSTM: recurrence",
}


class KernelTimer:
    """Device time per class of kernel inside a step, from CUDA events around every launch (the reference records
    one duration per pass, python/stride_worker/model.py:238-240,343-345; this splits it up). Use::

        with ops.KernelTimer() as timer:
            model.forward(ctx)              # eagerly: a captured graph has no place for events
        timer.milliseconds()                # {"attention (decode)": 1.52, "product 6144x4096 (qkv + rotation)": 1.18, ...}

    The events stand between the kernels, so launches do not overlap their predecessors' tails as they do in a
    real step: the classes' shares are right, their sum is somewhat above the step's own time."""

    def __init__(self):
        self.spans: list = []       # (class, start event, end event)

    def __enter__(self):
        global _timer
        if _timer is not None:
            raise KernelError("a KernelTimer is active already")
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None

    def timed(self, what: str, call):
        def run(*args):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = call(*args)
            end.record()
            self.spans.append((what, start, end))
            return code
        return run

    def milliseconds(self) -> dict:
        """Synchronises; class -> summed device time, largest first."""
        torch.cuda.synchronize()
        out: dict = {}
        for what, start, end in self.spans:
            out[what] = out.get(what, 0.0) + start.elapsed_time(end)
        return dict(sorted(out.items(), key=lambda kv: -kv[1]))


_timer: KernelTimer | None = None


# How many of the package's own kernels were launched (library matrix products
# are not counted). A captured graph counts its launches once, at capture.
counters = {"launches": 0}


def _check(code: int, name: str) -> None:
    if code == 0:
        counters["launches"] += 1
        return
    if code in _ERRORS:
        raise KernelError(f"{name}: {_ERRORS[code]}")
    raise KernelError(f"{name}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle. Asked for on every launch, so through the one C call when torch has it
    (``torch.cuda.current_stream()`` builds a Python object every time)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device; stride_b200 has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t, name: str, dtype=None) -> int | None:
    return None if t is None else _dev(t, name, dtype)


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)") from None


def require_device() -> None:
    """Fails loudly when the product path cannot run."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: stride_b200 runs its models on the GPU only")


# ------------------------------------------------------------------ elementwise
def embed_gather(ids, seq_of_token, table, out) -> None:
    tokens, hidden = out.shape
    _check(_fn("stride_embed_gather")(_dev(ids, "ids", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
                                      _dev(table, "table"), _dev(out, "out", torch.float32), tokens, hidden,
                                      table.shape[0], _code(table.dtype), _stream()), "embed_gather")


def add_rmsnorm(residual, delta, weight, out, eps: float, rows=None) -> None:
    """``x = residual (+ delta)``; writes x back to ``residual`` (unless ``rows``
    selects source rows) and ``rmsnorm(x) * weight`` to ``out``."""
    num_rows, hidden = out.shape
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("delta and out must have the same element type")
    _check(_fn("stride_add_rmsnorm")(_dev(residual, "residual", torch.float32), _opt(delta, "delta"),
                                     _dev(weight, "weight", torch.float32), _dev(out, "out"),
                                     _opt(rows, "rows", torch.int32), num_rows, hidden, float(eps), _code(out.dtype),
                                     _stream()), "add_rmsnorm")


def add_residual(residual, delta) -> None:
    _check(_fn("stride_add_residual")(_dev(residual, "residual", torch.float32), _dev(delta, "delta"), delta.numel(),
                                      _code(delta.dtype), _stream()), "add_residual")


def zero_fresh_state(state, state_slot, q_start, q_len, positions) -> None:
    """Clears ``state[slot]`` for every sequence of the step whose first token sits at position 0 (``state``:
    [num_slots, ...] of a 4-byte element type; the index arrays are the step's, at their layout's capacity)."""
    if state.element_size() != 4:
        raise KernelError("state rows must have a 4-byte element type")
    row_bytes = (state.numel() // state.shape[0]) * 4
    _check(_fn("stride_zero_fresh_state")(_dev(state, "state"), row_bytes, state.shape[0], _dev(state_slot, "state_slot", torch.int32),
                                          _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32),
                                          _dev(positions, "positions", torch.int32), q_len.shape[0], _stream()), "zero_fresh_state")


def rope_kv_write(qkv, bias, positions, slot_mapping, cos, sin, k_pages, v_pages, nq: int, nkv: int, hd: int,
                  page_size: int, rotate: bool = True) -> None:
    tokens = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * hd:
        raise KernelError("qkv has the wrong width")
    if k_pages.dtype != qkv.dtype or v_pages.dtype != qkv.dtype:
        raise KernelError("cache pages and activations must have the same element type")
    _check(_fn("stride_rope_kv_write")(_dev(qkv, "qkv"), _opt(bias, "bias", torch.float32),
                                       _dev(positions, "positions", torch.int32),
                                       _opt(slot_mapping, "slot_mapping", torch.int32), _dev(cos, "cos", torch.float32),
                                       _dev(sin, "sin", torch.float32), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
                                       tokens, nq, nkv, hd, page_size, int(rotate), _code(qkv.dtype), _stream()),
           "rope_kv_write")


def silu_mul(inp, out, block: int | None = None) -> None:
    """``out = silu(gate) * up`` for ``inp`` = [tokens, 2 * inter] whose gate and up columns alternate in
    blocks of ``block`` columns (default: all gate columns, then all up columns)."""
    tokens, inter = out.shape
    if inp.shape != (tokens, 2 * inter) or inp.dtype != out.dtype:
        raise KernelError("silu_mul wants [tokens, 2*inter] in and [tokens, inter] out of one element type")
    _check(_fn("stride_silu_mul")(_dev(inp, "in"), _dev(out, "out"), tokens, inter, inter if block is None else int(block),
                                  _code(out.dtype), _stream()), "silu_mul")


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}
EPILOGUE_ACTIVATIONS = ("silu", "gelu_tanh", "swish_clamped")      # what the tcgen05 gate/up product applies in its own epilogue


def gated_act(inp, out, block: int | None = None, activation: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> None:
    """``silu_mul`` for any activation of ``ACTIVATIONS``: ``out = act(gate) * up``, same layout of ``inp``.
    ``swish_clamped`` is ``g' sigmoid(alpha g') (u' + 1)`` with ``g' = min(gate, limit)`` and ``u' = clamp(up, -limit, limit)``."""
    tokens, inter = out.shape
    if inp.shape != (tokens, 2 * inter) or inp.dtype != out.dtype:
        raise KernelError("gated_act wants [tokens, 2*inter] in and [tokens, inter] out of one element type")
    _check(_fn("stride_gated_act")(_dev(inp, "in"), _dev(out, "out"), tokens, inter, inter if block is None else int(block),
                                   ACTIVATIONS[activation], float(limit), float(alpha), _code(out.dtype), _stream()), "gated_act")


def head_gate(x, gates, gate_stride: int, heads: int, width: int) -> None:
    """``x[t, h, :] *= sigmoid(gates[t * gate_stride + h])`` for ``x`` [tokens, heads * width]; ``gates`` may be a column
    block of a wider buffer of the same element type."""
    if x.shape[1] != heads * width or gates.dtype != x.dtype:
        raise KernelError("head_gate: x must be [tokens, heads * width] and the gates of its element type")
    if not gates.is_cuda:
        raise KernelError("gates must live on a CUDA device; stride_b200 has no CPU path")
    _check(_fn("stride_head_gate")(_dev(x, "x"), gates.data_ptr(), int(gate_stride), x.shape[0], heads, width, _code(x.dtype), _stream()),
           "head_gate")


def add_sinusoid(x, copy, positions, seq_of_token, freq) -> None:
    """``x[t, 2i] += sin(p_t freq[i])``, ``x[t, 2i + 1] += cos(p_t freq[i])`` for the float32 rows ``x``; angles in float64
    (``freq`` float64 [ceil(width / 2)]). ``copy`` (or None) receives the sums in its own element type."""
    tokens, width = x.shape
    if freq.dtype != torch.float64 or freq.numel() < (width + 1) // 2:
        raise KernelError("add_sinusoid: freq must be float64 with one entry per pair of columns")
    _check(_fn("stride_add_sinusoid")(_dev(x, "x", torch.float32), _opt(copy, "copy"), _dev(positions, "positions", torch.int32),
                                      _opt(seq_of_token, "seq_of_token", torch.int32), _dev(freq, "freq", torch.float64), tokens, width,
                                      _code(copy.dtype if copy is not None else torch.float32), _stream()), "add_sinusoid")


def norm_add(residual, delta, bias, weight, copy, eps: float, mult: float, next_weight=None, next_eps: float = 0.0, next_out=None) -> None:
    """``residual += mult * weight * y / sqrt(mean(y^2) + eps)`` with ``y = delta (+ bias)`` per row, in float32; ``copy`` (or
    None) receives the new rows in the compute dtype. ``delta`` None: only the copy is made. With ``next_weight`` and
    ``next_out`` (``delta``'s type) the kernel also leaves the RMS norm of the new rows with that weight and ``next_eps``: the
    norm in front of the next sublayer."""
    tokens, hidden = residual.shape
    kind = delta if delta is not None else copy
    if kind is None:
        return
    if delta is not None and copy is not None and delta.dtype != copy.dtype:
        raise KernelError("norm_add: delta and copy must have one element type")
    if next_out is not None and (delta is None or next_out.dtype != delta.dtype or next_out.shape != residual.shape):
        raise KernelError("norm_add: the next norm's output must have the delta's element type and the stream's shape")
    _check(_fn("stride_norm_add")(_dev(residual, "residual", torch.float32), _opt(delta, "delta"), _opt(bias, "bias", torch.float32),
                                  _opt(weight, "weight", torch.float32), _opt(copy, "copy"), tokens, hidden, float(eps), float(mult),
                                  _opt(next_weight, "next_weight", torch.float32), float(next_eps), _opt(next_out, "next_out"),
                                  _code(kind.dtype), _stream()), "norm_add")


def qkv_unit_norm(qkv, bias, slot_mapping, k_pages, v_pages, nq: int, nkv: int, hd: int, vd: int, page_size: int, eps: float,
                  norm_qk: bool = True, norm_v: bool = True) -> None:
    """For the fused projection ``qkv`` [tokens, >= (nq + nkv) * hd + nkv * vd] (query heads, key heads, value heads, then
    whatever else): adds ``bias``, divides every query and key head (and every value head) by its root mean square, in
    place, and with ``slot_mapping`` writes keys and values into the pages. ``nkv`` 0: queries only."""
    _check(_fn("stride_qkv_unit_norm")(_dev(qkv, "qkv"), qkv.shape[1], _opt(bias, "bias", torch.float32),
                                       _opt(slot_mapping, "slot_mapping", torch.int32), _opt(k_pages, "k_pages", qkv.dtype),
                                       _opt(v_pages, "v_pages", qkv.dtype), qkv.shape[0], nq, nkv, hd, vd, page_size, float(eps),
                                       int(norm_qk), int(norm_v), _code(qkv.dtype), _stream()), "qkv_unit_norm")


def sigmoid_gate(x, gate) -> None:
    """``x *= sigmoid(gate)`` elementwise, in float32 arithmetic."""
    if gate.shape != x.shape or gate.dtype != x.dtype:
        raise KernelError("sigmoid_gate: x and gate must agree in shape and element type")
    _check(_fn("stride_pointwise")(_dev(x, "x"), _dev(gate, "gate"), 0, 0.0, x.numel(), _code(x.dtype), _stream()), "sigmoid_gate")


def softcap_(x, cap: float) -> None:
    """``x = cap * tanh(x / cap)`` in place."""
    _check(_fn("stride_pointwise")(_dev(x, "x"), None, 1, float(cap), x.numel(), _code(x.dtype), _stream()), "softcap")


def weighted_sum(out, a, sa: float, b, sb: float) -> None:
    """``out = sa * a + sb * b`` elementwise, formed in float32 and rounded once; ``out`` may be ``a`` or ``b``."""
    if not (out.shape == a.shape == b.shape and out.dtype == a.dtype == b.dtype):
        raise KernelError("weighted_sum: one shape and one element type for all three")
    _check(_fn("stride_weighted_sum")(_dev(out, "out"), _dev(a, "a"), float(sa), _dev(b, "b"), float(sb), out.numel(), _code(out.dtype),
                                      _stream()), "weighted_sum")


def tanh_(x) -> None:
    _check(_fn("stride_pointwise")(_dev(x, "x"), None, 2, 0.0, x.numel(), _code(x.dtype), _stream()), "tanh")


# ------------------------------------------------------------ matrix memories (delta rule, decayed memory with a bonus)
MEMORY_PIECE = 64       # tokens a piece when a matrix memory runs its long portions in pieces
# The delta rule in pieces is off by default (0): a piece needs its D x D matrix besides its own sum, three passes over the
# tokens in all, and measured at 16 heads of 128 x 128 over 2,048 tokens that takes 1.94 ms against the chain's 0.91 ms.
# STRIDE_B200_DELTA_PIECES_MIN=256 switches it on for portions of that many tokens.
DELTA_PIECES_MIN_TOKENS = int(_os.environ.get("STRIDE_B200_DELTA_PIECES_MIN", "0"))

def delta_prepare(proj, conv_w, low, a_log, dt_bias, state, tail_off: int, seq_of_token, q_start, state_slot, qk, v, beta, decay,
                  G: int, H: int, D: int, DV: int, taps: int, unit_eps: float) -> None:
    """Per token of the step, from ``proj`` [tokens, >= 2GD + HV + H] (q, k, v, beta's projection) and ``low`` (float32,
    its first HD columns the decay's projection): convolution with SiLU, unit-length q and k, beta, and decay - 1, all
    float32. ``state`` [slots, n] float32 holds the convolution's tail [taps - 1, 2GD + HV] at ``tail_off``."""
    tokens = proj.shape[0]
    C = 2 * G * D + H * DV
    if proj.shape[1] < C + H or conv_w.shape != (C, taps) or low.shape[1] < H * D:
        raise KernelError("delta_prepare: shapes do not agree")
    _check(_fn("stride_delta_prepare")(
        _dev(proj, "proj"), proj.shape[1], _dev(conv_w, "conv_w", torch.float32), _dev(low, "low", torch.float32), low.shape[1],
        _dev(a_log, "a_log", torch.float32), _dev(dt_bias, "dt_bias", torch.float32), _dev(state, "state", torch.float32), state.shape[1],
        int(tail_off), _dev(seq_of_token, "seq_of_token", torch.int32), _dev(q_start, "q_start", torch.int32),
        _dev(state_slot, "state_slot", torch.int32), _dev(qk, "qk", torch.float32), _dev(v, "v", torch.float32),
        _dev(beta, "beta", torch.float32), _dev(decay, "decay", torch.float32), tokens, G, H, D, DV, taps, float(unit_eps),
        _code(proj.dtype), _stream()), "delta_prepare")


def delta_scan_scratch_floats(num_seqs: int, max_q_len: int, H: int, D: int, DV: int) -> int:
    return num_seqs * -(-max_q_len // MEMORY_PIECE) * H * D * (DV + D)


def delta_scan(qk, v, beta, decay, o, state, tail_off: int, proj, q_start, q_len, state_slot, num_seqs: int, G: int, H: int, D: int,
               DV: int, taps: int, max_q_len: int = 0, scratch=None) -> None:
    """The gated delta rule over every request of the step, in token order: ``o`` [tokens, H * DV] float32; S and the
    convolution's tail in ``state`` move on. With ``scratch`` (float32, ``delta_scan_scratch_floats`` for the step's longest
    portion ``max_q_len``) the portions run in pieces of ``MEMORY_PIECE`` tokens, parallel over the pieces."""
    piece = MEMORY_PIECE if scratch is not None else 0
    max_pieces = -(-max_q_len // MEMORY_PIECE) if piece else 0
    if piece and (max_pieces <= 0 or scratch.numel() < delta_scan_scratch_floats(num_seqs, max_q_len, H, D, DV)):
        raise KernelError("delta_scan: the scratch is too small")
    _check(_fn("stride_delta_scan")(
        _dev(qk, "qk", torch.float32), _dev(v, "v", torch.float32), _dev(beta, "beta", torch.float32), _dev(decay, "decay", torch.float32),
        _dev(o, "o", torch.float32), _dev(state, "state", torch.float32), state.shape[1], int(tail_off), _dev(proj, "proj"), proj.shape[1],
        _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32), _dev(state_slot, "state_slot", torch.int32), num_seqs,
        G, H, D, DV, taps, _code(proj.dtype), piece, max_pieces, _opt(scratch, "scratch", torch.float32), _stream()), "delta_scan")


def bonus_scan_scratch_floats(num_seqs: int, max_q_len: int, H: int, D: int) -> int:
    return num_seqs * -(-max_q_len // MEMORY_PIECE) * H * D * (D + 1)


def bonus_scan(r, k, v, wlog, w0, bonus, o, state, q_start, q_len, state_slot, num_seqs: int, H: int, D: int, max_q_len: int = 0,
               scratch=None) -> None:
    """Decayed memory with a bonus for the current token: ``o_t = (S + diag(bonus) k v^T)^T r``, then
    ``S = diag(exp(-exp(wlog + w0))) S + k v^T``; r, k, v [tokens, H * D] in one element type, the rest float32. With
    ``scratch`` (float32, ``bonus_scan_scratch_floats`` for the step's longest portion ``max_q_len``) the portions run in
    pieces of ``MEMORY_PIECE`` tokens, parallel over the pieces."""
    if not (r.dtype == k.dtype == v.dtype):
        raise KernelError("bonus_scan: r, k and v must have one element type")
    piece = MEMORY_PIECE if scratch is not None else 0
    max_pieces = -(-max_q_len // MEMORY_PIECE) if piece else 0
    if piece and (max_pieces <= 0 or scratch.numel() < bonus_scan_scratch_floats(num_seqs, max_q_len, H, D)):
        raise KernelError("bonus_scan: the scratch is too small")
    _check(_fn("stride_bonus_scan")(
        _dev(r, "r"), _dev(k, "k"), _dev(v, "v"), _dev(wlog, "wlog", torch.float32), _dev(w0, "w0", torch.float32),
        _dev(bonus, "bonus", torch.float32), _dev(o, "o", torch.float32), _dev(state, "state", torch.float32), state.shape[1],
        _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32), _dev(state_slot, "state_slot", torch.int32), num_seqs,
        H, D, _code(r.dtype), piece, max_pieces, _opt(scratch, "scratch", torch.float32), _stream()), "bonus_scan")


def shift_mix(x, mu, state, prev_off: int, seq_of_token, q_start, q_len, state_slot, out) -> None:
    """``out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s]`` with the request's last input before the step (``state`` at
    ``prev_off``) in front of its first token; the step's last input is stored there afterwards."""
    tokens, width = x.shape
    mixes = mu.shape[0]
    if out.shape != (mixes, tokens, width) or out.dtype != x.dtype or mu.shape[1] != width:
        raise KernelError("shift_mix: shapes do not agree")
    _check(_fn("stride_shift_mix")(
        _dev(x, "x"), _dev(mu, "mu", torch.float32), _dev(state, "state", torch.float32), state.shape[1], int(prev_off),
        _dev(seq_of_token, "seq_of_token", torch.int32), _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32),
        _dev(state_slot, "state_slot", torch.int32), _dev(out, "out"), tokens, width, mixes, _code(x.dtype), _stream()), "shift_mix")


def head_norm_gate(o, weight, per_head_weight: bool, gate, gate_kind: str, out, H: int, DV: int, eps: float, gate_off: int = 0) -> None:
    """``out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * gate`` per head. ``weight`` [DV] for all heads or
    [H * DV]; ``gate`` [tokens, >= gate_off + H * DV], read from column ``gate_off`` on: ``sigmoid`` of float32 values or
    ``silu`` of values in ``out``'s type."""
    tokens = o.shape[0]
    kind = {"sigmoid": 0, "silu": 1, "sigmoid_compute": 2}[gate_kind]      # the last: sigmoid of a gate in ``out``'s type
    _check(_fn("stride_head_norm_gate")(
        _dev(o, "o", torch.float32), _dev(weight, "weight", torch.float32), DV if per_head_weight else 0,
        _dev(gate, "gate", torch.float32 if kind == 0 else out.dtype) + gate_off * gate.element_size(), gate.shape[1], kind,
        _dev(out, "out"), tokens, H, DV, float(eps),
        _code(out.dtype), _stream()), "head_norm_gate")


def mlstm_state_floats(H: int, D: int, DV: int) -> int:
    return H * D * DV + H * D + H


def mlstm_scan(proj, q_off: int, k_off: int, v_off: int, gates, bias_i, bias_f, cap: float, q_scale: float, o, state, q_start, q_len,
               state_slot, num_seqs: int, H: int, D: int, DV: int) -> None:
    """The matrix memory with exponential gates over every request of the step, in token order. ``proj`` [tokens, ld] holds
    q, k ([H, D]) and v ([H, DV]) from the given columns on; ``gates`` (float32 [tokens, >= 2H]) the projections of the input
    gates (columns 0..H-1) and the forget gates (H..2H-1), to which ``bias_i`` / ``bias_f`` are added before
    ``cap * tanh(. / cap)``. ``o`` [tokens, H * DV] float32; ``state`` [slots, >= mlstm_state_floats]: S, n, m per head."""
    if state.shape[1] < mlstm_state_floats(H, D, DV) or o.shape[1] != H * DV or gates.shape[1] < 2 * H:
        raise KernelError("mlstm_scan: shapes do not agree")
    _check(_fn("stride_mlstm_scan")(
        _dev(proj, "proj"), proj.shape[1], int(q_off), int(k_off), int(v_off), _dev(gates, "gates", torch.float32), gates.shape[1],
        _dev(bias_i, "bias_i", torch.float32), _dev(bias_f, "bias_f", torch.float32), float(cap), float(q_scale),
        _dev(o, "o", torch.float32), _dev(state, "state", torch.float32), state.shape[1], _dev(q_start, "q_start", torch.int32),
        _dev(q_len, "q_len", torch.int32), _dev(state_slot, "state_slot", torch.int32), int(num_seqs), H, D, DV, _code(proj.dtype),
        _stream()), "mlstm_scan")


# ------------------------------------------------------------ short convolution with head norms
def conv_head_norm(raw, out, conv_w, state, tail_off: int, seq_of_token, q_start, state_slot, wq, wk, eps: float, slot_mapping, k_pages,
                   v_pages, nq: int, nkv: int, hd: int, vd: int, page_size: int) -> None:
    """From the fused projection ``raw`` [tokens, >= C] (query heads, key heads, value heads; C channels): the causal
    convolution ``conv_w`` (float32 [taps, C]: a tap's weights side by side; or None) over a request's projected rows, which before the step's first token
    come from the tail in ``state`` (float32 [slots, n], rows [taps - 1, C] at ``tail_off``); then the RMS norm of every query
    head with the weight ``wq`` and of every key head with ``wk`` (float32 [hd], or None for no norm); into ``out``, and with
    ``slot_mapping`` keys and values into their pages. The tail is not moved: ``conv_tail`` does that afterwards."""
    taps = 1 if conv_w is None else conv_w.shape[0]
    if out.dtype != raw.dtype or out.shape[0] != raw.shape[0]:
        raise KernelError("conv_head_norm: raw and out must agree in rows and element type")
    _check(_fn("stride_conv_head_norm")(
        _dev(raw, "raw"), raw.shape[1], _dev(out, "out"), out.shape[1], _opt(conv_w, "conv_w", torch.float32), taps,
        _opt(state, "state", torch.float32), 0 if state is None else state.shape[1], int(tail_off),
        _dev(seq_of_token, "seq_of_token", torch.int32), _dev(q_start, "q_start", torch.int32), _dev(state_slot, "state_slot", torch.int32),
        _opt(wq, "wq", torch.float32), _opt(wk, "wk", torch.float32), float(eps), _opt(slot_mapping, "slot_mapping", torch.int32),
        _opt(k_pages, "k_pages", raw.dtype), _opt(v_pages, "v_pages", raw.dtype), raw.shape[0], nq, nkv, hd, vd, page_size,
        _code(raw.dtype), _stream()), "conv_head_norm")


def conv_tail(raw, state, tail_off: int, q_start, q_len, state_slot, num_seqs: int, channels: int, taps: int) -> None:
    """Moves every request's convolution tail on by the step's rows of ``raw`` (its first ``channels`` columns)."""
    _check(_fn("stride_conv_tail")(
        _dev(raw, "raw"), raw.shape[1], _dev(state, "state", torch.float32), state.shape[1], int(tail_off),
        _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32), _dev(state_slot, "state_slot", torch.int32),
        int(num_seqs), int(channels), int(taps), _code(raw.dtype), _stream()), "conv_tail")


def rms_norm_cols(x, col_off: int, width: int, weight, out, eps: float) -> None:
    """``out[t] = y / sqrt(mean(y^2) + eps) * weight`` for ``y = x[t, col_off : col_off + width]``; ``out`` [tokens, >= width]."""
    if out.dtype != x.dtype or out.shape[0] != x.shape[0] or x.shape[1] < col_off + width or out.shape[1] < width or weight.numel() != width:
        raise KernelError("rms_norm_cols: shapes do not agree")
    _check(_fn("stride_rms_norm_cols")(_dev(x, "x") + int(col_off) * x.element_size(), x.shape[1], _dev(weight, "weight", torch.float32),
                                       _dev(out, "out"), out.shape[1], x.shape[0], int(width), float(eps), _code(x.dtype), _stream()),
           "rms_norm_cols")


def stream_concat(residual, second, out) -> None:
    """``out[t] = [residual[t] rounded to out's type | second[t]]`` ([tokens, 2 * hidden])."""
    tokens, hidden = residual.shape
    if second.shape != (tokens, hidden) or out.shape != (tokens, 2 * hidden) or second.dtype != out.dtype:
        raise KernelError("stream_concat: shapes or element types do not agree")
    _check(_fn("stride_stream_concat")(_dev(residual, "residual", torch.float32), _dev(second, "second"), _dev(out, "out"), tokens, hidden,
                                       _code(out.dtype), _stream()), "stream_concat")


def add_row_vector(residual, vector, seq_of_token=None) -> None:
    """``residual[t] += vector`` (float32) for every row that is not padding."""
    tokens, hidden = residual.shape
    if vector.numel() != hidden:
        raise KernelError("add_row_vector: the vector must have the rows' width")
    _check(_fn("stride_add_row_vector")(_dev(residual, "residual", torch.float32), _dev(vector, "vector", torch.float32),
                                        _opt(seq_of_token, "seq_of_token", torch.int32), tokens, hidden, _stream()), "add_row_vector")


# ------------------------------------------------------------ Dynamic Tanh, scaled sums
def add_dyt(residual, delta, scale: float, weight, bias, alpha: float, out, rows=None) -> None:
    """``x = residual (+ scale * delta)``; writes x back to ``residual`` (unless ``rows`` selects source rows) and
    ``tanh(alpha * x) * weight + bias`` to ``out``."""
    num_rows, hidden = out.shape
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("delta and out must have the same element type")
    _check(_fn("stride_add_dyt")(_dev(residual, "residual", torch.float32), _opt(delta, "delta"), float(scale),
                                 _dev(weight, "weight", torch.float32), _dev(bias, "bias", torch.float32), float(alpha), _dev(out, "out"),
                                 _opt(rows, "rows", torch.int32), num_rows, hidden, _code(out.dtype), _stream()), "add_dyt")


def add_scaled(residual, delta, scale: float) -> None:
    """``residual += scale * delta`` in float32."""
    _check(_fn("stride_add_scaled")(_dev(residual, "residual", torch.float32), _dev(delta, "delta"), float(scale), delta.numel(),
                                    _code(delta.dtype), _stream()), "add_scaled")


def token_side(residual, ids, seq_of_token, table, offset: int, w_gate, w_proj, norm_w, eps: float, scale: float) -> None:
    """``residual[t] += scale * unit_rms(w_proj (gelu_tanh(w_gate residual[t]) * table[ids[t], offset:offset+dim])) * norm_w``,
    in float32 on the stream itself, one CTA a token (the matrices are read once per token: for checks and small sizes;
    the part runs the two products as products). ``w_gate`` [dim, hidden], ``w_proj`` [hidden, dim]."""
    tokens, hidden = residual.shape
    dim = w_gate.shape[0]
    if w_gate.shape != (dim, hidden) or w_proj.shape != (hidden, dim) or table.dtype != w_gate.dtype or w_proj.dtype != w_gate.dtype:
        raise KernelError("token_side: the matrices do not fit the stream")
    _check(_fn("stride_token_side")(_dev(residual, "residual", torch.float32), _dev(ids, "ids", torch.int32),
                                    _opt(seq_of_token, "seq_of_token", torch.int32), _dev(table, "table"), table.shape[1], int(offset),
                                    table.shape[0], _dev(w_gate, "w_gate"), _dev(w_proj, "w_proj"), _dev(norm_w, "norm_w", torch.float32),
                                    tokens, hidden, dim, float(eps), float(scale), _code(w_gate.dtype), _stream()), "token_side")


def cast_rows(src, dst) -> None:
    """``dst = src`` (float32) rounded to ``dst``'s element type."""
    _check(_fn("stride_cast_rows")(_dev(src, "src", torch.float32), _dev(dst, "dst"), src.numel(), _code(dst.dtype), _stream()), "cast_rows")


def side_gate(pre, ids, seq_of_token, table, offset: int, out) -> None:
    """``out[t] = gelu_tanh(pre[t]) * table[ids[t], offset : offset + dim]`` (zeros for a padded row)."""
    tokens, dim = out.shape
    _check(_fn("stride_side_gate")(_dev(pre, "pre", out.dtype), _dev(ids, "ids", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
                                   _dev(table, "table", out.dtype), table.shape[1], int(offset), table.shape[0], _dev(out, "out"), tokens, dim,
                                   _code(out.dtype), _stream()), "side_gate")


def side_norm_add(residual, y, seq_of_token, norm_w, eps: float, scale: float) -> None:
    """``residual[t] += scale * y[t] / sqrt(mean(y[t]^2) + eps) * norm_w`` in float32; padded rows stay."""
    tokens, hidden = residual.shape
    _check(_fn("stride_side_norm_add")(_dev(residual, "residual", torch.float32), _dev(y, "y"), _opt(seq_of_token, "seq_of_token", torch.int32),
                                       _dev(norm_w, "norm_w", torch.float32), tokens, hidden, float(eps), float(scale), _code(y.dtype),
                                       _stream()), "side_norm_add")


# --------------------------------------------------------------- latent attention
def latent_prepare(proj, q_off: int, kv_off: int, qa, positions, seq_of_token, slot_mapping, cos, sin, latent_w, eps: float,
                   latent_pages, krot_pages, heads: int, dim: int, rot: int, rot_dims: int, rank: int, q=None) -> None:
    """From the projections of a step (``proj`` [tokens, ld]: queries at ``q_off``, the latent projection at ``kv_off``
    or ``kv_off`` < 0 for none): the rotated parts of the queries into ``qa`` [tokens, heads, rank + rot], and, when
    there is a latent projection and ``slot_mapping``, the normed latent and the rotated key part into their pages.
    ``q`` [tokens, >= heads * (dim + rot)]: the queries in a buffer of their own instead of ``proj``'s columns."""
    tokens = proj.shape[0]
    if qa.shape != (tokens, heads * (rank + rot)) or qa.dtype != proj.dtype:
        raise KernelError("latent_prepare: qa must be [tokens, heads * (rank + rot)] of the projections' type")
    if q is not None and (q.dtype != proj.dtype or q.shape[0] != tokens or q.shape[1] < heads * (dim + rot)):
        raise KernelError("latent_prepare: q must be [tokens, >= heads * (dim + rot)] of the projections' type")
    has_kv = kv_off >= 0
    q_ptr, ldq = (_dev(proj, "proj") + int(q_off) * proj.element_size(), proj.shape[1]) if q is None else (_dev(q, "q"), q.shape[1])
    _check(_fn("stride_latent_prepare")(
        q_ptr, ldq, _dev(proj, "proj"), proj.shape[1], int(kv_off), _dev(qa, "qa"), _dev(positions, "positions", torch.int32),
        _dev(seq_of_token, "seq_of_token", torch.int32), _opt(slot_mapping, "slot_mapping", torch.int32), _dev(cos, "cos", torch.float32),
        _dev(sin, "sin", torch.float32), _opt(latent_w if has_kv else None, "latent_w", torch.float32), float(eps),
        _opt(latent_pages if has_kv else None, "latent_pages", proj.dtype), _opt(krot_pages if has_kv else None, "krot_pages", proj.dtype),
        tokens, heads, dim, rot, rot_dims, rank, _code(proj.dtype), _stream()), "latent_prepare")


def head_gemm(a, lda: int, a_head_stride: int, b, b_head_stride: int, b_k_stride: int, b_n_stride: int, c, ldc: int, c_head_stride: int,
              rows: int, heads: int, n: int, k: int, gate=None, ldg: int = 0, gate_off: int = 0, a_off: int = 0,
              gate_per_output: bool = False) -> None:
    """Per head h: ``c[t, h, :n] = a[t, a_off + h * a_head_stride : ... + k] @ B_h`` with
    ``B_h[k, n] = b[h * b_head_stride + k * b_k_stride + n * b_n_stride]``, times ``sigmoid(gate[t * ldg + gate_off + h])``
    when a gate is given (``gate_per_output``: one gate per output, ``gate[t * ldg + gate_off + h * n + j]`` for column j).
    Float32 accumulation in a fixed order."""
    if a.dtype != b.dtype or c.dtype != a.dtype or (gate is not None and gate.dtype != a.dtype):
        raise KernelError("head_gemm: one element type for all operands")
    item = a.element_size()
    gate_ptr = None if gate is None else _dev(gate, "gate") + gate_off * item
    _check(_fn("stride_head_gemm")(_dev(a, "a") + a_off * item, lda, a_head_stride, _dev(b, "b"), b_head_stride, b_k_stride, b_n_stride,
                                   _dev(c, "c"), ldc, c_head_stride, gate_ptr, ldg, n if gate_per_output else 1, 1 if gate_per_output else 0,
                                   rows, heads, n, k, _code(a.dtype), _stream()),
           "head_gemm")


def latent_attention(qa, out, latent_pages, krot_pages, block_table, seq_of_token, positions, heads: int, rank: int, rot: int,
                     page_size: int, scale: float, sinks=None) -> None:
    """Causal attention of every token over its request's latent pages: ``qa`` [tokens, heads * (rank + rot)] holds the
    folded and the rotated query parts, ``out`` [tokens, heads * rank] receives the weighted sums of the latents.
    ``sinks`` (float32 [heads]): exp(sink_h) joins head h's denominator."""
    tokens = out.shape[0]
    if out.shape[1] != heads * rank or qa.shape != (tokens, heads * (rank + rot)):
        raise KernelError("latent_attention: shapes do not agree")
    _check(_fn("stride_latent_attention")(
        _dev(qa, "qa"), _dev(out, "out", qa.dtype), _dev(latent_pages, "latent_pages", qa.dtype), _dev(krot_pages, "krot_pages", qa.dtype),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(positions, "positions", torch.int32), tokens, heads, rank, rot, page_size, float(scale), _opt(sinks, "sinks", torch.float32),
        _code(qa.dtype), _stream()), "latent_attention")


def latent_tc_supported(dtype, heads: int, rank: int, rot: int) -> bool:
    """Sizes the tensor-core latent attention kernel takes; everything else runs the exact kernel."""
    return LATENT_TC and dtype == torch.bfloat16 and rank % 16 == 0 and rot % 16 == 0 and 0 < rank <= 512 and rank + rot <= 640


LATENT_TC = _os.environ.get("STRIDE_B200_LATENT_TC", "1") != "0"


def latent_attention_tc(qa, out, partial, latent_pages, krot_pages, block_table, q_start, q_len, ctx_len, seq_of_token, first_seq: int,
                        num_seqs: int, first_token: int, tokens: int, max_q_len: int, heads: int, rank: int, rot: int, page_size: int,
                        scale: float, splits: int = 1, keys_per_split: int = 0, sinks=None) -> None:
    """Latent attention on the tensor cores for the requests ``first_seq .. first_seq + num_seqs`` of the step, which own
    ``tokens`` rows from ``first_token`` on (``qa`` and ``out`` are the whole step's). ``max_q_len`` 1 runs the single-token
    form, whose keys may be cut into ``splits`` of ``keys_per_split`` with ``partial`` (float32,
    (first_token + tokens) * heads * splits * (rank + 2)) as scratch."""
    _check(_fn("stride_latent_attention_tc")(
        _dev(qa, "qa", torch.bfloat16), _dev(out, "out", torch.bfloat16), _opt(partial, "partial", torch.float32),
        _dev(latent_pages, "latent_pages", torch.bfloat16), _dev(krot_pages, "krot_pages", torch.bfloat16),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], _dev(q_start, "q_start", torch.int32),
        _dev(q_len, "q_len", torch.int32), _dev(ctx_len, "ctx_len", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
        first_seq, num_seqs, first_token, tokens, max_q_len, heads, rank, rot, page_size, float(scale), splits, keys_per_split,
        _opt(sinks, "sinks", torch.float32), _stream()), "latent_attention_tc")


# ---------------------------------------------------------------- recurrent block
def rglru_conv(xy, x_off: int, bias_x, conv_w, conv_b, state, seq_of_token, q_start, state_slot, u) -> None:
    tokens, width = u.shape
    taps = conv_w.shape[1]
    _check(_fn("stride_rglru_conv")(_dev(xy, "xy"), xy.shape[1], int(x_off), _dev(bias_x, "bias_x", torch.float32), _dev(conv_w, "conv_w", xy.dtype),
                                    _dev(conv_b, "conv_b", torch.float32), _dev(state, "state", torch.float32),
                                    _dev(seq_of_token, "seq_of_token", torch.int32), _dev(q_start, "q_start", torch.int32),
                                    _dev(state_slot, "state_slot", torch.int32), _dev(u, "u", torch.float32), tokens, width, taps,
                                    _code(xy.dtype), _stream()), "rglru_conv")


def rglru_gates(u, wa_t, wi_t, ba, bi, lam, decay: float, a_out, gx_out, blocks: int) -> None:
    """``wa_t`` / ``wi_t``: the gate matrices of every block transposed, [blocks, in, out]."""
    tokens, width = u.shape
    _check(_fn("stride_rglru_gates")(_dev(u, "u", torch.float32), _dev(wa_t, "wa_t"), _dev(wi_t, "wi_t", wa_t.dtype), _dev(ba, "ba", torch.float32),
                                     _dev(bi, "bi", torch.float32), _dev(lam, "lam", torch.float32), float(decay),
                                     _dev(a_out, "a", torch.float32), _dev(gx_out, "gx", torch.float32), tokens, width, blocks,
                                     _code(wa_t.dtype), _stream()), "rglru_gates")


def rglru_scan(a, gx, xy, x_off: int, y_off: int, bias_x, bias_y, state, q_start, q_len, state_slot, out, num_seqs: int, taps: int) -> None:
    width = out.shape[1]
    _check(_fn("stride_rglru_scan")(_dev(a, "a", torch.float32), _dev(gx, "gx", torch.float32), _dev(xy, "xy", out.dtype), xy.shape[1],
                                    int(x_off), int(y_off), _dev(bias_x, "bias_x", torch.float32), _dev(bias_y, "bias_y", torch.float32),
                                    _dev(state, "state", torch.float32), _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32),
                                    _dev(state_slot, "state_slot", torch.int32), _dev(out, "out"), num_seqs, width, taps,
                                    _code(out.dtype), _stream()), "rglru_scan")


SCAN_PIECES_MIN_TOKENS = int(_os.environ.get("STRIDE_B200_SCAN_PIECES_MIN", "256"))


def rglru_scan_pieces(a, gx, xy, x_off: int, y_off: int, bias_x, bias_y, state, q_start, q_len, state_slot, out, piece, num_seqs: int,
                      max_q_len: int, taps: int) -> None:
    """``rglru_scan`` in three passes over pieces of 64 tokens, parallel over the pieces (bfloat16 activations). ``piece``:
    float32 scratch of at least ``(tokens // 64 + num_seqs + 1) * 2 * width``."""
    width = out.shape[1]
    if piece.numel() < (out.shape[0] // 64 + num_seqs + 1) * 2 * width:
        raise KernelError("rglru_scan_pieces: the scratch is too small")
    _check(_fn("stride_rglru_scan_pieces")(
        _dev(a, "a", torch.float32), _dev(gx, "gx", torch.float32), _dev(xy, "xy", torch.bfloat16), xy.shape[1], int(x_off), int(y_off),
        _dev(bias_x, "bias_x", torch.float32), _dev(bias_y, "bias_y", torch.float32), _dev(state, "state", torch.float32),
        _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32), _dev(state_slot, "state_slot", torch.int32),
        _dev(out, "out", torch.bfloat16), _dev(piece, "piece", torch.float32), num_seqs, max_q_len, width, taps, _code(out.dtype), _stream()),
        "rglru_scan_pieces")


# ------------------------------------------------------------------ routed experts
def moe_route(h, w_router, bias, seq_of_token, ids, weights) -> None:
    tokens, hidden = h.shape
    experts, top = w_router.shape[0], ids.shape[1]
    _check(_fn("stride_moe_route")(_dev(h, "h"), _dev(w_router, "w_router", h.dtype), _opt(bias, "bias", torch.float32),
                                   _opt(seq_of_token, "seq_of_token", torch.int32), _dev(ids, "ids", torch.int32),
                                   _dev(weights, "weights", torch.float32), tokens, hidden, experts, top, _code(h.dtype), _stream()), "moe_route")


def moe_select(logits, bias, seq_of_token, ids, weights) -> None:
    """From router logits [tokens, experts] (float32, without the bias): the ``top`` largest of ``logits + bias`` (the lower
    index among equals) and the softmax over them."""
    tokens, experts = logits.shape
    _check(_fn("stride_moe_select")(_dev(logits, "logits", torch.float32), _opt(bias, "bias", torch.float32),
                                    _opt(seq_of_token, "seq_of_token", torch.int32), _dev(ids, "ids", torch.int32),
                                    _dev(weights, "weights", torch.float32), tokens, experts, ids.shape[1], _stream()), "moe_select")


def moe_select_sigmoid(logits, correction, seq_of_token, ids, weights, experts: int, groups: int, keep: int, route_scale: float) -> None:
    """From router logits (float32, the first ``experts`` columns of ``logits``' rows): scores ``sigmoid(z)``, choice scores
    ``score + correction``, only the experts of the ``keep`` best of ``groups`` equal groups (a group's score: its two largest
    choice scores) can be chosen, the ``top`` largest choice scores win; weights ``score / (sum + 1e-20) * route_scale``."""
    _check(_fn("stride_moe_select_sigmoid")(_dev(logits, "logits", torch.float32), logits.shape[1], _opt(correction, "correction", torch.float32),
                                            _opt(seq_of_token, "seq_of_token", torch.int32), _dev(ids, "ids", torch.int32),
                                            _dev(weights, "weights", torch.float32), logits.shape[0], int(experts), ids.shape[1], int(groups),
                                            int(keep), float(route_scale), _stream()), "moe_select_sigmoid")


def moe_select_groups(logits, correction, seq_of_token, ids, weights, experts: int, groups: int, keep: int, route_scale: float,
                      softmax: bool = False, group_max: bool = False, keep_scores: bool = False) -> None:
    """``moe_select_sigmoid`` with its rule opened up: ``softmax`` takes the softmax of the logits over all experts as
    scores (sigmoid otherwise), ``group_max`` counts a group as its largest choice score (the sum of its two largest
    otherwise), ``keep_scores`` leaves the weights at ``score * route_scale`` (divided by the chosen scores' sum otherwise)."""
    rule = (1 if softmax else 0) | (2 if group_max else 0) | (4 if keep_scores else 0)
    _check(_fn("stride_moe_select_groups")(_dev(logits, "logits", torch.float32), logits.shape[1], _opt(correction, "correction", torch.float32),
                                           _opt(seq_of_token, "seq_of_token", torch.int32), _dev(ids, "ids", torch.int32),
                                           _dev(weights, "weights", torch.float32), logits.shape[0], int(experts), ids.shape[1], int(groups),
                                           int(keep), float(route_scale), rule, _stream()), "moe_select_groups")


def moe_plan(ids, experts: int, offsets, perm_token, row_of, rank_tmp) -> None:
    tokens, top = ids.shape
    _check(_fn("stride_moe_plan")(_dev(ids, "ids", torch.int32), tokens, top, experts, _dev(offsets, "offsets", torch.int32),
                                  _dev(perm_token, "perm_token", torch.int32), _dev(row_of, "row_of", torch.int32),
                                  _dev(rank_tmp, "rank_tmp", torch.int32), _stream()), "moe_plan")


def grouped_gemm(a, row_map, w, offsets, c, max_rows: int, act: int = 0, limit: float = 0.0, alpha: float = 1.0) -> None:
    """For every expert e and row p in ``offsets[e] .. offsets[e+1]``: ``c[p] = act(a[row_map[p]] @ w[e].T)`` (``row_map`` None:
    row p itself). ``w`` [experts, n, k]; ``act`` 1 squares the positive part; ``act`` 2 takes rows 2i and 2i + 1 of ``w[e]`` as
    gate and up of unit i and leaves ``g' sigmoid(alpha g') (u' + 1)`` (clamped at ``limit``) in ``c`` [rows, n / 2]; ``act`` 3
    takes the same pairs and leaves ``g sigmoid(g) u``."""
    experts, n, k = w.shape
    if a.dtype == torch.float32:
        kind = 0
    elif c.dtype == torch.bfloat16:
        kind = 1
    else:
        kind = 2
    _check(_fn("stride_grouped_gemm")(_dev(a, "a"), a.shape[1], _opt(row_map, "row_map", torch.int32), _dev(w, "w", a.dtype),
                                      _dev(offsets, "offsets", torch.int32), experts, _dev(c, "c"), c.shape[1], int(max_rows), n, k, int(act),
                                      float(limit), float(alpha), kind, _stream()), "grouped_gemm")


# Steps with at least this many (token, choice) rows run the experts' products on the tcgen05 kernel (128-row tiles
# per expert); smaller ones, whose tiles would be mostly empty, stay on the 64-row mma.sync tiles. 0 turns it off.
GROUPED_TC_MIN_ROWS = int(_os.environ.get("STRIDE_GROUPED_TC_MIN_ROWS", "1024"))


def grouped_tc_wanted(dtype, rows: int) -> bool:
    return dtype == torch.bfloat16 and GROUPED_TC_MIN_ROWS > 0 and rows >= GROUPED_TC_MIN_ROWS


def gather_rows(x, perm, offsets, experts: int, xs, max_rows: int) -> bool:
    """``xs[p] = x[perm[p]]`` for the rows p that the plan filled (``offsets[experts]`` of them, at most ``max_rows``). False:
    the rows are not whole 16-byte pieces and nothing was done."""
    if x.dtype != xs.dtype or x.shape[1] != xs.shape[1] or xs.shape[0] < max_rows:
        raise KernelError("gather_rows wants rows of one width and element type and room for every row")
    code = _fn("stride_gather_rows")(_dev(x, "x"), x.stride(0) * x.element_size(), _dev(perm, "perm", torch.int32),
                                     _dev(offsets, "offsets", torch.int32), int(experts), _dev(xs, "xs"), x.shape[1] * x.element_size(),
                                     int(max_rows), _stream())
    if code == -2:
        return False
    _check(code, "gather_rows")
    return True


def grouped_gemm_tc(a, w, offsets, c, max_rows: int, act: int = 0, limit: float = 0.0, alpha: float = 1.0) -> bool:
    """``grouped_gemm`` without a row map (row p of ``a`` belongs to the expert whose range holds p) on the tcgen05 kernel,
    bfloat16 operands, ``c`` bfloat16 or float32. False when it does not take the sizes (nothing was done)."""
    experts, n, k = w.shape
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[1] != k or c.dtype not in (torch.bfloat16, torch.float32):
        return False
    code = _fn("stride_grouped_gemm_tc5")(_dev(a, "a"), a.stride(0), _dev(w, "w"), _dev(offsets, "offsets", torch.int32), experts, _dev(c, "c"),
                                          c.shape[1], int(max_rows), n, k, int(act), float(limit), float(alpha),
                                          1 if c.dtype == torch.float32 else 0, _status_ptr(a.device), _stream())
    if code == -2:
        return False
    _check(code, "grouped_gemm_tc5")
    return True


def moe_combine(y, row_of, weights, shared, out, shared_gate=None) -> None:
    """``shared_gate``: a float32 column (one logit per token, possibly a column of a wider buffer); the shared expert's
    output is then multiplied by its sigmoid."""
    tokens, hidden = out.shape
    gate_ptr, gate_stride = (None, 0) if shared_gate is None else (shared_gate.data_ptr(), shared_gate.stride(0))
    if shared_gate is not None and (shared_gate.dtype != torch.float32 or shared_gate.shape[0] != tokens):
        raise KernelError("moe_combine: the shared expert's gate must be one float32 logit per token")
    _check(_fn("stride_moe_combine")(_dev(y, "y", torch.float32), _dev(row_of, "row_of", torch.int32), _dev(weights, "weights", torch.float32),
                                     _opt(shared, "shared", out.dtype), gate_ptr, gate_stride, _dev(out, "out"), tokens, hidden,
                                     row_of.shape[1], _code(out.dtype), _stream()), "moe_combine")


def relu_squared(x) -> None:
    _check(_fn("stride_relu_squared")(_dev(x, "x"), x.numel(), _code(x.dtype), _stream()), "relu_squared")


# ----------------------------------------------------------------------- matmul
# Up to this many rows (tokens: a decode step) the bfloat16 products run on the package's own kernels, which
# stream the weights once; above it the library product is called, as the reference's engine does.
# STRIDE_B200_TC_GEMM=0 switches both off, STRIDE_TC_MAX_TOKENS moves the limit (the tcgen05 kernel takes up to
# 256 rows, the weight-streaming kernel 16; measured at 32 and 64 rows the library is level or faster).
import os as _os

TC_GEMM_MAX_TOKENS = 0 if _os.environ.get("STRIDE_B200_TC_GEMM", "1") == "0" else int(_os.environ.get("STRIDE_TC_MAX_TOKENS", "16"))
# The tcgen05 kernel (TMA ring, weight rows as the 128-row tile side) takes the weight matrices with at least this
# many 128-row tiles (gate/up, the head): with fewer, K has to be split over several CTAs and the partial tiles go
# through global memory. STRIDE_TC_MIN_TILES=0 sends every product to it.
TC_GEMM_MIN_TILES = int(_os.environ.get("STRIDE_TC_MIN_TILES", "100"))
# The smaller matrices (QKV, O, down) go to the weight-streaming kernel, which gives a CTA 16 rows and all of K.
# STRIDE_B200_STREAM_GEMM=0 sends them to the library product instead.
STREAM_GEMM = _os.environ.get("STRIDE_B200_STREAM_GEMM", "1") != "0"
_TC_TICKETS = 8192
_tc_state: dict = {}


def _device_key(device) -> torch.device:
    """``cuda`` and ``cuda:<current>`` are one device: state kept per device must not be kept twice."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return device


def _tc_buffers(device, partial_floats: int):
    device = _device_key(device)
    st = _tc_state.get(device)
    if st is None:
        st = {"tickets": torch.zeros(_TC_TICKETS, dtype=torch.int32, device=device),
              "status": torch.zeros(64, dtype=torch.int32, device=device), "partials": None, "retired": []}
        _tc_state[device] = st
    if partial_floats and (st["partials"] is None or st["partials"].numel() < partial_floats):
        if st["partials"] is not None:
            st["retired"].append(st["partials"])      # a captured graph may still use it
        st["partials"] = torch.empty(max(partial_floats, 1 << 20), dtype=torch.float32, device=device)
    return st


def _tc_scratch_floats(n_out: int, tokens: int, k: int) -> int:
    f = _bound.get("stride_gemm_tc_scratch_floats")
    if f is None:
        f = build.load_kernel_library("gemm_bf16_tc").stride_gemm_tc_scratch_floats
        f.argtypes = [c_int, c_int, c_int]
        f.restype = c_longlong
        _bound["stride_gemm_tc_scratch_floats"] = f
    return int(f(n_out, tokens, k))


def tc_status(device=None) -> int:
    """0, or the code of the first bounded wait that ran out inside the tcgen05
    kernels (1 producer, 2 tensor-core issuer, 3 epilogue). Synchronises."""
    codes = [int(st["status"][0].item()) for dev, st in _tc_state.items() if device is None or dev == _device_key(device)]
    return next((c for c in codes if c), 0)


_WAIT_CODES = {1: "matrix product: producer", 2: "matrix product: tensor-core issuer", 3: "matrix product: epilogue",
               31: "decode attention: a tile copy", 41: "weight-streaming product: a tile copy",
               51: "tokens-as-rows product: activation copies", 52: "tokens-as-rows product: weight copies",
               53: "tokens-as-rows product: tensor-core issuer", 54: "tokens-as-rows product: epilogue"}
_WAIT_CODES.update({c: "prefill attention (attention_prefill_tc.cu)" for c in range(11, 22)})
_OTHER_CODES = {32: "decode attention was given a token whose position is not below the context bound of its launch"}


def reset_kernel_status(device=None) -> None:
    """Sets the status word back to 0 (on ``device``, or wherever one exists), so that later steps are judged on
    their own: the kernels only ever write the first code into a word that is still 0."""
    for dev, st in _tc_state.items():
        if device is None or dev == _device_key(device):
            st["status"].zero_()


def raise_on_kernel_status(code: int, device=None) -> None:
    """Raises when ``code`` (the status word, read back by the caller) is not 0: a bounded wait inside a kernel ran
    out, or a kernel refused a row, so what the step wrote is not to be trusted. With ``device`` the word there is
    cleared first, so that the failure is reported once and the next step starts clean (the reference's worker
    reports a failed pass and keeps serving, python/stride_worker/worker.py:156-165)."""
    if not code:
        return
    if device is not None:
        reset_kernel_status(device)
    if code in _OTHER_CODES:
        raise KernelError(f"kernel status {code}: {_OTHER_CODES[code]}; the step's results are invalid")
    raise KernelError(f"a bounded wait inside a kernel ran out (code {code}: {_WAIT_CODES.get(code, 'unknown place')}); "
                      "the step's results are invalid")


def check_kernel_status(device=None) -> None:
    """Reads the status word (synchronises), clears it if it is set, and raises if a kernel recorded a failure."""
    code = tc_status(device)
    if code:
        reset_kernel_status(device)
    raise_on_kernel_status(code)


def status_tensor(device):
    """The device word that the tcgen05 kernels set on a timed-out wait (for callers that copy it with their own results)."""
    return _tc_buffers(device, 0)["status"]


def linear_tc(x, weight, out) -> bool:
    """``out = x @ weight.T`` on the tcgen05 kernel. Returns False when the kernel
    does not take the shape (the caller then uses the library product)."""
    m, k = x.shape
    n = weight.shape[0]
    st = _tc_buffers(x.device, _tc_scratch_floats(n, m, k))
    partials = st["partials"]
    code = _fn("stride_gemm_tc_skinny", f"product {n}x{k} (tcgen05)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"),
                                        m, n, k, int(out.dtype == torch.float32),
                                        None if partials is None else partials.data_ptr(),
                                        0 if partials is None else partials.numel(), st["tickets"].data_ptr(), _TC_TICKETS,
                                        st["status"].data_ptr(), _stream())
    if code == -2:
        return False
    _check(code, "gemm_tc_skinny")
    return True


# The tcgen05 kernel with the CTAs of an output tile in a cluster (the parts of K meet in the first CTA's shared
# memory, nothing goes through global memory) takes up to 64 tokens. Measured over whole decode steps of the 8B shape
# at a context of 2,048 it is level with the library product at 17 and 32 tokens (4.51 against 4.44 ms, 5.11 against
# 5.02) and slower at 64 (7.3 against 6.3: there the library streams the small matrices in 48- and 64-row tiles
# through a 15-stage ring at about 0.6 of the memory bandwidth, this kernel's 128-row tiles with K split four ways at
# 0.35), so it is off by default: STRIDE_TC_CLUSTER_MAX_TOKENS=64 switches it on.
TC_CLUSTER_MAX_TOKENS = int(_os.environ.get("STRIDE_TC_CLUSTER_MAX_TOKENS", "0"))


def linear_tc_clustered(x, weight, out) -> bool:
    """``out = x @ weight.T`` for up to 64 rows of ``x`` on the clustered tcgen05 kernel. Returns False when the
    kernel does not take the shape."""
    m, k = x.shape
    n = weight.shape[0]
    code = _fn("stride_gemm_tc_clustered", f"product {n}x{k} (tcgen05, clusters)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"), m, n, k,
        int(out.dtype == torch.float32), _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_tc_clustered")
    return True


# Decode steps of 17 to this many tokens (128 at the most) run the package's tcgen05 product with the tokens as the
# rows of the tile (gemm_bf16_rows.cu: one CTA per block of output features and all of K; residual sum and the
# statistics of the norm that follows, the norm's factor, rotation with cache write and SiLU * up in its epilogues).
# Off by default: it is level with the library product plus separate elementwise kernels where a 4096-row matrix
# gives every SM a CTA, and slower elsewhere. Whole decode steps from a graph, this kernel / library: 8B sizes at a
# context of 2,048, 17 tokens 4.43 / 4.44 ms, 24: 4.70 / 4.63, 32: 4.92 / 4.97, 40: 5.60 / 5.28, 64: 6.57 / 6.29,
# 128: 10.0 / 9.1; at a context of 1,024, 32 tokens 4.33 / 4.42; 3B sizes (3072-row matrices: 96 CTAs), 32 tokens at
# a context of 4,096 4.50 / 4.28. Every CTA reads all of the activations, which is more than its weights once there
# are more tokens than features in its block; the library shares them between the CTAs of a cluster.
ROWS_GEMM_MAX_TOKENS = min(128, int(_os.environ.get("STRIDE_ROWS_GEMM_MAX_TOKENS", "0")))


def rows_wanted(tokens: int) -> bool:
    """Whether a step of this many tokens runs its products on the tokens-as-rows kernel (the callers' policy; the
    ``linear_rows*`` functions themselves take up to 128 rows)."""
    return TC_GEMM_MAX_TOKENS < tokens <= ROWS_GEMM_MAX_TOKENS


def _rows_ok(x, m: int) -> bool:
    return m <= 128 and x.dtype == torch.bfloat16 and TC_GEMM_MAX_TOKENS > 0


def linear_rows(x, weight, out) -> bool:
    """``out = x @ weight.T`` (bfloat16 or float32 out) for up to 128 rows of ``x`` on the tokens-as-rows tcgen05 kernel.
    Returns False when the kernel does not take the shape."""
    m, k = x.shape
    n = weight.shape[0]
    code = _fn("stride_gemm_rows", f"product {n}x{k} (tcgen05, tokens as rows)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"), m, n, k,
        int(out.dtype == torch.float32), _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows")
    return True


def linear_rows_add(x, weight, residual) -> bool:
    """``residual += bf16(x @ weight.T)`` (float32 residual) in one kernel, for 17 to 128 rows. False: not done."""
    m, k = x.shape
    n = weight.shape[0]
    if not _rows_ok(x, m) or residual.shape != (m, n):
        return False
    code = _fn("stride_gemm_rows_add", f"product {n}x{k} (tcgen05, tokens as rows, + residual)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(residual, "residual", torch.float32), m, n, k,
        _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows_add")
    return True


def linear_rows_add_norm(x, weight, residual, norm_weight, xt, partials) -> int:
    """``linear_add_norm`` for 17 to 128 rows: ``partials[cta, token]`` has 128 tokens a CTA. Returns the number of
    producer CTAs, or 0 when the kernel does not take the sizes."""
    m, k = x.shape
    n = weight.shape[0]
    if not (FOLD_NORMS and _rows_ok(x, m)) or residual.shape != (m, n):
        return 0
    count = c_int(0)
    code = _fn("stride_gemm_rows_add_norm", f"product {n}x{k} (tcgen05, tokens as rows, + residual, norm statistics)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(xt, "xt", torch.bfloat16),
        _dev(residual, "residual", torch.float32), _dev(norm_weight, "norm_weight", torch.float32),
        _dev(partials, "partials", torch.float32), partials.numel(), m, n, k, ctypes.byref(count), _status_ptr(x.device), _stream())
    if code == -2:
        return 0
    _check(code, "gemm_rows_add_norm")
    return count.value


ROWS_FOLD_STRIDE = 128      # tokens a CTA in the partials that ``linear_rows_add_norm`` writes


def linear_rows_gated(x, weight, out, folded=None) -> bool:
    """``out = silu(x @ gate.T) * (x @ up.T)`` for 17 to 128 rows; ``weight`` as for ``linear_gated_tc``; ``folded``: a
    FoldedNorm from ``linear_rows_add_norm`` whose ``xt`` is ``x``. False: not done."""
    m, k = x.shape
    inter = weight.shape[0] // 2
    if not _rows_ok(x, m) or out.shape != (m, inter) or (folded is not None and folded.stride != ROWS_FOLD_STRIDE):
        return False
    partials, count, eps = _fold_args(folded, ROWS_FOLD_STRIDE)
    code = _fn("stride_gemm_rows_gated", f"product 2x{inter}x{k} (tcgen05, tokens as rows, silu * up)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out", torch.bfloat16), m, inter, k,
        partials, count, eps, _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows_gated")
    return True


def linear_rows_qkv_rope(x, weight, qkv, bias, positions, slot_mapping, cos, sin, k_pages, v_pages, nq: int, nkv: int, hd: int,
                         page_size: int, rotate: bool, folded=None) -> bool:
    """``linear_qkv_rope`` for 17 to 128 rows of ``x`` (``folded``: from ``linear_rows_add_norm``). False: not done."""
    m, k = x.shape
    if not _rows_ok(x, m) or qkv.shape != (m, (nq + 2 * nkv) * hd) or (folded is not None and folded.stride != ROWS_FOLD_STRIDE):
        return False
    partials, count, eps = _fold_args(folded, ROWS_FOLD_STRIDE)
    code = _fn("stride_gemm_rows_qkv_rope", f"product {weight.shape[0]}x{k} (tcgen05, tokens as rows, qkv + rotation + cache write)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(qkv, "qkv", torch.bfloat16),
        _opt(bias, "bias", torch.float32), _dev(positions, "positions", torch.int32), _opt(slot_mapping, "slot_mapping", torch.int32),
        _dev(cos, "cos", torch.float32), _dev(sin, "sin", torch.float32), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), m, nq, nkv, hd, page_size, k, int(rotate), partials, count, eps,
        _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows_qkv_rope")
    return True


GATED_BLOCK = 64      # rows of gate and up alternate in blocks of this many in a weight laid out for ``linear_gated_tc``


FOLD_NORMS = _os.environ.get("STRIDE_B200_FOLD_NORMS", "1") != "0"


class FoldedNorm:
    """The output of an RMS norm whose two halves were folded into the products around it: ``xt`` holds
    ``residual * weight`` in bfloat16 (no 1/rms yet), ``partials`` [count, 16] the sums of squares of the
    residual per producer CTA and token (``stride`` tokens a CTA: 16 from the kernels for at most 16 tokens, 128 from
    the tokens-as-rows kernel). A product that takes it applies ``rsqrt(sum / width + eps)`` to its
    accumulators; anything else asks for ``tensor()``, which runs the small kernel that finishes the norm."""

    def __init__(self, xt, partials, count: int, eps: float, make_buffer, stride: int = 16):
        self.xt, self.partials, self.count, self.eps, self.stride = xt, partials, int(count), float(eps), int(stride)
        self.shape, self.dtype, self.device = xt.shape, xt.dtype, xt.device
        self._make_buffer = make_buffer
        self._tensor = None

    def tensor(self):
        if self._tensor is None:
            out = self._make_buffer()
            _check(_fn("stride_scale_rows")(self.xt.data_ptr(), self.partials.data_ptr(), self.count, self.eps, out.data_ptr(),
                                            self.shape[0], self.shape[1], self.stride, _stream()), "scale_rows")
            self._tensor = out
        return self._tensor


def _fold_args(folded, stride: int = 16):
    if folded is None:
        return None, 0, 0.0
    if folded.stride != stride:
        raise ValueError(f"a folded norm with {folded.stride} tokens a CTA was given to a kernel that reads {stride}")
    return folded.partials.data_ptr(), folded.count, folded.eps


def linear_add_norm(x, weight, residual, norm_weight, xt, partials) -> int:
    """The product before an RMS norm, for at most 16 rows: ``residual += bf16(x @ weight.T)`` (float32),
    ``xt = residual * norm_weight`` in bfloat16, ``partials[cta, token]`` the sums of squares. Returns the number
    of producer CTAs (what a consumer has to add up), or 0 when the kernel does not take the sizes."""
    m, k = x.shape
    n = weight.shape[0]
    if not (FOLD_NORMS and STREAM_GEMM) or m > TC_GEMM_MAX_TOKENS or x.dtype != torch.bfloat16 or residual.shape != (m, n):
        return 0
    count = c_int(0)
    code = _fn("stride_gemm_stream_add_norm", f"product {n}x{k} (+ residual, norm statistics)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16),
                                              _dev(xt, "xt", torch.bfloat16), _dev(residual, "residual", torch.float32),
                                              _dev(norm_weight, "norm_weight", torch.float32), _dev(partials, "partials", torch.float32),
                                              partials.numel(), m, n, k, ctypes.byref(count), _status_ptr(x.device), _stream())
    if code == -2:
        return 0
    _check(code, "gemm_stream_add_norm")
    return count.value


def linear_gated_tc(x, weight, out, folded=None, activation: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> bool:
    """``out = act(x @ gate.T) * (x @ up.T)`` (``activation`` one of ``ACTIVATIONS``) in one tcgen05 kernel for at most 16 rows of ``x``; ``weight`` is
    [2 * inter, k] with gate and up rows alternating in blocks of ``GATED_BLOCK``. With ``folded`` (a FoldedNorm
    whose ``xt`` is ``x``) the kernel applies the norm's 1/rms itself. Returns False when the kernel does not take
    the sizes (the caller then runs the product and ``silu_mul`` with the same block). ``limit`` and ``alpha`` belong to
    ``swish_clamped``."""
    m, k = x.shape
    inter = weight.shape[0] // 2
    if m > TC_GEMM_MAX_TOKENS or out.shape != (m, inter) or x.dtype != torch.bfloat16:
        return False
    st = _tc_buffers(x.device, 0)
    partials, count, eps = _fold_args(folded)
    code = _fn("stride_gemm_tc_gated", f"product 2x{inter}x{k} (tcgen05, {activation} * up)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16),
                                       _dev(out, "out", torch.bfloat16), m, inter, k, st["status"].data_ptr(), partials, count, eps,
                                       ACTIVATIONS[activation], float(limit), float(alpha), _stream())
    if code == -2:
        return False
    _check(code, "gemm_tc_gated")
    return True


def _status_ptr(device) -> int:
    return _tc_buffers(device, 0)["status"].data_ptr()


def linear_stream(x, weight, out) -> bool:
    """``out = x @ weight.T`` on the weight-streaming kernel (at most 16 rows of ``x``).
    Returns False when the kernel does not take the shape."""
    m, k = x.shape
    n = weight.shape[0]
    code = _fn("stride_gemm_stream_bf16", f"product {n}x{k} (weight streaming)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"),
                                          m, n, k, int(out.dtype == torch.float32), _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_stream_bf16")
    return True


def linear_qkv_rope(x, weight, qkv, bias, positions, slot_mapping, cos, sin, k_pages, v_pages, nq: int, nkv: int, hd: int,
                    page_size: int, rotate: bool, folded=None) -> bool:
    """The projection of queries, keys and values with ``rope_kv_write`` in its epilogue, for at most 16 rows of
    ``x``: afterwards ``qkv`` holds the rotated queries (its key and value columns are not written) and the cache
    the rotated keys and the values. With ``folded`` (a FoldedNorm whose ``xt`` is ``x``) the kernel applies the
    norm's 1/rms itself. Returns False when the kernel does not take the sizes; the caller then runs ``linear`` and
    ``rope_kv_write``."""
    m, k = x.shape
    if not STREAM_GEMM or m > TC_GEMM_MAX_TOKENS or x.dtype != torch.bfloat16 or qkv.shape != (m, (nq + 2 * nkv) * hd):
        return False
    partials, count, eps = _fold_args(folded)
    code = _fn("stride_gemm_stream_qkv_rope", f"product {weight.shape[0]}x{k} (qkv + rotation + cache write)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(qkv, "qkv", torch.bfloat16),
        _opt(bias, "bias", torch.float32), _dev(positions, "positions", torch.int32), _opt(slot_mapping, "slot_mapping", torch.int32),
        _dev(cos, "cos", torch.float32), _dev(sin, "sin", torch.float32), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), m, nq, nkv, hd, page_size, k, int(rotate), partials, count, eps,
        _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_stream_qkv_rope")
    return True


def linear(x, weight, out) -> None:
    """``out = x @ weight.T`` for row-major ``weight`` [out_features, in_features].

    float32 runs the package's own FMA kernel (true 32-bit, order of the sum
    fixed). bfloat16 with few rows (decode steps) runs the package's own kernels:
    the tcgen05 kernel for large matrices, the weight-streaming kernel for the
    others; with many rows it calls the library matrix product, as the
    reference's engine does (python/stride_worker/model.py:258-260). ``out`` may
    be float32 for bfloat16 inputs to keep the accumulator's precision (the
    output head).
    """
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} do not agree")
    if x.dtype == torch.float32:
        _check(_fn("stride_gemm_nt_f32", f"product {n}x{k} (float32)")(_dev(x, "x", torch.float32), _dev(weight, "weight", torch.float32),
                                         _dev(out, "out", torch.float32), m, n, k, k, k, n, _stream()), "gemm_nt_f32")
        return
    _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out")
    if m == 0:
        return
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("linear: the output must be bfloat16 or float32")
    if m <= TC_GEMM_MAX_TOKENS:
        if -(-n // 128) >= TC_GEMM_MIN_TILES:
            if linear_tc(x, weight, out):
                return
        elif STREAM_GEMM and linear_stream(x, weight, out):
            return
    elif m <= TC_CLUSTER_MAX_TOKENS and TC_GEMM_MAX_TOKENS > 0 and linear_tc_clustered(x, weight, out):
        return
    def library(*_):
        if out.dtype == torch.float32:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, weight.t(), out=out)
        return 0
    (_timer.timed(f"product {n}x{k} (library)", library) if _timer is not None else library)()


# -------------------------------------------------------------------- attention
def paged_attention(q, q_stride: int, out, k_pages, v_pages, block_table, seq_of_token, positions, nq: int, nkv: int,
                    hd: int, page_size: int, scale: float, window: int = 0, softcap: float = 0.0, sinks=None, slopes=None,
                    vd: int | None = None) -> None:
    """Attention of every token in the flat batch over its request's pages.
    ``q`` holds head h of token t at ``q[t * q_stride + h * hd]``. ``softcap`` c > 0 caps the scaled scores at
    c tanh(s / c); ``sinks`` (float32 [nq]) adds exp(sink) of the head to the softmax's denominator; ``slopes`` (float32
    [nq]) takes slope_h times the key's distance off every score; ``vd`` is the values' width where it is not ``hd``."""
    tokens = out.shape[0]
    vd = hd if vd is None else int(vd)
    if out.shape[1] != nq * vd or k_pages.shape[-1] != hd or v_pages.shape[-1] != vd:
        raise KernelError("attention output or pages have the wrong width")
    _check(_fn("stride_paged_attention_generic")(
        _dev(q, "q"), q_stride, _dev(out, "out"), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(positions, "positions", torch.int32), tokens, nq, nkv, hd, vd, page_size, float(scale), int(window), float(softcap),
        _opt(sinks, "sinks", torch.float32), _opt(slopes, "slopes", torch.float32), _code(q.dtype), _stream()), "paged_attention")


def fast_attention_supported(dtype, nq: int, nkv: int, hd: int) -> bool:
    """Sizes that the tensor-core attention kernels run; others use the generic kernel."""
    return dtype == torch.bfloat16 and hd in (64, 128) and nq % nkv == 0 and nq // nkv <= 16


def decode_scratch_floats(tokens: int, nq: int, nkv: int, hd: int, max_context: int) -> int:
    """float32 elements of scratch that ``paged_attention_decode`` needs for these sizes."""
    f = _bound.get("stride_paged_decode_scratch_floats")
    if f is None:
        f = build.load_kernel_library("attention_decode").stride_paged_decode_scratch_floats
        f.argtypes = [c_int, c_int, c_int, c_int, c_int]
        f.restype = c_longlong
        _bound["stride_paged_decode_scratch_floats"] = f
    return int(f(tokens, nq, nkv, hd, max_context))


def paged_attention_decode(q, q_stride: int, out, k_pages, v_pages, block_table, seq_of_token, positions, scratch, nq: int,
                           nkv: int, hd: int, page_size: int, scale: float, window: int, max_context: int, softcap: float = 0.0,
                           sinks=None, slopes=None, gate_col: int = -1) -> None:
    """Attention for single decoded tokens (one query per row), split over the keys;
    ``scratch`` (float32, zero when first used) holds the ticket counters and the
    partial results of the splits. ``softcap``, ``sinks`` and ``slopes`` as for ``paged_attention``. ``gate_col`` >= 0: columns
    ``gate_col .. gate_col + nq - 1`` of a row of ``q`` hold one logit per head, and head h's output leaves the kernel
    multiplied by the sigmoid of its logit."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    _check(_fn("stride_paged_decode_attention_gated")(
        _dev(q, "q", torch.bfloat16), q_stride, _dev(out, "out", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), k_pages.shape[0], _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], _dev(seq_of_token, "seq_of_token", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(scratch, "scratch", torch.float32), scratch.numel(), tokens, nq, nkv, hd, page_size, float(scale), int(window),
        float(softcap), _opt(sinks, "sinks", torch.float32), _opt(slopes, "slopes", torch.float32), int(gate_col), int(max_context),
        _tc_buffers(q.device, 0)["status"].data_ptr(), _stream()),
        "paged_attention_decode")


TC_ATTENTION = _os.environ.get("STRIDE_B200_TC_ATTENTION", "1") != "0"


def paged_attention_prefill_tc(q, q_stride: int, out, k_pages, v_pages, block_table, q_start, q_len, ctx_len, num_seqs: int,
                               nq: int, nkv: int, hd: int, page_size: int, scale: float, window: int, softcap: float = 0.0,
                               sinks=None, slopes=None) -> bool:
    """The tcgen05 version of ``paged_attention_prefill`` (same arguments). Returns False
    when it does not take the sizes; the caller then uses the mma.sync kernel."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    st = _tc_buffers(q.device, 0)
    code = _fn("stride_paged_prefill_attention_tc")(
        _dev(q, "q", torch.bfloat16), q_stride, _dev(out, "out", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), k_pages.shape[0], _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32),
        _dev(ctx_len, "ctx_len", torch.int32), num_seqs, tokens, nq, nkv, hd, page_size, float(scale), int(window), float(softcap),
        _opt(sinks, "sinks", torch.float32), _opt(slopes, "slopes", torch.float32), st["status"].data_ptr(), _stream())
    if code == -2:
        return False
    _check(code, "paged_attention_prefill_tc")
    return True


def paged_attention_prefill(q, q_stride: int, out, k_pages, v_pages, block_table, q_start, q_len, ctx_len, num_seqs: int,
                            nq: int, nkv: int, hd: int, page_size: int, scale: float, window: int, softcap: float = 0.0,
                            sinks=None, slopes=None) -> None:
    """Attention for the first ``num_seqs`` requests of the step (portions of any
    length), which own the rows of ``out``. ``softcap`` and ``sinks`` as for ``paged_attention``."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    _check(_fn("stride_paged_prefill_attention")(
        _dev(q, "q", torch.bfloat16), q_stride, _dev(out, "out", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32), _dev(ctx_len, "ctx_len", torch.int32),
        num_seqs, tokens, nq, nkv, hd, page_size, float(scale), int(window), float(softcap), _opt(sinks, "sinks", torch.float32),
        _opt(slopes, "slopes", torch.float32), _stream()), "paged_attention_prefill")


# --------------------------------------------------------------------- sampling
_sample_scratch: dict = {}


def _sampling_scratch(device, rows: int, vocab: int):
    """Zeroed int32 words for the segment results and tickets of ``sample_rows`` (it leaves the tickets zero)."""
    f = _bound.get("stride_sample_scratch_words")
    if f is None:
        f = build.load_kernel_library("sampling").stride_sample_scratch_words
        f.argtypes = [c_int, c_int]
        f.restype = c_longlong
        _bound["stride_sample_scratch_words"] = f
    need = int(f(rows, vocab))
    st = _sample_scratch.setdefault(device, {"buf": None, "retired": []})
    if st["buf"] is None or st["buf"].numel() < need:
        if st["buf"] is not None:
            st["retired"].append(st["buf"])          # a captured graph may still use it
        st["buf"] = torch.zeros(max(need, 1 << 18), dtype=torch.int32, device=device)
    return st["buf"]


def sample_rows(logits, out, temperature=None, uniform=None, suppress=None) -> None:
    """Greedy (no ``temperature``, or 0) or temperature sampling per row."""
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("logits rows must be dense")
    if not logits.is_cuda:
        raise KernelError("logits must live on a CUDA device; stride_b200 has no CPU path")
    scratch = _sampling_scratch(logits.device, rows, vocab)
    _check(_fn("stride_sample_rows")(logits.data_ptr(), rows, vocab, logits.stride(0),
                                     _opt(temperature, "temperature", torch.float32),
                                     _opt(uniform, "uniform", torch.float32), _opt(suppress, "suppress", torch.int32),
                                     _dev(out, "out", torch.int32), scratch.data_ptr(), scratch.numel(), _stream()), "sample_rows")


_ranked_probs: dict = {}


def sample_ranked(logits, out, temperature, uniform, suppress, top_k, top_p) -> None:
    """Draws the rows with a temperature above 0 that ask for top-k (``top_k[r] > 0``) or a nucleus (``top_p[r] < 1``)
    by the reference sampler's rule and writes their tokens to ``out``; the other rows of ``out`` are left as they
    are (``sample_rows`` draws those). One [rows, vocab] float32 scratch per device, grown when a step needs more."""
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("logits rows must be dense")
    if not logits.is_cuda:
        raise KernelError("logits must live on a CUDA device; stride_b200 has no CPU path")
    key = _device_key(logits.device)
    probs = _ranked_probs.get(key)
    if probs is None or probs.numel() < rows * vocab:
        probs = torch.empty(rows * vocab, dtype=torch.float32, device=logits.device)
        _ranked_probs[key] = probs
    _check(_fn("stride_sample_ranked")(logits.data_ptr(), rows, vocab, logits.stride(0), _dev(temperature, "temperature", torch.float32),
                                       _dev(uniform, "uniform", torch.float32), _opt(suppress, "suppress", torch.int32),
                                       _dev(top_k, "top_k", torch.int32), _dev(top_p, "top_p", torch.float32),
                                       _dev(out, "out", torch.int32), probs.data_ptr(), probs.numel(), _stream()), "sample_ranked")
