"""Launchers of `csrc/linear_attention.cu`: the scan of a decaying matrix state over a step's new
tokens, the decay gate, and the gated group norm that follows the scan."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..errors import KernelLaunchError
from . import build
from .lib import _check, _dev, _ptr, dtype_code, stream_handle

MAX_KEY_DIM = 256
GATES = {"sigmoid": 0, "silu": 1}

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("linear_attention.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_linear_attention_scan.argtypes = [P, P, P, I, L, L, L, P, I, P, P, P, P, P, I, I, I, I, F, P]
        l.llm_decay_gate.argtypes = [P, I, L, P, P, P, I, I, I, F, P]
        l.llm_gated_group_norm.argtypes = [P, P, I, L, P, I, P, I, L, I, I, I, I, F, F, P]
        for name in ("llm_linear_attention_scan", "llm_decay_gate", "llm_gated_group_norm"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def scan(ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, per_channel: bool,
         state: torch.Tensor, out: torch.Tensor, heads: int, dk: int, dv: int, q_scale: float = 1.0) -> None:
    """For every sequence of the step, in token order: S = diag(a) S + k v^T, o = S^T (q * q_scale),
    with S in `state[slot]` ([heads, dk, dv] float32) read at the start and written at the end.
    q, k [rows, heads * dk] and v [rows, heads * dv] may be column views of a wider matrix;
    `decay` is [heads] or, with `per_channel`, [rows, heads * dk] float32.  out [rows, heads * dv]
    float32."""
    _dev(q, k, v, decay, state, out)
    if not (q.dtype == k.dtype == v.dtype) or state.dtype != torch.float32 or out.dtype != torch.float32 \
            or decay.dtype != torch.float32 or not out.is_contiguous() or not decay.is_contiguous():
        raise KernelLaunchError("linear_attention_scan: element types or layout not as the kernel needs")
    _check(lib().llm_linear_attention_scan(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), dtype_code(q.dtype), q.stride(0), k.stride(0), v.stride(0),
        decay.data_ptr(), 1 if per_channel else 0, state.data_ptr(), out.data_ptr(),
        ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr(), ctx.n_seqs, heads, dk, dv,
        float(q_scale), ctx.stream), "linear_attention_scan")


def decay_gate(low: torch.Tensor, up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, rows: int,
               tau: float, stream=None) -> None:
    """out[t, c] = sigmoid(up[c] . low[t] + bias[c]) ** (1 / tau), float32."""
    _dev(low, up, bias, out)
    channels, rank = up.shape
    _check(lib().llm_decay_gate(low.data_ptr(), dtype_code(low.dtype), low.stride(0), up.data_ptr(), _ptr(bias),
                                out.data_ptr(), rows, channels, rank, 1.0 / float(tau),
                                stream if stream is not None else stream_handle()), "decay_gate")


def gated_group_norm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, rows: int,
                     group: int, gate_kind: str, eps: float, out_scale: float = 1.0, stream=None) -> None:
    """out = rms_norm over groups of `group` neighbouring channels of x (float32 [rows, channels]) *
    weight[c % len(weight)] * gate_kind(gate) * out_scale; gate and out may be column views."""
    _dev(x, gate, weight, out)
    _check(lib().llm_gated_group_norm(x.data_ptr(), gate.data_ptr(), dtype_code(gate.dtype), gate.stride(0),
                                      weight.data_ptr(), weight.numel(), out.data_ptr(), dtype_code(out.dtype),
                                      out.stride(0), rows, x.shape[-1], group, GATES[gate_kind], float(eps),
                                      float(out_scale), stream if stream is not None else stream_handle()),
           "gated_group_norm")
