"""Launchers of `csrc/linear_attention.cu`: the scan of a decaying matrix state over a step's new
tokens, the decay gate, and the gated group norm that follows the scan."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..errors import KernelLaunchError
from . import build
from .lib import LAUNCHES, _check, _dev, _ptr, dtype_code, stream_handle

MAX_KEY_DIM = 256
GATES = {"sigmoid": 0, "silu": 1}

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("linear_attention.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_linear_attention_scan.argtypes = [P, P, P, I, L, L, L, P, I, P, P, P, P, P, I, I, I, I, F, I, I, P, P, P, I, P]
        l.llm_linear_attention_join.argtypes = [P, I, L, P, I, P, P, P, P, P, I, I, I, I, F, I, I, I, P, P, P, P]
        l.llm_decay_gate.argtypes = [P, I, L, P, P, P, I, I, I, F, P]
        l.llm_gated_group_norm.argtypes = [P, P, I, L, P, I, P, I, L, I, I, I, I, F, F, P]
        for name in ("llm_linear_attention_scan", "llm_linear_attention_join", "llm_decay_gate", "llm_gated_group_norm"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


STRETCH = 128                    # tokens of a stretch when a long portion is walked in stretches side by side
STRETCHES_FROM = 4 * STRETCH     # portions at least this long are
STRETCH_SCRATCH_BYTES = 256 << 20
_scratch = {}                    # device -> float32 scratch for the stretches' states (old ones are kept: graphs hold them)
_retired = []


def _stretches(ctx, q, heads: int, dk: int, dv: int) -> int:
    """How many stretches a step's longest portion is cut into (1: walked in one piece).  Only
    bfloat16 steps are cut (also where the scan's operands are float32 copies): the pieces' sums are
    joined in another order than one walk forms them."""
    if ctx.dtype != torch.bfloat16 or ctx.max_q_len < STRETCHES_FROM:
        return 1
    n = -(-ctx.max_q_len // STRETCH)
    if ctx.n_seqs * n * heads * (dk * dv + dk) * 4 > STRETCH_SCRATCH_BYTES or (dk * dv + 32 * dk) * 4 > 160 * 1024:
        return 1
    return n


def _stretch_scratch(device, floats: int) -> torch.Tensor:
    buf = _scratch.get(device)
    if buf is None or buf.numel() < floats:
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(floats, dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def scan(ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, per_channel,
         state: torch.Tensor, out: torch.Tensor, heads: int, dk: int, dv: int, q_scale: float = 1.0) -> None:
    """For every sequence of the step, in token order: S = diag(a) S + k v^T, o = S^T (q * q_scale),
    with S in `state[slot]` ([heads, dk, dv] float32) read at the start and written at the end.
    q, k [rows, heads * dk] and v [rows, heads * dv] may be column views of a wider matrix;
    `decay` is [heads] or, with `per_channel`, [rows, heads * dk] float32, or, with `per_channel`
    == "token", one number per token and head, [rows, heads].  out [rows, heads * dv]
    float32.  A long portion of a bfloat16 step is walked as stretches of `STRETCH` tokens side by
    side, each from an empty state, and joined afterwards (two more kernels)."""
    _dev(q, k, v, decay, state, out)
    if not (q.dtype == k.dtype == v.dtype) or state.dtype != torch.float32 or out.dtype != torch.float32 \
            or decay.dtype != torch.float32 or not out.is_contiguous() or not decay.is_contiguous():
        raise KernelLaunchError("linear_attention_scan: element types or layout not as the kernel needs")
    mode = 2 if per_channel == "token" else (1 if per_channel else 0)
    n_segs = _stretches(ctx, q, heads, dk, dv)
    seg_state = seg_decay = cum = 0
    if n_segs > 1:
        states = ctx.n_seqs * n_segs * heads * dk * dv
        scratch = _stretch_scratch(q.device, states + ctx.n_seqs * n_segs * heads * dk)
        seg_state, seg_decay = scratch.data_ptr(), scratch.data_ptr() + 4 * states
        if per_channel:
            cum = ctx.ws.get("scan_cum", (q.shape[0], heads * dk), torch.float32).data_ptr()
    _check(lib().llm_linear_attention_scan(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), dtype_code(q.dtype), q.stride(0), k.stride(0), v.stride(0),
        decay.data_ptr(), mode, state.data_ptr(), out.data_ptr(),
        ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr(), ctx.n_seqs, heads, dk, dv,
        float(q_scale), STRETCH, n_segs, seg_state, seg_decay, cum, int(ctx.max_q_len), ctx.stream),
        "linear_attention_scan")
    if n_segs > 1:
        _check(lib().llm_linear_attention_join(
            q.data_ptr(), dtype_code(q.dtype), q.stride(0), decay.data_ptr(), 1 if per_channel else 0,
            state.data_ptr(), out.data_ptr(), ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(),
            ctx.seq_q_len.data_ptr(), ctx.n_seqs, heads, dk, dv, float(q_scale), STRETCH, n_segs, ctx.max_q_len,
            seg_state, seg_decay, cum, ctx.stream), "linear_attention_join")
        LAUNCHES[0] += 1      # the join is two kernels


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
