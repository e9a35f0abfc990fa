"""Launchers of `csrc/mlstm.cu`: the gates and running maximum of an mLSTM head, the float32
operands for the state scan, and the quotient, unit norm and gate after it."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build
from .lib import _check, _dev, dtype_code

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("mlstm.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_mlstm_gates.argtypes = [P, L, I, I, P, P, I, F, P, P, P, P, P, I, I, P]
        l.llm_mlstm_operands.argtypes = [P, I, L, I, I, I, P, P, P, P, P, I, I, I, I, I, P]
        l.llm_mlstm_finish.argtypes = [P, P, P, P, L, P, L, I, I, I, I, I, F, P]
        l.llm_mlstm_step.argtypes = [P, I, L, I, I, I, I, P, L, I, I, P, P, F, P, P, P, P, L, P, P, P, I, I, I, I, I, F, F, P]
        for name in ("llm_mlstm_gates", "llm_mlstm_operands", "llm_mlstm_finish", "llm_mlstm_step"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def gates(ctx, z: torch.Tensor, i_col: int, f_col: int, i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float,
          m_state: torch.Tensor, coef: torch.Tensor, heads: int) -> None:
    """z [rows, columns] float32 holds the gates' projections (input gate of head h at column
    i_col + h, forget gate at f_col + h); coef [rows, heads, 4] float32 receives (decay, input
    weight, exp(-m), m) per new token; m_state [slots + 1, heads] carries m between steps."""
    _dev(z, i_bias, f_bias, m_state, coef)
    if z.dtype != torch.float32 or m_state.dtype != torch.float32 or coef.dtype != torch.float32:
        raise TypeError("mlstm gates: projections, state and coefficients must be float32")
    _check(lib().llm_mlstm_gates(z.data_ptr(), z.stride(0), i_col, f_col, i_bias.data_ptr(), f_bias.data_ptr(),
                                 dtype_code(i_bias.dtype), float(cap), m_state.data_ptr(), coef.data_ptr(),
                                 ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr(),
                                 ctx.n_seqs, heads, ctx.stream), "mlstm_gates")


def operands(ctx, u: torch.Tensor, q_col: int, k_col: int, v_col: int, coef: torch.Tensor, qf, kf, decay, vf,
             heads: int, dk: int, dv: int, dvp: int) -> None:
    _dev(u, coef, qf, kf, decay, vf)
    _check(lib().llm_mlstm_operands(u.data_ptr(), dtype_code(u.dtype), u.stride(0), q_col, k_col, v_col, coef.data_ptr(),
                                    qf.data_ptr(), kf.data_ptr(), decay.data_ptr(), vf.data_ptr(), ctx.n_tokens, heads,
                                    dk, dv, dvp, ctx.stream), "mlstm_operands")


def finish(ctx, scanned: torch.Tensor, coef: torch.Tensor, norm_w: torch.Tensor, gate: torch.Tensor, out: torch.Tensor,
           heads: int, dv: int, dvp: int, eps: float) -> None:
    _dev(scanned, coef, norm_w, gate, out)
    _check(lib().llm_mlstm_finish(scanned.data_ptr(), coef.data_ptr(), norm_w.data_ptr(), gate.data_ptr(),
                                  gate.stride(0), out.data_ptr(), out.stride(0), dtype_code(out.dtype), ctx.n_tokens,
                                  heads, dv, dvp, float(eps), ctx.stream), "mlstm_finish")


STEP_MAX_VALUE_COLUMNS = 288      # vdim + pad the one-token kernel keeps per warp
STEP_MAX_SHARED = 48 * 1024


def step_takes(dk: int, dvp: int) -> bool:
    return dvp <= STEP_MAX_VALUE_COLUMNS and (2 * dk + 9 * dvp + 8) * 4 <= STEP_MAX_SHARED


def step(ctx, u: torch.Tensor, q_col: int, k_col: int, v_col: int, g_col: int, z: torch.Tensor, i_col: int, f_col: int,
         i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float, state: torch.Tensor, m_state: torch.Tensor,
         norm_w: torch.Tensor, out: torch.Tensor, heads: int, dk: int, dv: int, dvp: int, q_scale: float, eps: float) -> None:
    """All of a head's work for a step of one token per request: gates, m, [S | n] updated in place,
    quotient, unit norm, weight and gate."""
    _dev(u, z, i_bias, f_bias, state, m_state, norm_w, out)
    if z.dtype != torch.float32 or state.dtype != torch.float32 or m_state.dtype != torch.float32:
        raise TypeError("mlstm step: gate projections and states must be float32")
    _check(lib().llm_mlstm_step(u.data_ptr(), dtype_code(u.dtype), u.stride(0), q_col, k_col, v_col, g_col, z.data_ptr(),
                                z.stride(0), i_col, f_col, i_bias.data_ptr(), f_bias.data_ptr(), float(cap),
                                state.data_ptr(), m_state.data_ptr(), norm_w.data_ptr(), out.data_ptr(), out.stride(0),
                                ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr(), ctx.n_seqs,
                                heads, dk, dv, dvp, float(q_scale), float(eps), ctx.stream), "mlstm_step")
