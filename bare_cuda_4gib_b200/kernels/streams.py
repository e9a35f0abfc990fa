"""Launchers of `csrc/stream_kernels.cu`: the embedding with scale and learned positions that
fills a residual kept as several streams, the kernel that writes a sublayer's result into the
streams, reads the next sublayer's input from them and norms it, and element-wise activations."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import Partials, _check, _dev, _ptr, dtype_code, stream_handle

ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}
MAX_STREAMS = 16

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("stream_kernels.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_embed_positions.argtypes = [P, P, I, P, P, P, I, I, I, F, P]
        l.llm_stream_step.argtypes = [P, I, P, I, I, L, L, P, P, P, P, P, P, I, P, I, I, F, P]
        l.llm_activation.argtypes = [P, I, I, L, L, P, I, L, I, I, I, P]
        for name in ("llm_embed_positions", "llm_stream_step", "llm_activation"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def embed_positions(table: torch.Tensor, pos_table: Optional[torch.Tensor], ids: torch.Tensor,
                    positions: torch.Tensor, out: torch.Tensor, n_tokens: int, width: int, streams: int,
                    scale: float, stream=None) -> None:
    """out[t, s, :] = table[ids[t]] * scale + pos_table[positions[t]] for every stream s (float32)."""
    _dev(table, pos_table, ids, positions, out)
    _check(lib().llm_embed_positions(table.data_ptr(), _ptr(pos_table), dtype_code(table.dtype), ids.data_ptr(),
                                     positions.data_ptr(), out.data_ptr(), n_tokens, width, streams, float(scale),
                                     stream if stream is not None else stream_handle()), "embed_positions")


class StreamWrite:
    """A sublayer's result that is not in the streams yet, with what writing it takes: `y` (a
    `Partials` [rows, width]), `scale` [width] or None, `write` [streams] and `mix` [streams,
    streams] indexed [from, to] (None: every stream keeps itself)."""

    __slots__ = ("y", "scale", "write", "mix")

    def __init__(self, y: Partials, scale, write, mix):
        self.y, self.scale, self.write, self.mix = y, scale, write, mix


def stream_step(streams_buf: torch.Tensor, n_streams: int, pending: Optional[StreamWrite],
                read: Optional[torch.Tensor], weight: Optional[torch.Tensor], out: Optional[torch.Tensor],
                eps: float, rows: int, width: int, row_index: Optional[torch.Tensor] = None, stream=None) -> None:
    """Writes `pending` into the streams ([tokens, streams, width] float32), then
    out = rms_norm(sum_t read[t] x_t) * weight (`read` None: the plain sum)."""
    y = pending.y if pending is not None else None
    yt = y.tensor if y is not None else None
    _dev(streams_buf, yt, read, weight, out)
    _check(lib().llm_stream_step(
        streams_buf.data_ptr(), n_streams, _ptr(yt), dtype_code(yt.dtype) if yt is not None else 0,
        y.n if y is not None else 0, y.stride if y is not None else 0, yt.stride(-2) if yt is not None else 0,
        _ptr(pending.scale) if pending is not None else 0, _ptr(pending.write) if pending is not None else 0,
        _ptr(pending.mix) if pending is not None else 0, _ptr(read), _ptr(weight), _ptr(out),
        dtype_code(out.dtype) if out is not None else 0, _ptr(row_index), rows, width, float(eps),
        stream if stream is not None else stream_handle()), "stream_step")


def activation(x: Partials, out: torch.Tensor, rows: int, kind: str, stream=None) -> None:
    """out = act(sum of the partial results of x), element by element."""
    _dev(x.tensor, out)
    _check(lib().llm_activation(x.tensor.data_ptr(), dtype_code(x.tensor.dtype), x.n, x.stride, x.tensor.stride(-2),
                                out.data_ptr(), dtype_code(out.dtype), out.stride(-2), rows, out.shape[-1],
                                ACTIVATIONS[kind], stream if stream is not None else stream_handle()), "activation")
