"""A residual kept as several parallel streams (hyper-connections), and the plain residual with a
per-channel scale on every sublayer's result as the one-stream case.

For a sublayer with read vector r [S], write vector w [S], mixing matrix M [S, S] (indexed
[from, to]) and per-channel scale g:

    u = sum_s r[s] x_s;   y = g * sublayer(norm(u));   x_t <- sum_s M[s, t] x_s + w[t] y   (all t at once)

The streams are float32 [tokens, S * width].  As with the plain residual of `parts.norm`, writing a
result and reading (and norming) the next sublayer's input are one kernel: a block hands its last
result on unwritten (`StreamWrite`), and the norm that reads the streams next writes it first.  The
model's final norm reads the plain sum of the streams.

Parts: norm "stream_rmsnorm" (params `size`, `eps`, `streams`, `read`: "vector" | "sum"; tensors
`weight`, and `read` [streams] with "vector"), `stream_write` (what a sublayer's result is written
with: params `size`, `streams`, `mixing`; tensors `scale` [size], and with `mixing` also `write`
[streams], `mix` [streams, streams]), block "stream_prenorm".
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import streams as SK
from .base import Part
from .registry import build_part, register_block, register_norm


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.to(torch.float32).contiguous()


@register_norm("stream_rmsnorm")
class StreamRMSNorm(Part):
    def local_weights(self):
        out = {"weight": ((int(self.params["size"]),), "norm")}
        if self.params.get("read", "sum") == "vector":
            out["read"] = ((int(self.params["streams"]),), "norm")
        return out

    def prepare(self, dtype, device) -> None:
        self.weight = _f32(self.tensors["weight"])
        self.read = _f32(self.tensors.get("read"))

    def forward(self, ctx, residual: torch.Tensor, delta: Optional[SK.StreamWrite], rows: int,
                row_index: Optional[torch.Tensor] = None, buffer: str = "normed", lazy: bool = False):
        size = int(self.params["size"])
        out = ctx.ws.get(buffer, (rows, size), ctx.dtype)
        SK.stream_step(residual, int(self.params.get("streams") or 1), delta, self.read, self.weight, out,
                       float(self.params["eps"]), rows, size, row_index, ctx.stream)
        return out


class StreamWriter(Part):
    """How one sublayer's result goes into the streams."""

    def local_weights(self):
        size, s = int(self.params["size"]), int(self.params.get("streams") or 1)
        out = {"scale": ((size,), "norm")}
        if self.params.get("mixing"):
            out["write"] = ((s,), "norm")
            out["mix"] = ((s, s), "identity")
        return out

    def prepare(self, dtype, device) -> None:
        self.scale = _f32(self.tensors["scale"])
        self.write = _f32(self.tensors.get("write"))
        self.mix = _f32(self.tensors.get("mix"))

    def pending(self, y) -> SK.StreamWrite:
        return SK.StreamWrite(y, self.scale, self.write, self.mix)


@register_block("stream_prenorm")
class StreamPreNormBlock:
    """x <- write1(mixer(norm1(read1(x)))), then (if the layer has a feed-forward) the same with
    the second set.  `layer_spec.extras` names the writers: "write1", "write2"."""

    def __init__(self, layer_spec):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.write1 = StreamWriter(layer_spec.extras["write1"])
        self.has_ffn = layer_spec.ffn is not None
        if self.has_ffn:
            self.ffn_norm = build_part("norm", layer_spec.ffn_norm)
            self.ffn = build_part("feed_forward", layer_spec.ffn)
            self.write2 = StreamWriter(layer_spec.extras["write2"])

    def parts(self):
        out = [self.mixer_norm, self.mixer, self.write1]
        if self.has_ffn:
            out += [self.ffn_norm, self.ffn, self.write2]
        return out

    def cache_demands(self):
        many = getattr(self.mixer, "cache_demands", None)
        return many() if many else [(self.mixer.cache_request(), self.mixer.state_request())]

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, ctx, call, residual, pending):
        n = ctx.n_tokens
        ctx.residual = None          # sublayers hand their result back; the streams are written by the norms
        ctx.following_norm = None
        h = self.mixer_norm.forward(ctx, residual, pending, n)
        pending = self.write1.pending(self.mixer.forward(ctx, call, h))
        if self.has_ffn:
            h = self.ffn_norm.forward(ctx, residual, pending, n)
            pending = self.write2.pending(self.ffn.forward(ctx, h))
        return pending
