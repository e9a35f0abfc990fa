"""Mixers with a decaying matrix state per (request, head) instead of a cache of keys and values:

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t       (S float32, in a state slot)

* "lightning_attention": q, k, v = silu of their projections; one fixed decay per head; all heads'
  outputs are RMS-normed together, multiplied by sigmoid(g) and projected.
  params: `hidden`, `heads`, `dim`, `vdim`, `decay` [heads], `eps`.
  tensors: `q`, `k`, `v`, `g`, `o`, `norm` [heads * vdim].
* "gated_linear_attention": q = projection / sqrt(dim), k, v plain; a decay per key channel from the
  token, a = sigmoid(W2 (W1 h) + b) ** (1 / tau); every head's output is RMS-normed by itself with one
  weight shared by the heads, multiplied by silu(g) and projected.
  params: `hidden`, `heads`, `dim`, `vdim`, `tau`, `rank` (-1: from the file), `eps`.
  tensors: `q`, `k`, `v`, `g`, `a1` [rank, hidden], `a2` [heads * dim, rank], `a2_bias`, `o`, `norm` [vdim].

All input projections of a mixer are one matrix product; the scan, the decays, the norms and the
gates are float32.  Both can run on their own or as a branch of "parallel" (`parts.parallel`), which
multiplies every branch's input projections as one matrix and sums the branches inside one output
projection: for that a branch states its projections in order (`PROJECTIONS`, `projection_widths`)
and computes what goes into the output projection from a view of the product (`inner`).
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import lib as K, linear_attention as LA, streams as SK
from .base import Part, StateRequest
from .linear import Linear
from .registry import register_mixer
from ..weights.loader import fused_rows


class BranchMixer(Part):
    """Common ground of mixers that can be a branch of "parallel"."""

    PROJECTIONS = ()          # local names of the input projections, in the order they are stacked
    embedded = False          # set by a parent that multiplies the projections itself
    takes_lazy_input = False

    def projection_widths(self):
        return [self.local_weights()[name][0][0] for name in self.PROJECTIONS]

    def out_width(self) -> int:
        return self.local_weights()["o"][0][1]

    def adjacent_weights(self):
        return [tuple(self.PROJECTIONS)]

    def cache_request(self):
        return None

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        self.prepare_inner(dtype, device)
        if not self.embedded:
            self.proj = Linear(fused_rows([self.tensors[n] for n in self.PROJECTIONS]), self.spec.kind + ".in")
            self.o = Linear(self.tensors["o"], self.spec.kind + ".o")
            self.proj.prepare(dtype)
            self.o.prepare(dtype)

    def forward(self, ctx, call, h):
        n = ctx.n_tokens
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        act = ctx.ws.get("mixer_act", (n, self.out_width()), ctx.dtype)
        self.inner(ctx, call.cache, call.state, call.writes_cache, u, act, 1.0)
        return self.o.forward(ctx, act, n, torch.float32, "mixer_out", allow_partials=True)


class _LinearAttention(BranchMixer):
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        if self.dim > LA.MAX_KEY_DIM:
            raise ConfigError(f"{spec.kind}: key size {self.dim} exceeds the {LA.MAX_KEY_DIM} the scan kernel takes")
        self.eps = float(p["eps"])

    def state_request(self):
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32)

    def _split(self, u):
        """Column views of the stacked projections, in `PROJECTIONS` order."""
        out, at = [], 0
        for w in self.projection_widths():
            out.append(u[:, at: at + w])
            at += w
        return out


@register_mixer("lightning_attention")
class LightningAttention(_LinearAttention):
    PROJECTIONS = ("q", "k", "v", "g")

    def local_weights(self):
        kd, vd = self.heads * self.dim, self.heads * self.vdim
        return {"q": ((kd, self.hidden), "matrix"), "k": ((kd, self.hidden), "matrix"),
                "v": ((vd, self.hidden), "matrix"), "g": ((vd, self.hidden), "matrix"),
                "o": ((self.hidden, vd), "matrix"), "norm": ((vd,), "norm")}

    def prepare_inner(self, dtype, device) -> None:
        decay = [float(x) for x in self.params["decay"]]
        if len(decay) != self.heads:
            raise ConfigError(f"lightning_attention: {len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        self.norm_w = self.tensors["norm"].to(torch.float32).contiguous()

    def inner(self, ctx, cache, state, writes, u, out, out_scale) -> None:
        n = ctx.n_tokens
        q, k, v, g = self._split(u)
        # silu on q, k and v where the projection left them (they are neighbouring columns)
        qkv = u[:, : 2 * self.heads * self.dim + self.heads * self.vdim]
        SK.activation(K.Partials(qkv), qkv, n, "silu", ctx.stream)
        o = ctx.ws.get("scan_out", (n, self.heads * self.vdim), torch.float32)
        LA.scan(ctx, q, k, v, self.decay, False, state, o, self.heads, self.dim, self.vdim)
        LA.gated_group_norm(o, g, self.norm_w, out, n, self.heads * self.vdim, "sigmoid", self.eps, out_scale, ctx.stream)


@register_mixer("gated_linear_attention")
class GatedLinearAttention(_LinearAttention):
    PROJECTIONS = ("q", "k", "v", "g", "a1")

    def local_weights(self):
        kd, vd, rank = self.heads * self.dim, self.heads * self.vdim, int(self.params.get("rank") or -1)
        return {"q": ((kd, self.hidden), "matrix"), "k": ((kd, self.hidden), "matrix"),
                "v": ((vd, self.hidden), "matrix"), "g": ((vd, self.hidden), "matrix"),
                "a1": ((rank, self.hidden), "matrix"), "a2": ((kd, rank), "unit"), "a2_bias": ((kd,), "unit"),
                "o": ((self.hidden, vd), "matrix"), "norm": ((self.vdim,), "norm")}

    def projection_widths(self):
        kd, vd = self.heads * self.dim, self.heads * self.vdim
        return [kd, kd, vd, vd, int(self.tensors["a1"].shape[0])]

    def prepare_inner(self, dtype, device) -> None:
        self.a2 = self.tensors["a2"].to(torch.float32).contiguous()
        self.a2_bias = self.tensors["a2_bias"].to(torch.float32).contiguous()
        self.norm_w = self.tensors["norm"].to(torch.float32).contiguous()
        self.tau = float(self.params["tau"])

    def inner(self, ctx, cache, state, writes, u, out, out_scale) -> None:
        n = ctx.n_tokens
        q, k, v, g, low = self._split(u)
        a = ctx.ws.get("scan_decay", (n, self.heads * self.dim), torch.float32)
        LA.decay_gate(low, self.a2, self.a2_bias, a, n, self.tau, ctx.stream)
        o = ctx.ws.get("scan_out", (n, self.heads * self.vdim), torch.float32)
        LA.scan(ctx, q, k, v, a, True, state, o, self.heads, self.dim, self.vdim, self.dim ** -0.5)
        LA.gated_group_norm(o, g, self.norm_w, out, n, self.vdim, "silu", self.eps, out_scale, ctx.stream)
