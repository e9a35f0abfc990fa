"""Several mixers side by side on the same input, summed with fixed weights:

    result = sum_b scale_b * branch_b(h)

Every branch is a mixer of its own kind (`parts.linear_attention.BranchMixer`).  Because all read
the same h and all end in a projection back to the model's width, the input projections of all
branches are ONE matrix product (their weights stacked, adjacent in memory), and the sum of the
branches is ONE output projection over the branches' gated outputs laid side by side, each already
multiplied by its scale: sum_b scale_b Wo_b a_b = [Wo_0 | Wo_1 | ...] [scale_0 a_0; scale_1 a_1; ...].

What each branch keeps per request (pages, state) is stated branch by branch, in order.

params: `hidden`, `branches` (a list of mixer `PartSpec`s), `scales`.  tensors: none of its own
(it binds the branches' projections a second time, under "<branch index>.<name>").
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from .base import Part
from .linear import Linear
from .registry import build_part, register_mixer
from ..weights.loader import fused_rows


@register_mixer("parallel")
class ParallelMixers(Part):
    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        self.branches = [build_part("mixer", b) for b in self.params["branches"]]
        self.scales = [float(s) for s in self.params["scales"]]
        if len(self.scales) != len(self.branches) or not self.branches:
            raise ConfigError("parallel: one scale per branch is needed")
        for b in self.branches:
            if not hasattr(b, "inner"):
                raise ConfigError(f"parallel: mixer '{b.spec.kind}' cannot run as a branch")
            b.embedded = True

    def children(self):
        return list(self.branches)

    def _names(self):
        return [(f"{i}.{name}", b, name) for i, b in enumerate(self.branches) for name in tuple(b.PROJECTIONS) + ("o",)]

    def local_weights(self):
        return {mine: b.local_weights()[name] for mine, b, name in self._names()}

    def weight_specs(self):
        out = {}
        for mine, b, name in self._names():
            out[mine] = b.weight_specs()[name]
        return out

    def adjacent_weights(self):
        return [tuple(mine for mine, _b, name in self._names() if name != "o")]

    def cache_demands(self):
        return [(b.cache_request(), b.state_request()) for b in self.branches]

    def cache_request(self):
        return self.branches[0].cache_request()

    def state_request(self):
        return self.branches[0].state_request()

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(fused_rows([t[mine] for mine, _b, name in self._names() if name != "o"]), "parallel.in")
        outs = [t[f"{i}.o"] for i in range(len(self.branches))]
        self.o = Linear(torch.cat(outs, dim=1).contiguous(), "parallel.o")
        self.proj.prepare(dtype)
        self.o.prepare(dtype)
        self.tensors = {}

    def forward(self, ctx, call, h):
        n = ctx.n_tokens
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        widths = [b.out_width() for b in self.branches]
        act = ctx.ws.get("mixer_act", (n, sum(widths)), ctx.dtype)
        at_in = at_out = 0
        for j, b in enumerate(self.branches):
            w_in = sum(b.projection_widths())
            b.inner(ctx, call.caches[j], call.states[j], call.writes_cache, u[:, at_in: at_in + w_in],
                    act[:, at_out: at_out + widths[j]], self.scales[j])
            at_in += w_in
            at_out += widths[j]
        return self.o.forward(ctx, act, n, torch.float32, "mixer_out", allow_partials=True)
