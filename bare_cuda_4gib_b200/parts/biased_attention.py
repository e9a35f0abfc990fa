"""Causal softmax attention over the paged cache with a learned bias by distance, for designs that
put no rotation on q and k:

    q, k, v = projections, each passed through a short causal convolution over time (per channel,
              `taps` taps, zeros before the sequence's start);
    q <- rms_norm(all of q) * wq * (1 + coef * ln(floor((p + 1) / every) + 1)) at position p;
    k <- rms_norm(all of k) * wk                                  (norms over all heads at once)
    score(i, j) = (q_i . k_j) * scale + rel[bucket(i - j), head];   softmax over j <= i.

bucket(n) = n below half the table's rows R/2, then R/2 + floor(ln(n / (R/2)) / ln(far / (R/2)) *
(R - R/2)), at most R - 1.  The table is expanded once per layer into a bias per (head, distance),
which the attention kernel reads by distance.  Key heads and value heads may differ in size.

Per request the mixer keeps its keys and values in pages and the convolution's last taps - 1
inputs in a state slot.

params: `hidden`, `heads`, `kv_heads`, `dim`, `vdim`, `taps`, `scale`, `bias_far`, `bias_rows`
(-1: from the file), `temp_coef`, `temp_every`, `eps`, `max_positions`, `window` (None: every key).
tensors: `q`, `k`, `v`, `o`, `q_norm`, `k_norm`, `q_conv`, `k_conv`, `v_conv` ([channels, taps]),
`rel` [rows, heads].
"""

from __future__ import annotations

import math

import torch

from ..errors import ConfigError
from ..kernels import biased_attention as BA
from .base import KVCacheRequest, StateRequest
from .linear_attention import BranchMixer
from .registry import register_mixer


def distance_rows(distances: int, rows: int, far: float):
    """For every distance 0 .. distances - 1 the row of a table with `rows` rows: exact up to half
    the table, logarithmic from there to `far`, the last row beyond."""
    half = rows // 2
    if rows < 1 or (half > 0 and not far > half):
        raise ConfigError(f"distance bias: a table of {rows} rows needs a far distance above {half}, got {far}")
    out = []
    for n in range(distances):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
        else:
            step = math.log(n / half) / math.log(far / half) * (rows - half)
            out.append(min(rows - 1, half + int(math.floor(step))))
    return out


@register_mixer("biased_attention")
class BiasedAttention(BranchMixer):
    PROJECTIONS = ("q", "k", "v")

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["taps"])
        if self.heads % self.kv_heads:
            raise ConfigError(f"biased_attention: {self.heads} heads cannot share {self.kv_heads} key/value heads")
        if self.vdim > 256:
            raise ConfigError(f"biased_attention: value head size {self.vdim} exceeds the 256 the kernel takes")
        self.window = p.get("window")
        self.qd, self.kd, self.vd = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim

    def local_weights(self):
        rows = int(self.params.get("bias_rows") or -1)
        return {"q": ((self.qd, self.hidden), "matrix"), "k": ((self.kd, self.hidden), "matrix"),
                "v": ((self.vd, self.hidden), "matrix"), "o": ((self.hidden, self.heads * self.vdim), "matrix"),
                "q_norm": ((self.qd,), "norm"), "k_norm": ((self.kd,), "norm"),
                "q_conv": ((self.qd, self.taps), "unit"), "k_conv": ((self.kd, self.taps), "unit"),
                "v_conv": ((self.vd, self.taps), "unit"), "rel": ((rows, self.heads), "unit")}

    def cache_request(self):
        return KVCacheRequest(self.kv_heads, self.dim, self.window, None if self.vdim == self.dim else self.vdim)

    def state_request(self):
        return StateRequest((max(self.taps - 1, 1), self.qd + self.kd + self.vd), torch.float32)

    def prepare_inner(self, dtype, device) -> None:
        t = self.tensors
        f = lambda x: x.to(torch.float32).contiguous()
        self.conv_w = f(torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], 0))
        self.q_norm_w, self.k_norm_w = f(t["q_norm"]), f(t["k_norm"])
        rel = t["rel"].to(torch.float32).cpu()
        rows = distance_rows(int(self.params["max_positions"]), rel.shape[0], float(self.params["bias_far"]))
        assert 0 <= min(rows) and max(rows) < rel.shape[0]
        # gathered on the host (every index checked there), then one copy: [heads, distances]
        self.bias = rel[torch.tensor(rows)].t().contiguous().to(device)
        # bfloat16 steps with key and value heads of one size the tensor-core kernel is built for run
        # there; everything else (float32, other sizes) runs the plain kernel
        self.fast = None
        if dtype == torch.bfloat16 and device.type == "cuda" and self.dim == self.vdim:
            from ..kernels import attention as fast
            self.fast = fast.plan_for(self.dim, self.heads, self.kv_heads, distance_bias=True)

    def plan_step(self, ctx) -> None:
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.step_tiles(ctx, self.fast)

    def inner(self, ctx, cache, state, writes, u, out, out_scale) -> None:
        n, p = ctx.n_tokens, self.params
        q = ctx.ws.get("biased_q", (n, self.qd), ctx.dtype)
        BA.conv_norm_cache(ctx, u, self.conv_w, state, self.q_norm_w, self.k_norm_w, q, cache, self.heads,
                           float(p["eps"]), float(p["temp_coef"]), int(p["temp_every"]), writes)
        if writes:
            BA.conv_ring_write(ctx, u, state, self.taps, self.qd + self.kd + self.vd)
        window = int(self.window) if self.window else 0
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            if fast.usable_with_bias(out, cache):
                fast.run(ctx, self.fast, q, out, cache, float(p["scale"]), window, self.bias, out_scale)
                return
        BA.attention(ctx, q, out, cache, self.bias, self.heads, float(p["scale"]), window, out_scale)
