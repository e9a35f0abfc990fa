"""The matrix memory of xLSTM (mLSTM) as a mixer over state slots.

Per head, q = Wq h / sqrt(dim), k = Wk h, v = Wv h, log gates i = cap tanh((Wi h + bi) / cap) and
f = logsigmoid(cap tanh((Wf h + bf) / cap)), a running maximum m (0 at the start):

    m_t = max(f + m_(t-1), i);  S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;  n_t likewise with k;
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

Every head's o is divided by its root mean square, the heads are concatenated, multiplied by `norm`
and by sigmoid(Wg h), then projected.  A request keeps S and n together as one float32 state
[heads, dim, vdim + pad] (n is the column behind the values) and m as a second one [heads].  The
walk over a step's tokens is the engine's state scan (`kernels.linear_attention.scan`), fed with
float32 operands; the kernels of csrc/mlstm.cu come before and after it.

params: `hidden`, `heads`, `dim`, `vdim`, `gate_cap`, `eps`.
tensors: `q`, `k` [heads * dim, hidden], `v`, `g` [heads * vdim, hidden], `o` [hidden, heads * vdim],
`norm` [heads * vdim], `i`, `f` [heads, hidden], `i_bias`, `f_bias` [heads].
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import linear_attention as LA, mlstm as MK
from .base import Part, StateRequest
from .linear import Linear
from .registry import register_mixer
from ..weights.loader import fused_rows


@register_mixer("mlstm")
class MLSTM(Part):
    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        if self.dim > LA.MAX_KEY_DIM:
            raise ConfigError(f"mlstm: key size {self.dim} exceeds the {LA.MAX_KEY_DIM} the scan kernel takes")
        self.cap, self.eps = float(p["gate_cap"]), float(p["eps"])
        self.vpad = (self.vdim + 1 + 3) // 4 * 4          # values, the column of n, zeros up to a multiple of four

    def local_weights(self):
        kd, vd, w, H = self.heads * self.dim, self.heads * self.vdim, self.hidden, self.heads
        return {"q": ((kd, w), "matrix"), "k": ((kd, w), "matrix"), "v": ((vd, w), "matrix"), "g": ((vd, w), "matrix"),
                "o": ((w, vd), "matrix"), "norm": ((vd,), "norm"), "i": ((H, w), "matrix"), "f": ((H, w), "matrix"),
                "i_bias": ((H,), "unit"), "f_bias": ((H,), "unit")}

    def adjacent_weights(self):
        return [("q", "k", "v", "g"), ("i", "f")]

    def cache_request(self):
        return None

    def state_request(self):
        return StateRequest((self.heads, self.dim, self.vpad), torch.float32)

    def cache_demands(self):
        """Two states per request: [S | n] and m."""
        return [(None, self.state_request()), (None, StateRequest((self.heads,), torch.float32))]

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(fused_rows([t["q"], t["k"], t["v"], t["g"]]), "mlstm.in")
        self.gates = Linear(fused_rows([t["i"], t["f"]]), "mlstm.gates")
        self.o = Linear(t["o"], "mlstm.o")
        for lin in (self.proj, self.gates, self.o):
            lin.prepare(dtype)
        self.i_bias, self.f_bias = t["i_bias"].to(dtype).contiguous(), t["f_bias"].to(dtype).contiguous()
        self.norm_w = t["norm"].to(dtype).contiguous()

    def forward(self, ctx, call, h):
        n, H, dk, dv, dvp = ctx.n_tokens, self.heads, self.dim, self.vdim, self.vpad
        kd, vd = H * dk, H * dv
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        z = self.gates.forward(ctx, h, n, torch.float32, "mlstm_gates").tensor
        out = ctx.ws.get("mixer_act", (n, vd), ctx.dtype)
        if ctx.max_q_len == 1 and MK.step_takes(dk, dvp):
            # one token per request: one kernel per step instead of gates, operands, scan and finish
            MK.step(ctx, u, 0, kd, 2 * kd, 2 * kd + vd, z, 0, H, self.i_bias, self.f_bias, self.cap, call.states[0],
                    call.states[1], self.norm_w, out, H, dk, dv, dvp, dk ** -0.5, self.eps)
            return self.o.forward(ctx, out, n, torch.float32, "mixer_out", allow_partials=True)
        coef = ctx.ws.get("mlstm_coef", (n, H * 4), torch.float32)
        MK.gates(ctx, z, 0, H, self.i_bias, self.f_bias, self.cap, call.states[1], coef, H)
        qf = ctx.ws.get("mlstm_q", (n, kd), torch.float32)
        kf = ctx.ws.get("mlstm_k", (n, kd), torch.float32)
        decay = ctx.ws.get("mlstm_decay", (n, H), torch.float32)
        vf = ctx.ws.get("mlstm_v", (n, H * dvp), torch.float32)
        MK.operands(ctx, u, 0, kd, 2 * kd, coef, qf, kf, decay, vf, H, dk, dv, dvp)
        scanned = ctx.ws.get("mlstm_scan", (n, H * dvp), torch.float32)
        LA.scan(ctx, qf, kf, vf, decay, "token", call.states[0], scanned, H, dk, dvp, dk ** -0.5)
        MK.finish(ctx, scanned, coef, self.norm_w, u[:, 2 * kd + vd:], out, H, dv, dvp, self.eps)
        return self.o.forward(ctx, out, n, torch.float32, "mixer_out", allow_partials=True)
