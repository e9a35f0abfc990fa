"""A plain, slow restatement of the Zadurax decoder in float64 torch, one function per mechanism.

It shares no code with the engine: tensors come in as a dictionary by file name, the configuration
as the dictionary that config.json holds, tokens as a list.  Everything is computed for a whole
sequence at once (or token by token where a recurrence says so), with no cache.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """Angle per position of every rotated pair, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot):
    """x [tokens, heads, d]: the first rot.dims entries of every head turned pair by pair
    (entry 2i with entry 2i + 1); the rest unchanged."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    a = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_attention(q, k, v, scale, window=None, sink=None):
    """q [T, H, d], k [T, H, d], v [T, H, e] (already one key head per query head).  Token i sees
    j <= i, and with `window` only i - j < window.  `sink` [H] adds exp(sink) to the denominator."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    s = s.masked_fill(~seen[None], -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.to(F64)[:, None, None])
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(F64)[:, None, None] - top)
    return torch.einsum("hij,jhe->ihe", e / den, v)


def windowed_attention(h, w, m, eps, positions):
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = k.clone()
    q = rotate_pairs(rms_norm(q, w["q.norm"], eps), positions, m["rot"])
    k = rotate_pairs(rms_norm(k, w["k.norm"], eps), positions, m["rot"])
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    o = softmax_attention(q, k, v, float(m["scale"]), window=int(m["mask"]["size"]))
    o = o.reshape(T, -1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def latent_attention(h, w, m, eps, positions):
    H, d, r, e, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, d + r)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, None, rank:], positions, m["rot"])
    q_rot = rotate_pairs(q[..., d:], positions, m["rot"])
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, e)
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, r)], -1)
    o = softmax_attention(qq, kk, v, float(m["scale"]), sink=w["sink"])
    o = o.reshape(T, -1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def mlstm(h, w, m, eps):
    H, d, e, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, e)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    S = torch.zeros(H, d, e, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    top = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, e, dtype=F64)
    for t in range(T):
        new = torch.maximum(gf[t] + top, gi[t])
        keep, take = torch.exp(gf[t] + top - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        top = new
        num = torch.einsum("hde,hd->he", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-top)) + 1e-6
        out[t] = num / den[:, None]
    o = rms_unit(out, eps).reshape(T, -1) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def feed_forward(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def sub(tensors, prefix):
    """The tensors whose names start with `prefix`, by the rest of their name, in float64."""
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, layers_out=None):
    """Logits [tokens, vocab] for one sequence.  `layers_out`, a list, receives the residual
    stream after every layer run."""
    eps = float(config["norm"]["eps"])
    t = {k: v.to(F64) for k, v in tensors.items()}
    positions = torch.arange(len(tokens))
    x = rms_norm(t["embed"][torch.tensor(tokens)], t["embed.norm"], eps)
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        name = f"l{src}."
        m = layer["mixer"]
        h = rms_norm(x, t[name + "norm1"], eps)
        w = sub(tensors, name + "mix.")
        if layer["type"] == "attention":
            y = windowed_attention(h, w, m, eps, positions)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, m, eps, positions)
        elif layer["type"] == "mlstm":
            y = mlstm(h, w, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, t[name + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, t[name + "norm2"], eps)
            x = x + rms_norm(feed_forward(h, sub(tensors, name + "mlp.")), t[name + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T
