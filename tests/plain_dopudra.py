"""A plain, slow restatement of the Dopudra decoder in float64 torch on the CPU: one function per
mechanism, a token loop wherever the definition is a recurrence, no cache and no batching.  It
shares no code with the engine; the tests compare the engine against it.

Notation: h [T, width] is a sublayer's input for one sequence whose positions are 0 .. T-1;
weights come as a dictionary from tensor name to tensor, linear weights stored [out, in].
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the learned distance table for a key n positions back: one row per distance below
    half the table, then logarithmic steps up to `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y += padded[j: j + T] * w[:, j]
    return y


def lightning_mixer(h, w, p, cfg, eps):
    """Linear attention with one fixed decay per head, silu on q, k and v, a norm over all heads
    together and a sigmoid gate."""
    H, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).view(T, H, dk)
    k = silu(h @ w[p + "k"].T).view(T, H, dk)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(cfg["decay"], dtype=F)
    S = torch.zeros(H, dk, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms(o.reshape(T, H * dv), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def biased_attention(h, w, p, cfg, eps):
    """Softmax attention whose q, k and v pass a short causal convolution, whose q and k are
    normed over the whole projection, with a query factor that grows with the position and a
    learned bias per (distance bucket, head)."""
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = short_conv(h @ w[p + "q"].T, w[p + "q.conv"])
    k = short_conv(h @ w[p + "k"].T, w[p + "k.conv"])
    v = short_conv(h @ w[p + "v"].T, w[p + "v.conv"])
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    temp = torch.tensor([query_temperature(t, cfg["q_temp"]["coef"], cfg["q_temp"]["every"]) for t in range(T)], dtype=F)
    q = (q * temp[:, None]).view(T, H, dk)
    k = k.view(T, G, dk)
    v = v.view(T, G, dv)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    by_distance = rel[[distance_bucket(n, rows, cfg["bias_max"]) for n in range(T)]]      # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, head]) * cfg["scale"] + by_distance[: i + 1, head].flip(0)
            out[i, head] = torch.softmax(s, 0) @ v[: i + 1, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def gated_linear_attention(h, w, p, cfg, eps):
    """Linear attention whose state decays per key channel by a factor computed from the token."""
    H, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T * dk ** -0.5).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / cfg["tau"]).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = (rms(o, eps) * w[p + "norm"]).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, cfg, eps):
    return (cfg["left_scale"] * biased_attention(h, w, p + "left.", cfg["left"], eps)
            + cfg["right_scale"] * gated_linear_attention(h, w, p + "right.", cfg["right"], eps))


def dense_ff(h, w, p):
    return torch.relu(h @ w[p + "up"].T).square() @ w[p + "down"].T


def stream_sublayer(xs, w, layer, q, norm_w, eps, fn):
    """xs [S, T, width]: reads one input from the streams, runs the sublayer on its norm, mixes the
    streams and writes the (layer-scaled) result back into each."""
    u = torch.einsum("s,stc->tc", w[f"{layer}.hc{q}.in"], xs)
    y = fn(rms(u, eps) * norm_w) * w[f"{layer}.ls{q}"]
    return torch.einsum("st,sjc->tjc", w[f"{layer}.hc{q}.mix"], xs) + w[f"{layer}.hc{q}.out"][:, None, None] * y


def forward(config, weights, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence (float64); with `want_layers` also the sum of the streams
    after every layer [layers, T, width]."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"] + w["pos"][:T]
    S = config["streams"]
    xs = x[None].repeat(S, 1, 1)
    after = []
    for i, layer in enumerate(config["layers"]):
        name = f"l{i}"
        mixer = {"lightning": lightning_mixer, "parallel": parallel_mixer}[layer["type"]]
        xs = stream_sublayer(xs, w, name, 1, w[name + ".norm1"], eps,
                             lambda h: mixer(h, w, name + ".mix.", layer["mixer"], eps))
        if layer["mlp"] is not None:
            xs = stream_sublayer(xs, w, name, 2, w[name + ".norm2"], eps, lambda h: dense_ff(h, w, name + ".mlp."))
        after.append(xs.sum(0))
    logits = (rms(xs.sum(0), eps) * w["final.norm"]) @ w["head"].T
    return (logits, torch.stack(after)) if want_layers else logits
