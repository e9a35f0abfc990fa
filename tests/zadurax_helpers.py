"""Small Zadurax configurations with random weights made here (names and shapes written out from
the configuration, independent of the engine's own list), their model folders, and the comparison
of replayed logits with the plain implementation."""

from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import torch

import helpers as H
import plain_zadurax as P


def _mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def attention(heads, kv_heads, dim, window, rot_dims, base=10000.0, scale=None, ff=None):
    return {"type": "attention", "mlp": _mlp(ff),
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dims}, "scale": dim ** -0.5 if scale is None else scale}}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None, ff=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"type": "latent_attention", "mlp": _mlp(ff),
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": rot,
                      "scale": scale}}


def mlstm(heads, dim, vdim, cap, ff=None):
    return {"type": "mlstm", "mlp": _mlp(ff), "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def again(layers, j):
    return dict(json.loads(json.dumps(layers[j])), weights_of=j)


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _cfg_p():
    layers = [attention(4, 2, 16, 24, 8, ff=80),
              mlstm(3, 8, 20, 15.0),
              latent(3, 12, 8, 20, 24, 0.2, base=5000.0, scaling=yarn(4.0, 64, 16.0, 2.0), ff=48)]
    layers += [again(layers, 2), again(layers, 0), again(layers, 1)]
    return {"architecture": "Zadurax", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "layers": layers}


def _cfg_q():
    layers = [latent(2, 24, 16, 8, 64, 0.15, base=100.0, ff=64),            # no scaling of the frequencies
              attention(2, 2, 64, 40, 64, base=500.0, scale=0.1),            # as many key heads as heads, all entries turned
              mlstm(1, 32, 8, 6.0, ff=72),
              attention(6, 1, 32, 1000, 2, ff=40)]                           # a window wider than any request
    layers += [again(layers, 1)]
    return {"architecture": "Zadurax", "vocab": 77, "width": 96, "norm": {"eps": 1e-6}, "layers": layers}


CFG_P, CFG_Q = _cfg_p(), _cfg_q()
CONFIGS = {"P": (CFG_P, 16), "Q": (CFG_Q, 32)}


def tensor_shapes(cfg) -> Dict[str, Tuple[int, ...]]:
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "embed.norm": (W,), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,)})
        if layer["type"] == "attention":
            qd, kd = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            out.update({p + "mix.q": (qd, W), p + "mix.k": (kd, W), p + "mix.g": (qd, W), p + "mix.o": (W, qd),
                        p + "mix.q.norm": (m["dim"],), p + "mix.k.norm": (m["dim"],)})
        elif layer["type"] == "latent_attention":
            H_, d, r, e, k = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H_ * (d + r), W), p + "mix.dkv": (k + r, W), p + "mix.dkv.norm": (k,),
                        p + "mix.uk": (H_ * d, k), p + "mix.uv": (H_ * e, k), p + "mix.sink": (H_,),
                        p + "mix.g": (H_ * e, W), p + "mix.o": (W, H_ * e)})
        else:
            kd, vd = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + "mix.q": (kd, W), p + "mix.k": (kd, W), p + "mix.v": (vd, W), p + "mix.g": (vd, W),
                        p + "mix.o": (W, vd), p + "mix.norm": (vd,), p + "mix.i": (m["heads"], W),
                        p + "mix.i.b": (m["heads"],), p + "mix.f": (m["heads"], W), p + "mix.f.b": (m["heads"],)})
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "norm2b": (W,), p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W),
                        p + "mlp.down": (W, ff)})
    return out


def random_tensors(cfg, seed: int) -> Dict[str, torch.Tensor]:
    """Values of a size that keeps every activation of order one; bfloat16, as files store them."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        x = torch.randn(shape, generator=g)
        last = name.rsplit(".", 1)[-1]
        if len(shape) == 1 and (last.startswith("norm") or name.endswith(".norm")):
            x = 1.0 + 0.2 * x
        elif last == "sink":
            x = 1.5 * x
        elif name.endswith("f.b"):
            x = 3.0 + x
        elif name.endswith("i.b"):
            x = 0.5 * x
        elif len(shape) == 2 and name != "embed":
            x = x / shape[1] ** 0.5
        out[name] = x.to(torch.bfloat16)
    return out


def write_folder(folder, cfg, tensors) -> None:
    from bare_cuda_4gib_b200.weights.safetensors_io import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    write_safetensors(folder / "model.safetensors", tensors)
    (folder / "config.json").write_text(json.dumps(cfg))


_tensors: Dict[str, Dict[str, torch.Tensor]] = {}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 3):
    cfg, _page = CONFIGS[name]
    folder = H.tmp_root() / f"zadurax{name}-{seed}"
    register(folder, cfg, random_tensors(cfg, seed))
    return folder


def register(folder, cfg, tensors) -> None:
    write_folder(folder, cfg, tensors)
    _tensors[str(folder)] = tensors


# Per logits row: max |got - want| / max |want| against the float64 plain implementation.  A logic
# fault (a key, a window's edge, a state or a sink lost or shifted) shows at 1e-2 and more in float32,
# where every row has to be within the tolerance.  In bfloat16 single rows are ill-conditioned: while
# one token dominates a matrix memory, a head's output is sign(q . k) times that token's value after
# the unit norm, and rounding can turn the sign of a small q . k.  So a bfloat16 run has to have
# `BF16_SHARE` of its rows within the tolerance and none beyond `BF16_WORST`.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}
BF16_SHARE, BF16_WORST = 0.97, 0.6

_plain: Dict[Tuple, torch.Tensor] = {}


def plain_logits(folder, ids: Sequence[int]) -> torch.Tensor:
    key = (str(folder), tuple(ids))
    if key not in _plain:
        cfg = json.loads((folder / "config.json").read_text())
        _plain[key] = P.forward(cfg, _tensors[str(folder)], list(ids))
    return _plain[key]


def check(folder, requests: Dict[str, List[int]], got, dtype: str, expect_all: bool = True) -> None:
    errors = []
    for rid, ids in requests.items():
        want = plain_logits(folder, ids)
        places = sorted(p for (r, p) in got if r == rid)
        if expect_all:
            assert places == list(range(len(ids))), f"request {rid}: places {places}"
        for p in places:
            err = H.row_error(got[(rid, p)], want[p])
            errors.append(err)
            if dtype == "float32":
                assert err <= TOLERANCE[dtype], f"request {rid} position {p} of {len(ids)}: error {err:.3e}"
    if dtype != "float32":
        errors.sort()
        over = sum(e > TOLERANCE[dtype] for e in errors)
        assert errors[-1] <= BF16_WORST, f"worst row: error {errors[-1]:.3e}"
        assert over <= (1.0 - BF16_SHARE) * len(errors) or over <= 1, \
            f"{over} of {len(errors)} rows beyond {TOLERANCE[dtype]:.0e}: {errors[-5:]}"


def check_most(folder, requests: Dict[str, List[int]], got, dtype: str, share: float = 0.9, worst: float = 2.0) -> None:
    """For configurations drawn at random in bfloat16 (gates, caps and sizes of any kind, where a
    matrix memory may be one token's for long): `share` of the rows within the tolerance, none beyond
    `worst`; that the fast kernels compute what the plain ones do is checked row by row beside this."""
    errors = sorted(H.row_error(got[(rid, p)], plain_logits(folder, requests[rid])[p]) for (rid, p) in got)
    assert errors[-1] <= worst, f"worst row: error {errors[-1]:.3e}"
    at = min(len(errors) - 1, int(share * len(errors)))
    assert errors[at] <= TOLERANCE[dtype], f"{share:.0%} of the rows: error {errors[at]:.3e}"
