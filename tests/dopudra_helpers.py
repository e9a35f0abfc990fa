"""Small Dopudra configurations with random weights made here (names and shapes written out from
the configuration, independent of the engine's own list), their model folders, and the comparison
of replayed logits with the plain implementation."""

from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import torch

import helpers as H
import plain_dopudra as P


def lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def parallel(left, right, left_scale, right_scale, ff=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def left(heads, kv_heads, dim, vdim, conv, scale, bias_max, coef, every):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
            "bias_max": bias_max, "q_temp": {"coef": coef, "every": every}}


def right(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


# Three streams, grouped heads with one key/value head, key and value heads of different sizes in
# both branches, an odd number of bias rows, a decay of exactly one.
CFG_X = {"architecture": "Dopudra", "vocab": 97, "width": 64, "max_positions": 160, "streams": 3,
         "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
         "layers": [parallel(left(4, 1, 16, 24, 3, 0.2, 50, 0.3, 7), right(2, 24, 16, 4.0), 0.7, 1.3, ff=80),
                    lightning(3, 16, 8, [1.0, 0.9, 0.5]),
                    lightning(2, 8, 32, [0.99, 0.7], ff=48)]}
# One stream, a convolution of one tap, no position factor, as many key/value heads as heads, a
# key size that is no power of two, one head, tau 1.
CFG_Y = {"architecture": "Dopudra", "vocab": 130, "width": 96, "max_positions": 256, "streams": 1,
         "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
         "layers": [lightning(2, 40, 40, [0.97, 0.3], ff=64),
                    parallel(left(2, 2, 32, 32, 1, 0.25, 20, 0.0, 1), right(1, 8, 64, 1.0), 1.0, 0.5),
                    parallel(left(6, 3, 8, 16, 5, 0.5, 100, 1.0, 32), right(3, 16, 16, 9.0), 1.5, 1.0, ff=40)]}
CONFIGS = {"X": (CFG_X, 16, {"rank": 5, "rows": 7}), "Y": (CFG_Y, 32, {"rank": 8, "rows": 16})}


def tensor_shapes(cfg, rank: int, rows: int) -> Dict[str, Tuple[int, ...]]:
    W, S = cfg["width"], cfg["streams"]
    out = {"embed": (cfg["vocab"], W), "pos": (cfg["max_positions"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = [1] + ([2] if layer["mlp"] else [])
        for q in subs:
            out.update({f"{p}norm{q}": (W,), f"{p}ls{q}": (W,), f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,),
                        f"{p}hc{q}.mix": (S, S)})
        if layer["type"] == "lightning":
            kd, vd = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + "mix.q": (kd, W), p + "mix.k": (kd, W), p + "mix.v": (vd, W), p + "mix.g": (vd, W),
                        p + "mix.o": (W, vd), p + "mix.norm": (vd,)})
        else:
            l, r = m["left"], m["right"]
            qd, kd, vd = l["heads"] * l["dim"], l["kv_heads"] * l["dim"], l["kv_heads"] * l["vdim"]
            out.update({p + "mix.left.q": (qd, W), p + "mix.left.k": (kd, W), p + "mix.left.v": (vd, W),
                        p + "mix.left.q.norm": (qd,), p + "mix.left.k.norm": (kd,),
                        p + "mix.left.q.conv": (qd, l["conv"]), p + "mix.left.k.conv": (kd, l["conv"]),
                        p + "mix.left.v.conv": (vd, l["conv"]), p + "mix.left.rel": (rows, l["heads"]),
                        p + "mix.left.o": (W, l["heads"] * l["vdim"])})
            kd, vd = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            out.update({p + "mix.right.q": (kd, W), p + "mix.right.k": (kd, W), p + "mix.right.v": (vd, W),
                        p + "mix.right.g": (vd, W), p + "mix.right.o": (W, vd), p + "mix.right.norm": (r["vdim"],),
                        p + "mix.right.a1": (rank, W), p + "mix.right.a2": (kd, rank), p + "mix.right.a2.b": (kd,)})
        if layer["mlp"]:
            out.update({p + "mlp.up": (layer["mlp"]["ff"], W), p + "mlp.down": (W, layer["mlp"]["ff"])})
    return out


def random_tensors(cfg, rank: int, rows: int, seed: int) -> Dict[str, torch.Tensor]:
    """Values of a size that keeps every activation of order one; bfloat16, as files store them."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rank, rows).items():
        x = torch.randn(shape, generator=g)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2", "ls1", "ls2", "out") or name == "final.norm":
            x = 1.0 + 0.2 * x
        elif last == "in":
            x = 1.0 / shape[0] + 0.2 * x
        elif last == "mix" and len(shape) == 2 and ".hc" in name:
            x = torch.eye(shape[0]) + 0.2 * x
        elif last == "conv":
            x = 0.6 * x
        elif last == "rel":
            x = 2.0 * x
        elif last == "b":
            x = 2.0 + x
        elif name == "pos":
            x = 0.3 * x
        elif len(shape) == 2 and name not in ("embed",) and last != "a2":
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
    cfg, _page, sizes = CONFIGS[name]
    folder = H.tmp_root() / f"dopudra{name}-{seed}"
    tensors = random_tensors(cfg, sizes["rank"], sizes["rows"], seed)
    write_folder(folder, cfg, tensors)
    _tensors[str(folder)] = tensors
    return folder


def register(folder, cfg, tensors) -> None:
    """A folder made by a test itself (planted weights)."""
    write_folder(folder, cfg, tensors)
    _tensors[str(folder)] = tensors
    (folder / "config.json").write_text(json.dumps(cfg))


# Per logits row: max |got - want| / max |want| against the float64 plain implementation, fixed before
# the first run of this file's final form.  Wider than the Llama tests' bounds: a unit norm directly
# on a rank-one state (the first positions of a linear-attention head, where o = (q . k) v) turns
# the rounding of a small q . k into an error of order one of that head, and these weights are of
# order one throughout.  A logic fault (a key, a tap, a state or a stream lost or shifted) shows at
# 1e-2 and more in float32.
TOLERANCE = {"float32": 1e-4, "bfloat16": 8e-2}

_plain: Dict[Tuple, torch.Tensor] = {}


def plain_logits(folder, ids: Sequence[int]) -> torch.Tensor:
    key = (str(folder), tuple(ids))
    if key not in _plain:
        cfg = json.loads((folder / "config.json").read_text())
        _plain[key] = P.forward(cfg, _tensors[str(folder)], list(ids))
    return _plain[key]


def check(folder, requests: Dict[str, List[int]], got, dtype: str, expect_all: bool = True) -> None:
    for rid, ids in requests.items():
        want = plain_logits(folder, ids)
        places = sorted(p for (r, p) in got if r == rid)
        if expect_all:
            assert places == list(range(len(ids))), f"request {rid}: places {places}"
        for p in places:
            err = H.row_error(got[(rid, p)], want[p])
            assert err <= TOLERANCE[dtype], f"request {rid} position {p} of {len(ids)}: error {err:.3e}"


def check_most(folder, requests: Dict[str, List[int]], got, dtype: str, share: float = 0.95, worst: float = 0.5) -> None:
    """For configurations drawn at random in bfloat16, where single positions can be ill-conditioned (see
    TOLERANCE): `share` of the rows within the tolerance, none beyond `worst`."""
    errors = sorted(H.row_error(got[(rid, p)], plain_logits(folder, requests[rid])[p]) for (rid, p) in got)
    assert errors[-1] <= worst, f"worst row: error {errors[-1]:.3e}"
    at = min(len(errors) - 1, int(share * len(errors)))
    assert errors[at] <= TOLERANCE[dtype], f"{share:.0%} of the rows: error {errors[at]:.3e}"
