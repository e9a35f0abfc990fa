"""Typed configuration of the Dopudra decoder, read from its own `config.json` layout:

    architecture, vocab, width, max_positions, streams, embedding.scale, norm.eps,
    layers: [{type: "lightning" | "parallel", mixer: {...}, mlp: {kind: "dense", ff} | null}, ...]

Every size and every constant that may differ between models of the design is read here and
nowhere else; a key that is wrong or missing is named in the error.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..errors import ConfigError

MIXER_TYPES = ("lightning", "parallel")
MAX_STREAMS = 16


def _get(d: Dict[str, Any], key: str, where: str, kind=int, positive: bool = True):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{where}{key}' must be an integer, got {v!r}")
    elif isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"config.json: '{where}{key}' must be a number, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: '{where}{key}' must be positive, got {v!r}")
    return kind(v)


def _linear_mixer(m, where: str, decay: bool) -> None:
    heads = _get(m, "heads", where)
    _get(m, "dim", where)
    _get(m, "vdim", where)
    if decay:
        d = m.get("decay")
        if not isinstance(d, list) or len(d) != heads or not all(isinstance(x, (int, float)) and 0.0 <= x <= 1.0 for x in d):
            raise ConfigError(f"config.json: '{where}decay' must list one number in [0, 1] per head ({heads})")
    else:
        _get(m, "tau", where, float)


def _left_mixer(m, where: str) -> None:
    heads, kv = _get(m, "heads", where), _get(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: '{where}heads' {heads} is not a multiple of '{where}kv_heads' {kv}")
    for key in ("dim", "vdim", "conv"):
        _get(m, key, where)
    _get(m, "scale", where, float)
    _get(m, "bias_max", where, float)
    _get(m.get("q_temp"), "coef", where + "q_temp.", float, positive=False)
    _get(m.get("q_temp"), "every", where + "q_temp.")


@dataclass
class DopudraConfig:
    vocab: int
    width: int
    max_positions: int
    layers: List[Dict[str, Any]] = field(default_factory=list)
    streams: Optional[int] = None          # None: a single residual with a plain sum
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6

    ARCHITECTURE = "Dopudra"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DopudraConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=_get(d, "vocab", ""), width=_get(d, "width", ""), max_positions=_get(d, "max_positions", ""),
                  layers=copy.deepcopy(layers),
                  streams=None if d.get("streams") is None else _get(d, "streams", ""),
                  embedding_scale=_get(d.get("embedding", {"scale": 1.0}), "scale", "embedding.", float),
                  norm_eps=_get(d.get("norm"), "eps", "norm.", float))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.streams is not None and self.streams > MAX_STREAMS:
            raise ConfigError(f"config.json: 'streams' {self.streams} exceeds the {MAX_STREAMS} the kernels take")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' must be one of {list(MIXER_TYPES)}, "
                                  f"got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            if layer["type"] == "lightning":
                _linear_mixer(m, where + "mixer.", decay=True)
            else:
                _left_mixer(m.get("left"), where + "mixer.left.")
                _linear_mixer(m.get("right"), where + "mixer.right.", decay=False)
                _get(m, "left_scale", where + "mixer.", float, positive=False)
                _get(m, "right_scale", where + "mixer.", float, positive=False)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: '{where}mlp.kind' must be 'dense' (or 'mlp' null)")
                _get(mlp, "ff", where + "mlp.")

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
             "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.streams is not None:
            d["streams"] = self.streams
        return d

    # the names the command line tools read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def stop_ids(self) -> List[int]:
        return []
