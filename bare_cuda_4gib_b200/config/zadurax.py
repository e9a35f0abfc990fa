"""Typed configuration of the Zadurax decoder, read from its own `config.json` layout:

    architecture, vocab, width, norm.eps,
    layers: [{type: "attention" | "latent_attention" | "mlstm", mixer: {...},
              mlp: {kind: "dense", ff} | null, weights_of: j (optional)}, ...]

A layer with `weights_of` j runs with layer j's tensors and keeps a cache or state of its own.
Every size and every constant that may differ between models of the design is read here and
nowhere else; a key that is wrong or missing is named in the error.  The design states no largest
position: a request is as long as the cache pool lets it be.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from ..errors import ConfigError
from .dopudra import _get

MIXER_TYPES = ("attention", "latent_attention", "mlstm")


def _rotation(rot, where: str, scaling_allowed: bool) -> None:
    dims = _get(rot, "dims", where)
    _get(rot, "base", where, float)
    if dims % 2:
        raise ConfigError(f"config.json: '{where}dims' must be even (entries are turned in pairs), got {dims}")
    sc = rot.get("scaling")
    if sc is not None:
        if not scaling_allowed:
            raise ConfigError(f"config.json: '{where}scaling' is not part of this mixer")
        for key in ("factor", "fast", "slow"):
            _get(sc, key, where + "scaling.", float)
        _get(sc, "original", where + "scaling.", float)


def _attention(m, where: str) -> None:
    heads, kv = _get(m, "heads", where), _get(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: '{where}heads' {heads} is not a multiple of '{where}kv_heads' {kv}")
    dim, vdim = _get(m, "dim", where), _get(m, "vdim", where)
    if vdim != dim:
        raise ConfigError(f"config.json: '{where}vdim' {vdim} must equal '{where}dim' {dim}: the values are the keys")
    _get(m, "scale", where, float)
    _get(m.get("mask"), "size", where + "mask.")
    _rotation(m.get("rot"), where + "rot.", scaling_allowed=False)
    if m["rot"]["dims"] > dim:
        raise ConfigError(f"config.json: '{where}rot.dims' {m['rot']['dims']} exceeds '{where}dim' {dim}")


def _latent(m, where: str) -> None:
    for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
        _get(m, key, where)
    _get(m, "scale", where, float)
    _rotation(m.get("rot"), where + "rot.", scaling_allowed=True)
    if m["rot"]["dims"] != m["rot_dim"]:
        raise ConfigError(f"config.json: '{where}rot.dims' {m['rot']['dims']} must equal '{where}rot_dim' {m['rot_dim']}")


def _mlstm(m, where: str) -> None:
    for key in ("heads", "dim", "vdim"):
        _get(m, key, where)
    _get(m, "gate_cap", where, float)


_CHECKS = {"attention": _attention, "latent_attention": _latent, "mlstm": _mlstm}


@dataclass
class ZaduraxConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]] = field(default_factory=list)
    norm_eps: float = 1e-6

    ARCHITECTURE = "Zadurax"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ZaduraxConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=_get(d, "vocab", ""), width=_get(d, "width", ""), layers=copy.deepcopy(layers),
                  norm_eps=_get(d.get("norm"), "eps", "norm.", float))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' must be one of {list(MIXER_TYPES)}, "
                                  f"got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            if not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            _CHECKS[layer["type"]](layer["mixer"], where + "mixer.")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: '{where}mlp.kind' must be 'dense' (or 'mlp' null)")
                _get(mlp, "ff", where + "mlp.")
            src = layer.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < len(self.layers)) or src == i:
                    raise ConfigError(f"config.json: '{where}weights_of' must name another layer, got {src!r}")
                other = self.layers[src]
                if isinstance(other, dict) and other.get("weights_of") is not None:
                    raise ConfigError(f"config.json: '{where}weights_of' names layer {src}, which has no tensors of its own")
                if not isinstance(other, dict) or other.get("type") != layer["type"]:
                    raise ConfigError(f"config.json: '{where}type' differs from layer {src}, whose tensors it uses")

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}

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
