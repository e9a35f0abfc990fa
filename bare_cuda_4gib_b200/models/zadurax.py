"""The Zadurax decoder laid out as parts.

The embedding is RMS-normed; every layer is a "sandwich" block, x += norm_b(sublayer(norm(x))),
first with its mixer and then, where it has one, with a gated feed-forward (tanh-form gelu).
Mixers, by the layer's `type`: "attention" (grouped heads, per-head norms of queries and keys,
pairwise rotation of the first entries of a head, a window of the last positions, the keys as
projected serving as values, a sigmoid gate on the output), "latent_attention" (keys and values
of all heads expanded from one cached latent vector, a rotated key part shared by the heads, a
learned sink in the softmax, the same gate), and "mlstm" (a matrix state with input and forget
gates per head).  A layer that names another with `weights_of` is a second run of that layer's
parts with a cache of its own, so the model's run order names that layer again.

Tensor names: `embed`, `embed.norm`, `final.norm`, `head`, and per layer i with tensors of its own
`l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down`.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zadurax import ZaduraxConfig
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _rotation(rot) -> PartSpec:
    return PartSpec("rotary_pairs", {"dims": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling")})


def _attention(cfg: ZaduraxConfig, m, p: str) -> PartSpec:
    return PartSpec("gated_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"],
                     "window": m["mask"]["size"], "scale": m["scale"], "eps": cfg.norm_eps, "values": "keys",
                     "position": _rotation(m["rot"])},
                    {"q": p + "q", "k": p + "k", "g": p + "g", "o": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm"})


def _latent(cfg: ZaduraxConfig, m, p: str) -> PartSpec:
    return PartSpec("latent_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                     "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": cfg.norm_eps, "sink": True, "window": None,
                     "position": _rotation(m["rot"])},
                    {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                     "sink": p + "sink", "g": p + "g", "o": p + "o"})


def _mlstm(cfg: ZaduraxConfig, m, p: str) -> PartSpec:
    return PartSpec("mlstm",
                    {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "gate_cap": m["gate_cap"], "eps": cfg.norm_eps},
                    {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o", "norm": p + "norm",
                     "i": p + "i", "i_bias": p + "i.b", "f": p + "f", "f_bias": p + "f.b"})


_MIXERS = {"attention": _attention, "latent_attention": _latent, "mlstm": _mlstm}


def zadurax_spec(cfg: ZaduraxConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("sandwich_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps}, {"weight": name})

    layers, own = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            continue
        name = f"l{i}"
        mlp = layer.get("mlp")
        extras = {"post1": norm(name + ".norm1b")}
        if mlp is not None:
            extras["post2"] = norm(name + ".norm2b")
        own[i] = len(layers)
        layers.append(LayerSpec(
            mixer_norm=norm(name + ".norm1"),
            mixer=_MIXERS[layer["type"]](cfg, layer["mixer"], name + ".mix."),
            ffn_norm=norm(name + ".norm2") if mlp is not None else None,
            ffn=PartSpec("glu", {"hidden": cfg.width, "intermediate": mlp["ff"], "activation": "gelu_tanh"},
                         {"gate": name + ".mlp.gate", "up": name + ".mlp.up", "down": name + ".mlp.down"})
            if mlp is not None else None,
            block="sandwich", extras=extras))
    # the run order follows the configuration; a layer without tensors of its own is one more run of the
    # layer it names (which may stand before or behind it)
    order = [LayerCall(own[i if layer.get("weights_of") is None else layer["weights_of"]])
             for i, layer in enumerate(cfg.layers)]
    sizes = {"vocab": cfg.vocab, "hidden": cfg.width}
    return ModelSpec(
        architecture=ZaduraxConfig.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=None,
        embed=PartSpec("table_norm", dict(sizes, eps=cfg.norm_eps), {"weight": "embed", "norm": "embed.norm"}),
        layers=layers, order=order, final_norm=norm("final.norm"), head=PartSpec("linear", sizes, {"weight": "head"}))


register_architecture(ZaduraxConfig.ARCHITECTURE, ZaduraxConfig, zadurax_spec)
