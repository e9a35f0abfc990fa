"""The Dopudra decoder laid out as parts.

Embedding times a scale plus a learned position vector, copied into `streams` residual streams;
layers in the order the configuration lists them, each a "stream_prenorm" block whose mixer is
either lightning attention (type "lightning") or two mixers side by side, softmax attention with a
distance bias beside gated linear attention (type "parallel"), and whose feed-forward, where the
layer has one, is a plain up / square-of-relu / down; the final norm reads the sum of the streams.
Without `streams` in the configuration the residual is a single stream with a plain sum.

Tensor names: `embed`, `pos`, `final.norm`, `head`, and per layer i `l<i>.norm1|norm2`,
`l<i>.ls1|ls2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.up|down`.
"""

from __future__ import annotations

from ..config.dopudra import DopudraConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _lightning(cfg: DopudraConfig, m, p: str) -> PartSpec:
    return PartSpec("lightning_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "decay": list(m["decay"]), "eps": cfg.norm_eps},
                    {n: p + n for n in ("q", "k", "v", "g", "o", "norm")})


def _parallel(cfg: DopudraConfig, m, p: str) -> PartSpec:
    l, r = m["left"], m["right"]
    left = PartSpec("biased_attention",
                    {"hidden": cfg.width, "heads": l["heads"], "kv_heads": l["kv_heads"], "dim": l["dim"],
                     "vdim": l["vdim"], "taps": l["conv"], "scale": l["scale"], "bias_far": l["bias_max"],
                     "bias_rows": l.get("bias_rows"), "temp_coef": l["q_temp"]["coef"],
                     "temp_every": l["q_temp"]["every"], "eps": cfg.norm_eps, "max_positions": cfg.max_positions,
                     "window": None},
                    {"q": p + "left.q", "k": p + "left.k", "v": p + "left.v", "o": p + "left.o",
                     "q_norm": p + "left.q.norm", "k_norm": p + "left.k.norm", "q_conv": p + "left.q.conv",
                     "k_conv": p + "left.k.conv", "v_conv": p + "left.v.conv", "rel": p + "left.rel"})
    right = PartSpec("gated_linear_attention",
                     {"hidden": cfg.width, "heads": r["heads"], "dim": r["dim"], "vdim": r["vdim"], "tau": r["tau"],
                      "rank": r.get("rank"), "eps": cfg.norm_eps},
                     {"q": p + "right.q", "k": p + "right.k", "v": p + "right.v", "g": p + "right.g",
                      "o": p + "right.o", "norm": p + "right.norm", "a1": p + "right.a1", "a2": p + "right.a2",
                      "a2_bias": p + "right.a2.b"})
    weights = {f"{i}.{local}": name for i, branch in enumerate((left, right)) for local, name in branch.weights.items()
               if local in ("q", "k", "v", "g", "a1", "o")}
    return PartSpec("parallel", {"hidden": cfg.width, "branches": [left, right],
                                 "scales": [m["left_scale"], m["right_scale"]]}, weights)


def dopudra_spec(cfg: DopudraConfig) -> ModelSpec:
    streams = cfg.streams or 1
    mixing = cfg.streams is not None

    def norm(name, read):
        weights = {"weight": name}
        if mixing and read:
            weights["read"] = read
        return PartSpec("stream_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "streams": streams,
                                           "read": "vector" if mixing and read else "sum"}, weights)

    def writer(layer, q):
        weights = {"scale": f"{layer}.ls{q}"}
        if mixing:
            weights.update(write=f"{layer}.hc{q}.out", mix=f"{layer}.hc{q}.mix")
        return PartSpec("stream_write", {"size": cfg.width, "streams": streams, "mixing": mixing}, weights)

    layers = []
    for i, layer in enumerate(cfg.layers):
        name = f"l{i}"
        build = _lightning if layer["type"] == "lightning" else _parallel
        mlp = layer.get("mlp")
        extras = {"write1": writer(name, 1)}
        if mlp is not None:
            extras["write2"] = writer(name, 2)
        layers.append(LayerSpec(
            mixer_norm=norm(name + ".norm1", f"{name}.hc1.in"),
            mixer=build(cfg, layer["mixer"], name + ".mix."),
            ffn_norm=norm(name + ".norm2", f"{name}.hc2.in") if mlp is not None else None,
            ffn=PartSpec("dense", {"hidden": cfg.width, "intermediate": mlp["ff"], "activation": "relu2"},
                         {"up": name + ".mlp.up", "down": name + ".mlp.down"}) if mlp is not None else None,
            block="stream_prenorm", extras=extras))
    sizes = {"vocab": cfg.vocab, "hidden": cfg.width}
    return ModelSpec(
        architecture=DopudraConfig.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embed=PartSpec("table_positions", dict(sizes, scale=cfg.embedding_scale, positions=cfg.max_positions,
                                               streams=streams), {"weight": "embed", "positions": "pos"}),
        layers=layers, order=[LayerCall(i) for i in range(len(layers))],
        final_norm=norm("final.norm", None),
        head=PartSpec("linear", sizes, {"weight": "head"}))


register_architecture(DopudraConfig.ARCHITECTURE, DopudraConfig, dopudra_spec)
