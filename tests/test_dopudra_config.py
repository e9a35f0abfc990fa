"""Host-side pieces of the Dopudra decoder: configuration, the layout as parts with its tensor
names, the distance table, value heads of their own size in the cache manager, random weights."""

import copy
import json

import pytest
import torch

import dopudra_helpers as D
import plain_dopudra as P

import bare_cuda_4gib_b200.models  # noqa: F401
from bare_cuda_4gib_b200.cache.manager import CacheDemand, CacheManager
from bare_cuda_4gib_b200.config.dopudra import DopudraConfig
from bare_cuda_4gib_b200.config.registry import resolve_architecture
from bare_cuda_4gib_b200.engine.model import expected_weights
from bare_cuda_4gib_b200.errors import ConfigError
from bare_cuda_4gib_b200.parts.base import KVCacheRequest, StateRequest


@pytest.mark.parametrize("name", ["X", "Y"])
def test_tensor_names_and_shapes(name):
    cfg, _page, sizes = D.CONFIGS[name]
    arch = resolve_architecture(cfg)
    assert arch.name == "Dopudra"
    config = arch.config_class.from_dict(cfg)
    assert config.to_dict() == json.loads(json.dumps(cfg))
    expected, model = expected_weights(arch.build_spec(config))
    want = D.tensor_shapes(cfg, sizes["rank"], sizes["rows"])
    assert sorted(expected) == sorted(want)
    for n, spec in expected.items():
        assert len(spec.shape) == len(want[n]) and all(a in (-1, b) for a, b in zip(spec.shape, want[n])), n
    # a parallel layer keeps pages and a convolution state for one branch and a matrix state for the other
    demands = model.cache_demands()
    for layer, run in zip(cfg["layers"], demands):
        if layer["type"] == "parallel":
            l, r = layer["mixer"]["left"], layer["mixer"]["right"]
            assert run[0].kv == KVCacheRequest(l["kv_heads"], l["dim"], None, None if l["dim"] == l["vdim"] else l["vdim"])
            channels = (l["heads"] + l["kv_heads"]) * l["dim"] + l["kv_heads"] * l["vdim"]
            assert run[0].state == StateRequest((max(l["conv"] - 1, 1), channels))
            assert run[1].kv is None and run[1].state == StateRequest((r["heads"], r["dim"], r["vdim"]))
        else:
            m = layer["mixer"]
            assert len(run) == 1 and run[0].kv is None and run[0].state == StateRequest((m["heads"], m["dim"], m["vdim"]))


def test_config_errors_name_the_key():
    def broken(change):
        cfg = copy.deepcopy(D.CFG_X)
        change(cfg)
        with pytest.raises(ConfigError) as e:
            DopudraConfig.from_dict(cfg)
        return str(e.value)

    assert "'width'" in broken(lambda c: c.pop("width"))
    assert "layers[1].type" in broken(lambda c: c["layers"][1].update(type="other"))
    assert "layers[0].mixer.left.kv_heads" in broken(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3))
    assert "layers[1].mixer.decay" in broken(lambda c: c["layers"][1]["mixer"].update(decay=[0.5]))
    assert "layers[0].mixer.right.tau" in broken(lambda c: c["layers"][0]["mixer"]["right"].pop("tau"))
    assert "layers[0].mlp.kind" in broken(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    assert "norm.eps" in broken(lambda c: c.pop("norm"))
    assert "streams" in broken(lambda c: c.update(streams=40))


def test_distance_rows_match_the_plain_buckets():
    from bare_cuda_4gib_b200.parts.biased_attention import distance_rows
    for rows, far in [(16, 240), (7, 50), (9, 9), (32, 128), (2, 5), (16, 20), (5, 1000)]:
        assert distance_rows(600, rows, far) == [P.distance_bucket(n, rows, far) for n in range(600)], (rows, far)
    with pytest.raises(ConfigError):      # the logarithmic part needs a far distance beyond the exact part
        distance_rows(600, 16, 6)


def test_value_heads_of_their_own_size_in_the_cache():
    kv = KVCacheRequest(2, 16, None, 24)
    cache = CacheManager([CacheDemand(kv), CacheDemand(kv)], page_tokens=8, max_seqs=2, max_tokens=32, num_pages=6,
                         dtype=torch.float32, device="cpu")
    g = cache.groups[0]
    assert g.key_elems == 2 * 8 * 16 and g.cache_elems == 2 * 8 * (16 + 24) and g.page_stride == 2 * g.cache_elems
    table = torch.zeros((2, 4), dtype=torch.int32)
    first, second = cache.cache_view(0, table), cache.cache_view(1, table)
    assert first.v_ptr - first.k_ptr == g.key_elems * 4 and second.k_ptr - first.k_ptr == g.cache_elems * 4
    assert first.head_dim == 16 and first.v_dim == 24
    same = CacheManager([CacheDemand(KVCacheRequest(2, 16))], page_tokens=8, max_seqs=1, max_tokens=8, num_pages=1,
                        dtype=torch.float32, device="cpu")
    assert same.cache_view(0, table).v_dim == 16


def test_random_weights_need_every_extent(tmp_path):
    from bare_cuda_4gib_b200.models.presets import preset_config
    from bare_cuda_4gib_b200.weights import write_random_model
    from bare_cuda_4gib_b200.weights.safetensors_io import SafetensorsFile

    config = preset_config("dopudra-tiny")
    write_random_model(tmp_path / "m", config, 1)
    with SafetensorsFile(tmp_path / "m" / "model.safetensors") as f:
        assert "l0.mix.q" in f.entries or "l0.mix.left.q" in f.entries
    bare = DopudraConfig.from_dict(D.CFG_X)      # no rank and no table rows: only a file can say
    with pytest.raises(ValueError):
        write_random_model(tmp_path / "n", bare, 1)


def test_plain_prompt_equals_plain_prefixes():
    """The plain implementation itself: a prefix's logits do not depend on what follows."""
    cfg, _page, sizes = D.CONFIGS["X"]
    t = D.random_tensors(cfg, sizes["rank"], sizes["rows"], 5)
    ids = list(range(3, 40))
    full = P.forward(cfg, t, ids)
    part = P.forward(cfg, t, ids[:17])
    assert float((full[:17] - part).abs().max()) < 1e-9
