"""The Zadurax decoder without a GPU: tensor names and shapes against a list written out
independently, the run order of layers that share tensors, what each run keeps per request,
configuration errors by key, the scaled rotary frequencies, and random weights."""

import copy
import math

import pytest
import torch

import plain_zadurax as P
import zadurax_helpers as Z
from bare_cuda_4gib_b200 import models  # noqa: F401
from bare_cuda_4gib_b200.config.registry import resolve_architecture
from bare_cuda_4gib_b200.config.zadurax import ZaduraxConfig
from bare_cuda_4gib_b200.engine.model import expected_weights
from bare_cuda_4gib_b200.errors import ConfigError
from bare_cuda_4gib_b200.parts.base import KVCacheRequest
from bare_cuda_4gib_b200.parts.registry import build_part
from bare_cuda_4gib_b200.parts.spec import PartSpec


def _spec(cfg):
    arch = resolve_architecture(cfg)
    return arch.build_spec(arch.config_class.from_dict(cfg))


@pytest.mark.parametrize("name", ["P", "Q"])
def test_tensor_names_and_shapes(name):
    cfg = Z.CONFIGS[name][0]
    expected, _ = expected_weights(_spec(cfg))
    assert {k: tuple(v.shape) for k, v in expected.items()} == Z.tensor_shapes(cfg)


def test_layers_that_share_tensors_run_again_with_a_cache_of_their_own():
    spec = _spec(Z.CFG_P)
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2, 2, 0, 1]
    assert all(c.cache_from is None for c in spec.order)
    _, model = expected_weights(spec)
    demands = model.cache_demands()
    assert demands[0][0].kv == KVCacheRequest(2, 16, 24) and demands[4][0].kv == demands[0][0].kv
    # the latent cache: one head of kv_rank + rot_dim entries and no values of its own
    assert demands[2][0].kv == KVCacheRequest(1, 32, None, v_head_dim=0) and demands[2][0].kv.value_dim == 0
    # an mLSTM run keeps [S | n] and m
    assert [d.state.shape for d in demands[1]] == [(3, 8, 24), (3,)] and demands[1][0].kv is None
    from bare_cuda_4gib_b200.cache.manager import CacheManager
    cache = CacheManager(demands, page_tokens=16, max_seqs=2, max_tokens=64, allocate=False)
    assert len(cache.groups) == 2 and sorted(len(g.members) for g in cache.groups) == [2, 2]
    assert len(cache.states) == 4


def test_a_layer_may_use_the_tensors_of_a_later_one():
    layers = [Z.again([None, Z.mlstm(2, 8, 8, 5.0)], 1), Z.mlstm(2, 8, 8, 5.0), Z.attention(2, 1, 16, 9, 4, ff=24)]
    cfg = {"architecture": "Zadurax", "vocab": 40, "width": 32, "norm": {"eps": 1e-6}, "layers": layers}
    spec = _spec(cfg)
    assert [c.layer for c in spec.order] == [0, 0, 1] and len(spec.layers) == 2
    expected, _ = expected_weights(spec)
    assert "l1.mix.q" in expected and "l2.mlp.gate" in expected and not any(k.startswith("l0.") for k in expected)


def test_configuration_errors_name_the_key():
    def broken(change):
        cfg = copy.deepcopy(Z.CFG_P)
        change(cfg)
        with pytest.raises(ConfigError) as e:
            ZaduraxConfig.from_dict(cfg)
        return str(e.value)

    assert "layers[0].mixer.kv_heads" in broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    assert "layers[0].mixer.vdim" in broken(lambda c: c["layers"][0]["mixer"].update(vdim=8))
    assert "layers[0].mixer.mask.size" in broken(lambda c: c["layers"][0]["mixer"].pop("mask"))
    assert "layers[0].mixer.rot.dims" in broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7))
    assert "layers[2].mixer.rot.scaling.slow" in broken(lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"))
    assert "layers[2].mixer.kv_rank" in broken(lambda c: c["layers"][2]["mixer"].pop("kv_rank"))
    assert "layers[1].mixer.gate_cap" in broken(lambda c: c["layers"][1]["mixer"].update(gate_cap=0))
    assert "layers[1].type" in broken(lambda c: c["layers"][1].update(type="lstm"))
    assert "layers[3].weights_of" in broken(lambda c: c["layers"][3].update(weights_of=9))
    assert "layers[0].mlp.kind" in broken(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    assert "norm.eps" in broken(lambda c: c.pop("norm"))
    assert ZaduraxConfig.from_dict(Z.CFG_Q).to_dict() == Z.CFG_Q


@pytest.mark.parametrize("rot", [{"dims": 8, "base": 5000.0, "scaling": Z.yarn(4.0, 64, 16.0, 2.0)},
                                 {"dims": 32, "base": 50.0, "scaling": Z.yarn(16.0, 300, 4.0, 0.5)},
                                 {"dims": 6, "base": 10000.0, "scaling": Z.yarn(2.0, 4096, 1.0, 1.0)},
                                 {"dims": 12, "base": 777.0}])
def test_rotary_frequencies(rot):
    part = build_part("position", PartSpec("rotary_pairs", {"dims": rot["dims"], "base": rot["base"],
                                                            "scaling": rot.get("scaling")}))
    part.prepare(torch.float32, torch.device("cpu"))
    want, mag = P.rotary_frequencies(rot)
    assert torch.allclose(part.inv_freq.double(), want, rtol=1e-6, atol=0)
    assert math.isclose(part.magnitude, mag, rel_tol=1e-12)
    if "scaling" not in rot:
        assert part.magnitude == 1.0


def test_random_weights_of_a_preset():
    from bare_cuda_4gib_b200.models.presets import preset_config
    from bare_cuda_4gib_b200.weights.random_init import random_tensors

    config = preset_config("zadurax-tiny")
    expected, _ = expected_weights(resolve_architecture(config.to_dict()).build_spec(config))
    tensors = random_tensors(expected, 5)
    assert set(tensors) == set(expected)
    assert abs(float(tensors["l0.norm1b"].float().mean()) - 1.0) < 0.05
