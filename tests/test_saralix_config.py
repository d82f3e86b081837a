"""Saralix without a device: the configuration's keys and refusals, the model description it gives, the tensors it
expects, random weights through the loader, the stretched rotation's frequencies against the plain ones."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_saralix as plain
import tiny_saralix as tiny
from xpu_serve_b200 import registry
from xpu_serve_b200.config import ConfigError, SaralixConfig
from xpu_serve_b200.parts.base import KVNeed, StateNeed
from xpu_serve_b200.parts.rope import ScaledRotaryTable
from xpu_serve_b200.weights import write_random_model
from xpu_serve_b200.weights.expected import expected_tensors
from xpu_serve_b200.weights.loader import load_weights
from xpu_serve_b200.weights.safetensors_io import WeightError


def test_the_architecture_is_found_by_its_key():
    arch = registry.architecture_for(tiny.CONFIGS["M"])
    assert arch.name == "saralix" and arch.config_class is SaralixConfig
    with pytest.raises(ConfigError, match="not supported"):
        registry.architecture_for({"architecture": "Nothing"})


def test_every_size_and_constant_comes_from_the_file():
    c = SaralixConfig.from_json(tiny.CONFIGS["M"])
    assert c.to_json() == tiny.CONFIGS["M"]
    spec = c.model_spec()
    assert spec.vocab == 203 and spec.hidden == 44 and spec.tied_head and spec.final_norm.kind == "layernorm"
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "mamba2", "latent_attention", "mamba2", "latent_attention"]
    a, m, w = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[2].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale) == (3, 12, 8, 20, 36, 0.21)
    assert a.head_gate and not a.sink and a.window == 0 and a.eps == 3e-6
    assert a.position.theta == 5000.0 and a.position.dims == 8 and a.position.scaling.factor == 4.0
    assert a.position.scaling.original == 48 and a.position.scaling.mscale_k == 0.1
    assert w.sink and not w.head_gate and w.window == 13 and w.position.scaling is None
    assert (m.heads, m.vdim, m.state, m.groups, m.taps, m.norm_groups) == (6, 6, 12, 3, 3, 3) and m.inner == 36
    assert spec.layers[0].ffn.kind == "clamped_glu" and spec.layers[0].ffn.limit == 1.5 and spec.layers[0].ffn.alpha == 1.702
    assert spec.layers[1].ffn.kind == "routed_experts" and (spec.layers[1].ffn.experts, spec.layers[1].ffn.top) == (6, 3)
    assert spec.layers[2].ffn is None and spec.layers[0].sandwich


def test_cache_needs():
    spec = SaralixConfig.from_json(tiny.CONFIGS["M"]).model_spec()
    needs = [registry.arrangement_class(l.kind).cache_need(l) for l in spec.layers]
    assert needs[0] == KVNeed(1, 44, 0, planes=1) and needs[2] == KVNeed(1, 34, 13, planes=1)
    assert needs[1] == (StateNeed((2, 108), "compute"), StateNeed((6, 12, 6), "float32"))


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "attention", "unknown layer type"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "dims"),
    (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 0, "mlp", "kind"), "other", "unknown feed-forward"),
    (("layers", 1, "mixer", "groups"), 4, "groups"),
    (("layers", 1, "mixer", "norm_groups"), 5, "norm groups"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 2, "mixer", "mask"), None, "mask"),
    (("norm", "eps"), 0.0, "eps"),
    (("width",), None, "width"),
])
def test_refusals_name_their_key(path, value, message):
    cfg = copy.deepcopy(tiny.CONFIGS["M"])
    at = cfg
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        SaralixConfig.from_json(cfg)


def test_expected_tensors_and_random_weights(tmp_path):
    spec = SaralixConfig.from_json(tiny.CONFIGS["M"]).model_spec()
    names = expected_tensors(spec)
    assert names["embed"].shape == (203, 44) and names["final.norm"].shape == (44,)
    assert names["l0.mix.q"].shape == (3 * 20, 44) and names["l0.mix.dkv"].shape == (44, 44)
    assert names["l0.mix.uk"].shape == (36, 36) and names["l0.mix.uv"].shape == (60, 36) and names["l0.mix.g"].shape == (3, 44)
    assert "l0.mix.sink" not in names and names["l2.mix.sink"].shape == (2,) and "l2.mix.g" not in names
    assert names["l1.mix.in"].shape == (2 * 36 + 2 * 3 * 12 + 6, 44) and names["l1.mix.conv"].shape == (36 + 2 * 3 * 12, 3)
    assert names["l1.mlp.e5.down"].shape == (44, 20) and names["l1.mlp.router"].shape == (6, 44)
    assert "l2.norm2" not in names and "l2.norm2b" not in names and "l2.norm1b" in names
    folder = tiny.make_folder(tmp_path, "M", "bfloat16")
    weights = load_weights(spec, folder)
    assert set(weights) == set(names) and weights["l1.mix.A_log"].dtype == torch.float32
    # a folder of another configuration is refused in one message
    other = SaralixConfig.from_json(tiny.CONFIGS["N"]).model_spec()
    with pytest.raises(WeightError, match="missing"):
        load_weights(other, folder)


def test_norms_of_an_absent_feed_forward_are_tolerated(tmp_path):
    """A layer without a feed-forward may still carry the two norms of one in its folder."""
    from xpu_serve_b200.weights.random_init import random_tensors
    from xpu_serve_b200.weights.safetensors_io import write_safetensors
    config = SaralixConfig.from_json(tiny.CONFIGS["windowed"])
    spec = config.model_spec()
    folder = str(tmp_path / "extra")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_json(), f)
    tensors = list(random_tensors(spec, 3)) + [("l0.norm2", torch.ones(40)), ("l0.norm2b", torch.ones(40))]
    write_safetensors(os.path.join(folder, "model.safetensors"), iter(tensors), metadata={"format": "pt"})
    assert "l0.norm2" not in load_weights(spec, folder)
    write_safetensors(os.path.join(folder, "model.safetensors"), iter(tensors + [("l0.other", torch.ones(2))]),
                      metadata={"format": "pt"})
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(spec, folder)


@pytest.mark.parametrize("name,layer", [("M", 0), ("M", 4), ("M", 2), ("N", 1), ("N", 2)])
def test_stretched_frequencies_match_the_plain_ones(name, layer):
    spec = SaralixConfig.from_json(tiny.CONFIGS[name]).model_spec()
    f, m = ScaledRotaryTable(spec.layers[layer].mixer.position, None).frequencies()
    want_f, want_m = plain.rotary_frequencies(tiny.CONFIGS[name]["layers"][layer]["mixer"]["rot"])
    assert np.allclose(f.numpy(), want_f, rtol=1e-13, atol=0) and abs(m - want_m) < 1e-15
    if spec.layers[layer].mixer.position.scaling is not None:
        assert not np.allclose(f.numpy(), plain.rotary_frequencies({**tiny.CONFIGS[name]["layers"][layer]["mixer"]["rot"], "scaling": None})[0])


def test_plain_routing_prefers_the_lower_index_among_equals_and_sums_to_one():
    t = {"r.router": np.array([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]])}
    for e in range(3):
        t[f"r.e{e}.gate"], t[f"r.e{e}.up"], t[f"r.e{e}.down"] = np.eye(2), np.eye(2), np.eye(2) * (e + 1)
    h = np.array([[2.0, 1.0]])
    out = plain.routed_ff(h, t, "r.", {"router": {"experts": 3, "top": 2}})
    act = plain.silu(h[0]) * h[0]
    assert np.allclose(out[0], 0.5 * act * 1 + 0.5 * act * 2)       # experts 0 and 1 tie at 2.0, expert 2 is left out
