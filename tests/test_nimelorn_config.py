"""Nimelorn without a device: the configuration's keys and refusals, the model description it gives, cache needs, the
tensors it expects, random weights through the loader, the padded head layout, and the oracle's own mechanisms against
hand-made cases."""
import copy
import os

import numpy as np
import pytest
import torch

import plain_nimelorn as plain
import tiny_nimelorn as tiny
from xpu_serve_b200 import registry
from xpu_serve_b200.cache import Cache
from xpu_serve_b200.config import ConfigError, NimelornConfig
from xpu_serve_b200.parts.attention import padded_head_dim
from xpu_serve_b200.parts.base import KVNeed, StateNeed
from xpu_serve_b200.weights.expected import expected_tensors
from xpu_serve_b200.weights.loader import load_weights
from xpu_serve_b200.weights.safetensors_io import WeightError


def test_the_architecture_is_found_by_its_key():
    arch = registry.architecture_for(tiny.CONFIGS["A"])
    assert arch.name == "nimelorn" and arch.config_class is NimelornConfig
    with pytest.raises(ConfigError, match="not supported"):
        registry.architecture_for({"architecture": "Nothing"})


def test_every_size_and_constant_comes_from_the_file():
    c = NimelornConfig.from_json(tiny.CONFIGS["A"])
    assert c.to_json() == tiny.CONFIGS["A"]
    spec = c.model_spec()
    assert spec.vocab == 203 and spec.hidden == 44 and not spec.tied_head and spec.final_norm.kind == "rmsnorm"
    assert spec.final_norm.eps == 3e-6
    e = spec.embedding
    assert (e.kind, e.scale, e.buckets, e.mul_prev, e.mul_cur, e.eps, e.theta) == ("pair_hash", 5.5, 211, 1009, 3, 3e-6, 10000.0)
    assert [l.mixer.kind for l in spec.layers] == ["attention", "attention", "mlstm", "attention", "mlstm"]
    assert all(l.kind == "branch_norm" for l in spec.layers)
    a, b, r = spec.layers[0].mixer, spec.layers[3].mixer, spec.layers[2].mixer
    assert (a.heads, a.kv_heads, a.head_dim, a.v_dim, a.chunk, a.scale, a.window) == (4, 2, 12, 20, 13, 0.21, 0)
    assert a.qk_norm and a.qk_norm_eps == 3e-6 and a.head_gate and a.position is None and a.own_kv
    assert not b.own_kv and b.chunk == 29 and spec.order[3].cache_of == 1 and spec.order[1].cache_of is None
    assert (r.heads, r.dim, r.vdim, r.gate_cap, r.eps) == (3, 10, 14, 9.0, 3e-6)
    f0, f1, f3 = spec.layers[0].ffn, spec.layers[1].ffn, spec.layers[3].ffn
    assert f0.kind == "squared_relu" and f0.intermediate == 70 and spec.layers[2].ffn is None
    assert (f1.kind, f1.experts, f1.top, f1.route_scale, f1.limit, f1.alpha, f1.up_shift) == ("routed_experts", 6, 3, 1.7, 1.5, 1.702, 1.0)
    assert (f1.shared.intermediate, f1.shared.limit) == (24, 0.8) and f3.shared is None and f3.limit == 0.6


def test_cache_needs_and_the_shared_cache():
    spec = NimelornConfig.from_json(tiny.CONFIGS["A"]).model_spec()
    needs = [registry.arrangement_class(l.kind).cache_need(l) for l in spec.layers]
    # key and value heads of 12 and 20 channels are laid out in 32, those of 10 and 6 in 16; a block mask keeps every key
    assert needs[0] == KVNeed(2, 32, 0) and needs[1] == KVNeed(3, 16, 0) and needs[3] == needs[1]
    assert needs[2] == (StateNeed((3, 10, 14), "float32"), StateNeed((3, 1, 11), "float32"))
    assert registry.embedding_class("pair_hash").cache_need(spec.embedding) == StateNeed((1,), "int32")
    shares = [c.cache_of for c in spec.order] + [None]
    cache = Cache(needs + [StateNeed((1,), "int32")], shares, 256, dtype=torch.float32, device="cpu")
    assert cache.views[3].storage is cache.views[1].storage and not cache.views[3].owner and cache.views[1].owner
    assert cache.views[5].storage.dtype == torch.int32 and cache.views[5].storage.shape[1:] == (1,)
    s = cache.open(2)
    cache.views[5].storage[s[0]] = 7
    cache.close(s)
    again = cache.open(2)                    # a slot that is used again starts with no last token
    assert int(cache.views[5].storage[again].abs().sum()) == 0


def test_padded_head_layout():
    class S:
        def __init__(self, d, v):
            self.head_dim, self.v_dim = d, v
    assert padded_head_dim(S(64, 0)) == 64 and padded_head_dim(S(64, 64)) == 64 and padded_head_dim(S(40, 40)) == 40
    assert padded_head_dim(S(64, 80)) == 96 and padded_head_dim(S(12, 20)) == 32 and padded_head_dim(S(100, 8)) == 128
    assert padded_head_dim(S(130, 7)) == 130 and padded_head_dim(S(131, 7)) == 132 and padded_head_dim(S(33, 33)) == 48


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "latent", "unknown layer type"),
    (("layers", 0, "mixer", "mask"), None, "mask"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 0, "mlp", "kind"), "other", "unknown feed-forward"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "expert", "limit"), 0.0, "limit"),
    (("layers", 1, "mlp", "shared", "ff"), 0, "shared"),
    (("layers", 2, "mixer", "gate_cap"), -1.0, "gate_cap"),
    (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
    (("layers", 3, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 3, "mixer", "kv_from"), 0, "head counts"),
    (("layers", 3, "mixer", "kv_from"), "1", "kv_from"),
    (("embedding", "bigram", "buckets"), 0, "buckets"),
    (("embedding", "scale"), None, "scale"),
    (("norm", "eps"), 0.0, "eps"),
    (("width",), None, "width"),
])
def test_refusals_name_their_key(path, value, message):
    cfg = copy.deepcopy(tiny.CONFIGS["A"])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        NimelornConfig.from_json(cfg)


def test_a_layer_cannot_borrow_from_a_borrower():
    cfg = copy.deepcopy(tiny.CONFIGS["borrowed"])
    cfg["layers"].append(copy.deepcopy(cfg["layers"][1]))
    cfg["layers"][2]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="kv_from"):
        NimelornConfig.from_json(cfg)


def test_tensor_names_and_random_weights_through_the_loader(tmp_path):
    c = NimelornConfig.from_json(tiny.CONFIGS["A"])
    spec = c.model_spec()
    exp = expected_tensors(spec)
    assert exp["embed"].shape == (203, 44) and exp["bigram"].shape == (212, 44) and exp["embed.norm"].shape == (44,)
    assert exp["head"].shape == (203, 44) and exp["final.norm"].shape == (44,)
    assert exp["l0.mix.q"].shape == (48, 44) and exp["l0.mix.v"].shape == (40, 44) and exp["l0.mix.o"].shape == (44, 80)
    assert exp["l0.mix.q.norm"].shape == (12,) and exp["l0.mix.g"].shape == (4, 44) and exp["l0.norm1"].shape == (44,)
    assert "l3.mix.k" not in exp and "l3.mix.v" not in exp and "l3.mix.k.norm" not in exp and "l3.mix.q.norm" in exp
    assert "l2.norm2" not in exp and "l0.norm2" in exp
    assert exp["l2.mix.i"].shape == (3, 44) and exp["l2.mix.i.b"].shape == (3,) and exp["l2.mix.norm"].shape == (42,)
    assert exp["l1.mlp.e5.down"].shape == (44, 20) and exp["l1.mlp.router"].shape == (6, 44)
    assert exp["l1.mlp.shared.sg"].shape == (1, 44) and exp["l1.mlp.shared.gate"].shape == (24, 44) and "l3.mlp.shared.sg" not in exp
    folder = tiny.make_folder(tmp_path, "A", "bfloat16")
    w = load_weights(spec, folder)
    assert set(w) == set(exp) and w["bigram"].dtype == torch.bfloat16 and w["l0.norm1"].dtype == torch.float32
    # a missing tensor and a wrong shape are named
    from xpu_serve_b200.weights.safetensors_io import WeightStore, write_safetensors
    st = WeightStore.open_dir(folder)
    tensors = [(n, st.get(n)) for n in st.names() if n != "bigram"]
    os.makedirs(tmp_path / "broken")
    with open(os.path.join(folder, "config.json")) as f, open(tmp_path / "broken" / "config.json", "w") as g:
        g.write(f.read())
    write_safetensors(str(tmp_path / "broken" / "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="bigram"):
        load_weights(spec, str(tmp_path / "broken"))


# ------------------------------------------------------------------------------------------- the oracle's mechanisms
def test_oracle_block_mask_and_shared_keys():
    """In the plain attention a query sees its own block only, and a layer that reads another layer's keys gives, with
    equal weights and mask, the same output as that layer."""
    cfg = tiny.CONFIGS["borrowed"]
    rng = np.random.default_rng(0)
    m0, m1 = cfg["layers"][0]["mixer"], dict(cfg["layers"][1]["mixer"], mask={"size": 16})
    w = {}
    for p in ("l0.mix.", "l1.mix."):
        w[p + "q"] = rng.standard_normal((16, 40)); w[p + "g"] = rng.standard_normal((2, 40))
        w[p + "o"] = rng.standard_normal((40, 24)); w[p + "q.norm"] = rng.uniform(0.5, 1.5, 8)
    w["l0.mix.k"] = rng.standard_normal((8, 40)); w["l0.mix.v"] = rng.standard_normal((12, 40))
    w["l0.mix.k.norm"] = rng.uniform(0.5, 1.5, 8)
    for k in ("q", "g", "o", "q.norm"):
        w["l1.mix." + k] = w["l0.mix." + k]
    h = rng.standard_normal((40, 40))
    y0, kv = plain.block_attention(cfg, m0, w, "l0.mix.", h)
    y1, _ = plain.block_attention(cfg, dict(m1, scale=m0["scale"]), w, "l1.mix.", h, kv)
    assert np.allclose(y0, y1)
    # position 16 opens a block: it sees itself alone, so its output is its own value through the gate and W_o
    v16 = kv[1][16, 0]
    gate = plain.sigmoid(h[16] @ w["l0.mix.g"].T)
    alone = np.concatenate([v16 * gate[0], v16 * gate[1]]) @ w["l0.mix.o"].T
    assert np.allclose(y0[16], alone)
    # changing a token of the block before changes nothing from position 16 on
    h2 = h.copy(); h2[15] += 1.0
    y2, _ = plain.block_attention(cfg, m0, w, "l0.mix.", h2)
    assert np.allclose(y0[16:], y2[16:]) and not np.allclose(y0[15], y2[15])


def test_oracle_recurrence_against_its_unrolled_sum():
    """With the running maximum taken out, the state is a sum of k v^T weighted by exp(i_s + f_(s+1) + ... + f_t)."""
    cfg = {"norm": {"eps": 1e-6}}
    m = {"heads": 1, "dim": 3, "vdim": 2, "gate_cap": 4.0}
    rng = np.random.default_rng(1)
    W = 5
    w = {"q": rng.standard_normal((3, W)), "k": rng.standard_normal((3, W)), "v": rng.standard_normal((2, W)),
         "i": rng.standard_normal((1, W)), "i.b": np.array([0.3]), "f": rng.standard_normal((1, W)), "f.b": np.array([1.0]),
         "g": rng.standard_normal((2, W)), "o": np.eye(2), "norm": np.ones(2)}
    h = rng.standard_normal((6, W))
    got = plain.mlstm(cfg, m, w, "", h)
    q, k, v = h @ w["q"].T / 3 ** 0.5, h @ w["k"].T, h @ w["v"].T
    gi = 4.0 * np.tanh((h @ w["i"].T + 0.3) / 4.0)[:, 0]
    gf = plain.log_sigmoid(4.0 * np.tanh((h @ w["f"].T + 1.0) / 4.0))[:, 0]
    for t in range(6):
        logw = np.array([gi[s] + gf[s + 1:t + 1].sum() for s in range(t + 1)])
        mt = 0.0
        for s in range(t + 1):                     # the maximum as the recurrence defines it, from 0
            mt = max(gf[s] + mt, gi[s])
        wts = np.exp(logw - mt)
        S = sum(wts[s] * np.outer(k[s], v[s]) for s in range(t + 1))
        n = sum(wts[s] * k[s] for s in range(t + 1))
        o = S.T @ q[t] / (max(abs(n @ q[t]), np.exp(-mt)) + 1e-6)
        o = o / np.sqrt((o * o).mean() + 1e-6) * plain.sigmoid(h[t] @ w["g"].T)
        assert np.allclose(got[t], o)


def test_oracle_router_and_embedding():
    f = {"router": {"top": 2, "scale": 2.5}, "expert": {"limit": 1.0}}
    w = {"router": np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [-1.0, 0.0]])}
    chosen, wts, z = plain.route(f, w, "", np.array([[2.0, 1.0]]))
    assert list(chosen[0]) == [2, 0] and np.isclose(wts.sum(), 2.5)
    assert np.isclose(wts[0, 0] / wts[0, 1], np.exp(3.0 - 2.0))
    cfg = {"width": 6, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0, "bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 2}}}
    rng = np.random.default_rng(2)
    w = {"embed": rng.standard_normal((9, 6)), "bigram": rng.standard_normal((6, 6)), "embed.norm": np.ones(6)}
    x = plain.embedding(cfg, w, [4, 7, 7])
    raw1 = w["embed"][7] * 2.0 + w["bigram"][(4 * 3 + 7 * 2) % 5]
    raw1[0::2] += np.sin(1.0 * 10000.0 ** (-2.0 * np.arange(3) / 6)); raw1[1::2] += np.cos(1.0 * 10000.0 ** (-2.0 * np.arange(3) / 6))
    assert np.allclose(x[1], plain.rms_norm(raw1, None, 1e-5))
    raw0 = w["embed"][4] * 2.0 + w["bigram"][5]
    raw0[1::2] += 1.0
    assert np.allclose(x[0], plain.rms_norm(raw0, None, 1e-5))


def test_the_command_line_writes_and_describes_a_model(tmp_path, capsys):
    """`random` with a Nimelorn config.json, then `info`: the architecture is found by the file's own key, and the count
    of parameters is the sum over the tensors the parts declare."""
    import json
    from xpu_serve_b200.cli.main import main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny.CONFIGS["B"]))
    out = str(tmp_path / "model")
    assert main(["random", out, "--config", str(cfg_path), "--seed", "3", "--dtype", "bfloat16"]) == 0
    assert capsys.readouterr().out.strip() == out
    assert main(["info", out]) == 0
    info = json.loads(capsys.readouterr().out)
    spec = NimelornConfig.from_json(tiny.CONFIGS["B"]).model_spec()
    assert info["architecture"] == "nimelorn" and info["layers"] == 4 and info["vocab"] == 384 and not info["tied_head"]
    assert info["mixers"] == ["mlstm", "attention", "attention", "attention"]
    assert info["parameters"] == sum(int(np.prod(ts.shape)) for ts in expected_tensors(spec).values())
    assert NimelornConfig.from_json(json.loads(open(os.path.join(out, "config.json")).read())).to_json() == tiny.CONFIGS["B"]
