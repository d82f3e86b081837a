"""Tiny Nimelorn configurations for the tests, and helpers to write them as model folders with random weights.

A mixes every mixer and feed-forward at sizes that are no multiple of 8 and differ from one another: attention whose value
heads are larger than its key heads, a block mask shorter than a cache page, a layer that reads an earlier layer's keys
and values under a mask of its own, two recurrences (one with more value columns than key rows, one with fewer), dense
and routed feed-forwards with and without a shared unit (top 3 of 6, top 2 of 5). B has widths that are multiples of 8,
key and value heads of one size, a block mask longer than a page, one query head per key head, one expert chosen of
three. C has every mixer and no experts. The single-layer configurations run one mechanism alone.
"""
import os

from xpu_serve_b200.config import NimelornConfig
from xpu_serve_b200.weights import write_random_model


def attention(heads, kv_heads, dim, vdim, size, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, scale, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared is not None:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def model(width, vocab, layers, eps=1e-5, scale=3.0, buckets=97, mul_prev=31, mul_cur=7):
    return {"architecture": "Nimelorn", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


CONFIGS = {
    "A": model(44, 203, [
        ("attention", attention(4, 2, 12, 20, 13, 0.21), dense(70)),
        ("attention", attention(6, 3, 10, 6, 40, 0.35), moe(20, 1.5, 6, 3, 1.7, shared=(24, 0.8))),
        ("mlstm", mlstm(3, 10, 14, 9.0), None),
        ("attention", attention(6, 3, 10, 6, 29, 0.3, kv_from=1), moe(12, 0.6, 5, 2, 0.9)),
        ("mlstm", mlstm(2, 6, 40, 5.0), dense(50)),
    ], eps=3e-6, scale=5.5, buckets=211, mul_prev=1009, mul_cur=3),
    "B": model(128, 384, [
        ("mlstm", mlstm(4, 32, 32, 15.0), moe(48, 2.0, 3, 1, 2.0, shared=(64, 3.0))),
        ("attention", attention(4, 4, 64, 64, 70, 0.11), dense(256)),
        ("attention", attention(8, 2, 16, 32, 128, 0.3), moe(64, 1.0, 8, 4, 1.0)),
        ("attention", attention(4, 4, 64, 64, 200, 0.2, kv_from=1), dense(96)),
    ], scale=11.0, buckets=509, mul_prev=2, mul_cur=65537),
    # every mixer, no experts: at reduced precision no router's close call stands between a fault and the bound
    "C": model(64, 180, [
        ("attention", attention(4, 2, 32, 48, 21, 0.2), dense(96)),
        ("mlstm", mlstm(4, 16, 24, 8.0), None),
        ("attention", attention(4, 2, 32, 48, 64, 0.15, kv_from=0), dense(40)),
        ("mlstm", mlstm(1, 8, 64, 20.0), dense(72)),
    ], scale=8.0, buckets=31, mul_prev=5, mul_cur=11),
    # one mechanism each (the feed-forward ones behind the smallest mixer)
    "blocked": model(40, 150, [("attention", attention(4, 2, 14, 10, 9, 0.25), None)]),
    "borrowed": model(40, 150, [("attention", attention(2, 1, 8, 12, 16, 0.3), None),
                                ("attention", attention(2, 1, 8, 12, 5, 0.4, kv_from=0), None)]),
    # three query heads a key head and one head size that no tensor-core kernel takes: the generic kernel in both types
    "odd": model(40, 150, [("attention", attention(6, 2, 20, 20, 7, 0.3), dense(30))]),
    "recurrent": model(40, 150, [("mlstm", mlstm(4, 10, 6, 7.0), None)]),
    "dense": model(40, 150, [("mlstm", mlstm(1, 4, 8, 10.0), dense(90))]),
    "routed": model(40, 150, [("mlstm", mlstm(1, 4, 8, 10.0), moe(30, 1.2, 7, 3, 2.5, shared=(16, 0.5)))]),
}

# What makes a lost part show: norm weights away from 1, and routers, gates and the pair table of a size that matters.
SCALE = {".mlp.router": 6.0, ".mix.g": 8.0, ".mlp.shared.sg": 10.0, "bigram": 20.0, ".mix.i": 2.0, ".mix.f": 2.0}


def make_folder(root, name: str, dtype: str, seed: int = 17, std: float = 0.08):
    folder = os.path.join(str(root), f"nimelorn_{name}_{dtype}")
    if not os.path.isdir(folder):
        write_random_model(folder, NimelornConfig.from_json(CONFIGS[name]), seed=seed, dtype=dtype, std=std,
                           norm_range=(0.5, 1.5), scale=SCALE)
    return folder


def prompt(name: str, length: int, salt: int = 0):
    V = CONFIGS[name]["vocab"]
    return [(i * 29 + 3 + 13 * salt + (i * i) % 11) % V for i in range(length)]


U_BF16 = 2.0 ** -9


def upper_limit(name: str, dtype: str) -> float:
    """Largest |difference| / largest |reference logit| that rounding alone may cause: float32 1e-5; bfloat16 about
    ten roundings to 8 bits a layer that add like a random walk, times 4 for the largest of many logits. The norms on
    the branches renormalise every branch, which costs a further factor (measured on layouts with such norms: ten times
    the others'); 3 is used here."""
    layers = len(CONFIGS[name]["layers"])
    return 1e-5 if dtype == "float32" else 3.0 * 4.0 * (10.0 * layers) ** 0.5 * U_BF16
