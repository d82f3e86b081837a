"""Tiny Saralix configurations for the tests, and helpers to write them as model folders with random weights.

M mixes every mixer and feed-forward at sizes that are no multiple of 8 and differ from one another (heads, head
sizes, ranks, groups, taps, experts): a gated latent attention with a stretched rotation, two Mamba-2 layers (one whose
state has more rows than a thread keeps at a time is in N), a windowed latent attention with sinks, an unstretched
rotation and no feed-forward at all, dense and routed feed-forwards (top 3 of 6). N has widths that are multiples of 8,
a window longer than a cache page, one head, one expert chosen of three, and a state of 160 rows. D has every mixer and
no experts. The single-layer configurations run one mechanism alone.
"""
import os

from xpu_serve_b200.config import SaralixConfig
from xpu_serve_b200.weights import write_random_model


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None, scaling=None, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims, "scaling": scaling}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(width, vocab, layers, eps=1e-5):
    return {"architecture": "Saralix", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


STRETCH = {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}

CONFIGS = {
    "M": model(44, 203, [
        ("latent_attention", latent(3, 12, 8, 20, 36, 0.21, base=5000.0, scaling=STRETCH), dense(70, 1.5)),
        ("mamba2", mamba(6, 6, 12, 3, 3, 3), moe(20, 6, 3)),
        ("latent_attention_2", latent(2, 10, 12, 14, 22, 0.3, base=300.0, window=13), None),
        ("mamba2", mamba(2, 20, 40, 1, 2, 1), dense(50, 0.7)),
        ("latent_attention", latent(5, 6, 4, 6, 18, 0.4, base=70.0, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 2.0}),
         moe(12, 5, 2)),
    ], eps=3e-6),
    "N": model(128, 384, [
        ("mamba2", mamba(4, 32, 160, 2, 5, 4), moe(48, 3, 1)),
        ("latent_attention_2", latent(1, 48, 16, 40, 96, 0.15, base=100000.0, scaling={"factor": 16.0, "original": 32, "fast": 16.0, "slow": 0.5},
                                      window=70), dense(256, 3.0)),
        ("latent_attention", latent(8, 16, 32, 8, 24, 0.18, base=777.0), moe(64, 8, 4)),
    ]),
    # every mixer, no experts: at reduced precision no router's close call stands between a fault and the bound
    "D": model(64, 180, [
        ("latent_attention_2", latent(4, 16, 16, 8, 48, 0.2, base=2000.0, scaling=STRETCH, window=21), dense(96, 2.5)),
        ("mamba2", mamba(4, 16, 32, 4, 4, 2), None),
        ("latent_attention", latent(2, 24, 8, 32, 16, 0.25, base=400.0), dense(40, 1.0)),
        ("mamba2", mamba(8, 8, 8, 1, 3, 8), dense(72, 4.0)),
    ]),
    # one mechanism each (the feed-forward ones behind the smallest mixer)
    # (only the first 4 of the 6 rotated channels turn: the rotation's own width may be smaller than the part it stands in)
    "gated": model(40, 150, [("latent_attention", latent(2, 14, 6, 10, 28, 0.25, base=900.0, dims=4, scaling=STRETCH), None)]),
    "windowed": model(40, 150, [("latent_attention_2", latent(3, 8, 10, 12, 20, 0.3, base=50.0, window=9), None)]),
    "recurrent": model(40, 150, [("mamba2", mamba(4, 10, 24, 2, 4, 2), None)]),
    "dense": model(40, 150, [("mamba2", mamba(1, 8, 4, 1, 2, 1), dense(90, 1.0))]),
    "routed": model(40, 150, [("mamba2", mamba(1, 8, 4, 1, 2, 1), moe(30, 7, 3))]),
}

# What makes a lost part show: norm weights away from 1, sinks and routers and decay rates of a size that matters.
SCALE = {".mix.sink": 30.0, ".mlp.router": 6.0, ".mix.g": 8.0}


def make_folder(root, name: str, dtype: str, seed: int = 11, std: float = 0.08):
    folder = os.path.join(str(root), f"saralix_{name}_{dtype}")
    if not os.path.isdir(folder):
        write_random_model(folder, SaralixConfig.from_json(CONFIGS[name]), seed=seed, dtype=dtype, std=std,
                           norm_range=(0.5, 1.5), scale=SCALE)
    return folder


def prompt(name: str, length: int, salt: int = 0):
    V = CONFIGS[name]["vocab"]
    return [(i * 29 + 3 + 13 * salt + (i * i) % 11) % V for i in range(length)]


U_BF16 = 2.0 ** -9


def upper_limit(name: str, dtype: str) -> float:
    """Largest |difference| / largest |reference logit| that rounding alone may cause: float32 1e-5; bfloat16 about
    ten roundings to 8 bits a layer that add like a random walk, times 4 for the largest of many logits. The norms on
    the branches renormalise every branch, which costs a further factor (measured on the LFM3 layouts with such norms:
    ten times the others'); 3 is used here."""
    layers = len(CONFIGS[name]["layers"])
    return 1e-5 if dtype == "float32" else 3.0 * 4.0 * (10.0 * layers) ** 0.5 * U_BF16
