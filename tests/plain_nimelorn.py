"""A plain, slow Nimelorn in float64 numpy: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json's keys itself and takes tensors by their
checkpoint names. Notation: T tokens, W the model's width. Weights are [out, in] and applied as
y = x W^T for rows x.

Embedding: table row times a constant, plus a row of a second table chosen by a hash of the previous and
the current token, plus a sine/cosine vector of the position, then an RMS norm. A layer is
x += norm1(mixer(x)); x += norm2(ff(x)): the sublayers read the stream itself, the norms act on what
they return. Mixers: grouped-query attention without rotation whose queries see the earlier keys of
their own block of positions only, with a sigmoid gate per head (a layer may read an earlier layer's
keys and values); and the matrix-memory recurrence of xLSTM. Feed-forwards: squared-ReLU, or routed
clamped gated units with a gated shared unit.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


def rms_norm(x: np.ndarray, w, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


# -------------------------------------------------------------------------------- embedding
def position_vector(pos: np.ndarray, width: int, angle_bits: int = 64) -> np.ndarray:
    """[T, width]: entry 2i is sin(p f_i), entry 2i + 1 cos(p f_i), f_i = 10000^(-2i / width)."""
    i = np.arange((width + 1) // 2, dtype=np.float64)
    f = 10000.0 ** (-2.0 * i / width)
    if angle_bits == 32:
        ang = (pos.astype(np.float32)[:, None] * f.astype(np.float32)[None, :]).astype(np.float64)
    else:
        ang = pos.astype(np.float64)[:, None] * f[None, :]
    out = np.zeros((len(pos), 2 * len(i)))
    out[:, 0::2] = np.sin(ang)
    out[:, 1::2] = np.cos(ang)
    return out[:, :width]


def embedding(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], angle_bits: int = 64) -> np.ndarray:
    e = cfg["embedding"]
    b = e["bigram"]
    buckets = int(b["buckets"])
    toks = np.asarray(tokens, dtype=np.int64)
    prev = np.concatenate([[0], toks[:-1]])
    rows = (prev * int(b["mul_prev"]) + toks * int(b["mul_cur"])) % buckets
    rows[0] = buckets                       # a sequence's first token has no previous one: the table's last row
    x = w["embed"][toks] * float(e["scale"]) + w["bigram"][rows]
    x = x + position_vector(np.arange(len(toks)), int(cfg["width"]), angle_bits)
    return rms_norm(x, w["embed.norm"], float(cfg["norm"]["eps"]))


# -------------------------------------------------------------------------------- attention
def block_attention(cfg: dict, m: dict, w: Dict[str, np.ndarray], p: str, h: np.ndarray,
                    shared_kv=None):
    """Returns (output [T, W], (k, v)): k normed [T, G, dim], v [T, G, vdim]. `shared_kv`: another layer's."""
    eps = float(cfg["norm"]["eps"])
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = rms_norm((h @ w[p + "q"].T).reshape(T, H, D), w[p + "q.norm"], eps)
    if shared_kv is None:
        k = rms_norm((h @ w[p + "k"].T).reshape(T, G, D), w[p + "k.norm"], eps)
        v = (h @ w[p + "v"].T).reshape(T, G, Dv)
    else:
        k, v = shared_kv
    size = int(m["mask"]["size"])
    pos = np.arange(T)
    visible = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    gate = sigmoid(h @ w[p + "g"].T)                     # [T, H]
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = np.where(visible, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        pr = np.exp(s)
        pr /= pr.sum(-1, keepdims=True)
        out[:, hd] = (pr @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * Dv) @ w[p + "o"].T, (k, v)


# ----------------------------------------------------------------------------------- mlstm
def mlstm(cfg: dict, m: dict, w: Dict[str, np.ndarray], p: str, h: np.ndarray) -> np.ndarray:
    eps = float(cfg["norm"]["eps"])
    H, D, Dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, Dv)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                   # [T, H] log input gate
    gf = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))      # [T, H] log forget gate
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        S = np.zeros((D, Dv))
        n = np.zeros(D)
        mx = 0.0
        for t in range(T):
            m_new = max(gf[t, hd] + mx, gi[t, hd])
            a, b = math.exp(gf[t, hd] + mx - m_new), math.exp(gi[t, hd] - m_new)
            S = a * S + b * np.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(n @ q[t, hd]), math.exp(-mx)) + 1e-6)
    out = rms_norm(out, None, eps).reshape(T, H * Dv) * w[p + "norm"]
    out = out * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forwards
def squared_relu_ff(w: Dict[str, np.ndarray], p: str, h: np.ndarray) -> np.ndarray:
    a = np.maximum(h @ w[p + "up"].T, 0.0)
    return (a * a) @ w[p + "down"].T


def clamped_unit(w: Dict[str, np.ndarray], p: str, h: np.ndarray, limit: float) -> np.ndarray:
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(f: dict, w: Dict[str, np.ndarray], p: str, h: np.ndarray):
    """(chosen [T, top], weights [T, top], logits [T, E])."""
    z = h @ w[p + "router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    top = int(f["router"]["top"])
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    cs = np.take_along_axis(s, chosen, -1)
    return chosen, cs / (cs.sum(-1, keepdims=True) + 1e-20) * float(f["router"]["scale"]), z


def routed_ff(f: dict, w: Dict[str, np.ndarray], p: str, h: np.ndarray) -> np.ndarray:
    chosen, wts, _ = route(f, w, p, h)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    limit = float(f["expert"]["limit"])
    for t in range(h.shape[0]):
        for c, e in enumerate(chosen[t]):
            out[t] += wts[t, c] * clamped_unit(w, f"{p}e{int(e)}.", h[t:t + 1], limit)[0]
    if f.get("shared") is not None:
        sh = clamped_unit(w, p + "shared.", h, float(f["shared"]["limit"]))
        out += sh * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------------ model
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], angle_bits: int = 64,
            layers_out: Optional[List[np.ndarray]] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence from its first token. `layers_out` collects the stream after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = embedding(cfg, w, tokens, angle_bits)
    kv: Dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            y, kv[i] = block_attention(cfg, m, w, p, x, None if src is None else kv[int(src)])
        elif layer["type"] == "mlstm":
            y = mlstm(cfg, m, w, p, x)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']}")
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            q = f"l{i}.mlp."
            y = squared_relu_ff(w, q, x) if f["kind"] == "dense" else routed_ff(f, w, q, x)
            x = x + rms_norm(y, w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def router_margins(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    """[T]: over the routed layers, the smallest gap between the last chosen and the first left-out
    router logit, divided by the largest |logit| (inf without routed layers)."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    streams: List[np.ndarray] = []
    forward(cfg, w, tokens, layers_out=streams)
    eps = float(cfg["norm"]["eps"])
    out = np.full(len(tokens), np.inf)
    x_in = embedding(cfg, w, tokens)
    for i, layer in enumerate(cfg["layers"]):
        f = layer.get("mlp")
        if f is not None and f["kind"] == "moe":
            # the feed-forward's input: the stream after the mixer's branch joined it
            p, m = f"l{i}.mix.", layer["mixer"]
            if layer["type"] == "attention":
                kvs: Dict[int, tuple] = {}
                src = m.get("kv_from")
                if src is not None:
                    prev_in = x_in if int(src) == 0 else streams[int(src) - 1]
                    _, kvs[int(src)] = block_attention(cfg, cfg["layers"][int(src)]["mixer"], w, f"l{int(src)}.mix.", prev_in)
                y, _ = block_attention(cfg, m, w, p, x_in, None if src is None else kvs[int(src)])
            else:
                y = mlstm(cfg, m, w, p, x_in)
            mid = x_in + rms_norm(y, w[f"l{i}.norm1"], eps)
            _, _, z = route(f, w, f"l{i}.mlp.", mid)
            zs = -np.sort(-z, axis=-1)
            top = int(f["router"]["top"])
            if top < z.shape[1]:
                out = np.minimum(out, (zs[:, top - 1] - zs[:, top]) / np.abs(z).max())
        x_in = streams[i]
    return out
