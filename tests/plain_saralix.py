"""A plain, slow Saralix in float64 numpy: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json's keys itself and takes tensors by their
checkpoint names. Notation: T tokens, W the model's width, H heads. Weights are [out, in] and applied
as y = x W^T for rows x.

A layer is  x += post1(mixer(pre1(x)));  x += post2(ff(pre2(x)))  with four weight-only layer norms,
the last two on the branches. Mixers: latent attention (all earlier keys, softmax, a sigmoid gate per
head), latent attention with a window and a sink, and a Mamba-2 recurrence. Feed-forwards: a clamped
gated unit, or routed experts. Logits are the embedding table applied to the normed stream.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


# ------------------------------------------------------------------------------------ norms
def layer_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w over the last axis."""
    mu = x.mean(-1, keepdims=True)
    d = x - mu
    var = (d * d).mean(-1, keepdims=True)
    return d / np.sqrt(var + eps) * w


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def silu(z: np.ndarray) -> np.ndarray:
    return z * sigmoid(z)


def softplus(z: np.ndarray) -> np.ndarray:
    return np.logaddexp(0.0, z)


# --------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict, angle_bits: int = 64) -> (np.ndarray, float):
    """The dims/2 frequencies of a rotation and the factor on cos and sin. Without `scaling` the
    frequencies are base^(-2i/dims) and the factor is 1. With it (factor s, original length L, fast and
    slow turn counts): pairs that turn fast keep their frequency, pairs that turn slowly are divided by
    s, with a linear ramp between, and cos and sin are multiplied by 0.1 ln s + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    ft = np.float32 if angle_bits == 32 else np.float64
    i = np.arange(dims // 2, dtype=ft)
    f = (ft(base) ** (-(2.0 * i) / ft(dims))).astype(ft)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    s, L = float(sc["factor"]), float(sc["original"])

    def where(turns: float) -> float:
        return dims * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - ft(lo)) / ft(max(hi - lo, 0.001)), 0.0, 1.0).astype(ft)
    f = (f / ft(s) * ramp + f * (1 - ramp)).astype(ft)
    return f, 0.1 * math.log(s) + 1.0


def rotate(x: np.ndarray, pos: np.ndarray, rot: dict, angle_bits: int = 64) -> np.ndarray:
    """x [T, ..., D]: the first rot.dims channels of the last axis turn, channel i with channel
    i + dims/2, by the angle pos * f_i; the others pass."""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot, angle_bits)
    if angle_bits == 32:
        ang = (pos.astype(np.float32)[:, None] * f[None, :]).astype(np.float32).astype(np.float64)
    else:
        ang = pos.astype(np.float64)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = (np.cos(ang) * m).reshape(shape), (np.sin(ang) * m).reshape(shape)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.copy()
    out[..., :dims // 2] = u * c - v * s
    out[..., dims // 2:dims] = v * c + u * s
    return out


# -------------------------------------------------------------------------- latent attention
def latent_attention(h: np.ndarray, t: Dict[str, np.ndarray], pre: str, m: dict, eps: float, *, window: int = 0,
                     sink: bool = False, gate: bool = False, angle_bits: int = 64) -> np.ndarray:
    """Keys and values of all heads are made from one latent vector per token (kv_rank numbers,
    unit-RMS times a weight) plus one rotated key part that the heads share."""
    T = h.shape[0]
    H, dn, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = np.arange(T)
    q = (h @ t[pre + "q"].T).reshape(T, H, dn + dr)
    down = h @ t[pre + "dkv"].T
    c = unit_rms(down[:, :R], eps) * t[pre + "dkv.norm"]
    k_rot = rotate(down[:, R:], pos, m["rot"], angle_bits)                 # [T, dr], one for all heads
    q_rot = rotate(q[:, :, dn:], pos, m["rot"], angle_bits)                # [T, H, dr]
    k_plain = (c @ t[pre + "uk"].T).reshape(T, H, dn)
    v = (c @ t[pre + "uv"].T).reshape(T, H, dv)
    s = (np.einsum("ihd,jhd->hij", q[:, :, :dn], k_plain) + np.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) if window <= 0 else ((j <= i) & (i - j < window))
    s = np.where(seen[None], s, -np.inf)
    top = s.max(-1, keepdims=True)
    if sink:
        top = np.maximum(top, t[pre + "sink"].reshape(H, 1, 1))
    e = np.exp(s - top)
    den = e.sum(-1, keepdims=True)
    if sink:       # one more term in the denominator, with no key and no value
        den = den + np.exp(t[pre + "sink"].reshape(H, 1, 1) - top)
    o = np.einsum("hij,jhd->ihd", e / den, v)
    if gate:
        o = o * sigmoid(h @ t[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ t[pre + "o"].T


# ---------------------------------------------------------------------------------- mamba-2
def mamba2(h: np.ndarray, t: Dict[str, np.ndarray], pre: str, m: dict, eps: float) -> np.ndarray:
    """Per head a state S [N, P] with S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T and
    y_t = S_t^T C_t + D x_t, behind a causal convolution with silu on x, B and C."""
    T = h.shape[0]
    Hh, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    taps, parts = int(m["conv"]), int(m["norm_groups"])
    inner = Hh * P
    proj = h @ t[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    w, b = t[pre + "conv"], t[pre + "conv.b"]
    padded = np.concatenate([np.zeros((taps - 1, xbc.shape[1])), xbc], 0)
    conv = np.zeros_like(xbc)
    for k in range(taps):                      # the last column of the taps belongs to the current token
        conv += padded[k:k + T] * w[:, k]
    xbc = silu(conv + b)
    x = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + t[pre + "dt_bias"])
    decay = np.exp(-np.exp(t[pre + "A_log"]) * dt)                       # [T, Hh]
    y = np.zeros((T, Hh, P))
    for hd in range(Hh):
        g = hd // (Hh // G)
        S = np.zeros((N, P))
        for i in range(T):
            S = decay[i, hd] * S + dt[i, hd] * np.outer(B[i, g], x[i, hd])
            y[i, hd] = S.T @ C[i, g] + t[pre + "D"][hd] * x[i, hd]
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * t[pre + "norm"]
    return y @ t[pre + "o"].T


# ---------------------------------------------------------------------------- feed-forwards
def dense_ff(h: np.ndarray, t: Dict[str, np.ndarray], pre: str, f: dict) -> np.ndarray:
    lim = float(f["limit"])
    g = np.minimum(h @ t[pre + "gate"].T, lim)
    u = np.clip(h @ t[pre + "up"].T, -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[pre + "down"].T


def routed_ff(h: np.ndarray, t: Dict[str, np.ndarray], pre: str, f: dict, margins: Optional[np.ndarray] = None) -> np.ndarray:
    """`margins` [T] is lowered to each token's gap between the last chosen and the first unchosen logit, relative to
    the largest |logit| (a comparison at reduced precision may then leave out the tokens whose choice is a close call)."""
    E, k = int(f["router"]["experts"]), int(f["router"]["top"])
    logits = h @ t[pre + "router"].T
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        order = np.argsort(-logits[i], kind="stable")
        chosen = order[:k]
        if margins is not None and k < E:
            margins[i] = min(margins[i], (logits[i, order[k - 1]] - logits[i, order[k]]) / np.abs(logits[i]).max())
        wts = np.exp(logits[i, chosen] - logits[i, chosen].max())
        wts = wts / wts.sum()
        for e, a in zip(chosen, wts):
            p = f"{pre}e{int(e)}."
            out[i] += a * ((silu(h[i] @ t[p + "gate"].T) * (h[i] @ t[p + "up"].T)) @ t[p + "down"].T)
    return out


# ------------------------------------------------------------------------------- the model
def forward(cfg: dict, t: Dict[str, np.ndarray], tokens: Sequence[int], angle_bits: int = 64,
            streams: Optional[List[np.ndarray]] = None, margins: Optional[np.ndarray] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence. `streams` collects the residual stream after every layer; `margins` [T]
    (start it at infinity) takes each token's smallest router margin over the layers."""
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][np.asarray(tokens, dtype=np.int64)]
    for i, layer in enumerate(cfg["layers"]):
        p, kind, m = f"l{i}.", layer["type"], layer["mixer"]
        h = layer_norm(x, t[p + "norm1"], eps)
        if kind == "latent_attention":
            y = latent_attention(h, t, p + "mix.", m, eps, gate=True, angle_bits=angle_bits)
        elif kind == "latent_attention_2":
            y = latent_attention(h, t, p + "mix.", m, eps, window=int(m["mask"]["size"]), sink=True, angle_bits=angle_bits)
        elif kind == "mamba2":
            y = mamba2(h, t, p + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown type {kind}")
        x = x + layer_norm(y, t[p + "norm1b"], eps)
        f = layer.get("mlp")
        if f is not None:
            h = layer_norm(x, t[p + "norm2"], eps)
            y = dense_ff(h, t, p + "mlp.", f) if f["kind"] == "dense" else routed_ff(h, t, p + "mlp.", f, margins)
            x = x + layer_norm(y, t[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.copy())
    return layer_norm(x, t["final.norm"], eps) @ t["embed"].T
