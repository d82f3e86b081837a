"""Mamba-2 mixer: in_proj, a causal depthwise convolution with silu over [x | B | C], the per-head recurrence

    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,   y_t = S_t^T C_t + D x_t,   dt_t = softplus(dt_raw_t + dt_bias)

then y * silu(z), a unit-RMS norm in `norm_groups` equal parts times a weight, and out_proj (csrc/mamba2.cu). A sequence
keeps the convolution's last taps - 1 inputs (activation type) and the state [heads, state, vdim] in float32; dt, the
decay and every sum of the recurrence are float32 in both precision modes. Long pieces of a prompt run chunk by chunk side
by side (two passes and a carry between them); single tokens and short pieces walk in order.
"""
from __future__ import annotations

import os
from typing import Dict

import numpy as np
import torch

from .. import registry
from ..ops import lib as ops
from .base import Mixer, StateNeed, TensorSpec


def chunk_plan(step, chunk: int, device):
    """The step's tokens cut into chunks of at most `chunk`, on the device: ([chunks, 3] (sequence, first token, tokens),
    [sequences + 1] first chunk of each), made once a step and shared by the step's layers (recurrent mixers that run
    long pieces chunk by chunk side by side)."""
    plans = step.__dict__.setdefault("_chunk_plans", {})
    if chunk not in plans:
        rows, first, t0 = [], [0], 0
        for i, n in enumerate(int(v) for v in step.q_lens_host):
            for c0 in range(0, n, chunk):
                rows.append((i, t0 + c0, min(chunk, n - c0)))
            first.append(len(rows))
            t0 += n
        plans[chunk] = (torch.from_numpy(np.asarray(rows, dtype=np.int32)).to(device),
                        torch.from_numpy(np.asarray(first, dtype=np.int32)).to(device))
    return plans[chunk]


class Mamba2Mixer(Mixer):
    kind = "mamba2"
    fixed_shape_ok = True      # a step captured for any lengths walks its tokens in order (no plan from the host)

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n, C = spec.names, spec.conv_channels
        return {
            n["in"]: TensorSpec((2 * spec.inner + 2 * spec.groups * spec.state + spec.heads, spec.hidden)),
            n["conv"]: TensorSpec((C, spec.taps), init="uniform:-0.5:0.5", role="vector"),
            n["conv_bias"]: TensorSpec((C,), role="vector"),
            n["dt_bias"]: TensorSpec((spec.heads,), init="uniform:-3:0", role="vector"),
            n["a_log"]: TensorSpec((spec.heads,), init="uniform:-1:1.5", role="vector"),
            n["d"]: TensorSpec((spec.heads,), init="uniform:0.5:1.5", role="vector"),
            n["norm"]: TensorSpec((spec.inner,), init="ones", role="vector"),
            n["out"]: TensorSpec((spec.hidden, spec.inner)),
        }

    @classmethod
    def cache_need(cls, spec):
        return (StateNeed((max(spec.taps - 1, 1), spec.conv_channels), "compute"),
                StateNeed((spec.heads, spec.state, spec.vdim), "float32"))

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if not 1 <= spec.taps <= 16:
            raise ValueError(f"mamba2: {spec.taps} taps (1 to 16 are supported)")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_in = rt.matrix(weights[n["in"]])
        self.w_out = rt.matrix(weights[n["out"]])
        self.taps = rt.vector(weights[n["conv"]].reshape(spec.conv_channels, spec.taps))
        self.conv_bias = rt.vector(weights[n["conv_bias"]])
        self.dt_bias = rt.vector(weights[n["dt_bias"]])
        self.a_log = rt.vector(weights[n["a_log"]])
        self.d_skip = rt.vector(weights[n["d"]])
        self.w_norm = rt.vector(weights[n["norm"]])
        # pieces of at least two chunks run chunk by chunk (XS_MAMBA2_CHUNK tokens each; 0: always in order)
        self.chunk = int(os.environ.get("XS_MAMBA2_CHUNK", "128"))

    def _plan(self, step):
        return chunk_plan(step, self.chunk, self.rt.device)

    def forward(self, x, step, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if cache is None or len(cache) != 2 or not cache.owner:
            raise RuntimeError("mamba2 keeps its own convolution inputs and state")
        T, inner, C = x.shape[0], s.inner, s.conv_channels
        proj = rt.linear(x, self.w_in, "m2_proj")
        xbc = rt.ws.get("m2_xbc", (T, C), rt.act_dtype)
        ops.mamba2_conv(proj, inner, self.taps, self.conv_bias, cache[0].storage, step.seq_of_token, step.cu_seqlens,
                        step.slots, xbc)
        y = rt.ws.get("m2_y", (T, inner), torch.float32)
        chunks = None
        if self.chunk > 0 and not step.fixed_shape and not step.decode and step.max_q_len >= 2 * self.chunk:
            chunk_seq, first_chunk = self._plan(step)
            n = chunk_seq.shape[0]
            chunks = (chunk_seq, first_chunk,
                      rt.ws.get("m2_chunk_state", (n, s.heads, s.state, s.vdim), torch.float32),
                      rt.ws.get("m2_chunk_decay", (n, s.heads), torch.float32))
        ops.mamba2_scan(xbc, proj, inner + C, self.dt_bias, self.a_log, self.d_skip, cache[1].storage, step.cu_seqlens,
                        step.slots, y, s.heads, s.vdim, s.state, s.groups, chunks)
        yn = rt.ws.get("m2_normed", (T, inner), rt.act_dtype)
        ops.grouped_rmsnorm(y, self.w_norm, yn, s.norm_groups, s.eps)
        return rt.linear(yn, self.w_out, "mixer_out")


registry.register_mixer(Mamba2Mixer.kind, Mamba2Mixer)
