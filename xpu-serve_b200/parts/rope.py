"""Rotary position encoding as a table of (cos, sin) per position and channel pair.

Pair i couples channels i and i + head_dim/2 (rotate-half); inv_freq[i] is the float32
value of theta^(-2i/head_dim) for the first `pairs` pairs and 0 beyond them, so the
unrotated tail of a partially rotated head passes through unchanged
(src/models/common/blocks.cpp:131-141). The angle pos * inv_freq and its cos and sin are
formed in float64, as the reference's CPU backend forms them
(src/backend/cpu_ref/ops.cpp:383-387), and stored as float32: a float32 angle alone would
be off by up to pos * 2^-24 rad.

A position encoding of another kind registers a class with the same two methods; the
attention kernels only see the table.
"""
from __future__ import annotations

import torch

from .. import registry


class RotaryTable:
    kind = "rope"

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.key = ("rope", spec.head_dim, float(spec.theta), spec.pairs)

    def inv_freq(self) -> torch.Tensor:
        s = self.spec
        i = torch.arange(s.head_dim // 2, dtype=torch.float64)
        inv = (1.0 / torch.pow(torch.tensor(float(s.theta), dtype=torch.float64), 2.0 * i / s.head_dim))
        inv = inv.to(torch.float32)
        inv[s.pairs:] = 0.0
        return inv

    def table(self, n_positions: int) -> torch.Tensor:
        """[n_positions or more, head_dim / 2, 2] float32 on the device."""
        have = self.rt.shared.get(self.key)
        if have is not None and have.shape[0] >= n_positions:
            return have
        inv = self.inv_freq().to(device=self.rt.device, dtype=torch.float64)
        pos = torch.arange(n_positions, dtype=torch.float64, device=self.rt.device)
        angle = pos[:, None] * inv[None, :]
        table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()
        if have is not None:     # a captured graph may still read the shorter table: keep it alive
            self.rt.shared.setdefault(("kept",), []).append(have)
        self.rt.shared[self.key] = table
        return table


class ScaledRotaryTable:
    """The table of a rotation over the first `dims` channels of a vector (pair i couples channels i and i + dims/2),
    with frequencies stretched for long sequences (config/spec.py: ScaledRopeSpec, RopeScalingSpec):

        f_i = theta^(-2i/dims);  where(t) = dims * ln(original / (2 pi t)) / (2 ln theta)
        lo = max(floor(where(fast)), 0);  hi = min(ceil(where(slow)), dims - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);  f'_i = f_i / factor * ramp_i + f_i * (1 - ramp_i)

    and cos and sin multiplied by mscale_k * ln(factor) + 1. Angles are formed in float64 as RotaryTable's are.
    table(n) is [n or more, dims / 2, 2] float32."""
    kind = "rope_scaled"

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        sc = spec.scaling
        self.key = ("rope_scaled", spec.dims, float(spec.theta),
                    None if sc is None else (sc.factor, sc.original, sc.fast, sc.slow, sc.mscale_k))

    def frequencies(self):
        """(float64 [dims / 2], the factor on cos and sin)."""
        import math
        s = self.spec
        i = torch.arange(s.dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(float(s.theta), dtype=torch.float64), -2.0 * i / s.dims)
        sc = s.scaling
        if sc is None:
            return f, 1.0

        def where(turns: float) -> float:
            return s.dims * math.log(sc.original / (2.0 * math.pi * turns)) / (2.0 * math.log(s.theta))

        lo = max(math.floor(where(sc.fast)), 0)
        hi = min(math.ceil(where(sc.slow)), s.dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / sc.factor * ramp + f * (1.0 - ramp), sc.mscale_k * math.log(sc.factor) + 1.0

    def table(self, n_positions: int) -> torch.Tensor:
        have = self.rt.shared.get(self.key)
        if have is not None and have.shape[0] >= n_positions:
            return have
        f, m = self.frequencies()
        pos = torch.arange(n_positions, dtype=torch.float64, device=self.rt.device)
        angle = pos[:, None] * f.to(self.rt.device)[None, :]
        table = (torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1) * m).to(torch.float32).contiguous()
        if have is not None:     # a captured graph may still read the shorter table: keep it alive
            self.rt.shared.setdefault(("kept",), []).append(have)
        self.rt.shared[self.key] = table
        return table


registry.register_position(RotaryTable.kind, RotaryTable)
registry.register_position(ScaledRotaryTable.kind, ScaledRotaryTable)
