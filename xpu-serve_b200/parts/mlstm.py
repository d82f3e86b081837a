"""The mLSTM mixer (the matrix memory of xLSTM): per head a state S [dim, vdim], a normaliser n [dim] and a running
maximum m, all float32 and zero at a sequence's start. For a token with input x:

    q = Wq x / sqrt(dim),  k = Wk x,  v = Wv x
    i = cap tanh((Wi x + bi) / cap)                        log of the input gate
    f = logsigmoid(cap tanh((Wf x + bf) / cap))            log of the forget gate
    m' = max(f + m, i);   S' = exp(f + m - m') S + exp(i - m') k v^T;   n' likewise with k alone
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

then every head's o divided by its root mean square, times a weight over all heads, times sigmoid(Wg x), and the output
projection. One product gives q, k, v and the output gate's logits in the activation type; the two gates' pre-activations
come from a second product whose output is float32, and everything behind them (soft cap, logsigmoid, the maximum, the
exponentials, the state and its sums, the heads' norm) is float32 in both precision modes (csrc/mlstm.cu). Single tokens
and short pieces walk in order; long pieces of a prompt run chunk by chunk side by side (a pass from the empty state, a
carry between the chunks, a second pass from each chunk's true state).
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import Mixer, StateNeed, TensorSpec
from .mamba2 import chunk_plan


def _copies(vdim: int) -> int:
    """Copies of n and m the kernel keeps per head: one per block of 64 value columns (csrc/mlstm.cu)."""
    return (vdim + 63) // 64


class MLstmMixer(Mixer):
    kind = "mlstm"
    fixed_shape_ok = True      # the kernel finds every sequence's tokens in the step's description on the device

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        qd, vd = spec.heads * spec.dim, spec.heads * spec.vdim
        return {
            n["q"]: TensorSpec((qd, spec.hidden)), n["k"]: TensorSpec((qd, spec.hidden)),
            n["v"]: TensorSpec((vd, spec.hidden)), n["gate"]: TensorSpec((vd, spec.hidden)),
            n["o"]: TensorSpec((spec.hidden, vd)), n["norm"]: TensorSpec((vd,), init="ones", role="vector"),
            n["i"]: TensorSpec((spec.heads, spec.hidden)), n["i_bias"]: TensorSpec((spec.heads,), init="uniform:-1:1", role="vector"),
            n["f"]: TensorSpec((spec.heads, spec.hidden)), n["f_bias"]: TensorSpec((spec.heads,), init="uniform:1:4", role="vector"),
        }

    @classmethod
    def cache_need(cls, spec):
        return (StateNeed((spec.heads, spec.dim, spec.vdim), "float32"),
                StateNeed((spec.heads, _copies(spec.vdim), spec.dim + 1), "float32"))

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.dim > 256:
            raise ValueError(f"mlstm: key size {spec.dim} (at most 256 is supported)")
        if not spec.gate_cap > 0:
            raise ValueError("mlstm: gate_cap must be positive")
        self.spec, self.rt = spec, rt
        n = spec.names
        f32 = torch.float32
        # [q; k; v; output gate] as one product; [input gates; forget gates] (padded to whole 16-row tiles) as another
        self.w_in = rt.matrix(torch.cat([weights[n[k]].to(f32) for k in ("q", "k", "v", "gate")], 0))
        g = torch.cat([weights[n["i"]].to(f32), weights[n["f"]].to(f32)], 0)
        pad = (-g.shape[0]) % 16
        if pad:
            g = torch.cat([g, torch.zeros(pad, g.shape[1])], 0)
        self.w_gates = rt.matrix(g)
        self.i_bias = rt.vector(weights[n["i_bias"]])
        self.f_bias = rt.vector(weights[n["f_bias"]])
        self.w_norm = rt.vector(weights[n["norm"]])
        self.w_o = rt.matrix(weights[n["o"]])
        # Pieces of at least two chunks run chunk by chunk side by side. XS_MLSTM_CHUNK: tokens a chunk (0: always in order);
        # unset: as many chunks as fill the device once with two CTAs an SM, between 64 and 512 tokens each (measured on
        # B200, 2,048 tokens, 16 heads of 64 x 128: chunks of 64 / 128 / 256 tokens take 0.68 / 0.51 / 0.42 ms a layer).
        self.chunk = int(os.environ["XS_MLSTM_CHUNK"]) if "XS_MLSTM_CHUNK" in os.environ else None

    def forward(self, x, step, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if cache is None or len(cache) != 2 or not cache.owner:
            raise RuntimeError("mlstm keeps its own state")
        T, qd, vd = x.shape[0], s.heads * s.dim, s.heads * s.vdim
        proj = rt.linear(x, self.w_in, "mlstm_proj")
        gates = rt.linear(x, self.w_gates, "mlstm_gates", out_dtype=torch.float32)
        y = rt.ws.get("mlstm_y", (T, vd), torch.float32)
        chunks = None
        chunk = self.chunk
        if chunk is None:
            at_once = max(1, (2 * rt.sm_count) // (s.heads * _copies(s.vdim)))
            chunk = min(512, max(64, -(-T // at_once // 8) * 8))
        if chunk > 0 and not step.fixed_shape and not step.decode and step.max_q_len >= 2 * chunk:
            # a long piece: its chunks from the empty state side by side, a carry over them in order, then the chunks again
            # from their true states (csrc/mlstm.cu)
            chunk_seq, first_chunk = chunk_plan(step, chunk, rt.device)
            n = chunk_seq.shape[0]
            chunks = (chunk_seq, first_chunk, rt.ws.get("mlstm_chunk_state", (n, s.heads, s.dim, s.vdim), torch.float32),
                      rt.ws.get("mlstm_chunk_nm", (n, s.heads, _copies(s.vdim), s.dim + 2), torch.float32))
        ops.mlstm_scan(proj, 0, qd, 2 * qd, gates, self.i_bias, self.f_bias, cache[0].storage, cache[1].storage,
                       step.cu_seqlens, step.slots, y, s.heads, s.dim, s.vdim, s.gate_cap, float(s.dim) ** -0.5, chunks)
        yn = rt.ws.get("mlstm_normed", (T, vd), rt.act_dtype)
        ops.grouped_rmsnorm(y, self.w_norm, yn, s.heads, s.eps, gate=proj[:, 2 * qd + vd:])
        return rt.linear(yn, self.w_o, "mixer_out")


registry.register_mixer(MLstmMixer.kind, MLstmMixer)
