"""Layer norm with a weight and no bias over the last dimension, in float32:
(x - mean(x)) * (mean((x - mean(x))^2) + eps)^(-1/2) * w. One kernel adds a pending branch to the stream (through the
branch's own layer norm when the layer norms its branches), writes the sum back and produces the normed rows
(csrc/layernorm.cu). The few-row products cannot carry it across themselves (it needs the mean before anything can be
scaled), so decode steps run the same kernel."""
from __future__ import annotations

from typing import Optional

import torch

from .. import registry
from ..ops import lib as ops
from .base import Norm


class LayerNorm(Norm):
    kind = "layernorm"
    carried = False

    def __init__(self, spec, weights, weight_name: str, rt):
        super().__init__(spec, weights, weight_name, rt)
        self.w = rt.vector(weights[weight_name])
        self.eps = float(spec.eps)

    def normed(self, x: torch.Tensor) -> torch.Tensor:
        h = x.float().contiguous()
        y = torch.empty(h.shape, dtype=self.rt.act_dtype, device=h.device)
        ops.add_layernorm(h, None, None, self.w, y, None, self.eps)
        return y

    def add_norm(self, h, branch, post: Optional[Norm], y, rows) -> None:
        if post is not None and not isinstance(post, LayerNorm):
            return super().add_norm(h, branch, post, y, rows)
        ops.add_layernorm(h, branch, None if post is None else post.w, self.w if y is not None else None, y, rows,
                          self.eps, self.eps if post is None else post.eps)


registry.register_norm(LayerNorm.kind, LayerNorm)
