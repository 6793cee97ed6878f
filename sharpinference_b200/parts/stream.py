"""Operations on the residual stream between scheduled blocks.

``ReinjectInput``: ``x <- W [x ; x0] + b``, the stream and the embedding output side by side through one
projection ``W [H, 2H]`` (the stream's half first), plus a vector ``b [H]``.  A model that runs a span of layers
several times with the same weights puts one of these before every pass, each with its own ``b``.  The product is
a matrix product like any other (operands in the activation dtype, float32 accumulation and output); the sum
that enters it and the vector added after it are float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import StepContext, StreamOp, register_part
from .linear import Linear


@register_part("stream", "reinject_input")
class ReinjectInput(StreamOp):
    graph_safe = True

    def __init__(self, *, proj: Linear, act_dtype: torch.dtype = torch.bfloat16):
        if proj.in_features != 2 * proj.out_features:
            raise ValueError(f"the re-injection projection is [{proj.out_features}, {proj.in_features}], "
                             f"expected [H, 2H]")
        self.proj, self.act_dtype = proj, act_dtype

    def forward(self, ctx: StepContext, x: torch.Tensor, pending: Optional[torch.Tensor], x0: torch.Tensor):
        both = ops.concat2(x, pending, x0, self.act_dtype)
        return self.proj(both), None
