"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..weights import TensorSpec, NORM, BIAS
from .base import Part, to_device_vector


class RMSNorm(Part):
    """y = x / sqrt(mean(x^2) + eps) * weight, statistics in 32-bit, the weight used as stored
    (src/math.br:18-36). Input: the 32-bit residual stream; output: the engine's activation dtype.
    `scalar_weight`: the checkpoint holds ONE number (a tensor without dimensions) that multiplies every coordinate; it is
    spread over the width when it is placed, so every kernel that takes an RMS norm's weight takes this one."""

    def __init__(self, dim: int, eps: float, names: Dict[str, str], scalar_weight: bool = False):
        super().__init__(names)
        self.dim, self.eps, self.scalar_weight = dim, float(eps), bool(scalar_weight)
        self.weight: Optional[torch.Tensor] = None

    def local_specs(self):
        return {"weight": TensorSpec(() if self.scalar_weight else (self.dim,), NORM)}

    def place(self, local, dtype, device):
        w = local["weight"]
        if self.scalar_weight:
            w = w.reshape(1).expand(self.dim).contiguous()
        self.weight = to_device_vector(w, dtype, device)

    def forward(self, ctx, x: torch.Tensor, row_idx: Optional[torch.Tensor] = None, pending_ok: bool = False):
        """The normed rows. `pending_ok`: the caller can finish a norm that the product before it has begun; it then
        gets `PendingNormRows` when the step holds them for this stream and this norm."""
        if pending_ok and row_idx is None:
            held = ctx.memo.get(("pending norm", id(x)))
            if held is not None and held.norm is self:
                return held
        rows = x.shape[0] if row_idx is None else row_idx.shape[0]
        out = ctx.empty((rows, self.dim))
        ops.rmsnorm(x, self.weight, self.eps, out, row_idx)
        return out


class LayerNorm(Part):
    """y = (x - mean) / sqrt(var + eps) * weight + bias over each row, var the mean of the squared deviations; statistics
    in 32-bit. Input: the 32-bit residual stream (or any 32-bit rows); output: the engine's activation dtype.
    `bias=False`: no bias tensor."""

    def __init__(self, dim: int, eps: float, names: Dict[str, str], bias: bool = True):
        super().__init__(names)
        self.dim, self.eps, self.has_bias = dim, float(eps), bool(bias)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def local_specs(self):
        s = {"weight": TensorSpec((self.dim,), NORM)}
        if self.has_bias:
            s["bias"] = TensorSpec((self.dim,), BIAS)
        return s

    def forward(self, ctx, x: torch.Tensor, row_idx: Optional[torch.Tensor] = None, pending_ok: bool = False):
        rows = x.shape[0] if row_idx is None else row_idx.shape[0]
        out = ctx.empty((rows, self.dim))
        ops.layernorm(x, self.weight, self.bias, self.eps, out, row_idx)
        return out
