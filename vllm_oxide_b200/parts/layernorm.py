"""Layer norm with weight and (optionally) bias: LN(z) = (z - mean) / sqrt(mean((z - mean)^2) + eps) * w + b, sums in float32.

Two uses. As any norm of this engine it normalises the float32 residual (after adding what is still
pending) for the part that follows: `forward`. In a block whose residual takes the NORMED result of each
sub-layer (`PostNormBlock`) it normalises that result and adds it into the residual: `add_normed`, which
can also leave the new residual in the activations' type for the sub-layer that reads it next.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Norm, StepContext, aligned


class LayerNorm(Norm):
    scale_and_weight = False      # the mean and the bias do not commute with a matrix product: no folded form

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, device):
        """`bias` None: a layer norm with a weight only."""
        if weight.dim() != 1 or (bias is not None and bias.shape != weight.shape):
            raise ValueError(f"layer norm needs a weight and a bias of one length, got {list(weight.shape)} and {list(bias.shape)}")
        self.weight = weight.to(device=device, dtype=torch.float32).contiguous()
        self.bias = bias.to(device=device, dtype=torch.float32).contiguous() if bias is not None else None
        self.eps = float(eps)
        self.width = weight.shape[0]

    def weight_bytes(self) -> int:
        return (2 if self.bias is not None else 1) * self.weight.numel() * 4

    def workspace_bytes(self, rows: int, act_bytes: int) -> int:
        return aligned(rows * self.width * act_bytes)

    def kernel_modules(self, dtype, max_rows):
        return ("elementwise",)

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                rows: Optional[torch.Tensor] = None, num_rows: Optional[int] = None,
                delta_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        if delta is not None:
            raise ValueError("this layer norm normalises the residual as it stands; a pending result must be added first")
        n = resid.shape[0] if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = ctx.alloc((n, self.width))
        kernels.layernorm_rows(resid, self.weight, self.bias, self.eps, out, rows[:n] if rows is not None else None)
        return out

    def add_normed(self, resid: torch.Tensor, result: torch.Tensor, copy: Optional[torch.Tensor] = None, depth=None, conv=None) -> None:
        """resid += LN(result); `copy`, if given, receives the new residual in its own type. `depth`, `conv`: work the kernel
        does on its way (see `kernels.layernorm_add`)."""
        kernels.layernorm_add(resid, result, self.weight, self.bias, self.eps, copy, depth=depth, conv=conv)
