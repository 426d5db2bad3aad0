"""Feed-forward that is not gated: down(act(up(x))), dense, no bias.

act = "xielu" with two learned numbers p and q (one pair per layer):
    z > 0:  softplus(p) z^2 + z / 2;      z <= 0:  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
The two factors are worked out once, in float32, when the part is built; the activation itself is float32
arithmetic on the product's result in the activations' type.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from .base import FeedForward, StepContext, aligned
from .linear import matmul, to_compute


def _softplus(z: float) -> float:
    return z if z > 30.0 else math.log1p(math.exp(z))


class ActMLP(FeedForward):
    def __init__(self, w_up: torch.Tensor, w_down: torch.Tensor, act_params: torch.Tensor, dtype=torch.bfloat16, device="cuda",
                 activation: str = "xielu"):
        inter, hidden = w_up.shape
        if w_down.shape != (hidden, inter):
            raise ValueError(f"feed-forward shapes do not fit: up {list(w_up.shape)}, down {list(w_down.shape)}")
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not known ({', '.join(kernels.ACTIVATIONS)})")
        if act_params.numel() != 2:
            raise ValueError(f"xielu takes two numbers, got {list(act_params.shape)}")
        p, q = (float(v) for v in act_params.float().reshape(2).tolist())
        self.activation = activation
        self.params = torch.tensor([_softplus(p), 0.5 + _softplus(q)], dtype=torch.float32, device=device)
        self.inter, self.hidden, self.dtype = inter, hidden, dtype
        self.w_up = to_compute(w_up, dtype, device)
        self.w_down = to_compute(w_down, dtype, device)

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def workspace_bytes(self, rows: int) -> int:
        es = 2 if self.dtype == torch.bfloat16 else 4
        return aligned(rows * self.inter * es) + aligned(rows * self.hidden * es)

    def kernel_modules(self, dtype, max_rows):
        return ("elementwise", "gemm_f32") if dtype == torch.float32 else ("elementwise", "gemm_sm100")

    def forward(self, x: torch.Tensor, ctx: StepContext, out=None) -> torch.Tensor:
        T = x.shape[0]
        h = matmul(x, self.w_up, ctx.alloc((T, self.inter)))
        kernels.activation(h, h, self.activation, self.params)
        return matmul(h, self.w_down, out if out is not None else ctx.alloc((T, self.hidden)))
