"""Feed-forward made of many small gated experts of which every token uses a few.

    z = W_router x (float32);  s = softmax(z) over all experts
    the experts form `groups` runs of neighbours; a run scores as its best expert; only experts of the `keep` best
    runs can be chosen (no groups: all can);  the `top` experts with the largest s are chosen
    out = sum over the chosen e of w_e * W_down[e] (silu(W_gate[e] x) * (W_up[e] x)),   w_e = s_e (or s_e / their sum)

Options: `activation` "clamped_swish" with `limit` (g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) *
(u + 1) in place of silu(gate) * up); `shared` = (w_gate, w_up, w_down, w_gate_scalar or None, limit): one more expert of the
same form that every token uses, added to the sum, times sigmoid(w_gate_scalar x) (one number per token) where that is given.
Softmax over all experts followed by `renormalize` over the chosen ones is the softmax over the chosen logits alone.

Per step: the election (one warp per token), the (token, expert) pairs put in order of their expert on the device
(no count ever goes to the host, so the step can be recorded in a CUDA graph), one grouped product for gate and up
with the gate in its epilogue, one for down with the weight in its epilogue, and the sum over a token's choices in
their own order. A step in which the experts get many pairs each takes tiles of 128 pairs, else of 32 (the same sums
either way). bfloat16 engines run the products on the tensor cores (`tensor_cores`), float32 engines as plain
multiply-add chains over the features in order.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from ..tuning import TUNING
from .base import FeedForward, StepContext, aligned
from .linear import to_compute


class RoutedExperts(FeedForward):
    def __init__(self, w_router: torch.Tensor, w_gate: Sequence[torch.Tensor], w_up: Sequence[torch.Tensor],
                 w_down: Sequence[torch.Tensor], top: int, groups: int = 0, keep: int = 0, renormalize: bool = False,
                 dtype=torch.bfloat16, device="cuda", activation: str = "silu", limit: float = 0.0, shared=None):
        E, hidden = w_router.shape
        if not (len(w_gate) == len(w_up) == len(w_down) == E):
            raise ValueError(f"the router names {E} experts, got {len(w_gate)} / {len(w_up)} / {len(w_down)} sets of weights")
        ff = w_gate[0].shape[0]
        for e in range(E):
            if w_gate[e].shape != (ff, hidden) or w_up[e].shape != (ff, hidden) or w_down[e].shape != (hidden, ff):
                raise ValueError(f"expert {e}: shapes {list(w_gate[e].shape)} / {list(w_up[e].shape)} / {list(w_down[e].shape)} do not "
                                 f"fit {ff} x {hidden}")
        self.E, self.ff, self.hidden, self.top = E, ff, hidden, int(top)
        self.groups, self.keep = (int(groups), int(keep)) if groups and groups > 1 else (0, 0)
        if not 0 < self.top <= E:
            raise ValueError(f"{top} choices among {E} experts")
        if self.groups and (E % self.groups or not 0 < self.keep <= self.groups or self.top > self.keep * (E // self.groups)):
            raise ValueError(f"{E} experts in {groups} groups of which {keep} are kept cannot give {top} choices")
        self.renorm = bool(renormalize)
        # the router is float32 whatever the engine computes in
        self.w_router = w_router.to(device=device, dtype=torch.float32).contiguous()
        self.w_gu = to_compute(torch.stack([torch.cat([g, u], dim=0) for g, u in zip(w_gate, w_up)]), dtype, device)
        self.w_down = to_compute(torch.stack(list(w_down)), dtype, device)
        self.dtype = dtype
        self.tensor_cores = dtype == torch.bfloat16
        self.meta = torch.zeros(4, dtype=torch.int32, device=device)
        if activation not in kernels.MOE_ACTIVATIONS or (activation == "clamped_swish" and not limit > 0):
            raise ValueError(f"activation {activation!r} with limit {limit}: known are {', '.join(kernels.MOE_ACTIVATIONS)}, and the "
                             f"clamped one needs a positive limit")
        self.activation, self.limit = activation, float(limit)
        self._side = None           # a second stream for the shared expert in steps of single tokens, made at first need
        self.shared = None
        if shared is not None:
            sg, su, sd, sgate, slimit = shared
            fs = sg.shape[0]
            if sg.shape != (fs, hidden) or su.shape != (fs, hidden) or sd.shape != (hidden, fs) or (sgate is not None and sgate.shape != (1, hidden)):
                raise ValueError(f"the shared expert's shapes {list(sg.shape)} / {list(su.shape)} / {list(sd.shape)} do not fit a width of {hidden}")
            # [gate; up; the gate's one row; zero rows up to a multiple of 8]: one product gives all of them
            rows = [sg, su] + ([sgate, torch.zeros((7, hidden), dtype=sg.dtype, device=sg.device)] if sgate is not None else [])
            self.shared = (to_compute(torch.cat([r.to(sg.device) for r in rows], dim=0), dtype, device), to_compute(sd, dtype, device), fs,
                           sgate is not None, float(slimit))
            if activation == "clamped_swish" and not slimit > 0:
                raise ValueError("the shared expert's limit must be positive")

    def weight_bytes(self) -> int:
        """What a step of one token reads: the router and `top` experts."""
        es = self.w_down.element_size()
        shared = (self.shared[0].numel() + self.shared[1].numel()) * es if self.shared is not None else 0
        return self.w_router.numel() * 4 + self.top * 3 * self.ff * self.hidden * es + shared

    def workspace_bytes(self, rows: int) -> int:
        es = 2 if self.dtype == torch.bfloat16 else 4
        P = rows * self.top
        cap = max(kernels.moe_sorted_rows(P, self.E, r) for r in (kernels.MOE_TILE_ROWS, kernels.MOE_LARGE_TILE_ROWS))
        shared = 0
        if self.shared is not None:
            shared = aligned(rows * self.shared[0].shape[0] * es) + aligned(rows * self.shared[2] * es) + aligned(rows * self.hidden * es)
        return shared + (2 * aligned(P * 4) + aligned(cap * 4) + aligned(cap // kernels.MOE_TILE_ROWS * 4) + aligned(P * self.ff * es)
                + aligned(P * self.hidden * 4) + aligned(rows * self.hidden * es))

    def kernel_modules(self, dtype, max_rows):
        if self.shared is None:
            return ("moe",)
        return ("moe", "elementwise") + (("gemm_f32",) if dtype == torch.float32 else ("gemm_sm100",))

    def _shared_expert(self, x, gu, hs, sh):
        w_gu, w_down, fs, gated, slimit = self.shared
        kernels.linear(x, w_gu, gu)
        if self.activation == "clamped_swish":
            kernels.glu_clamped(gu[:, :2 * fs], hs, slimit)
        else:
            kernels.glu(gu[:, :2 * fs], hs, "silu")
        kernels.linear(hs, w_down, sh)

    def forward(self, x: torch.Tensor, ctx: StepContext, out=None) -> torch.Tensor:
        T = x.shape[0]
        P = T * self.top
        idx, w = ctx.alloc((T, self.top), torch.int32), ctx.alloc((T, self.top), torch.float32)
        sh = sgate = side = None
        if self.shared is not None:
            w_gu, _, fs, gated, _ = self.shared
            gu, hs, sh = ctx.alloc((T, w_gu.shape[0])), ctx.alloc((T, fs)), ctx.alloc((T, self.hidden))
            sgate = gu[:, 2 * fs] if gated else None
            if ctx.decode_only and TUNING.moe_side_stream:
                # nothing of the shared expert depends on the routed ones: it runs beside them and joins before the sum
                if self._side is None:
                    self._side = torch.cuda.Stream(device=x.device)
                side, main = self._side, torch.cuda.current_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    self._shared_expert(x, gu, hs, sh)
            else:
                self._shared_expert(x, gu, hs, sh)
        kernels.moe_route(x, self.w_router, ctx.positions, self.top, self.groups, self.keep, self.renorm, idx, w)
        large = x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
        tile = kernels.moe_tile_rows(P, self.E, self.hidden, self.ff, self.tensor_cores and large)
        cap = kernels.moe_sorted_rows(P, self.E, tile)
        order, tile_expert = ctx.alloc((cap,), torch.int32), ctx.alloc((cap // tile,), torch.int32)
        kernels.moe_align(idx, self.E, order, tile_expert, self.meta, tile)
        h = ctx.alloc((P, self.ff))
        kernels.moe_gate_up(x, self.w_gu, order, tile_expert, self.top, h, self.tensor_cores, tile, self.activation, self.limit)
        y = ctx.alloc((P, self.hidden), torch.float32)
        kernels.moe_down(h, self.w_down, order, tile_expert, w, y, self.tensor_cores, tile)
        out = out if out is not None else ctx.alloc((T, self.hidden))
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        kernels.moe_combine(y, idx, out, sh, sgate)
        return out
