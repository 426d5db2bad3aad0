"""Attention whose cache holds one small latent vector per token instead of keys and values per head.

    q = W_q h, head by head [dim plain features | rot_dim rotated features]
    W_dkv h = [kv_rank columns | rot_dim columns];  c = RMSNorm(first kv_rank, weight);  kr = rotary(last rot_dim)
    key of head n = [W_uk,n c | kr],  value of head n = W_uv,n c
    score = (q_plain . k_plain + q_rot . kr) * scale,  causal, ordinary softmax;  out = W_o concat(heads)

Only c and kr are cached (`CacheSpec.tensors`: two tensors with one "head" each), and no key or value
is ever built from them. Since k_plain = W_uk,n c, the plain part of the score is (W_uk,n^T q_plain) . c:
the query is taken into the latent space once per row (a product per head), the attention kernel
works on c directly and returns sum_j p_j c_j, and W_uv,n is applied to that (softmax weights
sum to one, so W_uv (sum_j p_j c_j) = sum_j p_j W_uv c_j). A cached token costs kv_rank + rot_dim
elements whatever the number of heads, and a decode step reads each of them once for all heads.
Scores, softmax and the rotation are float32; the query in the latent space stays float32.

Options: `window` (a query sees itself and the window - 1 tokens before it; pages behind the window are given back) and
`pairing` of the rotated features: "half" (feature i with i + rot_dim / 2) or "interleaved" (2i with 2i + 1). The kernels
rotate halves; the interleaved pairing is the same rotation on another order of the rotated rows of W_q and W_dkv, the same
order for both (a score is a dot product, so a common order of q's and k's features changes nothing), applied here at load.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import CacheSpec, LayerCache, Mixer, PagedTensorSpec, StepContext, aligned
from .linear import matmul, to_compute
from .rotary import rotary_inv_freq


class LatentAttention(Mixer):
    def __init__(self, wq, wdkv, dkv_norm, wuk, wuv, wo, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 rot_base: float, eps: float, dtype=torch.bfloat16, device="cuda", window: int = 0, pairing: str = "half"):
        self.H, self.D, self.R, self.V, self.L = int(heads), int(dim), int(rot_dim), int(vdim), int(kv_rank)
        H, D, R, V, L = self.H, self.D, self.R, self.V, self.L
        hidden = wq.shape[1]
        if wq.shape != (H * (D + R), hidden) or wdkv.shape != (L + R, hidden) or wuk.shape != (H * D, L) or wuv.shape != (H * V, L) \
                or wo.shape != (hidden, H * V) or dkv_norm.shape != (L,):
            raise ValueError(f"projection shapes do not fit {H} heads of {D}+{R} / {V} with a latent of {L} over a width of {hidden}")
        if R % 2 or R <= 0:
            raise ValueError(f"the rotated part must have an even, positive size, got {R}")
        self.window = int(window) if window else 0
        if self.window < 0 or pairing not in ("half", "interleaved"):
            raise ValueError(f"window {window} must not be negative and pairing {pairing!r} is half or interleaved")
        if pairing == "interleaved":
            # rotated features in the order 0, 2, 4, ..., 1, 3, 5, ...: pairs (2i, 2i + 1) become (i, i + R / 2)
            order = torch.cat([torch.arange(0, R, 2), torch.arange(1, R, 2)])
            qrows = torch.arange(H * (D + R)).view(H, D + R).clone()
            qrows[:, D:] = qrows[:, D:][:, order]
            wq = wq[qrows.reshape(-1).to(wq.device)]
            krows = torch.cat([torch.arange(L), L + order])
            wdkv = wdkv[krows.to(wdkv.device)]
        self.w_in = to_compute(torch.cat([wq, wdkv], dim=0), dtype, device)
        # per head, as `linear` wants its weights ([out, in]): latent <- plain query features, values <- latent
        self.w_qlat = to_compute(wuk.reshape(H, D, L).transpose(1, 2), dtype, device)          # [H, L, D]
        self.w_val = to_compute(wuv.reshape(H, V, L), dtype, device)                            # [H, V, L]
        self.w_o = to_compute(wo, dtype, device)
        self.norm_weight = dkv_norm.to(device=device, dtype=torch.float32).contiguous()
        self.inv_freq = torch.from_numpy(rotary_inv_freq(R, rot_base).copy()).to(device)
        self.scale, self.eps, self.hidden, self.dtype = float(scale), float(eps), hidden, dtype
        self.batched = True       # bfloat16: the per-head products as one batched library product (False: one by one, tests)
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.splits = None        # a number forces so many blocks per row's keys (tests)
        self.tensor_cores = True  # False: prompt portions go through the float32 kernel too (tests)
        self._tc_ok = None

    def key_splits(self, rows: int) -> int:
        """Blocks that share a row's keys: steps of few rows would leave most of the GPU idle with one
        block per row and eight heads, so their keys are shared out until the grid is about twice the SMs."""
        if self.splits is not None:
            return int(self.splits)
        blocks = rows * -(-self.H // 8)
        return max(1, min(32, 2 * self.num_sms // blocks)) if blocks < self.num_sms else 1

    def cache_spec(self) -> Optional[CacheSpec]:
        kind = "window" if self.window else "full"
        return CacheSpec(kind=kind, window=self.window, tensors=(PagedTensorSpec(1, self.L), PagedTensorSpec(1, self.R)))

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_qlat.numel() + self.w_val.numel() + self.w_o.numel()) * self.w_in.element_size()

    def workspace_bytes(self, rows: int) -> int:
        es, H = self.w_in.element_size(), self.H
        parts = aligned(rows * H * self.key_splits(rows) * (self.L + 2) * 4) if self.key_splits(rows) > 1 else 0
        if self.splits is None:     # the most any step of at most `rows` rows takes: below one block per SM every row has 32 shares
            few = min(rows, self.num_sms // -(-H // 8))
            parts = max(parts, aligned(few * H * 32 * (self.L + 2) * 4))
        return (aligned(rows * self.w_in.shape[0] * es) + aligned(rows * H * self.R * 4) + aligned(rows * H * self.L * 4)
                + aligned(rows * H * self.L * es) + 2 * aligned(rows * H * self.V * es) + parts)

    def kernel_modules(self, dtype, max_rows):
        return ("gemm_f32", "latent_attention") if dtype == torch.float32 else ("gemm_sm100", "latent_attention")

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state=None, out=None) -> torch.Tensor:
        if cache is None:
            raise ValueError("latent attention needs a cache")
        H, D, R, V, L = self.H, self.D, self.R, self.V, self.L
        T = x.shape[0]
        lat, kr = cache.tensors
        proj = matmul(x, self.w_in, ctx.alloc((T, self.w_in.shape[0])))
        q_rot = ctx.alloc((T, H, R), torch.float32)
        kernels.latent_prep(proj, 0, H, D, R, H * (D + R), L, self.norm_weight, self.eps, ctx.positions,
                            ctx.slot_mapping[cache.group] if cache.write else None, self.inv_freq, lat, kr, q_rot)
        q_heads = proj[:, :H * (D + R)].view(T, H, D + R)[:, :, :D]                 # [T, H, D], strided
        bt = ctx.block_tables[cache.group]
        splits = self.key_splits(T)
        partials = ctx.alloc((T * H * splits * (L + 2),), torch.float32) if splits > 1 else None
        if self.dtype == torch.bfloat16 and self.batched:
            # head-major buffers, so that each of the two per-head products is one batched product
            q_lat = ctx.alloc((H, T, L), torch.float32)
            torch.bmm(q_heads.transpose(0, 1), self.w_qlat.transpose(1, 2), out_dtype=torch.float32, out=q_lat)
            out_lat = ctx.alloc((H, T, L))
            if self._tc_ok is None:
                self._tc_ok = kernels.latent_attend_tc_supported(H, L, R)
            if self.tensor_cores and self._tc_ok and not ctx.decode_only and ctx.max_new > 1:
                # prompt portions: scores and the weighted sum on the tensor cores, 16 tokens of a request at a time
                kernels.latent_attend_tc(q_lat.transpose(0, 1), q_rot, lat, kr, bt, ctx.seq_starts, ctx.positions, ctx.seqs,
                                         min(ctx.max_new, T), self.scale, out_lat.transpose(0, 1), self.window)
            else:
                kernels.latent_attend(q_lat.transpose(0, 1), q_rot, lat, kr, bt, ctx.row_seq, ctx.positions, self.scale,
                                      out_lat.transpose(0, 1), splits, partials, self.window)
            vals = ctx.alloc((H, T, V))
            torch.bmm(out_lat, self.w_val.transpose(1, 2), out=vals)
            attn = ctx.alloc((T, H * V))
            attn.view(T, H, V).copy_(vals.transpose(0, 1))
        else:
            q_lat = ctx.alloc((T, H, L), torch.float32)
            for h in range(H):
                kernels.linear(q_heads[:, h], self.w_qlat[h], q_lat[:, h])
            out_lat = ctx.alloc((T, H, L))
            kernels.latent_attend(q_lat, q_rot, lat, kr, bt, ctx.row_seq, ctx.positions, self.scale, out_lat, splits, partials, self.window)
            attn = ctx.alloc((T, H * V))
            for h in range(H):
                kernels.linear(out_lat[:, h], self.w_val[h], attn[:, h * V:(h + 1) * V])
        return matmul(attn, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))
