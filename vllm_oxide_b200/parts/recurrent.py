"""Mixers whose memory is a matrix state per request and head instead of a cache of keys: the state
S [key channels, value channels] is float32, lives in the request's state slot (`StateSpec`), starts
at zero when the request is admitted and is carried from token to token across steps.

`GeneralDelta`, the generalized delta rule, per head (all of size `dim`):
    r, k, v = W_r h, W_k h, W_v h;   u = k / sqrt(sum k^2 + 1e-6)
    w = exp(-exp(-1/2) sigmoid(W_w2 tanh(W_w1 h) + w0))     decay per key channel
    a = sigmoid(W_a h + a_bias)                              removal rate per key channel
    S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T;   o = S_t^T r
    out = W_o (rms_head(o) * norm_weight * sigmoid(W_g h))

`Retention`, linear attention with a fixed decay per head, no softmax and no denominator:
    q, k = rotary(W_q h), rotary(W_k h) * dim^-1/2;   v = W_v h  (heads of `vdim`)
    S_t = decay_h S_(t-1) + k v^T;   o = S_t^T q;   out = W_o (rms_head(o) * silu(W_g h))

`GatedDelta`, the gated delta rule, per value head (keys of `dim`, values of `vdim`; several value heads
may share one q and k head):
    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     short causal convolutions per channel
    q = q / sqrt(sum q^2 + 1e-6) * dim^-1/2;   k = k / sqrt(sum k^2 + 1e-6)
    beta = sigmoid(W_b h);   g = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias))   decay per key channel
    S' = diag(g) S_(t-1);   S_t = S' + k (beta (v - S'^T k))^T;   o = S_t^T q
    out = W_o (rms_head(o) * norm_weight * sigmoid(W_g2 W_g1 h))
  or, as options: one decay per head, g = exp(-exp(A_log_h) softplus(W_a h + dt_bias_h)) with W_a [heads, width] (no
  second matrix), and an output gate from one full projection, silu(W_g h) or sigmoid(W_g h).
Its state is the matrix S and, in a second tensor, the convolutions' last taps - 1 inputs.

`StateSpace`, a selective state-space mixer (the state-space duality form), per head of `vdim` values with a state of
`state` key channels, the heads in `groups` that share B and C:
    [z | x | B | C | dt] = W_in h;   x, B, C = silu(conv([x | B | C]) + conv_bias)    one short causal convolution per channel
    dt = softplus(dt + dt_bias);   S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T;   y_t = S_t^T C_t + D_h x_t
    out = W_o (rms_groups(y * silu(z)) * norm_weight)      the gate first, then an RMS norm over `norm_groups` equal parts
Its state is the matrix S [state, vdim] per head and the convolution's last taps - 1 inputs.

All run the same scan kernel (`kernels.recurrence_scan`) for prompt portions and single tokens
alike. The projections are one matrix product each side of it, in the compute dtype; everything
between them that enters the recurrence (unit key, decay, removal rate, rotation, the state, the
per-head norm and the gates) is float32.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .. import kernels
from .base import LayerCache, Mixer, StateSpec, StepContext, aligned
from .linear import matmul, to_compute
from .rotary import rotary_inv_freq


def _modules(dtype):
    return ("gemm_f32", "recurrence") if dtype == torch.float32 else ("gemm_sm100", "recurrence")


class GeneralDelta(Mixer):
    def __init__(self, wr, wk, wv, wa, a_bias, wg, w1, w2, w0, norm_weight, wo, heads: int, dim: int, eps: float,
                 dtype=torch.bfloat16, device="cuda"):
        self.H, self.D = int(heads), int(dim)
        hd, hidden = self.H * self.D, wr.shape[1]
        for name, t in (("r", wr), ("k", wk), ("v", wv), ("a", wa), ("g", wg)):
            if t.shape != (hd, hidden):
                raise ValueError(f"projection '{name}' is {list(t.shape)}, {self.H} heads of {self.D} over a width of {hidden} need [{hd}, {hidden}]")
        self.rank = w1.shape[0]
        if w1.shape != (self.rank, hidden) or w2.shape != (hd, self.rank) or wo.shape != (hidden, hd):
            raise ValueError(f"decay projection {list(w1.shape)} / {list(w2.shape)} or output projection {list(wo.shape)} do not fit")
        for name, t in (("a_bias", a_bias), ("w0", w0), ("norm", norm_weight)):
            if t.shape != (hd,):
                raise ValueError(f"'{name}' must have {hd} entries, got {list(t.shape)}")
        # one matrix [Wr; Wk; Wv; Wa; Wg; Ww1]: a single product gives every projection of the input
        self.w_in = to_compute(torch.cat([wr, wk, wv, wa, wg, w1], dim=0), dtype, device)
        self.w2t = to_compute(w2.t(), dtype, device)          # [rank, heads * dim]: the kernel reads it channel by channel
        self.w_o = to_compute(wo, dtype, device)
        f32 = dict(device=device, dtype=torch.float32)
        self.a_bias, self.w0, self.norm_weight = a_bias.to(**f32).contiguous(), w0.to(**f32).contiguous(), norm_weight.to(**f32).contiguous()
        self.eps, self.hidden, self.dtype = float(eps), hidden, dtype

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.H, self.D, self.D), torch.float32)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w2t.numel() + self.w_o.numel()) * self.w_in.element_size()

    def workspace_bytes(self, rows: int) -> int:
        es, hd = self.w_in.element_size(), self.H * self.D
        return aligned(rows * self.w_in.shape[0] * es) + 4 * aligned(rows * hd * 4) + aligned(rows * hd * es)

    def kernel_modules(self, dtype, max_rows):
        return _modules(dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state: Optional[torch.Tensor], out=None) -> torch.Tensor:
        if state is None:
            raise ValueError("the delta rule needs its state")
        T, hd = x.shape[0], self.H * self.D
        proj = matmul(x, self.w_in, ctx.alloc((T, self.w_in.shape[0])))
        w, b, u, o = (ctx.alloc((T, hd), torch.float32) for _ in range(4))
        kernels.delta_prep(proj, hd, 3 * hd, 5 * hd, self.rank, self.w2t, self.w0, self.a_bias, self.H, self.D, w, b, u)
        kernels.recurrence_scan(0, proj[:, :hd], proj[:, hd:2 * hd], proj[:, 2 * hd:3 * hd], w, b, u, state, ctx.seq_starts,
                                ctx.state_slots, ctx.seqs, self.H, o)
        gated = ctx.alloc((T, hd))
        kernels.recurrence_post(o, proj[:, 4 * hd:5 * hd], self.norm_weight, "sigmoid", self.eps, self.H, gated)
        return matmul(gated, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))


class Retention(Mixer):
    def __init__(self, wq, wk, wv, wg, wo, heads: int, dim: int, vdim: int, decay: Sequence[float], rot_dims: int, rot_base: float,
                 eps: float, dtype=torch.bfloat16, device="cuda"):
        self.H, self.D, self.V = int(heads), int(dim), int(vdim)
        hk, hv, hidden = self.H * self.D, self.H * self.V, wq.shape[1]
        if wq.shape != (hk, hidden) or wk.shape != (hk, hidden) or wv.shape != (hv, hidden) or wg.shape != (hv, hidden) or wo.shape != (hidden, hv):
            raise ValueError(f"projection shapes do not fit {self.H} heads of {self.D} / {self.V} over a width of {hidden}")
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decays for {self.H} heads")
        if rot_dims % 2 or not 0 <= rot_dims <= self.D:
            raise ValueError(f"{rot_dims} rotated features do not fit a head of {self.D}")
        self.w_in = to_compute(torch.cat([wq, wk, wv, wg], dim=0), dtype, device)
        self.w_o = to_compute(wo, dtype, device)
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=device)
        self.rot = int(rot_dims)
        self.inv_freq = torch.from_numpy(rotary_inv_freq(self.rot, rot_base).copy()).to(device) if self.rot else \
            torch.zeros(0, dtype=torch.float32, device=device)
        self.k_scale = float(self.D) ** -0.5
        self.eps, self.hidden, self.dtype = float(eps), hidden, dtype

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.H, self.D, self.V), torch.float32)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def workspace_bytes(self, rows: int) -> int:
        es, hk, hv = self.w_in.element_size(), self.H * self.D, self.H * self.V
        return aligned(rows * self.w_in.shape[0] * es) + 2 * aligned(rows * hk * 4) + aligned(rows * hv * 4) + aligned(rows * hv * es)

    def kernel_modules(self, dtype, max_rows):
        return _modules(dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state: Optional[torch.Tensor], out=None) -> torch.Tensor:
        if state is None:
            raise ValueError("retention needs its state")
        T, hk, hv = x.shape[0], self.H * self.D, self.H * self.V
        proj = matmul(x, self.w_in, ctx.alloc((T, self.w_in.shape[0])))
        q, k = ctx.alloc((T, hk), torch.float32), ctx.alloc((T, hk), torch.float32)
        kernels.rotate_scale(proj[:, :hk], ctx.positions, self.inv_freq, self.H, self.D, self.rot, 1.0, q)
        kernels.rotate_scale(proj[:, hk:2 * hk], ctx.positions, self.inv_freq, self.H, self.D, self.rot, self.k_scale, k)
        o = ctx.alloc((T, hv), torch.float32)
        kernels.recurrence_scan(1, q, k, proj[:, 2 * hk:2 * hk + hv], self.decay, None, None, state, ctx.seq_starts, ctx.state_slots,
                                ctx.seqs, self.H, o)
        gated = ctx.alloc((T, hv))
        kernels.recurrence_post(o, proj[:, 2 * hk + hv:], None, "silu", self.eps, self.H, gated)
        return matmul(gated, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))


class GatedDelta(Mixer):
    """See the module's head. `conv_q`, `conv_k`, `conv_v` are [channels, taps] with the last column the
    current token's. `w_a1` / `w_a2` and `w_g1` / `w_g2` are the two low-rank pairs (decay and output gate);
    `w_a2` None: `w_a1` is [heads, width] and gives one decay per head (`dt_bias` [heads]); `w_g2` None: `w_g1` is the
    full gate projection [heads * vdim, width]; `gate` names the gate's activation ("sigmoid" or "silu").
    `norm_weight` [vdim] is shared by the heads. Like `SoftmaxAttention` it offers its halves separately
    (`w_in`, `core`, `w_o`) for a layer that runs it beside another mixer."""

    def __init__(self, wq, wk, wv, conv_q, conv_k, conv_v, wb, a_log, w_a1, w_a2, dt_bias, w_g1, w_g2, norm_weight, wo, heads: int,
                 kv_heads: int, dim: int, vdim: int, eps: float, dtype=torch.bfloat16, device="cuda", gate: str = "sigmoid"):
        self.H, self.G, self.K, self.V = int(heads), int(kv_heads), int(dim), int(vdim)
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} q/k heads")
        if gate not in ("sigmoid", "silu"):
            raise ValueError(f"gate {gate!r} is not known (sigmoid or silu)")
        self.gate = gate
        if self.K > 512:
            raise ValueError(f"a key size of {self.K} is beyond the scan's 512")
        hidden = wq.shape[1]
        gk, hk, hv = self.G * self.K, self.H * self.K, self.H * self.V
        if wq.shape != (gk, hidden) or wk.shape != (gk, hidden) or wv.shape != (hv, hidden) or wb.shape != (self.H, hidden) or wo.shape != (hidden, hv):
            raise ValueError(f"projection shapes do not fit {self.H} heads on {self.G} of {self.K} / {self.V} over a width of {hidden}")
        self.taps = conv_q.shape[1]
        for name, c, n in (("q", conv_q, gk), ("k", conv_k, gk), ("v", conv_v, hv)):
            if c.shape != (n, self.taps):
                raise ValueError(f"convolution '{name}' is {list(c.shape)}, expected [{n}, {self.taps}]")
        ra, rg = w_a1.shape[0], w_g1.shape[0]
        self.decay_per_head, self.gate_direct = w_a2 is None, w_g2 is None
        if w_a1.shape != (ra, hidden) or w_g1.shape != (rg, hidden):
            raise ValueError(f"decay and gate projections {list(w_a1.shape)} / {list(w_g1.shape)} do not read a width of {hidden}")
        if (self.decay_per_head and ra != self.H) or (not self.decay_per_head and w_a2.shape != (hk, ra)):
            raise ValueError(f"decay projection {list(w_a1.shape)} fits neither {self.H} heads nor its second matrix")
        if (self.gate_direct and rg != hv) or (not self.gate_direct and w_g2.shape != (hv, rg)):
            raise ValueError(f"gate projection {list(w_g1.shape)} fits neither {hv} features nor its second matrix")
        n_decay = self.H if self.decay_per_head else hk
        if a_log.shape != (self.H,) or dt_bias.shape != (n_decay,) or norm_weight.shape != (self.V,):
            raise ValueError(f"A_log [heads], dt_bias [{n_decay}] and the norm weight [vdim] are needed")
        self.C = 2 * gk + hv
        # one matrix [Wq; Wk; Wv; Wa1; Wg1; Wb]: q, k, v side by side (the convolutions' channels), then the
        # two low-rank inputs side by side (one second product serves both), the strengths last
        self.w_in = to_compute(torch.cat([wq, wk, wv, w_a1, w_g1, wb], dim=0), dtype, device)
        self.low_off, self.ra, self.rg = self.C, ra, rg
        self.b_off = self.C + ra + rg
        self.b_in = None
        # [[Wa2, 0], [0, Wg2]]: the zero blocks add exact zeros, so each half is the product of its own pair. A half
        # without a second matrix is read from the first product as it is, and with neither there is no second product.
        self.w_low = None
        if not (self.decay_per_head and self.gate_direct):
            rows_a, rows_g = (0 if self.decay_per_head else hk), (0 if self.gate_direct else hv)
            cols_a, cols_g = (0 if self.decay_per_head else ra), (0 if self.gate_direct else rg)
            low = torch.zeros(rows_a + rows_g, cols_a + cols_g, dtype=torch.float32)
            if not self.decay_per_head:
                low[:hk, :ra] = w_a2.float().cpu()
            if not self.gate_direct:
                low[rows_a:, cols_a:] = w_g2.float().cpu()
            self.w_low = to_compute(low, dtype, device)
            if self.decay_per_head != self.gate_direct:
                raise ValueError("the decay and the gate are both low-rank pairs or both single projections")
        self.w_o = to_compute(wo, dtype, device)
        self.b_o = None
        self.n_pre = hv
        f32 = dict(device=device, dtype=torch.float32)
        self.conv_w = torch.cat([conv_q.to(**f32), conv_k.to(**f32), conv_v.to(**f32)], dim=0).contiguous()
        self.a_log, self.dt_bias = a_log.to(**f32).contiguous(), dt_bias.to(**f32).contiguous()
        self.norm_weight = norm_weight.to(**f32).repeat(self.H).contiguous()        # the kernel takes one weight per head and feature
        self.eps, self.hidden, self.dtype = float(eps), hidden, dtype

    def state_spec(self):
        s = StateSpec((self.H, self.K, self.V), torch.float32)
        return (s, StateSpec((self.taps - 1, self.C), torch.float32)) if self.taps > 1 else (s,)

    def weight_bytes(self) -> int:
        low = self.w_low.numel() if self.w_low is not None else 0
        return (self.w_in.numel() + low + self.w_o.numel()) * self.w_in.element_size()

    def core_workspace_bytes(self, rows: int) -> int:
        es, gk, hk, hv = self.w_in.element_size(), self.G * self.K, self.H * self.K, self.H * self.V
        return (aligned(rows * (hk + hv) * es) + 2 * aligned(rows * gk * 4) + aligned(rows * hv * es) + aligned(rows * hk * 4)
                + aligned(rows * self.H * 4) + aligned(rows * hv * 4))

    def workspace_bytes(self, rows: int) -> int:
        es = self.w_in.element_size()
        return aligned(rows * self.w_in.shape[0] * es) + aligned(rows * self.n_pre * es) + self.core_workspace_bytes(rows)

    def kernel_modules(self, dtype, max_rows):
        return _modules(dtype)

    def core(self, proj: torch.Tensor, ctx: StepContext, cache, state, pre_out: torch.Tensor, out_scale: float = 1.0) -> None:
        """proj [T, >= w_in rows] -> pre_out [T, heads * vdim]: everything between the two projections."""
        if state is None:
            raise ValueError("the gated delta rule needs its state")
        S, conv_state = state[0], (state[1] if self.taps > 1 else None)
        T, gk, hk, hv = proj.shape[0], self.G * self.K, self.H * self.K, self.H * self.V
        if self.w_low is not None:
            low = ctx.alloc((T, hk + hv))
            kernels.linear(proj[:, self.low_off:self.low_off + self.ra + self.rg], self.w_low, low)
            a_src, a_off, g_src = low, 0, low[:, hk:]
        else:       # [.. | W_a h (heads) | W_g h (heads * vdim) | ..] are columns of the first product
            a_src, a_off = proj, self.low_off
            g_src = proj[:, self.low_off + self.ra:self.low_off + self.ra + self.rg]
        q, k = ctx.alloc((T, gk), torch.float32), ctx.alloc((T, gk), torch.float32)
        v = ctx.alloc((T, hv))
        decay, strength = ctx.alloc((T, hk), torch.float32), ctx.alloc((T, self.H), torch.float32)
        kernels.gated_delta_prep(proj, 0, self.b_off, a_src, a_off, self.conv_w, conv_state, self.a_log, self.dt_bias, ctx.positions,
                                 ctx.row_seq, ctx.seq_starts, ctx.state_slots, ctx.seqs, self.H, self.G, self.K, self.V, q, k, v, decay,
                                 strength, self.decay_per_head)
        o = ctx.alloc((T, hv), torch.float32)
        # the scan also leaves the convolutions' last inputs in the request's slot (the preparation has read the old ones)
        kernels.recurrence_scan(2, q, k, v, decay, strength, None, S, ctx.seq_starts, ctx.state_slots, ctx.seqs, self.H, o, rk_heads=self.G,
                                conv_x=proj[:, :self.C] if conv_state is not None else None, conv_state=conv_state)
        kernels.recurrence_post(o, g_src, self.norm_weight, self.gate, self.eps, self.H, pre_out, out_scale)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state, out=None) -> torch.Tensor:
        T = x.shape[0]
        proj = matmul(x, self.w_in, ctx.alloc((T, self.w_in.shape[0])))
        pre = ctx.alloc((T, self.n_pre))
        self.core(proj, ctx, cache, state, pre)
        return matmul(pre, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))


class StateSpace(Mixer):
    """See the module's head. `w_in` [2 * heads * vdim + 2 * groups * state + heads, width] in the order z, x, B, C, dt;
    `conv_w` [heads * vdim + 2 * groups * state, taps] (last column the current token's) with `conv_b`; `dt_bias`, `a_log`,
    `d_skip` [heads]; `norm_weight` [heads * vdim]."""

    def __init__(self, w_in, conv_w, conv_b, dt_bias, a_log, d_skip, norm_weight, wo, heads: int, vdim: int, state: int, groups: int,
                 norm_groups: int, eps: float, dtype=torch.bfloat16, device="cuda"):
        self.H, self.P, self.N, self.G, self.NG = int(heads), int(vdim), int(state), int(groups), int(norm_groups)
        H, P, N, G = self.H, self.P, self.N, self.G
        if G <= 0 or H % G:
            raise ValueError(f"{H} heads are not a multiple of {G} groups")
        if N > 512:
            raise ValueError(f"a state of {N} channels is beyond the scan's 512")
        self.inner, self.GN = H * P, G * N
        if self.NG <= 0 or self.inner % self.NG:
            raise ValueError(f"{self.inner} features do not split into {self.NG} norm groups")
        self.C = self.inner + 2 * self.GN
        hidden = w_in.shape[1]
        rows = 2 * self.inner + 2 * self.GN + H
        if w_in.shape != (rows, hidden) or wo.shape != (hidden, self.inner):
            raise ValueError(f"projections {list(w_in.shape)} / {list(wo.shape)} do not fit {H} heads of {P} with a state of {N} in {G} "
                             f"groups over a width of {hidden}")
        if conv_w.dim() != 2 or conv_w.shape[0] != self.C or conv_b.shape != (self.C,):
            raise ValueError(f"the convolution takes [{self.C}, taps] weights and [{self.C}] biases, got {list(conv_w.shape)} / {list(conv_b.shape)}")
        self.taps = conv_w.shape[1]
        for name, t, n in (("dt_bias", dt_bias, H), ("A_log", a_log, H), ("D", d_skip, H), ("norm", norm_weight, self.inner)):
            if t.shape != (n,):
                raise ValueError(f"'{name}' must have {n} entries, got {list(t.shape)}")
        self.w_in = to_compute(w_in, dtype, device)
        self.w_o = to_compute(wo, dtype, device)
        f32 = dict(device=device, dtype=torch.float32)
        self.conv_w, self.conv_b = conv_w.to(**f32).t().contiguous(), conv_b.to(**f32).contiguous()     # tap by tap, as the kernel reads them
        self.dt_bias, self.a_log, self.d_skip = dt_bias.to(**f32).contiguous(), a_log.to(**f32).contiguous(), d_skip.to(**f32).contiguous()
        self.norm_weight = norm_weight.to(**f32).contiguous()
        self.eps, self.hidden, self.dtype = float(eps), hidden, dtype

    def state_spec(self):
        s = StateSpec((self.H, self.N, self.P), torch.float32)
        return (s, StateSpec((self.taps - 1, self.C), torch.float32)) if self.taps > 1 else (s,)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size() + (self.conv_w.numel() + self.conv_b.numel()) * 4

    def workspace_bytes(self, rows: int) -> int:
        es = self.w_in.element_size()
        return (aligned(rows * self.w_in.shape[0] * es) + aligned(rows * self.C * 4) + 2 * aligned(rows * self.H * 4)
                + aligned(rows * self.inner * 4) + aligned(rows * self.inner * es) + aligned(rows * self.hidden * es))

    def kernel_modules(self, dtype, max_rows):
        return _modules(dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state, out=None) -> torch.Tensor:
        if state is None:
            raise ValueError("the state-space mixer needs its state")
        S, conv_state = state[0], (state[1] if self.taps > 1 else None)
        T, inner, GN, C, H = x.shape[0], self.inner, self.GN, self.C, self.H
        proj = matmul(x, self.w_in, ctx.alloc((T, self.w_in.shape[0])))
        xbc = ctx.alloc((T, C), torch.float32)
        single = bool(ctx.decode_only and conv_state is not None)      # single tokens: the kernel moves the state on itself
        kernels.causal_conv(proj[:, inner:inner + C], self.conv_w, self.conv_b, conv_state, ctx.positions, ctx.row_seq, ctx.seq_starts,
                            ctx.state_slots, ctx.seqs, xbc, residual=False, act="silu", single=single)
        if conv_state is not None and not single:
            kernels.conv_state_update(proj, inner, conv_state, ctx.seq_starts, ctx.state_slots, ctx.seqs)
        dt, decay = ctx.alloc((T, H), torch.float32), ctx.alloc((T, H), torch.float32)
        kernels.ssm_steps(proj[:, inner + C:inner + C + H], self.dt_bias, self.a_log, dt, decay)
        o = ctx.alloc((T, inner), torch.float32)
        kernels.recurrence_scan(3, xbc[:, inner + GN:], xbc[:, inner:inner + GN], xbc[:, :inner], None, decay, dt, S, ctx.seq_starts,
                                ctx.state_slots, ctx.seqs, H, o, rk_heads=self.G)
        y = ctx.alloc((T, inner))
        kernels.ssm_post(o, xbc[:, :inner], proj[:, :inner], self.d_skip, self.norm_weight, self.eps, H, self.NG, y)
        return matmul(y, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))
