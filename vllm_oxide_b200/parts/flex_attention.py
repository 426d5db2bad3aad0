"""Softmax attention with options, over a paged cache whose keys and values have sizes of their own.

Per step: one fused projection [q | k | v (| gate)] (with its biases, if the design has them), one
preparation kernel (rotary positions on the first `rot_dims` features of each head, q and k divided
by their root mean square, the query factor, value mixing, the cache write), attention of every row
over its request's pages, the output projection. What a design may switch on, each with its constants
as parameters:

* `dim` / `vdim`     key and value sizes of a head (the cache holds two tensors of different widths);
* `bias_*`           biases of the q, k, v and output projections;
* `window`           a query sees itself and the window - 1 tokens before it (pages behind are given back);
* `rot_dims`, `rot_base`   partial rotary positions, feature i paired with i + rot_dims / 2;
* `unit_rms_eps`     q and k divided by sqrt(mean(x^2) + eps) per head, after the rotation;
* `q_norm_weight`, `k_norm_weight`   [dim] each, shared by the heads: q and k times it behind that division;
* `q_pre_norm`, `k_pre_norm`   [heads * dim] / [kv_heads * dim], with `pre_norm_eps`: BEFORE the rotation the whole q (k)
                     projection, all heads at once, is divided by its root mean square and multiplied by that weight;
* `pool`             (with `window`) beside the window's tokens a query sees one key and value for every block of `pool`
                     positions that lies wholly before the window: the means of the block's cached keys and values, in the
                     same softmax (the cache then keeps every token, and beside keys and values it holds, for every
                     size in `pooled_sizes`, the pooled keys and values: entry b where token b's would be);
* `pooled_sizes`     the block sizes the cache serves where several layers with blocks of different sizes read it
                     (default: this layer's own `pool`); the layer that writes the cache pools for all of them;
* `chunk`            a query sees only the keys of its own block of `chunk` positions, blocks counted from position 0
                     (pages of earlier blocks are given back);
* `softcap`          score <- softcap * tanh(score / softcap);
* `dist_bias`        (r1, r2), one number per head each: r1 * ln(1 + r2 * (i - j)) is taken off the score of key j;
* `shared_kv`        the layer has no key and value projections: it reads the cache another layer wrote (the run order
                     names it: `LayerCall(cache=that layer's, write=False)`), with its own queries, mask and the rest;
* `cache_keep`       ("full" | "window" | "chunk", size): what the cache keeps where that is more than this layer's own
                     mask asks for (a cache that layers with different masks read must serve them all);
* `q_temp`           (coef, every): q times 1 + coef * ln(floor((pos + 1) / every) + 1);
* `sink`             one number per head whose exponential joins the softmax's denominator (no key, no value);
* `gate_weight`      the heads' results times sigmoid(W_g x) before the output projection;
* `value_mix`        "first": this layer's values of the step's tokens are left in `ctx.shared[shared_name]`;
                     "mix": v <- (1 - lambda) v + lambda * those values, before v is cached.

A mixer that runs beside another one in one layer offers its halves separately: `w_in` / `b_in`,
`core(proj, ...)` (everything between the two projections, writing into a column range of a wider
buffer) and `w_o` / `b_o`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import kernels
from .attention import decode_split_rule
from .base import CacheSpec, LayerCache, Mixer, PagedTensorSpec, StepContext, aligned
from .linear import to_compute
from .rotary import rotary_inv_freq


class SoftmaxAttention(Mixer):
    def __init__(self, wq: torch.Tensor, wk: Optional[torch.Tensor], wv: Optional[torch.Tensor], wo: torch.Tensor, heads: int,
                 kv_heads: int, dim: int,
                 vdim: int, scale: float, *, bias_q=None, bias_k=None, bias_v=None, bias_o=None, window: int = 0, rot_dims: int = 0,
                 rot_base: float = 10000.0, unit_rms_eps: Optional[float] = None, q_temp: Optional[Tuple[float, int]] = None,
                 sink: Optional[torch.Tensor] = None, gate_weight: Optional[torch.Tensor] = None, value_mix: Optional[str] = None,
                 mix_weight: Optional[torch.Tensor] = None, shared_name: str = "v_first", q_norm_weight: Optional[torch.Tensor] = None,
                 k_norm_weight: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0, dist_bias=None,
                 shared_kv: bool = False, cache_keep: Optional[Tuple[str, int]] = None, dtype=torch.bfloat16, device="cuda",
                 q_pre_norm: Optional[torch.Tensor] = None, k_pre_norm: Optional[torch.Tensor] = None,
                 pre_norm_eps: Optional[float] = None, pool: int = 0, pooled_sizes: Optional[Tuple[int, ...]] = None):
        self.H, self.G, self.D, self.DV = int(heads), int(kv_heads), int(dim), int(vdim)
        self.shared_kv = bool(shared_kv)
        if self.shared_kv:
            if wk is not None or wv is not None or bias_k is not None or bias_v is not None or k_norm_weight is not None or value_mix:
                raise ValueError("a layer that reads another layer's keys and values has no key or value tensors of its own")
            wk = torch.zeros((0, wq.shape[1]), dtype=wq.dtype, device=wq.device)
            wv = torch.zeros((0, wq.shape[1]), dtype=wq.dtype, device=wq.device)
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if self.D > 256 or self.DV > 256:
            raise ValueError(f"head sizes {self.D} / {self.DV} are beyond 256")
        hidden = wq.shape[1]
        nq, nk, nv = self.H * self.D, self.G * self.D, self.G * self.DV
        if self.shared_kv:
            nk = nv = 0
        self.n_pre = self.H * self.DV
        if wq.shape != (nq, hidden) or wk.shape != (nk, hidden) or wv.shape != (nv, hidden) or wo.shape != (hidden, self.n_pre):
            raise ValueError(f"projection shapes {list(wq.shape)} / {list(wk.shape)} / {list(wv.shape)} / {list(wo.shape)} do not fit "
                             f"{self.H} heads on {self.G} of {self.D} / {self.DV} over a width of {hidden}")
        mats = [wq, wk, wv]
        self.gated = gate_weight is not None
        if self.gated:
            if gate_weight.shape != (self.n_pre, hidden):
                raise ValueError(f"gate projection {list(gate_weight.shape)} does not fit {self.n_pre} x {hidden}")
            mats.append(gate_weight)
        self.w_in = to_compute(torch.cat(mats, dim=0), dtype, device)
        self.q_off, self.k_off, self.v_off, self.g_off = 0, nq, nq + nk, nq + nk + nv
        biases = (bias_q, bias_k, bias_v)
        self.b_in = None
        if any(b is not None for b in biases):
            parts = []
            for b, n in zip(biases, (nq, nk, nv)):
                if b is not None and b.shape != (n,):
                    raise ValueError(f"a bias of {list(b.shape)} does not fit {n}")
                parts.append(b.float() if b is not None else torch.zeros(n))
            if self.gated:
                parts.append(torch.zeros(self.n_pre))
            self.b_in = to_compute(torch.cat([p.to("cpu") for p in parts]), dtype, device)
        self.w_o = to_compute(wo, dtype, device)
        if bias_o is not None and bias_o.shape != (hidden,):
            raise ValueError(f"output bias {list(bias_o.shape)} does not fit {hidden}")
        self.b_o = to_compute(bias_o, dtype, device) if bias_o is not None else None
        self.window = int(window) if window else 0
        self.chunk = int(chunk) if chunk else 0
        if self.window < 0 or self.chunk < 0 or (self.window and self.chunk):
            raise ValueError(f"a window of {window} and blocks of {chunk}: one of them at most, none negative")
        self.softcap = float(softcap) if softcap else 0.0
        if self.softcap < 0:
            raise ValueError(f"softcap {softcap} must be positive")
        self.pool = int(pool) if pool else 0
        if self.pool < 0 or (self.pool and not self.window):
            raise ValueError(f"pooled blocks of {pool} go with a window")
        self.pooled_sizes = tuple(int(x) for x in pooled_sizes) if pooled_sizes is not None else ((self.pool,) if self.pool else ())
        if (self.pool and self.pool not in self.pooled_sizes) or any(x <= 0 for x in self.pooled_sizes) \
                or len(set(self.pooled_sizes)) != len(self.pooled_sizes):
            raise ValueError(f"the cache's block sizes {self.pooled_sizes} must be distinct, positive and hold this layer's {self.pool}")
        own = ("full", 0) if self.pool else ("window", self.window) if self.window else ("chunk", self.chunk) if self.chunk else ("full", 0)
        self.cache_keep = (str(cache_keep[0]), int(cache_keep[1])) if cache_keep is not None else own
        if self.cache_keep != own and self.cache_keep[0] != "full":
            raise ValueError(f"a cache that keeps {self.cache_keep} cannot serve a layer that reads {own}")
        self.scale = float(scale)
        self.rot = int(rot_dims)
        if self.rot % 2 or not 0 <= self.rot <= self.D:
            raise ValueError(f"{self.rot} rotated features do not fit a head of {self.D}")
        self.inv_freq = torch.from_numpy(rotary_inv_freq(self.rot, rot_base).copy()).to(device) if self.rot else None
        self.unit_rms = unit_rms_eps is not None
        self.eps = float(unit_rms_eps) if self.unit_rms else 0.0
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        f32 = dict(device=device, dtype=torch.float32)
        for name, nw in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
            if nw is not None and (nw.shape != (self.D,) or not self.unit_rms):
                raise ValueError(f"{name} must have {self.D} entries and goes with unit_rms_eps, got {list(nw.shape)}")
        self.q_norm_w = q_norm_weight.to(**f32).contiguous() if q_norm_weight is not None else None
        self.k_norm_w = k_norm_weight.to(**f32).contiguous() if k_norm_weight is not None else None
        if (q_pre_norm is not None and q_pre_norm.shape != (nq,)) or (k_pre_norm is not None and (self.shared_kv or k_pre_norm.shape != (nk,))):
            raise ValueError(f"the norms over the whole projections take {nq} and {nk} weights (none for keys a layer does not make)")
        if (q_pre_norm is not None or k_pre_norm is not None) and (pre_norm_eps is None or self.unit_rms):
            raise ValueError("a norm over the whole projection needs its eps and does not go with the norm per head")
        self.q_pre_w = q_pre_norm.to(**f32).contiguous() if q_pre_norm is not None else None
        self.k_pre_w = k_pre_norm.to(**f32).contiguous() if k_pre_norm is not None else None
        if pre_norm_eps is not None and not self.unit_rms:
            self.eps = float(pre_norm_eps)
        self.dist_bias = None
        if dist_bias is not None:
            r1, r2 = dist_bias
            if r1.shape != (self.H,) or r2.shape != (self.H,):
                raise ValueError(f"the distance bias takes two numbers per head, got {list(r1.shape)} and {list(r2.shape)}")
            self.dist_bias = (r1.to(**f32).contiguous(), r2.to(**f32).contiguous())
        if sink is not None and sink.shape != (self.H,):
            raise ValueError(f"sink {list(sink.shape)} does not fit {self.H} heads")
        self.sink = sink.to(**f32).contiguous() if sink is not None else None
        if value_mix not in (None, "first", "mix"):
            raise ValueError(f"value_mix {value_mix!r} is not known (first or mix)")
        self.v_mode = {None: 0, "first": 1, "mix": 2}[value_mix]
        if self.v_mode == 2 and (mix_weight is None or mix_weight.numel() != 1):
            raise ValueError("value mixing needs its weight, one number")
        self.mix_weight = mix_weight.to(**f32).reshape(1).contiguous() if self.v_mode == 2 else None
        self.shared_name = shared_name
        self.hidden, self.dtype = hidden, dtype
        self.impl = "auto"            # "general" forces the general kernel (tests)
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
        self._partials = None         # scratch of the decode kernel's merge through global memory, made at first need
        self._arrived = None

    # ------------------------------------------------------------------ what the runtime asks
    def cache_spec(self) -> Optional[CacheSpec]:
        kv = (PagedTensorSpec(self.G, self.D), PagedTensorSpec(self.G, self.DV))
        return CacheSpec(kind=self.cache_keep[0], window=self.cache_keep[1], tensors=kv * (1 + len(self.pooled_sizes)))

    def shared_buffer(self) -> Optional[Tuple[str, int]]:
        """(name, columns) of the step buffer this mixer writes or reads, or None."""
        return (self.shared_name, self.G * self.DV) if self.v_mode else None

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def core_workspace_bytes(self, rows: int) -> int:
        return aligned(rows * self.H * self.D * self.w_in.element_size())

    def workspace_bytes(self, rows: int) -> int:
        es = self.w_in.element_size()
        return aligned(rows * self.w_in.shape[0] * es) + aligned(rows * self.n_pre * es) + self.core_workspace_bytes(rows)

    def plain_scores(self) -> bool:
        """Scores that are q . k * scale and nothing else, over all earlier keys or a window: what the framework's
        tensor-core attention kernels compute."""
        return not (self.chunk or self.softcap or self.dist_bias is not None or self.pool)

    def tensor_core_sizes(self) -> bool:
        """Keys and values of one size that the framework's tensor-core attention kernels are built for."""
        return self.plain_scores() and self.D == self.DV and self.D in kernels.TENSOR_CORE_HEAD_DIMS and self.H // self.G <= 16

    def shape_args(self) -> dict:
        """What shapes this layer's scores before the softmax, as the kernels' keyword arguments."""
        return dict(chunk=self.chunk, softcap=self.softcap, dist_bias=self.dist_bias)

    def padded_tile_sizes(self) -> bool:
        """Keys and values of sizes the portion kernel with padded tiles takes."""
        return self.D % 8 == 0 and self.DV % 8 == 0 and self.D <= 128 and self.DV <= 128

    def shaped_decode_sizes(self) -> bool:
        """Shaped scores with keys and values of one size the split-key decode kernel is built for."""
        return not self.plain_scores() and self.D == self.DV and self.D in kernels.TENSOR_CORE_HEAD_DIMS and self.H // self.G <= 16

    def kernel_modules(self, dtype, max_rows):
        if dtype == torch.float32:
            return ("gemm_f32", "attention_flex")
        mods = ["gemm_sm100", "attention_flex"]
        if self.pool and self.padded_tile_sizes():
            mods += ["attention_mma"]
        elif self.tensor_core_sizes():
            mods += ["attention_mma"] + ([] if self.window or self.gated else ["attention_sm100"])
        elif self.padded_tile_sizes():
            mods += ["attention_mma"]
        return tuple(mods)

    # ------------------------------------------------------------------ the step
    def core(self, proj: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state, pre_out: torch.Tensor,
             out_scale: float = 1.0) -> None:
        """proj [T, >= w_in rows] -> pre_out [T, n_pre]: everything between the two projections."""
        if cache is None:
            raise ValueError("attention needs a cache")
        T = proj.shape[0]
        kc, vc = cache.tensors[0], cache.tensors[1]
        q = ctx.alloc((T, self.H * self.D))
        v_first = ctx.shared.get(self.shared_name) if self.v_mode else None
        if self.v_mode and v_first is None:
            raise ValueError(f"the step has no buffer {self.shared_name!r} for the values that layers mix")
        if self.shared_kv == cache.write:
            raise ValueError("a layer writes the cache exactly when it has keys and values of its own")
        kernels.flex_prep(proj, self.q_off, self.k_off, self.v_off, ctx.positions, ctx.slot_mapping[cache.group] if cache.write else None,
                          self.inv_freq, self.rot, self.unit_rms, self.eps, self.q_temp, self.mix_weight, v_first, self.v_mode, q,
                          None if self.shared_kv else kc, None if self.shared_kv else vc, self.H, self.G, self.D, self.DV,
                          self.q_norm_w, self.k_norm_w, self.q_pre_w, self.k_pre_w)
        if cache.write:        # the blocks that this step's tokens complete, in every size the cache serves
            for i, size in enumerate(self.pooled_sizes):
                kernels.pool_blocks(kc, vc, cache.tensors[2 + 2 * i], cache.tensors[3 + 2 * i], ctx.block_tables[cache.group], ctx.row_seq,
                                    ctx.positions, size)
        gate = proj[:, self.g_off:self.g_off + self.n_pre] if self.gated else None
        self.attend(q, pre_out, ctx, cache, gate, out_scale)

    def attend(self, q, out, ctx: StepContext, cache: LayerCache, gate, out_scale: float) -> None:
        """bfloat16 with keys and values of one size the framework's tensor-core kernels take (64 or 128): steps of
        single tokens go to the split-key decode kernel, portions to the tcgen05 kernel (no window, no gate) or the
        mma.sync one, each of which ends with this mixer's sink, gate and factor; a mixed step's leading single tokens
        go to the decode kernel and the portions behind them to the portion kernel. bfloat16 with keys and values of
        other sizes (multiples of 8 up to 128 each, different or not): portions and mixed steps go to the mma.sync
        portion kernel that pads its tiles, steps of single tokens to the general kernel. Scores that are shaped
        before the softmax (blocks of positions, a cap, a distance bias) take the same two mma.sync kernels in their
        shaped build: the padded portion kernel for portions and mixed steps of any of those sizes, the split-key
        decode kernel for steps of single tokens with keys and values of one size of 64 or 128. Everything else
        (float32, other sizes) goes to the general kernel."""
        kc, vc = cache.tensors[0], cache.tensors[1]
        page, bt = kc.shape[2], ctx.block_tables[cache.group]
        H, G, D = self.H, self.G, self.D
        if (self.dtype == torch.bfloat16 and self.impl != "general" and self.scale > 0 and self.tensor_core_sizes()
                and kernels.attn_mma_supported(H, G, D, page, True) and out.data_ptr() % 4 == 0 and out.stride(0) % 2 == 0):
            if ctx.decode_only:
                self._attend_single(q, out, ctx, cache, bt, ctx.rows, gate, out_scale)
                return
            if ctx.max_new > 0:
                lead = ctx.lead_single if 0 < ctx.lead_single < ctx.seqs else 0
                if lead:
                    self._attend_single(q, out, ctx, cache, bt, lead, gate, out_scale)
                if (self.window == 0 and gate is None and out_scale == 1.0 and out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0
                        and kernels.attn_prefill_sm100_supported(H, G, D, page, bt.shape[1])):
                    kernels.attn_prefill_sm100(q, out, kc, vc, bt[lead:], ctx.seq_starts[lead:], ctx.context_lens[lead:], ctx.seqs - lead,
                                               ctx.max_new, H, G, D, self.scale, self.sink)
                else:
                    kernels.attn_prefill_mma(q, out, kc, vc, bt[lead:], ctx.seq_starts[lead:], ctx.context_lens[lead:], ctx.seqs - lead,
                                             ctx.max_new, H, G, D, self.scale, self.window, self.sink, gate, out_scale)
                return
        shaped = not self.plain_scores()
        if (self.pool and self.dtype == torch.bfloat16 and self.impl != "general" and self.dist_bias is None and ctx.max_new > 0
                and kernels.attn_prefill_mma_any_supported(H, G, D, self.DV, page) and out.data_ptr() % 4 == 0 and out.stride(0) % 2 == 0):
            # pooled blocks on the tensor cores: the padded portion kernel walks the pooled entries, then the window's tokens
            # (steps of single tokens too: a tile then holds one token's heads)
            i = self.pooled_sizes.index(self.pool)
            kernels.attn_prefill_mma_any(q, out, kc, vc, bt, ctx.seq_starts, ctx.context_lens, ctx.seqs, ctx.max_new, H, G, D, self.DV,
                                         self.scale, self.window, self.sink, gate, out_scale, softcap=self.softcap,
                                         pooled=(cache.tensors[2 + 2 * i], cache.tensors[3 + 2 * i], self.pool))
            return
        if self.pool:       # pooled blocks, float32 or sizes the tensor cores do not take: the general kernel pools on its way
            kernels.flex_attention(q, out, kc, vc, bt, ctx.row_seq, ctx.positions, H, G, D, self.DV, self.scale, self.window, self.sink,
                                   gate, out_scale, self.chunk, self.softcap, self.dist_bias, self.pool)
            return
        if (self.dtype == torch.bfloat16 and self.impl != "general" and shaped and ctx.decode_only and self.shaped_decode_sizes()
                and kernels.attn_mma_supported(H, G, D, page, True) and out.data_ptr() % 4 == 0 and out.stride(0) % 2 == 0):
            self._attend_single(q, out, ctx, cache, bt, ctx.rows, gate, out_scale)
            return
        if (self.dtype == torch.bfloat16 and self.impl != "general" and (self.scale > 0 or shaped) and not ctx.decode_only and ctx.max_new > 1
                and kernels.attn_prefill_mma_any_supported(H, G, D, self.DV, page) and out.data_ptr() % 4 == 0 and out.stride(0) % 2 == 0):
            kernels.attn_prefill_mma_any(q, out, kc, vc, bt, ctx.seq_starts, ctx.context_lens, ctx.seqs, ctx.max_new, H, G, D, self.DV,
                                         self.scale, self.window, self.sink, gate, out_scale, **self.shape_args())
            return
        kernels.flex_attention(q, out, kc, vc, bt, ctx.row_seq, ctx.positions, H, G, D, self.DV, self.scale, self.window, self.sink,
                               gate, out_scale, self.chunk, self.softcap, self.dist_bias)

    def _attend_single(self, q, out, ctx: StepContext, cache: LayerCache, bt, count: int, gate, out_scale: float) -> None:
        """The decode kernel on the first `count` rows, row i belonging to request i."""
        splits, wide = decode_split_rule(count, self.G, self.num_sms, ctx.long_context and not self.window and not self.chunk)
        if wide and self._partials is None:
            floats = kernels.attn_decode_partial_floats(1, 1, self.D, 3 * self.num_sms)    # requests x kv heads x splits <= 3 SMs
            self._partials = torch.empty(floats, dtype=torch.float32, device=q.device)
            self._arrived = torch.zeros(self.num_sms, dtype=torch.int32, device=q.device)
        kernels.attn_decode_mma(q[:count], out[:count], cache.tensors[0], cache.tensors[1], bt, ctx.positions[:count], self.H, self.G,
                                self.D, self.scale, self.window, splits, self._partials if wide else None,
                                self._arrived if wide else None, self.sink, gate[:count] if gate is not None else None, out_scale,
                                **self.shape_args())

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state=None, out=None) -> torch.Tensor:
        T = x.shape[0]
        proj = ctx.alloc((T, self.w_in.shape[0]))
        kernels.linear(x, self.w_in, proj, self.b_in)
        pre = ctx.alloc((T, self.n_pre))
        self.core(proj, ctx, cache, state, pre)
        out = out if out is not None else ctx.alloc((T, self.hidden))
        kernels.linear(pre, self.w_o, out, self.b_o)
        return out
