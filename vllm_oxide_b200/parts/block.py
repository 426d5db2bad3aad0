"""The arrangements of parts in one layer: the pre-norm residual block (`Block`), the block whose
residual takes the normed result of each sub-layer (`PostNormBlock`) and the block with a norm on both sides of
each sub-layer (`SandwichBlock`, at the end of the file).

    residual += mixer(norm1(residual));  residual += feed_forward(norm2(residual))
(crates/engine/src/model.rs:302-332). The residual is float32. Each part's output is not added
at once: it is handed on as `pending` and the next norm's kernel adds it while it normalises
(one pass over the row instead of two). The model's final norm takes the last `pending`.

Options: a per-feature scale on each part's output before it is added (`mixer_scale`, `ff_scale`:
the norm's kernel multiplies while it adds; `pending_scale` tells whoever adds this block's
output which one goes with it), and a block without a feed-forward (`feed_forward` None:
    residual += mixer(norm1(residual)) only; `norm2` is None then).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..tuning import TUNING
from .base import FeedForward, FoldedState, LayerCache, Mixer, Norm, StateSpec, StepContext, aligned


class Block:
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], feed_forward: Optional[FeedForward],
                 mixer_scale: Optional[torch.Tensor] = None, ff_scale: Optional[torch.Tensor] = None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        dev = getattr(norm1, "weight", None)

        def vec(t):
            if t is None:
                return None
            return t.to(device=dev.device if dev is not None else t.device, dtype=torch.float32).contiguous()
        self.mixer_scale, self.ff_scale = vec(mixer_scale), vec(ff_scale)
        # the scale that goes with the output this block hands on
        self.pending_scale = self.ff_scale if feed_forward is not None else self.mixer_scale

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def weight_bytes(self) -> int:
        scales = sum(t.numel() * 4 for t in (self.mixer_scale, self.ff_scale) if t is not None)
        return scales + sum(getattr(p, "weight_bytes", lambda: 0)() for p in self._parts())

    def workspace_bytes(self, rows: int, hidden: int, act_bytes: int) -> int:
        """Peak scratch of one run of the block, read off the scopes of `forward`: the mixer's
        output, then the larger of (first norm's output + mixer scratch) and (second norm's output +
        feed-forward scratch)."""
        if self.feed_forward is None:
            return self.norm1.workspace_bytes(rows, act_bytes) + self.mixer.workspace_bytes(rows)
        mixed = aligned(rows * hidden * act_bytes)
        return mixed + max(self.norm1.workspace_bytes(rows, act_bytes) + self.mixer.workspace_bytes(rows),
                           self.norm2.workspace_bytes(rows, act_bytes) + self.feed_forward.workspace_bytes(rows))

    def folded_workspace_bytes(self, rows: int) -> int:
        """Peak scratch of `forward_folded` (0 for parts that do not say)."""
        return max(getattr(self.mixer, "folded_workspace_bytes", lambda r: 0)(rows),
                   getattr(self.feed_forward, "folded_workspace_bytes", lambda r: 0)(rows))

    def kernel_modules(self, dtype, max_rows):
        mods = []
        for p in self._parts():
            mods += list(getattr(p, "kernel_modules", lambda d, r: ())(dtype, max_rows))
        return tuple(mods)

    def can_fold(self) -> bool:
        """Whether this block can run in folded form (see FoldedState): both norms are a per-token
        scale and a per-feature weight (`Norm.scale_and_weight`), which is what folds into the
        neighbouring products, and mixer and feed-forward both offer it."""
        if self.feed_forward is None or self.mixer_scale is not None or self.ff_scale is not None:
            return False
        return (self.norm1.scale_and_weight and self.norm2.scale_and_weight
                and getattr(self.mixer, "can_fold", lambda: False)() and getattr(self.feed_forward, "can_fold", lambda: False)()
                and self.mixer.state_spec() is None)

    def forward_folded(self, st: FoldedState, ctx: StepContext, cache: Optional[LayerCache], next_norm: Norm) -> None:
        """The block on the folded residual: no norm kernel, no separate residual add. `next_norm`
        is the norm that will read the residual after this block (the next block's first norm, or
        the model's final norm)."""
        with ctx.workspace.scope():
            self.mixer.forward_folded(st, self.norm1.eps, ctx, cache, self.norm2.weight)
        with ctx.workspace.scope():
            self.feed_forward.forward_folded(st, self.norm2.eps, ctx, next_norm.weight)

    def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[LayerCache], state, out: torch.Tensor, pending_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the block. `pending` is the previous block's output that is still to be added to
        the residual (times `pending_scale`, if that block had one); the feed-forward's output
        (again not yet added) is written to `out`, which outlives the block's own scratch."""
        ws = ctx.workspace

        def first_norm():
            if pending is not None and pending_scale is not None:
                return self.norm1.forward(resid, pending, ctx, delta_scale=pending_scale)
            return self.norm1.forward(resid, pending, ctx)
        if self.feed_forward is None:
            with ws.scope():
                m = self.mixer.forward(first_norm(), ctx, cache, state, out=out)
                if m.data_ptr() != out.data_ptr():
                    out.copy_(m)
            return out
        with ws.scope():
            mixed = ctx.alloc(out.shape, out.dtype)
            with ws.scope():
                m = self.mixer.forward(first_norm(), ctx, cache, state, out=mixed)
                if m.data_ptr() != mixed.data_ptr():
                    mixed.copy_(m)
            if self.mixer_scale is not None:
                normed2 = self.norm2.forward(resid, mixed, ctx, delta_scale=self.mixer_scale)
            else:
                normed2 = self.norm2.forward(resid, mixed, ctx)
            ff = self.feed_forward.forward(normed2, ctx, out=out)
            if ff.data_ptr() != out.data_ptr():
                out.copy_(ff)
        return out


class PostNormBlock:
    """residual += norm1(mixer(residual));  residual += norm2(feed_forward(residual))

    The sub-layers read the residual itself and the norms sit on their results only. The residual is float32; in an
    engine whose activations are narrower, a sub-layer reads the residual rounded to that type: the kernel that adds a
    normed result also leaves the new residual in that type, in `out` (which outlives the block), and names it in
    `ctx.shared[STREAM_COPY]` for the next block of this arrangement, so only the first block of a step runs a kernel
    that does nothing but round. The norms offer `add_normed(resid, result, copy)` (`LayerNorm`). A block without
    feed-forward has no second norm. Nothing is left pending: the block returns None."""

    STREAM_COPY = "_residual_in_act_type"

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], feed_forward: Optional[FeedForward]):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        for n in (norm1, norm2):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError("the norms of this arrangement must offer add_normed(resid, result, copy)")
        self.pending_scale = None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def weight_bytes(self) -> int:
        return sum(getattr(p, "weight_bytes", lambda: 0)() for p in self._parts())

    def workspace_bytes(self, rows: int, hidden: int, act_bytes: int) -> int:
        """The residual in the activations' type (where that is not float32), one sub-layer's result, and the larger of the
        two sub-layers' own scratch."""
        copy = aligned(rows * hidden * act_bytes) if act_bytes != 4 else 0
        result = aligned(rows * hidden * act_bytes)
        ff = self.feed_forward.workspace_bytes(rows) if self.feed_forward is not None else 0
        return 2 * copy + result + max(self.mixer.workspace_bytes(rows), ff)

    def folded_workspace_bytes(self, rows: int) -> int:
        return 0

    def kernel_modules(self, dtype, max_rows):
        mods = ["elementwise"]
        for p in self._parts():
            mods += list(getattr(p, "kernel_modules", lambda d, r: ())(dtype, max_rows))
        return tuple(mods)

    def can_fold(self) -> bool:
        return False

    def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[LayerCache], state, out: torch.Tensor, pending_scale: Optional[torch.Tensor] = None):
        if pending is not None:
            raise ValueError("a block of this arrangement follows blocks that leave nothing pending")
        from .. import kernels
        ws = ctx.workspace
        narrow = ctx.dtype != torch.float32
        with ws.scope():
            x = resid
            if narrow:
                x = ctx.shared.pop(self.STREAM_COPY, None)
                if x is None or x.data_ptr() == out.data_ptr():
                    x = ctx.alloc(resid.shape)
                    kernels.cast_rows(resid, x)
            mid = ctx.alloc(resid.shape) if narrow and self.feed_forward is not None else None
            with ws.scope():
                m = self.mixer.forward(x, ctx, cache, state)
                self.norm1.add_normed(resid, m, (mid if self.feed_forward is not None else out) if narrow else None)
            if self.feed_forward is not None:
                with ws.scope():
                    f = self.feed_forward.forward(mid if narrow else resid, ctx)
                    self.norm2.add_normed(resid, f, out if narrow else None)
        if narrow:
            ctx.shared[self.STREAM_COPY] = out
        return None


class SandwichBlock:
    """residual += post1(mixer(c1(pre1(residual))));  residual += post2(feed_forward(c2(pre2(residual))))

    A norm in front of each sub-layer and another on its result. Options, each off when its argument is None:

    * `canon1`, `canon2` ([width, taps] each): what a sub-layer reads, h, is first replaced by h + conv(h), a short causal
      convolution over time on each feature, conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j); the last taps - 1 inputs of
      a request are part of its state (the block answers `state_spec()` for them and for its mixer);
    * `depth_weights` ([n + 1], with `depth_index` = n - 1 and `depth_slots`): the stream is a learned sum over depth. The
      block files its result as entry n of `ctx.shared[depth_name]` (float32 [rows, depth_slots * width]; entry 0 is the
      embedding's output, filed by the block with `depth_index` 0) and hands on sum_j depth_weights[j] * entry j.

    The pre-norms offer `forward(resid, None, ctx)`, the post-norms `add_normed(resid, result, copy)` (`LayerNorm`). A block
    without feed-forward has neither second norm. Nothing is left pending: the block returns None."""

    def __init__(self, pre1: Norm, mixer: Mixer, post1: Norm, pre2: Optional[Norm], feed_forward: Optional[FeedForward],
                 post2: Optional[Norm], canon1: Optional[torch.Tensor] = None, canon2: Optional[torch.Tensor] = None,
                 depth_weights: Optional[torch.Tensor] = None, depth_index: int = 0, depth_slots: int = 0,
                 depth_name: str = "depth_stack", device="cuda"):
        self.norm1, self.mixer, self.post1 = pre1, mixer, post1
        self.norm2, self.feed_forward, self.post2 = pre2, feed_forward, post2
        if (pre2 is None) != (feed_forward is None) or (post2 is None) != (feed_forward is None):
            raise ValueError("a block has its second pair of norms exactly when it has a feed-forward")
        for n in (post1, post2):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError("the norms behind the sub-layers must offer add_normed(resid, result, copy)")
        if canon2 is not None and feed_forward is None:
            raise ValueError("a convolution in front of a feed-forward that is not there")
        f32 = dict(device=device, dtype=torch.float32)
        for c in (canon1, canon2):
            if c is not None and (c.dim() != 2 or c.shape[1] < 1):
                raise ValueError(f"a convolution's weights are [width, taps], got {list(c.shape)}")
        # kept tap by tap ([taps, width]), as the kernel reads them
        self.canon1 = canon1.to(**f32).t().contiguous() if canon1 is not None else None
        self.canon2 = canon2.to(**f32).t().contiguous() if canon2 is not None else None
        self.depth_weights = depth_weights.to(**f32).contiguous() if depth_weights is not None else None
        self.depth_index, self.depth_slots, self.depth_name = int(depth_index), int(depth_slots), depth_name
        if self.depth_weights is not None and (self.depth_weights.shape != (self.depth_index + 2,) or self.depth_slots < self.depth_index + 2):
            raise ValueError(f"the block at depth {depth_index} takes {self.depth_index + 2} weights and as many entries, got "
                             f"{list(self.depth_weights.shape)} and {depth_slots}")
        self.pending_scale = None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.post1, self.norm2, self.feed_forward, self.post2) if p is not None]

    def _own_states(self):
        return [c for c in (self.canon1, self.canon2) if c is not None and c.shape[0] > 1]

    def state_spec(self):
        """The convolutions' last inputs (one tensor each, [taps - 1, width]), then the mixer's own state."""
        own = [StateSpec((c.shape[0] - 1, c.shape[1]), torch.float32) for c in self._own_states()]
        ms = self.mixer.state_spec()
        ms = [] if ms is None else list(ms) if isinstance(ms, (tuple, list)) else [ms]
        return tuple(own + ms) if own or ms else None

    def weight_bytes(self) -> int:
        own = sum(t.numel() * 4 for t in (self.canon1, self.canon2, self.depth_weights) if t is not None)
        return own + sum(getattr(p, "weight_bytes", lambda: 0)() for p in self._parts())

    def workspace_bytes(self, rows: int, hidden: int, act_bytes: int) -> int:
        """The normed input, its convolved form, one sub-layer's result, and the larger of the two sub-layers' own scratch."""
        ff = self.feed_forward.workspace_bytes(rows) if self.feed_forward is not None else 0
        return 3 * aligned(rows * hidden * act_bytes) + max(self.mixer.workspace_bytes(rows), ff)

    def folded_workspace_bytes(self, rows: int) -> int:
        return 0

    def kernel_modules(self, dtype, max_rows):
        mods = ["elementwise"] + (["recurrence"] if self.canon1 is not None or self.canon2 is not None else [])
        for p in self._parts():
            mods += list(getattr(p, "kernel_modules", lambda d, r: ())(dtype, max_rows))
        return tuple(mods)

    def can_fold(self) -> bool:
        return False

    def _read(self, norm: Norm, canon, conv_state, resid, ctx: StepContext):
        """What a sub-layer reads: the normed residual, with its convolution added where there is one. Returns it and what the
        norm behind the sub-layer is to do on its way: move the convolution's state on (every read of the old one is over then)."""
        from .. import kernels
        h = norm.forward(resid, None, ctx)
        if canon is None:
            return h, None
        hc = ctx.alloc(h.shape)
        # a step of single tokens: the convolution's kernel moves the state on itself
        single = bool(ctx.decode_only and conv_state is not None)
        kernels.causal_conv(h, canon, None, conv_state, ctx.positions, ctx.row_seq, ctx.seq_starts, ctx.state_slots, ctx.seqs, hc,
                            residual=True, single=single)
        if conv_state is None or single:
            return hc, None
        if not TUNING.norm_tail:
            kernels.conv_state_update(h, 0, conv_state, ctx.seq_starts, ctx.state_slots, ctx.seqs)
            return hc, None
        return hc, (h, conv_state, ctx.row_seq, ctx.seq_starts, ctx.state_slots, ctx.positions)

    def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[LayerCache], state, out: torch.Tensor, pending_scale: Optional[torch.Tensor] = None):
        if pending is not None:
            raise ValueError("a block of this arrangement follows blocks that leave nothing pending")
        from .. import kernels
        ws = ctx.workspace
        states = list(state) if isinstance(state, (tuple, list)) else [] if state is None else [state]
        own = [states.pop(0) for _ in self._own_states()]
        cs1 = own.pop(0) if self.canon1 is not None and self.canon1.shape[0] > 1 else None
        cs2 = own.pop(0) if self.canon2 is not None and self.canon2.shape[0] > 1 else None
        ms = self.mixer.state_spec()
        mixer_state = None if ms is None else tuple(states) if isinstance(ms, (tuple, list)) else states[0]
        depth = None
        if self.depth_weights is not None:
            stack = ctx.shared[self.depth_name].view(resid.shape[0], self.depth_slots, resid.shape[1])
            if self.depth_index == 0:
                kernels.depth_average(stack, resid, None, 0)
            # the sum over depth rides on the block's last norm
            depth = (stack, self.depth_weights, self.depth_index + 1) if TUNING.norm_tail else None
        with ws.scope():
            x, conv = self._read(self.norm1, self.canon1, cs1, resid, ctx)
            m = self.mixer.forward(x, ctx, cache, mixer_state)
            self.post1.add_normed(resid, m, None, depth=depth if self.feed_forward is None else None, conv=conv)
        if self.feed_forward is not None:
            with ws.scope():
                x, conv = self._read(self.norm2, self.canon2, cs2, resid, ctx)
                f = self.feed_forward.forward(x, ctx)
                self.post2.add_normed(resid, f, None, depth=depth, conv=conv)
        if self.depth_weights is not None and depth is None:
            kernels.depth_average(stack, resid, self.depth_weights, self.depth_index + 1)
        return None
