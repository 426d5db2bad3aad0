"""Launch wrappers of the CUDA kernels: every shape, dtype, device and alignment is checked
here, on the host, before a pointer reaches a kernel (the reference's rule for its launch
wrappers, CLAUDE.md:79, and the checks of crates/engine/src/arena/ops.rs:30-268).

There is no CPU path and no fallback: a tensor that is not on a CUDA device, or a kernel
library that cannot be built or loaded, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import load_cuda_module
from .errors import KernelError, ShapeError
from .tuning import TUNING

_CODES = {torch.float32: 0, torch.bfloat16: 1}
_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_STATUS = {2001: "bad argument", 2002: "size not supported by this kernel"}


def _code(t: torch.Tensor, op: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise ShapeError(op, f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(op: str, *tensors: Optional[torch.Tensor]) -> None:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError(f"{op}: tensor on {t.device}; the kernels run on a CUDA device only "
                              "(there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ShapeError(op, f"tensors on different devices: {dev} and {t.device}")


def _ptr(t: Optional[torch.Tensor]):
    return _P(t.data_ptr()) if t is not None else _P(0)


def _stream() -> _P:
    # the raw handle straight from the runtime: torch.cuda.current_stream() builds a Python object
    # each time (some 15 us), which adds up over the two hundred launches of a step
    return _P(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


_launches = 0      # kernels of this package launched (or replayed from a graph) so far


def launch_count() -> int:
    return _launches


def count_launches(n: int) -> None:
    """Account for launches that did not pass through a wrapper (a CUDA graph replay)."""
    global _launches
    _launches += n


def _check(status: int, op: str, launches: int = 1) -> None:
    global _launches
    if status != 0:
        what = _STATUS.get(status, f"CUDA error {status}")
        raise KernelError(f"{op}: launch failed: {what}")
    _launches += launches


def _rows_2d(t: torch.Tensor, op: str, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ShapeError(op, f"{name} must be 2-D with unit inner stride, got shape {list(t.shape)} "
                             f"strides {list(t.stride())}")


def _int32_vec(t: torch.Tensor, n: int, op: str, name: str) -> None:
    if t.dtype != torch.int32 or t.dim() != 1 or t.numel() < n or not t.is_contiguous():
        raise ShapeError(op, f"{name} must be a contiguous int32 vector of at least {n}, got "
                             f"{t.dtype} {list(t.shape)}")


_fn_cache = {}
_MODULES = ("elementwise", "gemm_f32", "gemm_sm100", "gemm_sm100_pair", "attention", "attention_mma", "attention_sm100", "sampling",
            "streams", "recurrence", "latent_attention", "attention_flex", "moe")

# Per-op device timing, off unless a profile is being taken: CUDA events around each wrapper
# (the reference times ops by wall clock on the CPU and notes that a CUDA backend must use
# events and add no synchronisation, crates/engine/src/arena.rs:66-68,243-255).
_profile = None


class OpProfile:
    """with OpProfile() as p: ...steps...; p.totals() -> [(op, calls, total_ms)] by time."""

    def __init__(self):
        self.events = []

    def __enter__(self):
        global _profile
        _profile = self
        return self

    def __exit__(self, *exc):
        global _profile
        _profile = None
        return False

    def totals(self):
        torch.cuda.synchronize()
        agg = {}
        for name, a, b in self.events:
            c, t = agg.get(name, (0, 0.0))
            agg[name] = (c + 1, t + a.elapsed_time(b))
        return sorted(((n, c, t) for n, (c, t) in agg.items()), key=lambda x: -x[2])


def _timed(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if _profile is None:
            return fn(*args, **kwargs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            return fn(*args, **kwargs)
        finally:
            b.record()
            _profile.events.append((fn.__name__, a, b))
    return wrapper


def _fn(module: str, name: str, argtypes):
    key = (module, name)
    f = _fn_cache.get(key)
    if f is None:
        lib = _load(module)
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise KernelError(f"kernel library '{module}' has no entry point {name}") from None
        f.argtypes = argtypes
        f.restype = _I
        _fn_cache[key] = f
    return f


_pdl_on = False


TENSOR_CORE_HEAD_DIMS = (64, 128)       # head sizes the tensor-core attention kernels are built for


def preload(modules=_MODULES) -> None:
    """Build (side by side) and load kernel modules now, so that compile time is spent at start-up."""
    from .csrc.build import ensure_built
    ensure_built(modules)
    for m in modules:
        _load(m)


def _load(module: str):
    """dlopen a module and hand it the current launch switches."""
    from .csrc.build import _loaded
    fresh = module not in _loaded
    lib = load_cuda_module(module)
    if fresh:
        f = getattr(lib, f"vob_set_pdl_{module}")
        f.argtypes = [_I]
        f.restype = None
        f(1 if _pdl_on else 0)
    return lib


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off for every kernel of this package: with it, a
    kernel's set-up (and a matrix product's first weight loads) overlaps the end of the kernel
    before it; each kernel still waits for its predecessors before it reads or writes anything
    they touch. Modules loaded later take the switch over."""
    global _pdl_on
    from .csrc.build import _loaded
    _pdl_on = bool(on)
    for m in _MODULES:
        if m in _loaded:
            f = getattr(_loaded[m], f"vob_set_pdl_{m}")
            f.argtypes = [_I]
            f.restype = None
            f(1 if _pdl_on else 0)


# ------------------------------------------------------------------------------------ embedding
@_timed
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, err_flag: Optional[torch.Tensor] = None,
          scale: float = 1.0, pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[tokens[t]] * scale (+ pos_table[positions[t]]) as float32; `tokens` int32 [T], `out` float32 [T, h].
    `pos_table` [max positions, h] of the table's type: a learned vector per position (rows of negative position get none)."""
    op = "embed"
    _cuda(op, table, tokens, out, err_flag, pos_table, positions)
    if pos_table is not None:
        if pos_table.dim() != 2 or pos_table.shape[1] != table.shape[1] or pos_table.dtype != table.dtype or not pos_table.is_contiguous():
            raise ShapeError(op, f"pos_table must be contiguous {table.dtype} [positions, {table.shape[1]}], got {pos_table.dtype} {list(pos_table.shape)}")
        if positions is None:
            raise ShapeError(op, "a position table needs the rows' positions")
        _int32_vec(positions, out.shape[0], op, "positions")
    T = out.shape[0]
    if table.dim() != 2 or not table.is_contiguous():
        raise ShapeError(op, f"table must be contiguous [vocab, h], got {list(table.shape)}")
    _int32_vec(tokens, T, op, "tokens")
    if out.dtype != torch.float32 or out.dim() != 2 or out.shape[1] != table.shape[1] or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous float32 [T, {table.shape[1]}], got {out.dtype} {list(out.shape)}")
    f = _fn("elementwise", "vob_embed", [_P, _I, _P, _P, _I, _I, _I, _P, _F, _P, _P, _I, _P])
    _check(f(_ptr(table), _code(table, op), _ptr(tokens), _ptr(out), T, table.shape[1], table.shape[0],
             _ptr(err_flag), float(scale), _ptr(pos_table), _ptr(positions) if pos_table is not None else _P(0),
             pos_table.shape[0] if pos_table is not None else 0, _stream()), op)


# ------------------------------------------------------------------------------------ norm
@_timed
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, delta_scale: Optional[torch.Tensor] = None) -> None:
    """resid (+= delta, times `delta_scale` per feature if given); out = weight * (x / sqrt(mean(x^2) + eps)).
    With `rows` (int32 [R]) only those rows are normalised into out [R, h] and resid is left as it is."""
    op = "add_rmsnorm"
    _cuda(op, resid, delta, weight, out, rows, delta_scale)
    if resid.dtype != torch.float32 or resid.dim() != 2 or not resid.is_contiguous():
        raise ShapeError(op, f"the residual must be contiguous float32 [T, h], got {resid.dtype} {list(resid.shape)}")
    T, h = resid.shape
    if weight.dtype != torch.float32 or weight.shape != (h,) or not weight.is_contiguous():
        raise ShapeError(op, f"weight must be float32 [{h}], got {weight.dtype} {list(weight.shape)}")
    if delta is not None and (delta.shape != resid.shape or not delta.is_contiguous()):
        raise ShapeError(op, f"delta must be contiguous {list(resid.shape)}, got {list(delta.shape)}")
    R = T
    if rows is not None:
        R = rows.numel()
        _int32_vec(rows, R, op, "rows")
    if out.dim() != 2 or out.shape[0] < R or out.shape[1] != h or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous [>={R}, {h}], got {list(out.shape)}")
    if h * 4 > 48 * 1024:
        raise ShapeError(op, f"width {h} is beyond this kernel's limit of {48 * 1024 // 4}")
    if delta_scale is not None and (delta is None or delta_scale.dtype != torch.float32 or delta_scale.shape != (h,)
                                    or not delta_scale.is_contiguous()):
        raise ShapeError(op, f"delta_scale must be float32 [{h}] and come with a delta, got {delta_scale.dtype} {list(delta_scale.shape)}")
    f = _fn("elementwise", "vob_add_rmsnorm", [_P, _P, _I, _P, _P, _P, _I, _I, _I, _F, _P, _P])
    _check(f(_ptr(resid), _ptr(delta), _code(delta, op) if delta is not None else 0, _ptr(weight), _ptr(rows),
             _ptr(out), _code(out, op), R, h, float(eps), _ptr(delta_scale), _stream()), op)


@_timed
def layernorm_add(resid: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float,
                  copy: Optional[torch.Tensor] = None, depth=None, conv=None) -> None:
    """resid += LN(delta) with LN(z) = (z - mean) / sqrt(mean((z - mean)^2) + eps) * weight + bias; `copy` ([T, h] in the
    activations' type), if given, receives the new residual. On the way, where asked for (not together with `copy`):
    `depth` = (stack float32 [T, slots, h], weights float32 [n + 1], n): what `depth_average` does with the new residual;
    `conv` = (conv_x [T, h] of delta's type, conv_state float32 [slots, taps - 1, h], row_seq, seq_starts, state_slots,
    positions): what `conv_state_update` does for a convolution that read conv_x in front of the sub-layer."""
    op = "layernorm_add"
    _cuda(op, resid, delta, weight, bias, copy)
    if depth is not None or conv is not None:
        if copy is not None:
            raise ShapeError(op, "the residual's copy and the work on the way do not go together")
        T, h = resid.shape
        if resid.dtype != torch.float32 or resid.dim() != 2 or not resid.is_contiguous() or delta.shape != resid.shape or not delta.is_contiguous():
            raise ShapeError(op, f"a contiguous float32 residual [T, h] and a contiguous delta of its shape are needed")
        _f32_vec(weight, h, op, "weight")
        _f32_vec(bias, h, op, "bias")
        if h * 4 > 48 * 1024:
            raise ShapeError(op, f"width {h} is beyond this kernel's limit of {48 * 1024 // 4}")
        stack = dw = cx = cs = rs = ss = sl = ps = None
        slots = n = taps = 0
        if depth is not None:
            stack, dw, n = depth
            _cuda(op, resid, stack, dw)
            if stack.dtype != torch.float32 or stack.dim() != 3 or stack.shape[0] != T or stack.shape[2] != h or not stack.is_contiguous() \
                    or not 0 < n < stack.shape[1]:
                raise ShapeError(op, f"stack must be contiguous float32 [{T}, > {n}, {h}], got {stack.dtype} {list(stack.shape)}")
            _f32_vec(dw, n + 1, op, "depth weights")
            slots = stack.shape[1]
        if conv is not None:
            cx, cs, rs, ss, sl, ps = conv
            _cuda(op, resid, cx, cs, rs, ss, sl, ps)
            if cx.shape != resid.shape or cx.dtype != delta.dtype or not cx.is_contiguous():
                raise ShapeError(op, f"conv_x must be contiguous {delta.dtype} {list(resid.shape)}, got {cx.dtype} {list(cx.shape)}")
            if cs.dtype != torch.float32 or cs.dim() != 3 or cs.shape[2] != h or cs.shape[1] < 1 or not cs.is_contiguous():
                raise ShapeError(op, f"conv_state must be contiguous float32 [slots, taps - 1, {h}], got {cs.dtype} {list(cs.shape)}")
            taps = cs.shape[1] + 1
            _int32_vec(rs, T, op, "row_seq")
            _int32_vec(ps, T, op, "positions")
        f = _fn("elementwise", "vob_layernorm_tail", [_P, _P, _I, _P, _P, _I, _I, _F, _P, _P, _I, _I, _P, _P, _I, _P, _P, _P, _P, _P])
        _check(f(_ptr(resid), _ptr(delta), _code(delta, op), _ptr(weight), _ptr(bias), T, h, float(eps), _ptr(stack), _ptr(dw), slots, int(n),
                 _ptr(cx), _ptr(cs), taps, _ptr(rs), _ptr(ss), _ptr(sl), _ptr(ps), _stream()), op)
        return
    if resid.dtype != torch.float32 or resid.dim() != 2 or not resid.is_contiguous():
        raise ShapeError(op, f"the residual must be contiguous float32 [T, h], got {resid.dtype} {list(resid.shape)}")
    T, h = resid.shape
    _f32_vec(weight, h, op, "weight")
    _f32_vec(bias, h, op, "bias")
    if delta.shape != resid.shape or not delta.is_contiguous():
        raise ShapeError(op, f"delta must be contiguous {list(resid.shape)}, got {list(delta.shape)}")
    if copy is not None and (copy.shape != resid.shape or not copy.is_contiguous()):
        raise ShapeError(op, f"copy must be contiguous {list(resid.shape)}, got {list(copy.shape)}")
    if h * 4 > 48 * 1024:
        raise ShapeError(op, f"width {h} is beyond this kernel's limit of {48 * 1024 // 4}")
    f = _fn("elementwise", "vob_layernorm", [_P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _F, _P])
    _check(f(_ptr(resid), _ptr(delta), _code(delta, op), _ptr(weight), _ptr(bias), _P(0), _ptr(copy),
             _code(copy, op) if copy is not None else 0, T, h, float(eps), _stream()), op)


@_timed
def layernorm_rows(resid: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                   rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = LN(resid[rows[r]]) (every row in order without `rows`); the residual is left as it is."""
    op = "layernorm_rows"
    _cuda(op, resid, weight, bias, out, rows)
    if resid.dtype != torch.float32 or resid.dim() != 2 or not resid.is_contiguous():
        raise ShapeError(op, f"the residual must be contiguous float32 [T, h], got {resid.dtype} {list(resid.shape)}")
    T, h = resid.shape
    _f32_vec(weight, h, op, "weight")
    _f32_vec(bias, h, op, "bias")
    R = T
    if rows is not None:
        R = rows.numel()
        _int32_vec(rows, R, op, "rows")
    if out.dim() != 2 or out.shape[0] < R or out.shape[1] != h or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous [>={R}, {h}], got {list(out.shape)}")
    if h * 4 > 48 * 1024:
        raise ShapeError(op, f"width {h} is beyond this kernel's limit of {48 * 1024 // 4}")
    f = _fn("elementwise", "vob_layernorm", [_P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _F, _P])
    _check(f(_ptr(resid), _P(0), 0, _ptr(weight), _ptr(bias), _ptr(rows), _ptr(out), _code(out, op), R, h, float(eps), _stream()), op)


@_timed
def cast_rows(src: torch.Tensor, out: torch.Tensor) -> None:
    """out = src (float32, contiguous) in out's type, element by element."""
    op = "cast_rows"
    _cuda(op, src, out)
    if src.dtype != torch.float32 or not src.is_contiguous() or out.shape != src.shape or not out.is_contiguous():
        raise ShapeError(op, f"a contiguous float32 source and a contiguous result of its shape are needed, got {src.dtype} "
                             f"{list(src.shape)} and {list(out.shape)}")
    f = _fn("elementwise", "vob_cast_rows", [_P, _P, _I, _L, _P])
    _check(f(_ptr(src), _ptr(out), _code(out, op), src.numel(), _stream()), op)


ACTIVATIONS = {"xielu": 0}


@_timed
def activation(x: torch.Tensor, out: torch.Tensor, kind: str, params: torch.Tensor) -> None:
    """out[t, j] = act(x[t, j]), float32 arithmetic. "xielu" with params = float32 [ap, an] on the device:
    z > 0: ap z^2 + z / 2; z <= 0: an (exp(z) - 1 - z) + z / 2. `out` may be `x` itself."""
    op = "activation"
    _cuda(op, x, out, params)
    _rows_2d(x, op, "x")
    if kind not in ACTIVATIONS:
        raise ShapeError(op, f"activation {kind!r} is not known ({', '.join(ACTIVATIONS)})")
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous {x.dtype} {list(x.shape)}, got {out.dtype} {list(out.shape)}")
    _f32_vec(params, 2, op, "params")
    f = _fn("elementwise", "vob_act", [_P, _L, _P, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(x), x.stride(0), _ptr(out), _code(out, op), x.shape[0], x.shape[1], ACTIVATIONS[kind], _ptr(params), _stream()), op)


# ------------------------------------------------------------------------------------ rope + cache write
@_timed
def rope_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], positions: torch.Tensor,
                  slots: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                  kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate q and k in place (float32 angles position * inv_freq) and write k, v to their cache
    slots. q [T, H*hd], k and v [T, KV*hd] may be column slices of one wider tensor. kcache and
    vcache are one layer's pages [num_pages, KV, page_size, hd]."""
    op = "rope_kv_write"
    _cuda(op, q, k, v, positions, slots, inv_freq, kcache, vcache)
    _rows_2d(q, op, "q")
    T = q.shape[0]
    if q.shape[1] != num_heads * head_dim:
        raise ShapeError(op, f"q has {q.shape[1]} columns, expected heads*head_dim = {num_heads * head_dim}")
    if head_dim % 2 != 0:
        raise ShapeError(op, f"head_dim {head_dim} must be even")
    _int32_vec(positions, T, op, "positions")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (head_dim // 2,) or not inv_freq.is_contiguous()):
        raise ShapeError(op, f"inv_freq must be float32 [{head_dim // 2}], got {inv_freq.dtype} {list(inv_freq.shape)}")
    page_size = 1
    if k is not None:
        _rows_2d(k, op, "k")
        if k.shape != (T, num_kv_heads * head_dim) or k.dtype != q.dtype:
            raise ShapeError(op, f"k must be {q.dtype} [{T}, {num_kv_heads * head_dim}], got {k.dtype} {list(k.shape)}")
        if slots is not None:
            _int32_vec(slots, T, op, "slots")
            if v is None or kcache is None or vcache is None:
                raise ShapeError(op, "a cache write needs v, kcache and vcache")
            _rows_2d(v, op, "v")
            if v.shape != k.shape or v.dtype != q.dtype:
                raise ShapeError(op, f"v must match k, got {v.dtype} {list(v.shape)}")
            for name, c in (("kcache", kcache), ("vcache", vcache)):
                if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous() or c.dtype != q.dtype:
                    raise ShapeError(op, f"{name} must be contiguous {q.dtype} [pages, {num_kv_heads}, page_size, "
                                         f"{head_dim}], got {c.dtype} {list(c.shape)}")
            if kcache.shape != vcache.shape:
                raise ShapeError(op, "kcache and vcache differ in shape")
            page_size = kcache.shape[2]
    f = _fn("elementwise", "vob_rope_kv_write", [_P, _L, _P, _L, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0, _ptr(v),
             v.stride(0) if v is not None else 0, _ptr(positions), _ptr(slots), _ptr(inv_freq), _ptr(kcache),
             _ptr(vcache), _code(q, op), T, num_heads, num_kv_heads if k is not None else 0, head_dim, page_size,
             _stream()), op)


# ------------------------------------------------------------------------------------ swiglu
@_timed
def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j]."""
    op = "swiglu"
    _cuda(op, gate_up, out)
    _rows_2d(gate_up, op, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2 != 0:
        raise ShapeError(op, f"gate_up has an odd number of columns: {two_i}")
    if out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous {gate_up.dtype} [{T}, {two_i // 2}], got {out.dtype} {list(out.shape)}")
    f = _fn("elementwise", "vob_swiglu", [_P, _L, _P, _I, _I, _I, _P])
    _check(f(_ptr(gate_up), gate_up.stride(0), _ptr(out), _code(out, op), T, two_i // 2, _stream()), op)


GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


@_timed
def glu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[t, j] = act(gate_up[t, j]) * gate_up[t, I + j]; act is "silu" or "gelu_tanh" (the tanh form of gelu)."""
    op = "glu"
    _cuda(op, gate_up, out)
    _rows_2d(gate_up, op, "gate_up")
    T, two_i = gate_up.shape
    if activation not in GLU_ACTIVATIONS:
        raise ShapeError(op, f"activation {activation!r} is not known ({', '.join(GLU_ACTIVATIONS)})")
    if two_i % 2 != 0:
        raise ShapeError(op, f"gate_up has an odd number of columns: {two_i}")
    if out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous {gate_up.dtype} [{T}, {two_i // 2}], got {out.dtype} {list(out.shape)}")
    f = _fn("elementwise", "vob_glu", [_P, _L, _P, _I, _I, _I, _I, _P])
    _check(f(_ptr(gate_up), gate_up.stride(0), _ptr(out), _code(out, op), T, two_i // 2, GLU_ACTIVATIONS[activation], _stream()), op)


# ------------------------------------------------------------------------------------ matrix products
@_timed
def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias[N]) in true float32 (FMA chains in k order; no tensor cores)."""
    op = "gemm_f32"
    _cuda(op, a, w, out, bias)
    for name, t in (("a", a), ("w", w), ("out", out)):
        _rows_2d(t, op, name)
        if t.dtype != torch.float32:
            raise ShapeError(op, f"{name} must be float32, got {t.dtype}")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ShapeError(op, f"a has {K} columns, w has {w.shape[1]}")
    if out.shape != (M, N):
        raise ShapeError(op, f"out must be [{M}, {N}], got {list(out.shape)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (N,) or not bias.is_contiguous()):
        raise ShapeError(op, f"bias must be contiguous float32 [{N}], got {bias.dtype} {list(bias.shape)}")
    f = _fn("gemm_f32", "vob_gemm_f32", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K, _ptr(bias), _stream()), op)


class _GemmScratch:
    """Per device: the error word that a timed-out wait inside the tensor-core product raises."""

    def __init__(self, device):
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count


_gemm_scratch = {}


def _scratch_for(device) -> _GemmScratch:
    s = _gemm_scratch.get(device)
    if s is None:
        s = _gemm_scratch[device] = _GemmScratch(device)
    return s


def gemm_sm100_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes these operands: bfloat16, K a multiple of 8, 16-byte
    aligned rows (what TMA asks for)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


@_timed
def gemm_sm100(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None) -> None:
    """out[T, N] = a[T, K] @ w[N, K]^T on the tcgen05 tensor cores: bfloat16 operands fetched by
    TMA, float32 accumulation in tensor memory, bfloat16 or float32 out. `splits` > 1 (at most 8) splits K over
    the blocks of a cluster (for few tokens); None picks it from the sizes."""
    op = "gemm_sm100"
    _cuda(op, a, w, out)
    if not gemm_sm100_supported(a, w):
        raise ShapeError(op, f"operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows, got "
                             f"{a.dtype} {list(a.shape)} strides {list(a.stride())} and {w.dtype} {list(w.shape)}")
    T, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N) or out.stride(1) != 1:
        raise ShapeError(op, f"shapes do not fit: a {list(a.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ShapeError(op, f"out must be bfloat16 or float32, got {out.dtype}")
    sc = _scratch_for(a.device)
    if splits is None:
        f = _fn("gemm_sm100", "vob_gemm_sm100_pick_splits", [_I, _I, _I, _I])
        splits = int(f(T, N, K, sc.num_sms))
    f = _fn("gemm_sm100", "vob_gemm_sm100", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _code(out, op), T, N, K, int(splits),
             _ptr(sc.err), _stream()), op)


@_timed
def gemm_sm100_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, N] = a[T, K] @ w[N, K]^T for many rows, on pairs of SMs: tcgen05.mma with cta_group::2
    (256 weight rows x 256 tokens per instruction, operands split over the two blocks' shared
    memory), persistent over output tiles, accumulators double buffered in tensor memory. bfloat16
    operands, bfloat16 or float32 out."""
    op = "gemm_sm100_pair"
    _cuda(op, a, w, out)
    if not gemm_sm100_supported(a, w):
        raise ShapeError(op, f"operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows, got "
                             f"{a.dtype} {list(a.shape)} strides {list(a.stride())} and {w.dtype} {list(w.shape)}")
    T, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N) or out.stride(1) != 1:
        raise ShapeError(op, f"shapes do not fit: a {list(a.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ShapeError(op, f"out must be bfloat16 or float32, got {out.dtype}")
    f = _fn("gemm_sm100_pair", "vob_gemm_sm100_pair", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _code(out, op), T, N, K,
             _ptr(_scratch_for(a.device).err), _stream()), op)


@_timed
def gemm_pair_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[T, I] = act(a @ Wg^T) * (a @ Wu^T) with w_gate_up = [Wg; Wu] ([2I, K], bfloat16) for many rows:
    the two-SM tcgen05 product whose epilogue applies the activation (gate and up never go to memory);
    act is "silu" or "gelu_tanh"."""
    op = "gemm_pair_swiglu"
    if activation not in GLU_ACTIVATIONS:
        raise ShapeError(op, f"activation {activation!r} is not known ({', '.join(GLU_ACTIVATIONS)})")
    _cuda(op, a, w_gate_up, out)
    if not gemm_sm100_supported(a, w_gate_up):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    if w_gate_up.shape[0] % 2 != 0 or w_gate_up.shape[1] != K:
        raise ShapeError(op, f"w_gate_up must be [2I, {K}], got {list(w_gate_up.shape)}")
    I = w_gate_up.shape[0] // 2
    if out.shape != (T, I) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ShapeError(op, f"out must be bfloat16 [{T}, {I}], got {out.dtype} {list(out.shape)}")
    f = _fn("gemm_sm100_pair", "vob_gemm_sm100_pair_glu", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w_gate_up), w_gate_up.stride(0), _ptr(out), out.stride(0), T, I, K,
             GLU_ACTIVATIONS[activation], _ptr(_scratch_for(a.device).err), _stream()), op)


def _pick_splits(T: int, N: int, K: int, device) -> int:
    f = _fn("gemm_sm100", "vob_gemm_sm100_pick_splits", [_I, _I, _I, _I])
    return int(f(T, N, K, _scratch_for(device).num_sms))


FUSED_GEMM_MAX_ROWS = 64      # what the fused kernels take


@_timed
def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None,
                activation: str = "silu") -> None:
    """out[T, I] = act(a @ Wg^T) * (a @ Wu^T) with w_gate_up = [Wg; Wu] ([2I, K], bfloat16): one tcgen05
    kernel with two accumulators whose epilogue applies the activation ("silu" or "gelu_tanh"), for at most 64 rows."""
    op = "gemm_swiglu"
    if activation not in GLU_ACTIVATIONS:
        raise ShapeError(op, f"activation {activation!r} is not known ({', '.join(GLU_ACTIVATIONS)})")
    _cuda(op, a, w_gate_up, out)
    if not gemm_sm100_supported(a, w_gate_up):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    if w_gate_up.shape[0] % 2 != 0 or w_gate_up.shape[1] != K:
        raise ShapeError(op, f"w_gate_up must be [2I, {K}], got {list(w_gate_up.shape)}")
    I = w_gate_up.shape[0] // 2
    if T > FUSED_GEMM_MAX_ROWS:
        raise ShapeError(op, f"{T} rows: the fused kernel takes at most {FUSED_GEMM_MAX_ROWS}")
    if out.shape != (T, I) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ShapeError(op, f"out must be bfloat16 [{T}, {I}], got {out.dtype} {list(out.shape)}")
    if splits is None:
        splits = _pick_splits(T, 2 * I, K, a.device)
    f = _fn("gemm_sm100", "vob_gemm_sm100_glu", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w_gate_up), w_gate_up.stride(0), _ptr(out), out.stride(0), T, I, K, int(splits),
             GLU_ACTIVATIONS[activation], _ptr(_scratch_for(a.device).err), _stream()), op)


def gemm_qkv_rope_supported(head_dim: int) -> bool:
    return head_dim > 0 and head_dim % 2 == 0 and 128 % head_dim == 0


@_timed
def gemm_qkv_rope(a: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                  slots: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], kcache: torch.Tensor, vcache: torch.Tensor,
                  num_heads: int, num_kv_heads: int, head_dim: int, splits: Optional[int] = None) -> None:
    """[q | k | v] = a @ [Wq; Wk; Wv]^T in one tcgen05 kernel whose epilogue rotates q and k (float32
    angles position * inv_freq), writes q to q_out [T, H*hd] and the rotated k and v straight to their
    cache slots. At most 64 rows; 128 must be a multiple of head_dim."""
    op = "gemm_qkv_rope"
    _cuda(op, a, w_qkv, q_out, positions, slots, inv_freq, kcache, vcache)
    if not gemm_sm100_supported(a, w_qkv):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    H, KV, hd = num_heads, num_kv_heads, head_dim
    if not gemm_qkv_rope_supported(hd):
        raise ShapeError(op, f"head_dim {hd}: 128 must be a multiple of it")
    if w_qkv.shape != ((H + 2 * KV) * hd, K):
        raise ShapeError(op, f"w_qkv must be [{(H + 2 * KV) * hd}, {K}], got {list(w_qkv.shape)}")
    if T > FUSED_GEMM_MAX_ROWS:
        raise ShapeError(op, f"{T} rows: the fused kernel takes at most {FUSED_GEMM_MAX_ROWS}")
    if q_out.shape != (T, H * hd) or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1:
        raise ShapeError(op, f"q_out must be bfloat16 [{T}, {H * hd}], got {q_out.dtype} {list(q_out.shape)}")
    _int32_vec(positions, T, op, "positions")
    if slots is not None:
        _int32_vec(slots, T, op, "slots")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (hd // 2,) or not inv_freq.is_contiguous()):
        raise ShapeError(op, f"inv_freq must be float32 [{hd // 2}]")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != KV or c.shape[3] != hd or not c.is_contiguous() or c.dtype != torch.bfloat16:
            raise ShapeError(op, f"{name} must be contiguous bfloat16 [pages, {KV}, page_size, {hd}], got {c.dtype} {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if splits is None:
        splits = _pick_splits(T, (H + 2 * KV) * hd, K, a.device)
    f = _fn("gemm_sm100", "vob_gemm_sm100_qkv",
            [_P, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w_qkv), w_qkv.stride(0), _ptr(q_out), q_out.stride(0), T, K, int(splits),
             _ptr(_scratch_for(a.device).err), _ptr(positions), _ptr(slots), _ptr(inv_freq), _ptr(kcache), _ptr(vcache),
             H, KV, hd, kcache.shape[2], _stream()), op)


# ------------------------------------------------------------------------------------ folded norms (few rows)
EPI_STORE, EPI_SWIGLU, EPI_QKV, EPI_RESID, EPI_PICK = 0, 1, 2, 3, 4


class _EpiArgs(ctypes.Structure):
    """Mirror of `EpiArgs` in csrc/gemm_sm100.cu."""
    _fields_ = [("positions", _P), ("slots", _P), ("inv_freq", _P), ("kcache", _P), ("vcache", _P),
                ("ssq_in", _P), ("resid", _P), ("next_w", _P), ("xn_out", _P), ("ssq_out", _P),
                ("ld_resid", _L), ("ld_xn", _L),
                ("q_dim", _I), ("kv_dim", _I), ("hd", _I), ("KV", _I), ("page_size", _I),
                ("ssq_tiles", _I), ("ld_ssq", _I), ("inv_h", _F), ("eps", _F), ("act", _I),
                ("temperature", _P), ("seeds", _P), ("steps", _P), ("part_val", _P), ("part_idx", _P), ("nan_flags", _P),
                ("ld_part", _L)]


def _dp(t: Optional[torch.Tensor]) -> int:
    return t.data_ptr() if t is not None else 0


@_timed
def embed_fold(table: torch.Tensor, tokens: torch.Tensor, resid: torch.Tensor, next_w: torch.Tensor, xn: torch.Tensor,
               ssq: torch.Tensor, err_flag: Optional[torch.Tensor] = None) -> None:
    """resid[t] = table[tokens[t]] (float32), xn[t] = bf16(resid * next_w), ssq[tile, t] = sum of squares of
    resid over features 128*tile .. +127: the embedding with the first norm's input prepared."""
    op = "embed_fold"
    _cuda(op, table, tokens, resid, next_w, xn, ssq, err_flag)
    T, h = resid.shape
    if table.dim() != 2 or table.shape[1] != h or not table.is_contiguous():
        raise ShapeError(op, f"table must be contiguous [vocab, {h}], got {list(table.shape)}")
    _int32_vec(tokens, T, op, "tokens")
    if resid.dtype != torch.float32 or not resid.is_contiguous() or xn.dtype != torch.bfloat16 or xn.shape != resid.shape or not xn.is_contiguous():
        raise ShapeError(op, "resid must be contiguous float32 [T, h] and xn contiguous bfloat16 of the same shape")
    if next_w.dtype != torch.float32 or next_w.shape != (h,) or not next_w.is_contiguous():
        raise ShapeError(op, f"next_w must be float32 [{h}]")
    tiles = -(-h // 128)
    if ssq.dtype != torch.float32 or ssq.dim() != 2 or ssq.shape[0] < tiles or ssq.shape[1] < T or not ssq.is_contiguous():
        raise ShapeError(op, f"ssq must be contiguous float32 [>={tiles}, >={T}], got {list(ssq.shape)}")
    f = _fn("elementwise", "vob_embed_fold", [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(table), _code(table, op), _ptr(tokens), _ptr(resid), _ptr(next_w), _ptr(xn), _ptr(ssq), ssq.shape[1], T, h,
             table.shape[0], _ptr(err_flag), _stream()), op)


@_timed
def gemm_fused(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], mode: int, n_features: int, *,
               ssq_in: Optional[torch.Tensor] = None, eps: float = 0.0, qkv=None, resid=None, pick=None,
               splits: Optional[int] = None) -> None:
    """The tcgen05 product for at most 64 rows with a fused epilogue and, optionally, the RMSNorm of
    its input folded in: `a` holds bf16(x * norm weight), `ssq_in` [tiles, ld] the per-tile sums of
    squares of x, and each token's accumulator is multiplied by 1 / sqrt(mean(x^2) + eps).
      EPI_STORE  out[T, n] (bfloat16 or float32) = result
      EPI_SWIGLU out[T, n] = silu(gate) * up, w = [Wg; Wu] of shape [2n, K]
      EPI_QKV    qkv = (positions, slots, inv_freq, kcache, vcache, H, KV, hd): out[T, H*hd] = rotated q,
                 rotated k and v go to their cache slots
      EPI_RESID  resid = (resid float32 [T, n] updated in place, next_w float32 [n], xn_out bfloat16 [T, n],
                 ssq_out float32 [tiles(n), ld]); out is None
      EPI_PICK   the output head when only the picked tokens are wanted: pick = (temperature float32 [T] or None,
                 seeds int32 [T, 2], steps int32 [T], part_val float32 [T, ld], part_idx int32 [T, ld],
                 nan_flags int32 [T]), ld >= pick_tiles(n): every block leaves the best (value, index) pair of
                 its 128 logits per token (the rule of `pick_tokens`); `pick_final` finishes; out is None"""
    op = "gemm_fused"
    _cuda(op, a, w, out, ssq_in)
    if not gemm_sm100_supported(a, w):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    if T > FUSED_GEMM_MAX_ROWS:
        raise ShapeError(op, f"{T} rows: the fused kernel takes at most {FUSED_GEMM_MAX_ROWS}")
    w_rows = 2 * n_features if mode == EPI_SWIGLU else n_features
    if w.shape != (w_rows, K):
        raise ShapeError(op, f"w must be [{w_rows}, {K}], got {list(w.shape)}")
    ea = _EpiArgs()
    if ssq_in is not None:
        if ssq_in.dtype != torch.float32 or ssq_in.dim() != 2 or ssq_in.shape[0] != -(-K // 128) or ssq_in.shape[1] < T or not ssq_in.is_contiguous():
            raise ShapeError(op, f"ssq_in must be contiguous float32 [{-(-K // 128)}, >={T}], got {list(ssq_in.shape)}")
        ea.ssq_in, ea.ssq_tiles, ea.ld_ssq, ea.inv_h, ea.eps = _dp(ssq_in), ssq_in.shape[0], ssq_in.shape[1], 1.0 / K, float(eps)
    out_code, ldc, out_ptr = 1, n_features, 0
    if mode in (EPI_STORE, EPI_SWIGLU):
        if out is None or out.shape != (T, n_features) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
            raise ShapeError(op, f"out must be [{T}, {n_features}] bfloat16 or float32")
        if mode == EPI_SWIGLU and out.dtype != torch.bfloat16:
            raise ShapeError(op, "the SwiGLU epilogue writes bfloat16")
        out_code, ldc, out_ptr = _code(out, op), out.stride(0), out.data_ptr()
    elif mode == EPI_QKV:
        positions, slots, inv_freq, kcache, vcache, H, KV, hd = qkv
        _cuda(op, positions, slots, inv_freq, kcache, vcache)
        if not gemm_qkv_rope_supported(hd) or n_features != (H + 2 * KV) * hd:
            raise ShapeError(op, f"qkv sizes do not fit: heads {H}/{KV}, head_dim {hd}, features {n_features}")
        if out is None or out.shape != (T, H * hd) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise ShapeError(op, f"out must be bfloat16 [{T}, {H * hd}]")
        _int32_vec(positions, T, op, "positions")
        if slots is not None:
            _int32_vec(slots, T, op, "slots")
        for name, c in (("kcache", kcache), ("vcache", vcache)):
            if c.dim() != 4 or c.shape[1] != KV or c.shape[3] != hd or not c.is_contiguous() or c.dtype != torch.bfloat16:
                raise ShapeError(op, f"{name} must be contiguous bfloat16 [pages, {KV}, page_size, {hd}]")
        if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (hd // 2,)):
            raise ShapeError(op, f"inv_freq must be float32 [{hd // 2}]")
        ea.positions, ea.slots, ea.inv_freq, ea.kcache, ea.vcache = _dp(positions), _dp(slots), _dp(inv_freq), _dp(kcache), _dp(vcache)
        ea.q_dim, ea.kv_dim, ea.hd, ea.KV, ea.page_size = H * hd, KV * hd, hd, KV, kcache.shape[2]
        ldc, out_ptr = out.stride(0), out.data_ptr()
    elif mode == EPI_RESID:
        r, next_w, xn_out, ssq_out = resid
        _cuda(op, r, next_w, xn_out, ssq_out)
        tiles = -(-n_features // 128)
        if r.dtype != torch.float32 or r.shape != (T, n_features) or r.stride(1) != 1:
            raise ShapeError(op, f"resid must be float32 [{T}, {n_features}]")
        if xn_out.dtype != torch.bfloat16 or xn_out.shape != (T, n_features) or xn_out.stride(1) != 1:
            raise ShapeError(op, f"xn_out must be bfloat16 [{T}, {n_features}]")
        if next_w.dtype != torch.float32 or next_w.shape != (n_features,) or not next_w.is_contiguous():
            raise ShapeError(op, f"next_w must be float32 [{n_features}]")
        if ssq_out.dtype != torch.float32 or ssq_out.dim() != 2 or ssq_out.shape[0] < tiles or ssq_out.shape[1] < T or not ssq_out.is_contiguous():
            raise ShapeError(op, f"ssq_out must be contiguous float32 [>={tiles}, >={T}]")
        ea.resid, ea.next_w, ea.xn_out, ea.ssq_out = _dp(r), _dp(next_w), _dp(xn_out), _dp(ssq_out)
        ea.ld_resid, ea.ld_xn = r.stride(0), xn_out.stride(0)
        if ea.ld_ssq == 0:
            ea.ld_ssq = ssq_out.shape[1]
        elif ea.ld_ssq != ssq_out.shape[1]:
            raise ShapeError(op, "ssq_in and ssq_out must have the same row length")
    elif mode == EPI_PICK:
        temperature, seeds, steps, part_val, part_idx, nan_flags = pick
        _cuda(op, temperature, seeds, steps, part_val, part_idx, nan_flags)
        tiles = pick_tiles(n_features)
        for name, t_, dt in (("part_val", part_val, torch.float32), ("part_idx", part_idx, torch.int32)):
            if t_.dtype != dt or t_.dim() != 2 or t_.shape[0] < T or t_.shape[1] < tiles or not t_.is_contiguous():
                raise ShapeError(op, f"{name} must be contiguous {dt} [>={T}, >={tiles}], got {t_.dtype} {list(t_.shape)}")
        if part_val.shape[1] != part_idx.shape[1]:
            raise ShapeError(op, "part_val and part_idx must have the same row length")
        _int32_vec(nan_flags, T, op, "nan_flags")
        if temperature is not None:
            if temperature.dtype != torch.float32 or temperature.numel() < T or not temperature.is_contiguous():
                raise ShapeError(op, f"temperature must be float32 [{T}]")
            if seeds is None or steps is None or seeds.dtype != torch.int32 or seeds.numel() < 2 * T or not seeds.is_contiguous():
                raise ShapeError(op, f"temperature sampling needs seeds int32 [{T}, 2] and steps")
            _int32_vec(steps, T, op, "steps")
        ea.temperature, ea.seeds, ea.steps = _dp(temperature), _dp(seeds), _dp(steps)
        ea.part_val, ea.part_idx, ea.nan_flags, ea.ld_part = _dp(part_val), _dp(part_idx), _dp(nan_flags), part_val.shape[1]
        out_code = 0
        splits = 1
    else:
        raise ShapeError(op, f"unknown epilogue mode {mode}")
    if splits is None:
        splits = _pick_splits(T, w_rows, K, a.device)
    f = _fn("gemm_sm100", "vob_gemm_sm100_ex", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, ctypes.POINTER(_EpiArgs), _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _P(out_ptr), ldc, out_code, T, n_features, K, int(splits), int(mode),
             ctypes.byref(ea), _ptr(_scratch_for(a.device).err), _stream()), op)


def gemm_sm100_test_hooks(extra_tx_bytes: int = 0, wait_limit_ms: float = 0.0) -> None:
    """For the test of the kernels' give-up path only: the next one-block launches of the few-token
    product expect `extra_tx_bytes` more than their loads bring (their waits then run out), and
    waits give up after `wait_limit_ms` (0: the default of two seconds). (0, 0) restores both."""
    f = _fn("gemm_sm100", "vob_gemm_sm100_test_hooks", [_I, ctypes.c_ulonglong])
    _check(f(int(extra_tx_bytes), int(wait_limit_ms * 1e6)), "gemm_sm100_test_hooks", launches=0)


def gemm_sm100_check() -> None:
    """Raise if a bounded wait inside a tcgen05 kernel (matrix product or attention) ever expired
    (reads one word from the device)."""
    for dev, sc in _gemm_scratch.items():
        code = int(sc.err.item())
        if code:
            sc.err.zero_()
            raise KernelError(f"a bounded wait expired inside a tensor-core kernel (code {code}: 1-4 = matrix product: TMA "
                              "producer, MMA issuer, epilogue, peers of a split; 11-21 = attention: 11-12 TMA producer, 13-17 MMA issuer, "
                              "18-21 softmax rows); its result is not valid")


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out = a @ w^T (+ bias, a vector of the operands' type: added to the float32 sum before the result is
    rounded; with a bias the bfloat16 product is the library's, whose epilogue adds it). float32 operands: the true 32-bit kernel. bfloat16 operands: this package's
    tcgen05 kernel (TMA operands, float32 accumulation in tensor memory); for many rows, or
    operands TMA cannot address (K not a multiple of 8, unaligned rows), the library product
    (cuBLAS through torch, float32 accumulation; above `TUNING.few_rows` rows), as the reference plans for its own matrix
    products (CLAUDE.md:107). `out` may be bfloat16 or float32."""
    op = "linear"
    if a.dtype == torch.float32:
        gemm_f32(a, w, out, bias)
        return
    _cuda(op, a, w, out, bias)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ShapeError(op, f"operands must both be float32 or both bfloat16, got {a.dtype} and {w.dtype}")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or out.shape != (a.shape[0], w.shape[0]):
        raise ShapeError(op, f"shapes do not fit: a {list(a.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ShapeError(op, f"out must be bfloat16 or float32, got {out.dtype}")
    if bias is not None:
        if bias.dtype != torch.bfloat16 or bias.shape != (w.shape[0],) or out.dtype != torch.bfloat16:
            raise ShapeError(op, f"a bias must be bfloat16 [{w.shape[0]}] with a bfloat16 result, got {bias.dtype} {list(bias.shape)}")
        _library_gemm_bf16(a, w, out, bias)
    elif a.shape[0] <= TUNING.few_rows and gemm_sm100_supported(a, w):
        gemm_sm100(a, w, out)
    else:
        _library_gemm_bf16(a, w, out)


@_timed
def _library_gemm_bf16(a, w, out, bias=None):
    if bias is not None:
        torch.addmm(bias, a, w.t(), out=out)
    elif out.dtype == torch.bfloat16:
        torch.mm(a, w.t(), out=out)
    else:
        torch.mm(a, w.t(), out_dtype=torch.float32, out=out)


# ------------------------------------------------------------------------------------ residual in streams
def _f32_vec(t: Optional[torch.Tensor], n: int, op: str, name: str) -> None:
    if t is None:
        return
    if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
        raise ShapeError(op, f"{name} must be contiguous float32 with {n} elements, got {t.dtype} {list(t.shape)}")


@_timed
def stream_norm(streams: torch.Tensor, y: Optional[torch.Tensor], mix: Optional[torch.Tensor], out_coef: Optional[torch.Tensor],
                in_coef: Optional[torch.Tensor], weight: torch.Tensor, groups: int, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
    """The read of a residual kept as S streams, with the write that was still pending done first and
    an RMS norm in `groups` groups behind it. streams float32 [T, S, W]. With `y` [T, W]: every stream
    t becomes sum_s mix[s, t] * stream s + out_coef[t] * y (stored, unless `rows` is given: then the
    rows are only looked at). Then u = sum_s in_coef[s] * stream s (all ones if None), each of the
    `groups` consecutive parts of u divided by sqrt(mean(part^2) + eps), times weight.
    out [R, copies, W] (or [R, W]) receives the result, `copies` times side by side."""
    op = "stream_norm"
    _cuda(op, streams, y, mix, out_coef, in_coef, weight, out, rows)
    if streams.dtype != torch.float32 or streams.dim() != 3 or not streams.is_contiguous():
        raise ShapeError(op, f"streams must be contiguous float32 [T, S, W], got {streams.dtype} {list(streams.shape)}")
    T, S, W = streams.shape
    if groups < 1 or W % groups != 0:
        raise ShapeError(op, f"a width of {W} cannot be cut into {groups} equal groups")
    if S > 8:
        raise ShapeError(op, f"{S} streams: at most 8 are supported")
    _f32_vec(weight, W, op, "weight")
    _f32_vec(in_coef, S, op, "in_coef")
    if y is not None:
        if mix is None or out_coef is None:
            raise ShapeError(op, "a pending write needs its mix and out coefficients")
        _f32_vec(mix, S * S, op, "mix")
        _f32_vec(out_coef, S, op, "out_coef")
        if y.shape != (T, W) or not y.is_contiguous():
            raise ShapeError(op, f"y must be contiguous [{T}, {W}], got {list(y.shape)}")
    R = T
    if rows is not None:
        R = rows.numel()
        _int32_vec(rows, R, op, "rows")
    if not out.is_contiguous() or out.numel() % (R * W) != 0 or out.shape[0] != R or out.numel() == 0 and R:
        raise ShapeError(op, f"out must be contiguous [{R}, copies, {W}], got {list(out.shape)}")
    copies = out.numel() // (R * W) if R else 1
    f = _fn("streams", "vob_stream_norm", [_P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P])
    _check(f(_ptr(streams), _ptr(y), _code(y, op) if y is not None else 0, _ptr(mix), _ptr(out_coef), _ptr(in_coef), _ptr(weight),
             _ptr(rows), _ptr(out), _code(out, op), R, S, W, int(groups), float(eps), copies, _stream()), op)


# ------------------------------------------------------------------------------------ linear recurrences
@_timed
def delta_prep(proj: torch.Tensor, k_off: int, a_off: int, low_off: int, rank: int, w2t: torch.Tensor, w0: torch.Tensor,
               a_bias: torch.Tensor, heads: int, dim: int, w_out: torch.Tensor, b_out: torch.Tensor, u_out: torch.Tensor) -> None:
    """What the delta-rule recurrence reads besides r, k, v, per token, head and key channel, all float32
    [T, heads * dim]: u = k / sqrt(sum k^2 + 1e-6) per head; b = sigmoid(a + a_bias) * u;
    w = exp(-exp(-1/2) * sigmoid(w0 + w2 tanh(low))). k, a and low (width `rank`) are the columns
    k_off.., a_off.., low_off.. of `proj` [T, ld]; `w2t` is w2 transposed, [rank, heads * dim]."""
    op = "delta_prep"
    _cuda(op, proj, w2t, w0, a_bias, w_out, b_out, u_out)
    _rows_2d(proj, op, "proj")
    T, hd = proj.shape[0], heads * dim
    if w2t.shape != (rank, hd) or not w2t.is_contiguous() or w2t.dtype != proj.dtype:
        raise ShapeError(op, f"w2t must be contiguous {proj.dtype} [{rank}, {hd}], got {w2t.dtype} {list(w2t.shape)}")
    _f32_vec(w0, hd, op, "w0")
    _f32_vec(a_bias, hd, op, "a_bias")
    for name, t in (("w_out", w_out), ("b_out", b_out), ("u_out", u_out)):
        if t.dtype != torch.float32 or t.shape != (T, hd) or not t.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous float32 [{T}, {hd}], got {t.dtype} {list(t.shape)}")
    for off, n in ((k_off, hd), (a_off, hd), (low_off, rank)):
        if off < 0 or off + n > proj.shape[1]:
            raise ShapeError(op, f"columns {off}..{off + n} lie outside proj's {proj.shape[1]}")
    f = _fn("recurrence", "vob_delta_prep", [_P, _I, _L, _I, _I, _I, _I, _P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _P])
    _check(f(_ptr(proj), _code(proj, op), proj.stride(0), k_off, a_off, low_off, rank, _ptr(w2t), _code(w2t, op), _ptr(w0), _ptr(a_bias),
             T, heads, dim, _ptr(w_out), _ptr(b_out), _ptr(u_out), _stream()), op)


@_timed
def rotate_scale(src: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, heads: int, dim: int, rot: int, scale: float,
                 out: torch.Tensor) -> None:
    """out float32 [T, heads * dim] = scale * (src with the first `rot` features of every head rotated by
    position * inv_freq, feature i paired with i + rot / 2). src: [T, heads * dim] with any row stride."""
    op = "rotate_scale"
    _cuda(op, src, positions, inv_freq, out)
    _rows_2d(src, op, "src")
    T = src.shape[0]
    if src.shape[1] != heads * dim or out.shape != (T, heads * dim) or out.dtype != torch.float32 or not out.is_contiguous():
        raise ShapeError(op, f"src [{T}, {heads * dim}] and a contiguous float32 out of the same shape are needed, got "
                             f"{list(src.shape)} and {out.dtype} {list(out.shape)}")
    if rot % 2 or rot > dim or rot < 0:
        raise ShapeError(op, f"{rot} rotated features do not fit a head of {dim}")
    _int32_vec(positions, T, op, "positions")
    _f32_vec(inv_freq, rot // 2, op, "inv_freq")
    f = _fn("recurrence", "vob_rotate_scale", [_P, _I, _L, _P, _P, _I, _I, _I, _I, _F, _P, _P])
    _check(f(_ptr(src), _code(src, op), src.stride(0), _ptr(positions), _ptr(inv_freq), T, heads, dim, rot, float(scale), _ptr(out),
             _stream()), op)


@_timed
def recurrence_scan(mode: int, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor],
                    u: Optional[torch.Tensor], state: torch.Tensor, seq_starts: torch.Tensor, state_slots: torch.Tensor,
                    num_seqs: int, heads: int, out: torch.Tensor, rk_heads: Optional[int] = None, conv_x: Optional[torch.Tensor] = None,
                    conv_state: Optional[torch.Tensor] = None) -> None:
    """The recurrence over each request's rows of this step, from and to its state slot.
    mode 0: S = diag(w_t) S - b_t (u_t^T S) + k_t v_t^T with w, b, u float32 [T, heads * K];
    mode 1: S = w[h] S + k_t v_t^T with w float32 [heads];
    mode 2: S' = diag(w_t) S; S = S' + k_t (b_t (v_t - S'^T k_t))^T with w float32 [T, heads * K], b float32
    [T, heads], and r, k float32 [T, rk_heads * K] (head h reads r and k of head h // (heads / rk_heads));
    mode 3: S = b_t S + k_t (u_t v_t)^T with b (a decay) and u (a step size) float32 [T, heads], r, k, v float32, heads
    sharing r and k as in mode 2.
    o_t = S^T r_t -> out float32 [T, heads * V].
    state float32 [slots, heads, K, V]; r, k [T, heads * K] and v [T, heads * V] with any row stride.
    Mode 2 with `conv_x` ([T, C] of v's type, any row stride) and `conv_state` (float32 [slots, taps - 1, C]) also does
    what `conv_state_update` does, on its way."""
    op = "recurrence_scan"
    _cuda(op, r, k, v, w, b, u, state, seq_starts, state_slots, out)
    for name, t in (("r", r), ("k", k), ("v", v)):
        _rows_2d(t, op, name)
    if state.dtype != torch.float32 or state.dim() != 4 or not state.is_contiguous() or state.shape[1] != heads:
        raise ShapeError(op, f"state must be contiguous float32 [slots, {heads}, K, V], got {state.dtype} {list(state.shape)}")
    K, V = state.shape[2], state.shape[3]
    T = r.shape[0]
    rk_heads = heads if rk_heads is None else int(rk_heads)
    if rk_heads <= 0 or heads % rk_heads != 0 or (mode not in (2, 3) and rk_heads != heads):
        raise ShapeError(op, f"{heads} heads cannot share the r and k of {rk_heads} heads in mode {mode}")
    if r.shape != (T, rk_heads * K) or k.shape != (T, rk_heads * K) or v.shape != (T, heads * V) or r.dtype != k.dtype:
        raise ShapeError(op, f"r, k [{T}, {rk_heads * K}] and v [{T}, {heads * V}] are needed, got {list(r.shape)}, {list(k.shape)}, {list(v.shape)}")
    if out.shape != (T, heads * V) or out.dtype != torch.float32 or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous float32 [{T}, {heads * V}], got {out.dtype} {list(out.shape)}")
    if mode == 0:
        for name, t in (("w", w), ("b", b), ("u", u)):
            if t is None or t.dtype != torch.float32 or t.shape != (T, heads * K) or not t.is_contiguous():
                raise ShapeError(op, f"{name} must be contiguous float32 [{T}, {heads * K}]")
    elif mode == 1:
        _f32_vec(w, heads, op, "w")
    elif mode == 2:
        if r.dtype != torch.float32:
            raise ShapeError(op, f"mode 2 takes float32 r and k, got {r.dtype}")
        if w is None or w.dtype != torch.float32 or w.shape != (T, heads * K) or not w.is_contiguous():
            raise ShapeError(op, f"w must be contiguous float32 [{T}, {heads * K}]")
        if b is None or b.dtype != torch.float32 or b.shape != (T, heads) or not b.is_contiguous():
            raise ShapeError(op, f"b must be contiguous float32 [{T}, {heads}]")
    elif mode == 3:
        if r.dtype != torch.float32 or v.dtype != torch.float32:
            raise ShapeError(op, f"mode 3 takes float32 r, k and v, got {r.dtype} and {v.dtype}")
        for name, t in (("b", b), ("u", u)):
            if t is None or t.dtype != torch.float32 or t.shape != (T, heads) or not t.is_contiguous():
                raise ShapeError(op, f"{name} must be contiguous float32 [{T}, {heads}]")
    else:
        raise ShapeError(op, f"mode {mode} is not known")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(state_slots, num_seqs, op, "state_slots")
    conv_c = conv_taps = 0
    if conv_x is not None:
        _cuda(op, conv_x, conv_state)
        _rows_2d(conv_x, op, "conv_x")
        if (mode != 2 or conv_state is None or conv_state.dtype != torch.float32 or conv_state.dim() != 3 or not conv_state.is_contiguous()
                or conv_state.shape[1] < 1 or conv_x.shape != (T, conv_state.shape[2]) or conv_x.dtype != v.dtype):
            raise ShapeError(op, "conv_x [T, C] of v's type goes with mode 2 and a contiguous float32 conv_state [slots, taps - 1, C]")
        conv_c, conv_taps = conv_state.shape[2], conv_state.shape[1] + 1
    f = _fn("recurrence", "vob_recurrence_scan", [_I, _P, _L, _P, _L, _I, _P, _L, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                                                  _P, _L, _I, _I, _P, _P])
    _check(f(mode, _ptr(r), r.stride(0), _ptr(k), k.stride(0), _code(r, op), _ptr(v), v.stride(0), _code(v, op), _ptr(w), _ptr(b), _ptr(u),
             _ptr(state), _ptr(seq_starts), _ptr(state_slots), _ptr(out), num_seqs, heads, K, V, heads // rk_heads,
             _ptr(conv_x), conv_x.stride(0) if conv_x is not None else 0, conv_c, conv_taps,
             _ptr(conv_state) if conv_x is not None else _P(0), _stream()), op)


@_timed
def recurrence_post(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], gate_mode: str, eps: float, heads: int,
                    out: torch.Tensor, out_scale: float = 1.0) -> None:
    """out = o / sqrt(mean_head(o^2) + eps) * weight * act(gate) * out_scale, head by head; act is "sigmoid" or "silu".
    o float32 [T, heads * V]; gate and out [T, heads * V] (any row stride) in the activations' type."""
    op = "recurrence_post"
    _cuda(op, o, gate, weight, out)
    _rows_2d(gate, op, "gate")
    _rows_2d(out, op, "out")
    T, hv = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or hv % heads != 0:
        raise ShapeError(op, f"o must be contiguous float32 [T, heads * V], got {o.dtype} {list(o.shape)}")
    if gate.shape != (T, hv) or out.shape != (T, hv) or out.dtype != gate.dtype:
        raise ShapeError(op, f"gate and out must be [{T}, {hv}] of one type, got {list(gate.shape)} and {list(out.shape)}")
    _f32_vec(weight, hv, op, "weight")
    if gate_mode not in ("sigmoid", "silu"):
        raise ShapeError(op, f"gate {gate_mode!r} is not known (sigmoid or silu)")
    f = _fn("recurrence", "vob_recurrence_post", [_P, _P, _I, _L, _P, _I, _F, _I, _I, _I, _P, _L, _F, _P])
    _check(f(_ptr(o), _ptr(gate), _code(gate, op), gate.stride(0), _ptr(weight), 1 if gate_mode == "silu" else 0, float(eps), T, heads,
             hv // heads, _ptr(out), out.stride(0), float(out_scale), _stream()), op)


@_timed
def gated_delta_prep(proj: torch.Tensor, x_off: int, b_off: int, low: torch.Tensor, a_off: int, conv_w: torch.Tensor,
                     conv_state: Optional[torch.Tensor], a_log: torch.Tensor, dt_bias: torch.Tensor, positions: torch.Tensor,
                     row_seq: torch.Tensor, seq_starts: torch.Tensor, state_slots: torch.Tensor, num_seqs: int, heads: int,
                     rk_heads: int, dim: int, vdim: int, q_out: torch.Tensor, k_out: torch.Tensor, v_out: torch.Tensor,
                     decay: torch.Tensor, strength: torch.Tensor, decay_per_head: bool = False) -> None:
    """What the gated delta rule reads, per token. Columns x_off.. of `proj` [T, ld] hold q, k (rk_heads heads of
    `dim` each) and v (heads of `vdim`) side by side: each channel passes a causal convolution over the request's
    tokens (conv_w float32 [C, taps], last column the current token's; inputs before the step's first row from
    conv_state float32 [slots, taps - 1, C]) and silu; q and k are then scaled to unit length per head (1e-6 under
    the root), q also by dim^-1/2. strength = sigmoid(proj[b_off + h]); decay = exp(-exp(a_log[h]) *
    softplus(low[a_off + h * dim + c] + dt_bias)). q_out, k_out float32 [T, rk_heads * dim]; v_out [T, heads * vdim]
    in proj's type; decay float32 [T, heads * dim]; strength float32 [T, heads]. `decay_per_head`: one decay per head,
    exp(-exp(a_log[h]) * softplus(low[a_off + h] + dt_bias[h])), written to all of the head's key channels."""
    op = "gated_delta_prep"
    _cuda(op, proj, low, conv_w, conv_state, a_log, dt_bias, positions, row_seq, seq_starts, state_slots, q_out, k_out, v_out, decay, strength)
    _rows_2d(proj, op, "proj")
    _rows_2d(low, op, "low")
    T = proj.shape[0]
    C = 2 * rk_heads * dim + heads * vdim
    if conv_w.dtype != torch.float32 or conv_w.dim() != 2 or conv_w.shape[0] != C or not conv_w.is_contiguous():
        raise ShapeError(op, f"conv_w must be contiguous float32 [{C}, taps], got {conv_w.dtype} {list(conv_w.shape)}")
    taps = conv_w.shape[1]
    if taps > 1 and (conv_state is None or conv_state.dtype != torch.float32 or conv_state.dim() != 3 or conv_state.shape[1:] != (taps - 1, C)
                     or not conv_state.is_contiguous()):
        raise ShapeError(op, f"conv_state must be contiguous float32 [slots, {taps - 1}, {C}]")
    n_decay = heads if decay_per_head else heads * dim
    if low.dtype != proj.dtype or low.shape[0] != T or a_off < 0 or a_off + n_decay > low.shape[1]:
        raise ShapeError(op, f"low must be {proj.dtype} [{T}, >= {a_off + n_decay}], got {low.dtype} {list(low.shape)}")
    if x_off < 0 or x_off + C > proj.shape[1] or b_off < 0 or b_off + heads > proj.shape[1]:
        raise ShapeError(op, f"columns {x_off}..{x_off + C} or {b_off}..{b_off + heads} lie outside proj's {proj.shape[1]}")
    _f32_vec(a_log, heads, op, "a_log")
    _f32_vec(dt_bias, n_decay, op, "dt_bias")
    for name, t, cols in (("q_out", q_out, rk_heads * dim), ("k_out", k_out, rk_heads * dim), ("decay", decay, heads * dim),
                          ("strength", strength, heads)):
        if t.dtype != torch.float32 or t.shape != (T, cols) or not t.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous float32 [{T}, {cols}], got {t.dtype} {list(t.shape)}")
    if v_out.dtype != proj.dtype or v_out.shape != (T, heads * vdim) or not v_out.is_contiguous():
        raise ShapeError(op, f"v_out must be contiguous {proj.dtype} [{T}, {heads * vdim}], got {v_out.dtype} {list(v_out.shape)}")
    _int32_vec(positions, T, op, "positions")
    _int32_vec(row_seq, T, op, "row_seq")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(state_slots, num_seqs, op, "state_slots")
    f = _fn("recurrence", "vob_gated_delta_prep", [_P, _I, _L, _I, _I, _P, _L, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                                                   _P, _P, _P, _P, _P, _I, _P])
    _check(f(_ptr(proj), _code(proj, op), proj.stride(0), x_off, b_off, _ptr(low), low.stride(0), a_off, _ptr(conv_w), taps,
             _ptr(conv_state), _ptr(a_log), _ptr(dt_bias), _ptr(positions), _ptr(row_seq), _ptr(seq_starts), _ptr(state_slots), T,
             heads, rk_heads, dim, vdim, _ptr(q_out), _ptr(k_out), _ptr(v_out), _ptr(decay), _ptr(strength),
             1 if decay_per_head else 0, _stream()), op)


@_timed
def conv_state_update(proj: torch.Tensor, x_off: int, conv_state: torch.Tensor, seq_starts: torch.Tensor, state_slots: torch.Tensor,
                      num_seqs: int) -> None:
    """Leave every request's last taps - 1 convolution inputs (columns x_off .. x_off + C - 1 of proj) in its state slot;
    a request that brought fewer rows keeps the newest of what it had. conv_state float32 [slots, taps - 1, C]."""
    op = "conv_state_update"
    _cuda(op, proj, conv_state, seq_starts, state_slots)
    _rows_2d(proj, op, "proj")
    if conv_state.dtype != torch.float32 or conv_state.dim() != 3 or not conv_state.is_contiguous():
        raise ShapeError(op, f"conv_state must be contiguous float32 [slots, taps - 1, C], got {conv_state.dtype} {list(conv_state.shape)}")
    C = conv_state.shape[2]
    if x_off < 0 or x_off + C > proj.shape[1]:
        raise ShapeError(op, f"columns {x_off}..{x_off + C} lie outside proj's {proj.shape[1]}")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(state_slots, num_seqs, op, "state_slots")
    f = _fn("recurrence", "vob_conv_state_update", [_P, _I, _L, _I, _I, _I, _P, _P, _P, _I, _P])
    _check(f(_ptr(proj), _code(proj, op), proj.stride(0), x_off, C, conv_state.shape[1] + 1, _ptr(conv_state), _ptr(seq_starts),
             _ptr(state_slots), num_seqs, _stream()), op)


@_timed
def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], conv_state: Optional[torch.Tensor],
                positions: torch.Tensor, row_seq: torch.Tensor, seq_starts: torch.Tensor, state_slots: torch.Tensor, num_seqs: int,
                out: torch.Tensor, residual: bool = False, act: str = "none", single: bool = False) -> None:
    """A short causal convolution over time on each channel: y[t, c] = bias[c] + sum_j weight[j, c] * x[t - taps + 1 + j, c]
    (weight float32 [taps, C]: tap by tap, the last row the current token's),
    inputs before the step's rows taken from `conv_state` (float32 [slots, taps - 1, C], the request's last inputs; zero at its
    start); out = act(y + x) with `residual`, act(y) without; act "none" or "silu". x [T, C] (a column range of a projection,
    any row stride), out [T, C] in x's type or float32. The state is only read: `conv_state_update` moves it on afterwards;
    with `single` (the caller knows that every request brings exactly one row) the kernel moves it on itself."""
    op = "causal_conv"
    _cuda(op, x, weight, bias, conv_state, positions, row_seq, seq_starts, state_slots, out)
    _rows_2d(x, op, "x")
    _rows_2d(out, op, "out")
    T, C = x.shape
    if weight.dtype != torch.float32 or weight.dim() != 2 or weight.shape[1] != C or not weight.is_contiguous():
        raise ShapeError(op, f"weight must be contiguous float32 [taps, {C}], got {weight.dtype} {list(weight.shape)}")
    taps = weight.shape[0]
    _f32_vec(bias, C, op, "bias")
    if taps > 1 and (conv_state is None or conv_state.dtype != torch.float32 or conv_state.dim() != 3 or not conv_state.is_contiguous()
                     or conv_state.shape[1:] != (taps - 1, C)):
        raise ShapeError(op, f"conv_state must be contiguous float32 [slots, {taps - 1}, {C}]")
    if out.shape != (T, C) or out.dtype not in (x.dtype, torch.float32):
        raise ShapeError(op, f"out must be [{T}, {C}] of x's type or float32, got {out.dtype} {list(out.shape)}")
    if act not in ("none", "silu"):
        raise ShapeError(op, f"act {act!r} is not known (none or silu)")
    _int32_vec(positions, T, op, "positions")
    _int32_vec(row_seq, T, op, "row_seq")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(state_slots, num_seqs, op, "state_slots")
    f = _fn("recurrence", "vob_causal_conv", [_P, _I, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _I, _L, _I, _I, _P])
    _check(f(_ptr(x), _code(x, op), x.stride(0), C, taps, _ptr(weight), _ptr(bias), _ptr(conv_state) if taps > 1 else _P(0),
             _ptr(positions), _ptr(row_seq), _ptr(seq_starts), _ptr(state_slots), 1 if residual else 0, 1 if act == "silu" else 0,
             _ptr(out), _code(out, op), out.stride(0), T, 1 if single else 0, _stream()), op)


@_timed
def ssm_steps(raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, dt_out: torch.Tensor, decay_out: torch.Tensor) -> None:
    """dt = softplus(raw + dt_bias[h]) and decay = exp(-exp(a_log[h]) * dt) per token and head, float32 [T, heads] each; raw
    [T, heads] is a column range of a projection output."""
    op = "ssm_steps"
    _cuda(op, raw, dt_bias, a_log, dt_out, decay_out)
    _rows_2d(raw, op, "raw")
    T, H = raw.shape
    _f32_vec(dt_bias, H, op, "dt_bias")
    _f32_vec(a_log, H, op, "a_log")
    for name, t in (("dt_out", dt_out), ("decay_out", decay_out)):
        if t.dtype != torch.float32 or t.shape != (T, H) or not t.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous float32 [{T}, {H}], got {t.dtype} {list(t.shape)}")
    f = _fn("recurrence", "vob_ssm_steps", [_P, _I, _L, _P, _P, _I, _I, _P, _P, _P])
    _check(f(_ptr(raw), _code(raw, op), raw.stride(0), _ptr(dt_bias), _ptr(a_log), T, H, _ptr(dt_out), _ptr(decay_out), _stream()), op)


@_timed
def ssm_post(o: torch.Tensor, x: torch.Tensor, z: torch.Tensor, skip: torch.Tensor, weight: torch.Tensor, eps: float, heads: int,
             groups: int, out: torch.Tensor) -> None:
    """out = rms_groups((o + skip[head] * x) * silu(z)) * weight: the gate first, then an RMS norm over each of `groups` equal
    parts of the row. o float32 [T, n] contiguous; x float32 [T, n] (any row stride); z and out [T, n] in the activations' type
    (any row stride); skip float32 [heads]; weight float32 [n]."""
    op = "ssm_post"
    _cuda(op, o, x, z, skip, weight, out)
    _rows_2d(x, op, "x")
    _rows_2d(z, op, "z")
    _rows_2d(out, op, "out")
    if o.dtype != torch.float32 or o.dim() != 2 or not o.is_contiguous():
        raise ShapeError(op, f"o must be contiguous float32 [T, n], got {o.dtype} {list(o.shape)}")
    T, n = o.shape
    if x.shape != (T, n) or x.dtype != torch.float32 or z.shape != (T, n) or out.shape != (T, n) or out.dtype != z.dtype:
        raise ShapeError(op, f"x float32, z and out of one type, all [{T}, {n}], are needed")
    if heads <= 0 or groups <= 0 or n % heads or n % groups:
        raise ShapeError(op, f"{n} features do not split into {heads} heads and {groups} groups")
    _f32_vec(skip, heads, op, "skip")
    _f32_vec(weight, n, op, "weight")
    f = _fn("recurrence", "vob_ssm_post", [_P, _P, _L, _P, _I, _L, _P, _P, _F, _I, _I, _I, _I, _P, _L, _P])
    _check(f(_ptr(o), _ptr(x), x.stride(0), _ptr(z), _code(z, op), z.stride(0), _ptr(skip), _ptr(weight), float(eps), T, n, int(heads),
             int(groups), _ptr(out), out.stride(0), _stream()), op)


@_timed
def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float) -> None:
    """out[t, j] = g * sigmoid(1.702 g) * (u + 1) with g = min(gate_up[t, j], limit), u = clamp(gate_up[t, I + j], -limit, limit)."""
    op = "glu_clamped"
    _cuda(op, gate_up, out)
    _rows_2d(gate_up, op, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype or not out.is_contiguous() or not limit > 0:
        raise ShapeError(op, f"gate_up [{T}, 2 I], a contiguous out [{T}, I] of its type and a positive limit are needed, got "
                             f"{list(gate_up.shape)}, {out.dtype} {list(out.shape)}, {limit}")
    f = _fn("elementwise", "vob_glu_clamped", [_P, _L, _P, _I, _I, _I, _F, _P])
    _check(f(_ptr(gate_up), gate_up.stride(0), _ptr(out), _code(out, op), T, two_i // 2, float(limit), _stream()), op)


@_timed
def depth_average(stack: torch.Tensor, x: torch.Tensor, weights: Optional[torch.Tensor], n: int) -> None:
    """stack[:, n] = x; then, with `weights` (float32 [n + 1]), x = sum_j weights[j] * stack[:, j] over j = 0 .. n. Without
    weights only the filing is done (slot 0 takes the embedding's output). stack float32 [T, slots, h], x float32 [T, h]."""
    op = "depth_average"
    _cuda(op, stack, x, weights)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise ShapeError(op, f"x must be contiguous float32 [T, h], got {x.dtype} {list(x.shape)}")
    T, h = x.shape
    if stack.dtype != torch.float32 or stack.dim() != 3 or stack.shape[0] != T or stack.shape[2] != h or not stack.is_contiguous():
        raise ShapeError(op, f"stack must be contiguous float32 [{T}, slots, {h}], got {stack.dtype} {list(stack.shape)}")
    if not 0 <= n < stack.shape[1]:
        raise ShapeError(op, f"slot {n} lies outside the stack's {stack.shape[1]}")
    _f32_vec(weights, n + 1, op, "weights")
    f = _fn("elementwise", "vob_depth_average", [_P, _P, _P, _I, _I, _I, _I, _I, _P])
    _check(f(_ptr(stack), _ptr(x), _ptr(weights), T, stack.shape[1], h, int(n), 0 if weights is not None else 1, _stream()), op)


# ------------------------------------------------------------------------------------ mixture of experts
MOE_TILE_ROWS = 32           # rows of a tile of (token, expert) pairs (VOB_MOE_BM of csrc/moe.cu)
MOE_LARGE_TILE_ROWS = 128    # the pipelined tensor-core products also take tiles of this many
MOE_ACTIVATIONS = {"silu": 0, "clamped_swish": 1}    # how an expert's gate acts on its hidden values
MOE_LARGE_TILE_FROM = 64     # pairs an expert gets on average from which the large tiles are taken


def moe_tile_rows(pairs: int, experts: int, width: int, ff: int, tensor_cores: bool) -> int:
    """Rows of a tile for a step of `pairs` pairs: 128 where the tensor-core products can fetch their rows 16 bytes at a
    time (width and ff multiples of 8) and the experts get enough pairs each to fill such tiles, else 32."""
    if tensor_cores and width % 8 == 0 and ff % 8 == 0 and pairs >= MOE_LARGE_TILE_FROM * experts:
        return MOE_LARGE_TILE_ROWS
    return MOE_TILE_ROWS


def moe_sorted_rows(pairs: int, experts: int, tile_rows: int = MOE_TILE_ROWS) -> int:
    """Rows the ordered list of `pairs` (token, expert) pairs takes: every expert's run is padded to whole tiles."""
    return -(-pairs // tile_rows) * tile_rows + experts * tile_rows


@_timed
def moe_route(x: torch.Tensor, w_router: torch.Tensor, positions: Optional[torch.Tensor], top: int, groups: int, keep: int,
              renorm: bool, idx_out: torch.Tensor, w_out: torch.Tensor) -> None:
    """Per row of x [T, width]: softmax over the E router logits (w_router float32 [E, width], float32 sums), election of
    `top` experts among those of the `keep` best of `groups` runs of neighbours (groups <= 1: among all), weights = their
    scores (renorm: divided by their sum). idx_out int32 [T, top] (-1 for rows of negative position), w_out float32 [T, top]."""
    op = "moe_route"
    _cuda(op, x, w_router, positions, idx_out, w_out)
    _rows_2d(x, op, "x")
    T, width = x.shape
    if w_router.dtype != torch.float32 or w_router.dim() != 2 or w_router.shape[1] != width or not w_router.is_contiguous():
        raise ShapeError(op, f"w_router must be contiguous float32 [experts, {width}], got {w_router.dtype} {list(w_router.shape)}")
    E = w_router.shape[0]
    if not 0 < top <= E:
        raise ShapeError(op, f"{top} choices among {E} experts")
    if groups > 1 and (E % groups or not 0 < keep <= groups or top > keep * (E // groups)):
        raise ShapeError(op, f"{E} experts in {groups} groups of which {keep} are kept cannot give {top} choices")
    if idx_out.dtype != torch.int32 or idx_out.shape != (T, top) or not idx_out.is_contiguous():
        raise ShapeError(op, f"idx_out must be contiguous int32 [{T}, {top}], got {idx_out.dtype} {list(idx_out.shape)}")
    if w_out.dtype != torch.float32 or w_out.shape != (T, top) or not w_out.is_contiguous():
        raise ShapeError(op, f"w_out must be contiguous float32 [{T}, {top}], got {w_out.dtype} {list(w_out.shape)}")
    if positions is not None:
        _int32_vec(positions, T, op, "positions")
    f = _fn("moe", "vob_moe_route", [_P, _I, _L, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P])
    _check(f(_ptr(x), _code(x, op), x.stride(0), _ptr(w_router), _ptr(positions), T, width, E, int(top), int(groups), int(keep),
             1 if renorm else 0, _ptr(idx_out), _ptr(w_out), _stream()), op)


@_timed
def moe_align(idx: torch.Tensor, experts: int, sorted_pairs: torch.Tensor, tile_expert: torch.Tensor, meta: torch.Tensor,
              tile_rows: int = MOE_TILE_ROWS) -> None:
    """The pairs idx [T, top] (expert of token t's k-th choice, -1: none) in order of their expert: sorted_pairs int32 [cap]
    (pair number t * top + k, -1: padding; cap >= moe_sorted_rows(T * top, experts, tile_rows)), tile_expert int32
    [cap / tile_rows], meta int32 [>= 1] (meta[0]: tiles in use)."""
    op = "moe_align"
    _cuda(op, idx, sorted_pairs, tile_expert, meta)
    if idx.dtype != torch.int32 or idx.dim() != 2 or not idx.is_contiguous():
        raise ShapeError(op, f"idx must be contiguous int32 [T, top], got {idx.dtype} {list(idx.shape)}")
    P, cap = idx.numel(), sorted_pairs.numel()
    if tile_rows not in (MOE_TILE_ROWS, MOE_LARGE_TILE_ROWS):
        raise ShapeError(op, f"tiles have {MOE_TILE_ROWS} or {MOE_LARGE_TILE_ROWS} rows, not {tile_rows}")
    if cap % tile_rows or cap < moe_sorted_rows(P, experts, tile_rows):
        raise ShapeError(op, f"sorted_pairs has {cap} rows, {moe_sorted_rows(P, experts, tile_rows)} (a multiple of {tile_rows}) are needed")
    _int32_vec(sorted_pairs, cap, op, "sorted_pairs")
    _int32_vec(tile_expert, cap // tile_rows, op, "tile_expert")
    _int32_vec(meta, 1, op, "meta")
    f = _fn("moe", "vob_moe_align", [_P, _I, _I, _P, _I, _P, _P, _I, _P])
    _check(f(_ptr(idx), P, int(experts), _ptr(sorted_pairs), cap, _ptr(tile_expert), _ptr(meta), int(tile_rows), _stream()), op)


def _moe_tiles(op, sorted_pairs, tile_expert, tile_rows, tensor_cores, width, ff):
    cap = sorted_pairs.numel()
    _int32_vec(sorted_pairs, cap, op, "sorted_pairs")
    if tile_rows != MOE_TILE_ROWS and not (tile_rows == MOE_LARGE_TILE_ROWS and tensor_cores and width % 8 == 0 and ff % 8 == 0):
        raise ShapeError(op, f"tiles of {tile_rows} rows: {MOE_TILE_ROWS}, or {MOE_LARGE_TILE_ROWS} with the tensor-core form and "
                             f"width and ff multiples of 8")
    if cap % tile_rows:
        raise ShapeError(op, f"sorted_pairs must hold whole tiles of {tile_rows}, got {cap}")
    _int32_vec(tile_expert, cap // tile_rows, op, "tile_expert")
    return cap // tile_rows


@_timed
def moe_gate_up(x: torch.Tensor, w_gu: torch.Tensor, sorted_pairs: torch.Tensor, tile_expert: torch.Tensor, top: int,
                h_out: torch.Tensor, tensor_cores: bool = False, tile_rows: int = MOE_TILE_ROWS, activation: str = "silu",
                limit: float = 0.0) -> None:
    """h_out[pair] = silu(W_gate[e] x[token]) * (W_up[e] x[token]) for every pair of the ordered list; w_gu [E, 2 ff, width]
    (an expert's gate rows, then its up rows) and h_out [T * top, ff] of x's type. `tensor_cores`: the bfloat16 tile form.
    `activation` "clamped_swish": g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1)."""
    op = "moe_gate_up"
    if activation not in MOE_ACTIVATIONS or (activation == "clamped_swish" and not limit > 0):
        raise ShapeError(op, f"activation {activation!r} (limit {limit}) is not known ({', '.join(MOE_ACTIVATIONS)}; the clamped one "
                             f"needs a positive limit)")
    _cuda(op, x, w_gu, sorted_pairs, tile_expert, h_out)
    _rows_2d(x, op, "x")
    T, width = x.shape
    if w_gu.dim() != 3 or w_gu.shape[2] != width or w_gu.shape[1] % 2 or w_gu.dtype != x.dtype or not w_gu.is_contiguous():
        raise ShapeError(op, f"w_gu must be contiguous {x.dtype} [experts, 2 ff, {width}], got {w_gu.dtype} {list(w_gu.shape)}")
    ff = w_gu.shape[1] // 2
    if h_out.shape != (T * top, ff) or h_out.dtype != x.dtype or not h_out.is_contiguous():
        raise ShapeError(op, f"h_out must be contiguous {x.dtype} [{T * top}, {ff}], got {h_out.dtype} {list(h_out.shape)}")
    if tensor_cores and x.dtype != torch.bfloat16:
        raise ShapeError(op, "the tensor-core form takes bfloat16")
    tiles = _moe_tiles(op, sorted_pairs, tile_expert, tile_rows, tensor_cores, width, ff)
    if tile_rows != MOE_TILE_ROWS and (x.stride(0) % 8 or x.data_ptr() % 16):
        raise ShapeError(op, f"tiles of {tile_rows} rows need rows of x that start on 16-byte boundaries")
    f = _fn("moe", "vob_moe_gate_up", [_P, _I, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _F, _P])
    _check(f(_ptr(x), _code(x, op), x.stride(0), _ptr(w_gu), _ptr(sorted_pairs), _ptr(tile_expert), tiles, int(tile_rows), int(top), width, ff,
             _ptr(h_out), 1 if tensor_cores else 0, MOE_ACTIVATIONS[activation], float(limit), _stream()), op)


@_timed
def moe_down(h: torch.Tensor, w_down: torch.Tensor, sorted_pairs: torch.Tensor, tile_expert: torch.Tensor, pair_w: torch.Tensor,
             y: torch.Tensor, tensor_cores: bool = False, tile_rows: int = MOE_TILE_ROWS) -> None:
    """y[pair] = pair_w[pair] * (W_down[e] h[pair]), float32 [T * top, width]; w_down [E, width, ff] of h's type; pair_w
    float32 [T, top]."""
    op = "moe_down"
    _cuda(op, h, w_down, sorted_pairs, tile_expert, pair_w, y)
    if h.dim() != 2 or not h.is_contiguous():
        raise ShapeError(op, f"h must be contiguous [pairs, ff], got {list(h.shape)}")
    P, ff = h.shape
    if w_down.dim() != 3 or w_down.shape[2] != ff or w_down.dtype != h.dtype or not w_down.is_contiguous():
        raise ShapeError(op, f"w_down must be contiguous {h.dtype} [experts, width, {ff}], got {w_down.dtype} {list(w_down.shape)}")
    width = w_down.shape[1]
    if pair_w.dtype != torch.float32 or pair_w.numel() != P or not pair_w.is_contiguous():
        raise ShapeError(op, f"pair_w must be contiguous float32 of {P} entries, got {pair_w.dtype} {list(pair_w.shape)}")
    if y.dtype != torch.float32 or y.shape != (P, width) or not y.is_contiguous():
        raise ShapeError(op, f"y must be contiguous float32 [{P}, {width}], got {y.dtype} {list(y.shape)}")
    if tensor_cores and h.dtype != torch.bfloat16:
        raise ShapeError(op, "the tensor-core form takes bfloat16")
    tiles = _moe_tiles(op, sorted_pairs, tile_expert, tile_rows, tensor_cores, width, ff)
    f = _fn("moe", "vob_moe_down", [_P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _P])
    _check(f(_ptr(h), _code(h, op), _ptr(w_down), _ptr(sorted_pairs), _ptr(tile_expert), _ptr(pair_w), tiles, int(tile_rows), width, ff, _ptr(y),
             1 if tensor_cores else 0, _stream()), op)


@_timed
def moe_combine(y: torch.Tensor, idx: torch.Tensor, out: torch.Tensor, shared: Optional[torch.Tensor] = None,
                shared_gate: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum over k, in order, of y[t * top + k] where idx[t, k] >= 0; out [T, width] in the activations' type.
    `shared` [T, width] (out's type): the result of an expert every token uses, added; `shared_gate` [T] (a column of a
    projection output, out's type): `shared` is first multiplied by its sigmoid, token by token."""
    op = "moe_combine"
    _cuda(op, y, idx, out, shared, shared_gate)
    if shared is not None and (shared.shape != out.shape or shared.dtype != out.dtype or not shared.is_contiguous()):
        raise ShapeError(op, f"shared must be contiguous {out.dtype} {list(out.shape)}, got {shared.dtype} {list(shared.shape)}")
    if shared_gate is not None and (shared is None or shared_gate.dim() != 1 or shared_gate.shape[0] != out.shape[0]
                                    or shared_gate.dtype != out.dtype):
        raise ShapeError(op, f"shared_gate must be {out.dtype} [{out.shape[0]}] and go with shared, got {shared_gate.dtype} "
                             f"{list(shared_gate.shape)}")
    if idx.dtype != torch.int32 or idx.dim() != 2 or not idx.is_contiguous():
        raise ShapeError(op, f"idx must be contiguous int32 [T, top], got {idx.dtype} {list(idx.shape)}")
    T, top = idx.shape
    if y.dtype != torch.float32 or y.dim() != 2 or y.shape[0] != T * top or not y.is_contiguous():
        raise ShapeError(op, f"y must be contiguous float32 [{T * top}, width], got {y.dtype} {list(y.shape)}")
    if out.shape != (T, y.shape[1]) or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous [{T}, {y.shape[1]}], got {list(out.shape)}")
    f = _fn("moe", "vob_moe_combine", [_P, _P, _I, _I, _I, _P, _I, _P, _P, _L, _P])
    _check(f(_ptr(y), _ptr(idx), T, top, y.shape[1], _ptr(out), _code(out, op), _ptr(shared), _ptr(shared_gate),
             shared_gate.stride(0) if shared_gate is not None else 0, _stream()), op)


# ------------------------------------------------------------------------------------ attention over a latent cache
@_timed
def latent_prep(proj: torch.Tensor, q_off: int, heads: int, dim: int, rot: int, down_off: int, rank: int, norm_w: torch.Tensor,
                eps: float, positions: torch.Tensor, slots: Optional[torch.Tensor], inv_freq: torch.Tensor, lat: torch.Tensor,
                kr: torch.Tensor, q_rot: torch.Tensor) -> None:
    """Per token: the latent (first `rank` columns of the down projection, RMS norm with weight) and the
    rotated key part (its last `rot` columns, rotary positions) go to the token's cache slot (lat
    [pages, 1, page, rank], kr [pages, 1, page, rot]); the rotated query part of every head (the last
    `rot` of its dim + rot columns) goes to q_rot float32 [T, heads, rot]."""
    op = "latent_prep"
    _cuda(op, proj, norm_w, positions, slots, inv_freq, lat, kr, q_rot)
    _rows_2d(proj, op, "proj")
    T = proj.shape[0]
    if q_off < 0 or q_off + heads * (dim + rot) > proj.shape[1] or down_off < 0 or down_off + rank + rot > proj.shape[1]:
        raise ShapeError(op, f"the query or down-projection columns lie outside proj's {proj.shape[1]}")
    for name, t, w in (("lat", lat, rank), ("kr", kr, rot)):
        if t.dim() != 4 or t.shape[1] != 1 or t.shape[3] != w or not t.is_contiguous() or t.dtype != proj.dtype:
            raise ShapeError(op, f"{name} must be contiguous {proj.dtype} [pages, 1, page, {w}], got {t.dtype} {list(t.shape)}")
    if q_rot.shape != (T, heads, rot) or q_rot.dtype != torch.float32 or not q_rot.is_contiguous():
        raise ShapeError(op, f"q_rot must be contiguous float32 [{T}, {heads}, {rot}], got {q_rot.dtype} {list(q_rot.shape)}")
    _f32_vec(norm_w, rank, op, "norm_w")
    _f32_vec(inv_freq, rot // 2, op, "inv_freq")
    _int32_vec(positions, T, op, "positions")
    if slots is not None:
        _int32_vec(slots, T, op, "slots")
    f = _fn("latent_attention", "vob_latent_prep", [_P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _F, _P, _P, _P, _P, _P, _I, _P, _I, _P])
    _check(f(_ptr(proj), _code(proj, op), proj.stride(0), q_off, heads, dim, rot, down_off, rank, _ptr(norm_w), float(eps), _ptr(positions),
             _ptr(slots), _ptr(inv_freq), _ptr(lat), _ptr(kr), _code(lat, op), _ptr(q_rot), T, _stream()), op)


@_timed
def latent_attend(q_lat: torch.Tensor, q_rot: torch.Tensor, lat: torch.Tensor, kr: torch.Tensor, block_tables: torch.Tensor,
                  row_seq: torch.Tensor, positions: torch.Tensor, scale: float, out: torch.Tensor, splits: int = 1,
                  partials: Optional[torch.Tensor] = None, window: int = 0) -> None:
    """Causal attention of every row over its request's latent pages: score = (q_lat . c + q_rot . kr) *
    scale, softmax in float32, out_lat = sum of weights * c. q_lat float32 and out (cache type) are
    indexed [T, heads, rank] through their strides (last stride 1); q_rot float32 [T, heads, rot].
    `splits` > 1 shares every row's keys over that many blocks; `partials` (float32, at least
    T * heads * splits * (rank + 2) elements) is their scratch, and a second launch merges them. `window` > 0: a row sees
    itself and the window - 1 tokens before it."""
    op = "latent_attend"
    _cuda(op, q_lat, q_rot, lat, kr, block_tables, row_seq, positions, out)
    if q_lat.dim() != 3 or q_lat.dtype != torch.float32 or q_lat.stride(2) != 1:
        raise ShapeError(op, f"q_lat must be float32 [T, heads, rank] with unit inner stride, got {q_lat.dtype} {list(q_lat.shape)}")
    T, H, L = q_lat.shape
    R = kr.shape[3]
    if out.shape != (T, H, L) or out.stride(2) != 1 or out.dtype != lat.dtype:
        raise ShapeError(op, f"out must be {lat.dtype} [{T}, {H}, {L}] with unit inner stride, got {out.dtype} {list(out.shape)}")
    if q_rot.shape != (T, H, R) or q_rot.dtype != torch.float32 or not q_rot.is_contiguous():
        raise ShapeError(op, f"q_rot must be contiguous float32 [{T}, {H}, {R}], got {q_rot.dtype} {list(q_rot.shape)}")
    if lat.dim() != 4 or lat.shape[1] != 1 or lat.shape[3] != L or kr.shape[:3] != lat.shape[:3] or kr.dtype != lat.dtype \
            or not lat.is_contiguous() or not kr.is_contiguous():
        raise ShapeError(op, f"lat [pages, 1, page, {L}] and kr [pages, 1, page, {R}] of one type are needed, got {list(lat.shape)} and {list(kr.shape)}")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, "block_tables must be contiguous int32 [requests, max_pages]")
    _int32_vec(row_seq, T, op, "row_seq")
    _int32_vec(positions, T, op, "positions")
    splits = int(splits)
    if splits > 1:
        _cuda(op, partials)
        if partials is None or partials.dtype != torch.float32 or not partials.is_contiguous() or partials.numel() < T * H * splits * (L + 2):
            raise ShapeError(op, f"{splits} splits need contiguous float32 partials of {T * H * splits * (L + 2)} elements")
    f = _fn("latent_attention", "vob_latent_attend", [_P, _L, _L, _P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _I, _L, _L, _I, _P, _I, _P])
    _check(f(_ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), _ptr(lat), _ptr(kr), _code(lat, op), _ptr(block_tables),
             block_tables.shape[1], _ptr(row_seq), _ptr(positions), lat.shape[2], T, H, L, R, float(scale), _ptr(out), _code(out, op),
             out.stride(0), out.stride(1), splits, _ptr(partials) if splits > 1 else _P(0), int(window), _stream()), op, 2 if splits > 1 else 1)


def latent_attend_tc_supported(heads: int, rank: int, rot: int) -> bool:
    """Whether the tensor-core kernel for prompt portions takes these sizes (bfloat16 only)."""
    f = _fn("latent_attention", "vob_latent_attend_tc_supported", [_I, _I, _I])
    return bool(f(int(heads), int(rank), int(rot)))


@_timed
def latent_attend_tc(q_lat: torch.Tensor, q_rot: torch.Tensor, lat: torch.Tensor, kr: torch.Tensor, block_tables: torch.Tensor,
                     seq_starts: torch.Tensor, positions: torch.Tensor, num_seqs: int, max_new: int, scale: float, out: torch.Tensor,
                     window: int = 0) -> None:
    """`latent_attend` for prompt portions in bfloat16 on the tensor cores: request s owns rows seq_starts[s] ..
    seq_starts[s + 1] - 1 (consecutive positions), none more than `max_new`. Same operands and result."""
    op = "latent_attend_tc"
    _cuda(op, q_lat, q_rot, lat, kr, block_tables, seq_starts, positions, out)
    if q_lat.dim() != 3 or q_lat.dtype != torch.float32 or q_lat.stride(2) != 1:
        raise ShapeError(op, f"q_lat must be float32 [T, heads, rank] with unit inner stride, got {q_lat.dtype} {list(q_lat.shape)}")
    T, H, L = q_lat.shape
    R = kr.shape[3]
    if lat.dtype != torch.bfloat16 or kr.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise ShapeError(op, "the caches and out must be bfloat16")
    if out.shape != (T, H, L) or out.stride(2) != 1:
        raise ShapeError(op, f"out must be [{T}, {H}, {L}] with unit inner stride, got {list(out.shape)}")
    if q_rot.shape != (T, H, R) or q_rot.dtype != torch.float32 or not q_rot.is_contiguous():
        raise ShapeError(op, f"q_rot must be contiguous float32 [{T}, {H}, {R}], got {q_rot.dtype} {list(q_rot.shape)}")
    if lat.dim() != 4 or lat.shape[1] != 1 or lat.shape[3] != L or kr.shape[:3] != lat.shape[:3] or not lat.is_contiguous() or not kr.is_contiguous():
        raise ShapeError(op, f"lat [pages, 1, page, {L}] and kr [pages, 1, page, {R}] are needed, got {list(lat.shape)} and {list(kr.shape)}")
    if not latent_attend_tc_supported(H, L, R):
        raise ShapeError(op, f"a latent of {L} with a rotated part of {R} is not supported (multiples of 16 that fit shared memory)")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous() or block_tables.shape[0] < num_seqs:
        raise ShapeError(op, "block_tables must be contiguous int32 [requests, max_pages]")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(positions, T, op, "positions")
    f = _fn("latent_attention", "vob_latent_attend_tc", [_P, _L, _L, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _L, _L, _I, _P])
    _check(f(_ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), _ptr(lat), _ptr(kr), _ptr(block_tables), block_tables.shape[1],
             _ptr(seq_starts), _ptr(positions), lat.shape[2], int(num_seqs), int(max_new), H, L, R, float(scale), _ptr(out), out.stride(0),
             out.stride(1), int(window), _stream()), op)


# ------------------------------------------------------------------------------------ attention with options
def _kv_caches(op, kcache, vcache, kv_heads, dim, vdim, dtype):
    for name, c, w in (("kcache", kcache, dim), ("vcache", vcache, vdim)):
        if c.dim() != 4 or c.shape[1] != kv_heads or c.shape[3] != w or not c.is_contiguous() or c.dtype != dtype:
            raise ShapeError(op, f"{name} must be contiguous {dtype} [pages, {kv_heads}, page_size, {w}], got {c.dtype} {list(c.shape)}")
    if kcache.shape[:3] != vcache.shape[:3]:
        raise ShapeError(op, "kcache and vcache differ in pages, heads or page size")
    if kcache.numel() // dim >= 2 ** 31:
        raise ShapeError(op, "one layer's cache has 2^31 rows or more")


@_timed
def flex_prep(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, positions: torch.Tensor, slots: Optional[torch.Tensor],
              inv_freq: Optional[torch.Tensor], rot: int, unit_rms: bool, eps: float, q_temp, vmix: Optional[torch.Tensor],
              v_first: Optional[torch.Tensor], v_mode: int, q_out: torch.Tensor, kcache: Optional[torch.Tensor],
              vcache: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int,
              q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None,
              q_pre_w: Optional[torch.Tensor] = None, k_pre_w: Optional[torch.Tensor] = None) -> None:
    """Per token, from the columns q_off.., k_off.., v_off.. of `proj`: q and k with their first `rot` features rotated
    (feature i with i + rot / 2, by position * inv_freq[i]), then (unit_rms) divided by sqrt(mean(x^2) + eps) per head;
    q times 1 + coef * ln(floor((pos + 1) / every) + 1) for q_temp = (coef, every). q goes to q_out [T, heads * dim], k
    and v to their cache slots. v_mode 1 also leaves v in v_first [T, kv_heads * vdim]; v_mode 2 mixes
    v <- (1 - vmix) v + vmix v_first before the write (vmix: one float32 on the device). `q_norm_w`, `k_norm_w` (float32
    [dim], shared by the heads) multiply q and k behind the division. `q_pre_w` (float32 [heads * dim]) / `k_pre_w` (float32
    [kv_heads * dim]): BEFORE the rotation the whole projection, all its heads at once, is divided by sqrt(mean(x^2) + eps) and
    multiplied by that weight. Without caches (`kcache` None: a layer that reads
    what another layer cached) only q is prepared and `proj` needs no k and v columns."""
    op = "flex_prep"
    _cuda(op, proj, positions, slots, inv_freq, vmix, v_first, q_out, kcache, vcache, q_norm_w, k_norm_w, q_pre_w, k_pre_w)
    _f32_vec(q_pre_w, heads * dim, op, "q_pre_w")
    _f32_vec(k_pre_w, kv_heads * dim, op, "k_pre_w")
    _rows_2d(proj, op, "proj")
    _rows_2d(q_out, op, "q_out")
    T = proj.shape[0]
    if (kcache is None) != (vcache is None):
        raise ShapeError(op, "both caches or none")
    spans = ((q_off, heads * dim),) if kcache is None else ((q_off, heads * dim), (k_off, kv_heads * dim), (v_off, kv_heads * vdim))
    for off, n in spans:
        if off < 0 or off + n > proj.shape[1]:
            raise ShapeError(op, f"columns {off}..{off + n} lie outside proj's {proj.shape[1]}")
    if q_out.shape != (T, heads * dim) or q_out.dtype != proj.dtype:
        raise ShapeError(op, f"q_out must be {proj.dtype} [{T}, {heads * dim}], got {q_out.dtype} {list(q_out.shape)}")
    if kcache is not None:
        _kv_caches(op, kcache, vcache, kv_heads, dim, vdim, proj.dtype)
    elif v_mode or slots is not None:
        raise ShapeError(op, "without caches there is nothing to write and no value to mix")
    _f32_vec(q_norm_w, dim, op, "q_norm_w")
    _f32_vec(k_norm_w, dim, op, "k_norm_w")
    _int32_vec(positions, T, op, "positions")
    if slots is not None:
        _int32_vec(slots, T, op, "slots")
    if rot:
        _f32_vec(inv_freq, rot // 2, op, "inv_freq")
    if v_mode not in (0, 1, 2):
        raise ShapeError(op, f"v_mode {v_mode} is not known")
    if v_mode and (v_first is None or v_first.dtype != proj.dtype or v_first.shape != (T, kv_heads * vdim) or not v_first.is_contiguous()):
        raise ShapeError(op, f"v_first must be contiguous {proj.dtype} [{T}, {kv_heads * vdim}]")
    if v_mode == 2:
        _f32_vec(vmix, 1, op, "vmix")
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    f = _fn("attention_flex", "vob_flex_prep", [_P, _I, _L, _I, _I, _I, _P, _P, _P, _I, _I, _F, _F, _I, _P, _P, _P, _P, _P, _P, _I, _P, _L,
                                                _P, _P, _I, _I, _I, _I, _I, _I, _P])
    _check(f(_ptr(proj), _code(proj, op), proj.stride(0), q_off, k_off, v_off, _ptr(positions), _ptr(slots), _ptr(inv_freq), int(rot),
             1 if unit_rms else 0, float(eps), coef, every, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(q_pre_w), _ptr(k_pre_w), _ptr(vmix), _ptr(v_first), int(v_mode),
             _ptr(q_out), q_out.stride(0), _ptr(kcache), _ptr(vcache), T, heads, kv_heads, dim, vdim,
             kcache.shape[2] if kcache is not None else 1, _stream()), op)


@_timed
def pool_blocks(kcache: torch.Tensor, vcache: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, block_tables: torch.Tensor,
                row_seq: torch.Tensor, positions: torch.Tensor, pool: int) -> None:
    """For every row whose position p ends a block of `pool` tokens ((p + 1) % pool == 0): the mean of the block's cached keys
    and the mean of its cached values (float32 sums in token order) go to kpool and vpool, laid out like the caches, at the
    place a token at position p // pool would have. Runs behind the kernel that wrote the step's keys and values."""
    op = "pool_blocks"
    _cuda(op, kcache, vcache, kpool, vpool, block_tables, row_seq, positions)
    if kcache.dim() != 4 or vcache.dim() != 4 or kpool.shape != kcache.shape or vpool.shape != vcache.shape or kpool.dtype != kcache.dtype \
            or vpool.dtype != kcache.dtype or vcache.dtype != kcache.dtype or kcache.shape[:3] != vcache.shape[:3]:
        raise ShapeError(op, "caches [pages, heads, page, width] and pooled tensors of their shapes and type are needed")
    for t in (kcache, vcache, kpool, vpool):
        if not t.is_contiguous():
            raise ShapeError(op, "caches and pooled tensors must be contiguous")
    if pool <= 0:
        raise ShapeError(op, f"a block of {pool} tokens")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, "block_tables must be contiguous int32 [requests, max_pages]")
    T = positions.numel()
    _int32_vec(positions, T, op, "positions")
    _int32_vec(row_seq, T, op, "row_seq")
    f = _fn("attention_flex", "vob_pool_blocks", [_P, _P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P])
    _check(f(_ptr(kcache), _ptr(vcache), _ptr(kpool), _ptr(vpool), _code(kcache, op), _ptr(block_tables), block_tables.shape[1], _ptr(row_seq),
             _ptr(positions), T, kcache.shape[1], kcache.shape[3], vcache.shape[3], kcache.shape[2], int(pool), _stream()), op)


@_timed
def flex_attention(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                   row_seq: torch.Tensor, positions: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                   window: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   out_scale: float = 1.0, chunk: int = 0, softcap: float = 0.0, dist_bias=None, pool: int = 0) -> None:
    """Causal attention of every row of q [T, heads * dim] over its request's pages, keys of `dim` and values of `vdim`
    features: out [T, heads * vdim] (any row stride) = softmax(q . K * scale) V, over the last `window` keys (0: all), the
    denominator also holding exp(sink[head]) if `sink` (float32 [heads]) is given; times sigmoid(gate) ([T, heads * vdim],
    any row stride) and `out_scale`. `chunk` > 0: a query reads only the keys of its own block of `chunk` positions (blocks
    counted from position 0). `softcap` > 0: score <- softcap * tanh(score / softcap). `dist_bias` = (r1, r2), float32 [heads]
    each: r1 * ln(1 + r2 * distance) is taken off the score. `pool` > 0 (with a window): every block of `pool` positions that
    ends at or before position - window is seen as one key and one value, the means of the block's cached keys and values, in
    the same softmax as the window's tokens."""
    op = "flex_attention"
    if pool < 0 or (pool and (window <= 0 or chunk)):
        raise ShapeError(op, f"pooled blocks of {pool} go with a window and without blocks of positions")
    r1, r2 = dist_bias if dist_bias is not None else (None, None)
    _cuda(op, q, out, kcache, vcache, block_tables, row_seq, positions, sink, gate, r1, r2)
    _f32_vec(r1, heads, op, "dist_bias[0]")
    _f32_vec(r2, heads, op, "dist_bias[1]")
    if chunk < 0 or softcap < 0:
        raise ShapeError(op, f"chunk {chunk} and softcap {softcap} must not be negative")
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    T = q.shape[0]
    if q.shape[1] != heads * dim or out.shape != (T, heads * vdim) or out.dtype != q.dtype:
        raise ShapeError(op, f"q [{T}, {heads * dim}] and out [{T}, {heads * vdim}] of one dtype are needed, got {list(q.shape)} "
                             f"{q.dtype} and {list(out.shape)} {out.dtype}")
    if kv_heads <= 0 or heads % kv_heads != 0:
        raise ShapeError(op, f"{heads} heads are not a multiple of {kv_heads} kv heads")
    if dim > 256 or vdim > 256:
        raise ShapeError(op, f"head sizes {dim} / {vdim} are beyond this kernel's 256")
    _kv_caches(op, kcache, vcache, kv_heads, dim, vdim, q.dtype)
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, f"block_tables must be contiguous int32 [S, max_pages], got {block_tables.dtype} {list(block_tables.shape)}")
    _int32_vec(row_seq, T, op, "row_seq")
    _int32_vec(positions, T, op, "positions")
    _f32_vec(sink, heads, op, "sink")
    if gate is not None:
        _rows_2d(gate, op, "gate")
        if gate.shape != (T, heads * vdim) or gate.dtype != q.dtype:
            raise ShapeError(op, f"gate must be {q.dtype} [{T}, {heads * vdim}], got {gate.dtype} {list(gate.shape)}")
    f = _fn("attention_flex", "vob_flex_attention", [_P, _L, _P, _L, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P,
                                                     _L, _F, _I, _F, _P, _P, _I, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _code(q, op), _ptr(block_tables),
             block_tables.shape[1], _ptr(row_seq), _ptr(positions), T, heads, kv_heads, dim, vdim, kcache.shape[2], int(window),
             float(scale), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, float(out_scale), int(chunk),
             float(softcap), _ptr(r1), _ptr(r2), int(pool), _stream()), op)


# ------------------------------------------------------------------------------------ attention
@_timed
def paged_attention(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal GQA attention of every row of q [T, H*hd] over its request's pages.
    block_tables int32 [S, max_pages]; row_seq, positions int32 [T]; window 0 = all keys."""
    op = "paged_attention"
    _cuda(op, q, out, kcache, vcache, block_tables, row_seq, positions)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    T = q.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape or out.dtype != q.dtype:
        raise ShapeError(op, f"q and out must be [{T}, {num_heads * head_dim}] of one dtype, got {list(q.shape)} "
                             f"{q.dtype} and {list(out.shape)} {out.dtype}")
    if num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
        raise ShapeError(op, f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
    if head_dim % 8 != 0 or head_dim > 256:
        raise ShapeError(op, f"head_dim {head_dim} is not supported (multiples of 8 up to 256)")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous() or c.dtype != q.dtype:
            raise ShapeError(op, f"{name} must be contiguous {q.dtype} [pages, {num_kv_heads}, page_size, {head_dim}], "
                                 f"got {c.dtype} {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if kcache.numel() // head_dim >= 2 ** 31:
        raise ShapeError(op, "one layer's cache has 2^31 rows or more")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, f"block_tables must be contiguous int32 [S, max_pages], got {block_tables.dtype} {list(block_tables.shape)}")
    _int32_vec(row_seq, T, op, "row_seq")
    _int32_vec(positions, T, op, "positions")
    f = _fn("attention", "vob_paged_attention",
            [_P, _L, _P, _L, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _code(q, op),
             _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), T, num_heads,
             num_kv_heads, head_dim, kcache.shape[2], int(window), float(scale), _stream()), op)


def attn_mma_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, decode: bool) -> bool:
    """Whether the tensor-core attention kernels take these sizes (bfloat16 only)."""
    if head_dim not in TENSOR_CORE_HEAD_DIMS:
        return False                      # answered here: a model of another head size never builds the module
    f = _fn("attention_mma", "vob_attn_mma_supported", [_I, _I, _I, _I, _I])
    return bool(f(num_heads, num_kv_heads, head_dim, page_size, int(decode)))


def _attn_tail(op, q, sink, gate, num_heads, out_scale):
    """Checked arguments of what may follow the weighted sum: a sink per head (float32 [H]), a gate ([T, H * hd] bfloat16,
    any row stride: the result times its sigmoid) and a constant factor."""
    _cuda(op, q, sink, gate)
    _f32_vec(sink, num_heads, op, "sink")
    if gate is not None:
        _rows_2d(gate, op, "gate")
        if gate.shape != q.shape or gate.dtype != torch.bfloat16:
            raise ShapeError(op, f"gate must be bfloat16 {list(q.shape)}, got {gate.dtype} {list(gate.shape)}")
    return _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, float(out_scale)


def _score_shape(op, q, num_heads, chunk, softcap, dist_bias):
    """Checked arguments of what may shape a score before the softmax, or None where there is nothing: blocks of `chunk`
    positions (a query reads its own block's keys only), score <- softcap * tanh(score / softcap), and dist_bias = (r1, r2),
    float32 [H] each: r1 * ln(1 + r2 * distance) taken off."""
    if not chunk and not softcap and dist_bias is None:
        return None
    if chunk < 0 or softcap < 0:
        raise ShapeError(op, f"blocks of {chunk} and a cap of {softcap} must not be negative")
    r1, r2 = dist_bias if dist_bias is not None else (None, None)
    _cuda(op, q, r1, r2)
    _f32_vec(r1, num_heads, op, "dist_bias[0]")
    _f32_vec(r2, num_heads, op, "dist_bias[1]")
    return int(chunk), float(softcap), _ptr(r1), _ptr(r2)


def _attn_common_checks(op, q, out, kcache, vcache, block_tables, num_heads, num_kv_heads, head_dim):
    _cuda(op, q, out, kcache, vcache, block_tables)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
        raise ShapeError(op, "the tensor-core attention kernels are bfloat16 only")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise ShapeError(op, f"q and out must be [T, {num_heads * head_dim}], got {list(q.shape)} and {list(out.shape)}")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous [pages, {num_kv_heads}, page_size, {head_dim}], got {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, "block_tables must be contiguous int32 [S, max_pages]")
    if q.stride(0) % 8 != 0 or q.data_ptr() % 16 != 0 or out.stride(0) % 2 != 0 or out.data_ptr() % 4 != 0:
        raise ShapeError(op, "q rows must be 16-byte aligned and out rows 4-byte aligned")
    if not attn_mma_supported(num_heads, num_kv_heads, head_dim, kcache.shape[2], False):
        raise ShapeError(op, f"sizes not supported by the tensor-core kernels: heads {num_heads}/{num_kv_heads}, "
                             f"head_dim {head_dim}, page {kcache.shape[2]} (head_dim 64 or 128, page size dividing 64)")


@_timed
def attn_prefill_mma(q, out, kcache, vcache, block_tables, seq_starts, context_lens, num_seqs: int, max_new: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0, sink=None, gate=None,
                     out_scale: float = 1.0) -> None:
    """Tensor-core attention for portions of prompts and mixed batches (bfloat16). q/out [T, H*hd];
    seq_starts int32 [S+1] (first row of each request), context_lens int32 [S] (keys cached before
    the step), max_new = the longest portion. `sink`, `gate`, `out_scale`: see `_attn_tail`."""
    op = "attn_prefill_mma"
    if not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _attn_common_checks(op, q, out, kcache, vcache, block_tables, num_heads, num_kv_heads, head_dim)
    _cuda(op, seq_starts, context_lens)
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(context_lens, num_seqs, op, "context_lens")
    if block_tables.shape[0] < num_seqs:
        raise ShapeError(op, f"block_tables has {block_tables.shape[0]} rows for {num_seqs} requests")
    tail = _attn_tail(op, q, sink, gate, num_heads, out_scale)
    f = _fn("attention_mma", "vob_attn_prefill_mma",
            [_P, _L, _P, _L, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _L, _F, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
             block_tables.shape[1], _ptr(seq_starts), _ptr(context_lens), num_seqs, max_new, num_heads, num_kv_heads,
             head_dim, kcache.shape[2], int(window), float(scale), *tail, _stream()), op)


def attn_prefill_mma_any_supported(num_heads: int, num_kv_heads: int, dim: int, vdim: int, page_size: int) -> bool:
    """Whether the portion kernel for keys and values of sizes of their own takes these (bfloat16 only): multiples of 8 up to
    128 each, a page size that divides 64."""
    return (num_kv_heads > 0 and num_heads % num_kv_heads == 0 and 0 < dim <= 128 and 0 < vdim <= 128 and dim % 8 == 0
            and vdim % 8 == 0 and page_size > 0 and 64 % page_size == 0)


@_timed
def attn_prefill_mma_any(q, out, kcache, vcache, block_tables, seq_starts, context_lens, num_seqs: int, max_new: int,
                         num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, window: int = 0, sink=None, gate=None,
                         out_scale: float = 1.0, chunk: int = 0, softcap: float = 0.0, dist_bias=None, pooled=None) -> None:
    """Tensor-core attention for portions of prompts and mixed batches (bfloat16) with keys of `dim` and values of `vdim`
    features: q [T, H * dim], out [T, H * vdim] (any row stride), kcache [pages, KV, page, dim], vcache [pages, KV, page, vdim].
    The tiles in shared memory are padded with zero columns to the sizes the kernel is built for. Everything else as
    `attn_prefill_mma`. `chunk`, `softcap`, `dist_bias`: see `_score_shape` (the kernel built for shaped scores runs then).
    `pooled` = (kpool, vpool, pool), with a window: beside the window's tokens a query at position p sees the first
    floor((p + 1 - window) / pool) entries of kpool and vpool (laid out like the caches, entry b where a token at position b
    would be: the mean key and value of tokens b * pool .. b * pool + pool - 1, as `pool_blocks` leaves them)."""
    op = "attn_prefill_mma_any"
    shape = _score_shape(op, q, num_heads, chunk, softcap, dist_bias)
    pool_args = (_P(0), _P(0), 0)
    if pooled is not None:
        kpool, vpool, pool = pooled
        _cuda(op, q, kpool, vpool)
        if kpool.shape != kcache.shape or vpool.shape != vcache.shape or kpool.dtype != kcache.dtype or vpool.dtype != vcache.dtype \
                or not kpool.is_contiguous() or not vpool.is_contiguous():
            raise ShapeError(op, "the pooled entries are laid out like the caches")
        if pool <= 0 or window <= 0 or chunk or dist_bias is not None:
            raise ShapeError(op, "pooled entries go with a window, without blocks of positions and without a distance bias")
        pool_args = (_ptr(kpool), _ptr(vpool), int(pool))
        if shape is None:
            shape = (0, 0.0, _P(0), _P(0))
    if shape is None and not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _cuda(op, q, out, kcache, vcache, block_tables, seq_starts, context_lens)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    T = q.shape[0]
    if any(t.dtype != torch.bfloat16 for t in (q, out, kcache, vcache)):
        raise ShapeError(op, "the tensor-core attention kernels are bfloat16 only")
    if q.shape[1] != num_heads * dim or out.shape != (T, num_heads * vdim):
        raise ShapeError(op, f"q [{T}, {num_heads * dim}] and out [{T}, {num_heads * vdim}] are needed, got {list(q.shape)} and {list(out.shape)}")
    _kv_caches(op, kcache, vcache, num_kv_heads, dim, vdim, torch.bfloat16)
    if not attn_prefill_mma_any_supported(num_heads, num_kv_heads, dim, vdim, kcache.shape[2]):
        raise ShapeError(op, f"sizes not supported: heads {num_heads}/{num_kv_heads}, sizes {dim}/{vdim}, page {kcache.shape[2]}")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous() or block_tables.shape[0] < num_seqs:
        raise ShapeError(op, f"block_tables must be contiguous int32 [>= {num_seqs}, max_pages]")
    if q.stride(0) % 8 != 0 or q.data_ptr() % 16 != 0 or out.stride(0) % 2 != 0 or out.data_ptr() % 4 != 0:
        raise ShapeError(op, "q rows must be 16-byte aligned and out rows 4-byte aligned")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(context_lens, num_seqs, op, "context_lens")
    _cuda(op, q, sink, gate)
    _f32_vec(sink, num_heads, op, "sink")
    if gate is not None:
        _rows_2d(gate, op, "gate")
        if gate.shape != out.shape or gate.dtype != torch.bfloat16:
            raise ShapeError(op, f"gate must be bfloat16 {list(out.shape)}, got {gate.dtype} {list(gate.shape)}")
    sig = [_P, _L, _P, _L, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _L, _F]
    args = (_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
            block_tables.shape[1], _ptr(seq_starts), _ptr(context_lens), num_seqs, max_new, num_heads, num_kv_heads,
            dim, vdim, kcache.shape[2], int(window), float(scale), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
            float(out_scale))
    if shape is None:
        _check(_fn("attention_mma", "vob_attn_prefill_mma_any", sig + [_P])(*args, _stream()), op)
    else:
        _check(_fn("attention_mma", "vob_attn_prefill_shaped", sig + [_I, _F, _P, _P, _P, _P, _I, _P])(*args, *shape, *pool_args, _stream()), op)


def attn_prefill_sm100_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, max_pages: int) -> bool:
    """Whether the tcgen05 attention kernel for prompt portions takes these sizes (bfloat16, no window)."""
    if head_dim not in TENSOR_CORE_HEAD_DIMS:
        return False
    f = _fn("attention_sm100", "vob_attn_prefill_sm100_supported", [_I, _I, _I, _I, _I])
    return bool(f(num_heads, num_kv_heads, head_dim, page_size, max_pages))


@_timed
def attn_prefill_sm100(q, out, kcache, vcache, block_tables, seq_starts, context_lens, num_seqs: int, max_new: int,
                       num_heads: int, num_kv_heads: int, head_dim: int, scale: float, sink=None) -> None:
    """`sink` (float32 [H], optional): exp(sink[head]) joins every row's softmax denominator, a key with no value.
    Attention for portions of prompts and mixed batches on the tcgen05 tensor cores (bfloat16,
    head_dim 64 or 128, no window): Q, K and V tiles by TMA straight from the pages of the cache, scores
    and output in tensor memory. Arguments as `attn_prefill_mma`."""
    op = "attn_prefill_sm100"
    if not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _cuda(op, q, out, kcache, vcache, block_tables, seq_starts, context_lens)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
        raise ShapeError(op, "the tensor-core attention kernels are bfloat16 only")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise ShapeError(op, f"q and out must be [T, {num_heads * head_dim}], got {list(q.shape)} and {list(out.shape)}")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous [pages, {num_kv_heads}, page_size, {head_dim}], got {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, "block_tables must be contiguous int32 [S, max_pages]")
    if block_tables.shape[0] < num_seqs:
        raise ShapeError(op, f"block_tables has {block_tables.shape[0]} rows for {num_seqs} requests")
    for name, t in (("q", q), ("out", out)):
        if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
            raise ShapeError(op, f"{name} rows must be 16-byte aligned")
    if not attn_prefill_sm100_supported(num_heads, num_kv_heads, head_dim, kcache.shape[2], block_tables.shape[1]):
        raise ShapeError(op, f"sizes not supported: heads {num_heads}/{num_kv_heads}, head_dim {head_dim}, page "
                             f"{kcache.shape[2]}, {block_tables.shape[1]} pages per request (head_dim 64 or 128, at most 128 "
                             "heads per kv head, page size a power of two from 8 to 128)")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(context_lens, num_seqs, op, "context_lens")
    _cuda(op, q, sink)
    _f32_vec(sink, num_heads, op, "sink")
    f = _fn("attention_sm100", "vob_attn_prefill_sm100",
            [_P, _L, _L, _P, _L, _P, _P, _L, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P])
    _check(f(_ptr(q), q.shape[0], q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), kcache.shape[0],
             _ptr(block_tables), block_tables.shape[1], _ptr(seq_starts), _ptr(context_lens), num_seqs, max_new, num_heads,
             num_kv_heads, head_dim, kcache.shape[2], float(scale), _ptr(_scratch_for(q.device).err), _ptr(sink), _stream()), op)


@_timed
def attn_decode_mma(q, out, kcache, vcache, block_tables, positions, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int = 0, splits: int = 1, partials=None, arrived=None, sink=None, gate=None,
                    out_scale: float = 1.0, chunk: int = 0, softcap: float = 0.0, dist_bias=None) -> None:
    """`sink`, `gate`, `out_scale`: see `_attn_tail`; `chunk`, `softcap`, `dist_bias`: see `_score_shape`.
    Tensor-core attention for a step of single tokens, row i belonging to request i (bfloat16).
    With splits > 1 (at most 8) each request's keys are shared out over the blocks of a cluster,
    which merge their partial results through distributed shared memory. With `partials` (float32,
    `attn_decode_partial_floats` elements) and `arrived` (int32 zeros, one per request and kv head;
    the kernel leaves them zero) up to 64 blocks share a request without a cluster and merge
    through global memory: for few requests with long contexts."""
    op = "attn_decode_mma"
    shape = _score_shape(op, q, num_heads, chunk, softcap, dist_bias)
    if shape is None and not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _attn_common_checks(op, q, out, kcache, vcache, block_tables, num_heads, num_kv_heads, head_dim)
    _cuda(op, positions)
    S = q.shape[0]
    _int32_vec(positions, S, op, "positions")
    if block_tables.shape[0] < S:
        raise ShapeError(op, f"block_tables has {block_tables.shape[0]} rows for {S} requests")
    if num_heads // num_kv_heads > 16:
        raise ShapeError(op, f"{num_heads // num_kv_heads} heads per kv head: the decode kernel takes at most 16")
    if (partials is None) != (arrived is None):
        raise ShapeError(op, "partials and arrived go together")
    most = 8 if partials is None else 64
    if not 1 <= splits <= most:
        raise ShapeError(op, f"splits must be 1..{most}, got {splits}")
    if partials is not None:
        _cuda(op, partials, arrived)
        need = attn_decode_partial_floats(S, num_kv_heads, head_dim, splits)
        if partials.dtype != torch.float32 or not partials.is_contiguous() or partials.numel() < need or partials.data_ptr() % 16:
            raise ShapeError(op, f"partials must be contiguous float32, 16-byte aligned, with at least {need} elements")
        if arrived.dtype != torch.int32 or not arrived.is_contiguous() or arrived.numel() < S * num_kv_heads:
            raise ShapeError(op, f"arrived must be contiguous int32 with at least {S * num_kv_heads} elements")
    tail = _attn_tail(op, q, sink, gate, num_heads, out_scale)
    sig = [_P, _L, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P, _P, _P, _L, _F]
    args = (_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
            block_tables.shape[1], _ptr(positions), S, num_heads, num_kv_heads, head_dim, kcache.shape[2], int(window),
            float(scale), int(splits), _ptr(partials), _ptr(arrived), *tail)
    if shape is None:
        _check(_fn("attention_mma", "vob_attn_decode_mma", sig + [_P])(*args, _stream()), op)
    else:
        _check(_fn("attention_mma", "vob_attn_decode_shaped", sig + [_I, _F, _P, _P, _P])(*args, *shape, _stream()), op)


def attn_decode_partial_floats(num_seqs: int, num_kv_heads: int, head_dim: int, splits: int) -> int:
    """Elements of the float32 scratch that `attn_decode_mma` needs for its merge through global memory."""
    return num_seqs * num_kv_heads * splits * (16 * head_dim + 32)


# ------------------------------------------------------------------------------------ sampling
def pick_tiles(vocab: int) -> int:
    """Pairs per row that the output head's picking epilogue (EPI_PICK) leaves: one per 128 logits."""
    return -(-int(vocab) // 128)


class HostInts:
    """A page-locked host buffer of int32 that kernels write to directly (`also` of the pick
    functions): `tensor` is the host's view, `address` what the device reaches it under."""

    def __init__(self, shape):
        self.tensor = torch.zeros(shape, dtype=torch.int32, pin_memory=True)
        f = _fn("sampling", "vob_host_device_pointer", [_P, _P])
        dev = ctypes.c_void_p()
        rc = f(_P(self.tensor.data_ptr()), ctypes.byref(dev))
        if rc != 0 or not dev.value:
            raise KernelError(f"the device cannot address page-locked host memory (error {rc})")
        self.address = int(dev.value)

    def at(self, element: int) -> "_Address":
        if not 0 <= element <= self.tensor.numel():
            raise ShapeError("HostInts", f"element {element} lies outside {self.tensor.numel()} elements")
        return _Address(self.address + 4 * element, self.tensor.numel() - element)


class _Address:
    """A raw device-reachable address with the int32 elements that follow it."""

    def __init__(self, address: int, elements: int):
        self.address, self.elements = address, elements


def _also_pointers(op: str, also, rows: int):
    """Up to two further places the picked tokens go to: int32 device tensors or addresses of a `HostInts`."""
    if len(also) > 2:
        raise ShapeError(op, f"at most two further destinations, got {len(also)}")
    ptrs = []
    for a in also:
        if isinstance(a, _Address):
            if a.elements < rows:
                raise ShapeError(op, f"a further destination has room for {a.elements} of {rows} tokens")
            ptrs.append(_P(a.address))
        else:
            _cuda(op, a)
            _int32_vec(a, rows, op, "a further destination")
            ptrs.append(_ptr(a))
    return ptrs + [_P(0)] * (2 - len(ptrs))


@_timed
def pick_final(part_val: torch.Tensor, part_idx: torch.Tensor, rows: int, vocab: int, nan_flags: torch.Tensor,
               out: torch.Tensor, also=()) -> None:
    """The pick's second pass alone: out[r] = index of the best of row r's (value, index) pairs
    (part_val / part_idx [>= rows, pairs per row]); -1 for a row whose NaN flag is up (the flag is cleared).
    `also`: up to two further places the same tokens are written to."""
    op = "pick_final"
    _cuda(op, part_val, part_idx, nan_flags, out)
    if (part_val.dtype != torch.float32 or part_idx.dtype != torch.int32 or part_val.dim() != 2 or part_val.shape != part_idx.shape
            or part_val.shape[0] < rows or not part_val.is_contiguous() or not part_idx.is_contiguous()):
        raise ShapeError(op, f"part_val float32 and part_idx int32 must be contiguous [>={rows}, pairs], got {list(part_val.shape)} "
                             f"and {list(part_idx.shape)}")
    _int32_vec(out, rows, op, "out")
    _int32_vec(nan_flags, rows, op, "nan_flags")
    a, b = _also_pointers(op, also, rows)
    f = _fn("sampling", "vob_pick_final_to", [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P])
    _check(f(_ptr(part_val), _ptr(part_idx), rows, part_val.shape[1], int(vocab), _ptr(nan_flags), _ptr(out), a, b, _stream()), op)


def pick_splits(vocab: int) -> int:
    f = _fn("sampling", "vob_pick_splits", [_I])
    return int(f(vocab))


@_timed
def pick_tokens(logits: torch.Tensor, out: torch.Tensor, nan_flags: torch.Tensor, scratch_val: torch.Tensor,
                scratch_idx: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                seeds: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None, also=()) -> None:
    """One token per row of float32 logits [R, V]: greedy where temperature is 0 or absent,
    Gumbel-max sampling elsewhere. seeds int32 [R, 2] (low, high word), steps int32 [R]
    (index of the generated token), nan_flags int32 [R] raised for rows that hold a NaN.
    scratch_val float32 and scratch_idx int32 need R * pick_splits(V) elements each.
    `also`: up to two further places the same tokens are written to."""
    op = "pick_tokens"
    _cuda(op, logits, out, nan_flags, scratch_val, scratch_idx, temperature, seeds, steps)
    _rows_2d(logits, op, "logits")
    if logits.dtype != torch.float32:
        raise ShapeError(op, f"logits must be float32, got {logits.dtype}")
    R, V = logits.shape
    splits = pick_splits(V)
    _int32_vec(out, R, op, "out")
    _int32_vec(nan_flags, R, op, "nan_flags")
    if scratch_val.dtype != torch.float32 or scratch_val.numel() < R * splits or not scratch_val.is_contiguous():
        raise ShapeError(op, f"scratch_val must hold {R * splits} float32")
    if scratch_idx.dtype != torch.int32 or scratch_idx.numel() < R * splits or not scratch_idx.is_contiguous():
        raise ShapeError(op, f"scratch_idx must hold {R * splits} int32")
    if temperature is not None:
        if temperature.dtype != torch.float32 or temperature.numel() < R or not temperature.is_contiguous():
            raise ShapeError(op, f"temperature must be float32 [{R}]")
        if seeds is None or steps is None:
            raise ShapeError(op, "temperature sampling needs seeds and steps")
        if seeds.dtype != torch.int32 or seeds.numel() < 2 * R or not seeds.is_contiguous():
            raise ShapeError(op, f"seeds must be int32 [{R}, 2]")
        _int32_vec(steps, R, op, "steps")
    a, b = _also_pointers(op, also, R)
    f = _fn("sampling", "vob_pick_tokens_to", [_P, _L, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(seeds), _ptr(steps), splits,
             _ptr(scratch_val), _ptr(scratch_idx), _ptr(nan_flags), _ptr(out), a, b, _stream()), op, launches=2)
