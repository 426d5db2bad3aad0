"""The Pironex decoder in the engine against the plain implementation (tests/plain/pironex_plain.py): small
configurations made here, random weights, float32 and bfloat16. Each mechanism alone (the kernels on inputs made so that
a fault shows: one key that stands out far back inside a pooled block, at a page's border, just inside and just outside
the window, in the block that is just seen and the one that is not yet; the convolution's state over portions of one and
two tokens; the state-space scan in portions against token by token; a gate beyond its limit), models of one layer, whole
prompts against tokens one by one, portions down to two tokens, unequal requests side by side against each alone, pages
and state slots that are given back and used again, long decoding over windows and blocks, and greedy generation through
`LLM`, the command line and the trace program."""
import json
import os
import random

import pytest
import torch

from tests.plain import pironex_plain as plain
from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _configs():
    from vllm_oxide_b200.config import (ClampedExpertsConfig as FF, PironexConfig as C, PironexLayer as L, PooledAttentionConfig as AT,
                                        StateSpaceConfig as SS, WindowLatentConfig as LA)
    att = AT(heads=4, kv_heads=2, dim=24, vdim=40, scale=0.2, softcap=6.0, rot_dims=8, rot_base=100.0, window=10, pool=4)
    att_reader = AT(heads=6, kv_heads=2, dim=24, vdim=40, scale=0.3, softcap=3.0, rot_dims=8, rot_base=100.0, window=7, pool=3, kv_from=1)
    att_small = AT(heads=3, kv_heads=3, dim=10, vdim=6, scale=0.35, window=5, pool=8)                       # blocks longer than the window
    att_win = AT(heads=2, kv_heads=1, dim=16, vdim=8, scale=0.25, softcap=10.0, rot_dims=16, rot_base=50.0, window=9)   # nothing behind it
    att_all = AT(heads=1, kv_heads=1, dim=8, vdim=8, scale=0.4)                                             # every earlier token
    att_one = AT(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.4, softcap=2.0, window=1, pool=1)              # itself, and every other token as a block
    att_tc = AT(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.1, softcap=8.0, rot_dims=32, rot_base=10000.0, window=40)
    att_tc_pool = AT(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.12, rot_dims=32, rot_base=10000.0, window=16, pool=8, kv_from=0)
    ssm = SS(heads=4, vdim=16, state=8, groups=2, norm_groups=1, conv=3)
    ssm_b = SS(heads=3, vdim=8, state=12, groups=3, norm_groups=3, conv=2)
    ssm_one = SS(heads=2, vdim=12, state=5, groups=1, norm_groups=2, conv=1)                                # no convolution state
    lat = LA(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=32, scale=0.2, rot_base=1000.0, window=13)
    lat_all = LA(heads=2, dim=10, rot_dim=6, vdim=6, kv_rank=20, scale=0.3, rot_base=30.0)                  # no window; sizes the tensor cores do not take
    lat_tc = LA(heads=4, dim=32, rot_dim=16, vdim=16, kv_rank=48, scale=0.15, rot_base=10000.0, window=20)
    moe = FF(ff=24, limit=1.0, experts=6, top=2, shared_ff=40, shared_limit=2.5)
    moe_one = FF(ff=20, limit=0.7, experts=5, top=1)                                                        # one choice, no shared expert
    moe_three = FF(ff=16, limit=3.0, experts=5, top=3, shared_ff=8, shared_limit=0.5)
    return {
        "A": C(vocab=97, width=64, norm_eps=1e-5, embedding_scale=6.0, canon_taps=3, layers=(
            L("mamba2", ssm=ssm, mlp=moe), L("attention", attention=att, mlp=moe), L("latent_attention", latent=lat, mlp=None),
            L("attention", attention=att_reader, mlp=moe_one), L("mamba2", ssm=ssm_b, mlp=None))),
        # a width that is no multiple of 4 or 8, one tap (no convolution state), a latent layer first
        "B": C(vocab=131, width=42, norm_eps=1e-6, embedding_scale=1.0, canon_taps=1, layers=(
            L("latent_attention", latent=lat_all, mlp=moe_three), L("attention", attention=att_small, mlp=moe_one),
            L("attention", attention=att_win, mlp=None), L("mamba2", ssm=ssm_one, mlp=moe_three),
            L("attention", attention=att_all, mlp=None), L("attention", attention=att_one, mlp=None))),
        # sizes of the tensor-core kernels, four taps, no `canon` would be `canon_taps=0`
        "T": C(vocab=77, width=96, norm_eps=1e-5, embedding_scale=3.0, canon_taps=4, layers=(
            L("attention", attention=att_tc, mlp=moe), L("latent_attention", latent=lat_tc, mlp=moe_one),
            L("attention", attention=att_tc_pool, mlp=None), L("mamba2", ssm=ssm, mlp=moe))),
        "attention": C(vocab=50, width=48, norm_eps=1e-5, canon_taps=2, layers=(L("attention", attention=att, mlp=None),)),
        "mamba2": C(vocab=50, width=48, norm_eps=1e-5, canon_taps=0, layers=(L("mamba2", ssm=ssm, mlp=None),)),
        "latent": C(vocab=50, width=48, norm_eps=1e-5, canon_taps=3, layers=(L("latent_attention", latent=lat, mlp=None),)),
        "moe": C(vocab=50, width=48, norm_eps=1e-5, canon_taps=3, layers=(L("attention", attention=att_one, mlp=moe),)),
    }


def _model_dir(tmp_path, name, seed=11):
    """Random weights; routers, step sizes, decays, skips and the depth weights are made large enough to matter."""
    from vllm_oxide_b200.models import pironex_manifest
    from vllm_oxide_b200.weights import random_tensors
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    from vllm_oxide_b200.config.model_config import write_config_json
    d = os.path.join(str(tmp_path), f"pironex_{name}_{seed}")
    if os.path.exists(os.path.join(d, "model.safetensors")):
        return d
    cfg = _configs()[name]
    tensors = random_tensors(pironex_manifest(cfg), seed, 0.25, torch.bfloat16, "cpu", norm_jitter=0.3)
    g = torch.Generator().manual_seed(seed)
    for n in list(tensors):
        shape = tensors[n].shape
        if n.endswith(".router"):
            tensors[n] = (tensors[n].float() * 6).bfloat16()
        elif n.endswith(".dwa"):
            tensors[n] = (torch.rand(shape, generator=g) * 0.8 + 0.2).bfloat16()
        elif n.endswith(".A_log"):
            tensors[n] = (torch.rand(shape, generator=g) * 2 - 2).bfloat16()
        elif n.endswith(".dt_bias") or n.endswith(".conv.b") or n.endswith(".D"):
            tensors[n] = torch.randn(shape, generator=g).bfloat16()
        elif n.endswith(".mix.in") or n.endswith(".mix.q") or n.endswith(".mix.k"):
            tensors[n] = (tensors[n].float() * 2).bfloat16()
    os.makedirs(d, exist_ok=True)
    write_config_json(d, cfg.to_dict())
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


def _plain_logits(model_dir, tokens, layers_out=None):
    from safetensors.torch import load_file
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    tensors = load_file(os.path.join(model_dir, "model.safetensors"))
    want = plain.forward(cfg, tensors, tokens, torch.float64, layers_out)
    low = plain.forward(cfg, tensors, tokens, torch.float32).double()       # what float32 rounding alone does to each row
    want.spread = (low - want).abs().amax(-1) / want.abs().max()
    return want


def _runner(model_dir, dtype, page=8, pages=24, max_seqs=3, rows=192):
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import ModelRunner
    eng = EngineConfig(max_batch_tokens=rows, max_seqs=max_seqs, max_model_len=page * pages, block_size=page, num_pages=pages,
                       dtype=dtype, cuda_graphs=False)
    return ModelRunner.from_dir(model_dir, eng)


def _tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


TOL = {"float32": 3e-5}


def _row_errors(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


def _close(got, want, dtype) -> bool:
    """float32: every logit within TOL of the largest, plus twice what float32 rounding does to that row of the plain model.
    bfloat16: the typical row tight (a router's close call may go to another expert than in float64, so single rows are
    judged in float32 only; a key that is skipped, a window one token off or a lost state moves all later rows by far more)."""
    if dtype == "float32":
        rows = (got.double().cpu() - want).abs().amax(-1) / want.abs().max()
        return bool((rows < TOL[dtype] + 2 * getattr(want, "spread", 0.0)).all())
    err = _row_errors(got, want)
    return float(err.median()) < 4e-2 and float(err.quantile(0.7)) < 1e-1


def _poison(runner):
    """Whatever lies in pages that nobody holds must never be read."""
    for ts in runner.pools.kv.values():
        for t in ts:
            t.fill_(float("nan"))


def _replay(session, reqs, schedule, first_step=0):
    """schedule: a list of steps, each a list of (name, count). Returns {name: logits of all its tokens}."""
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for n, step in enumerate(schedule):
        entries, end = [], []
        for name, count in step:
            lo = at[name]
            entries.append({"id": name, "tokens": reqs[name][lo:lo + count], "want": list(range(count))})
            at[name] = lo + count
            if at[name] == len(reqs[name]):
                end.append(name)
        out = session.run_step({"step": first_step + n, "entries": entries, "end": end})
        r = 0
        for name, count in step:
            got[name].append(out[r:r + count])
            r += count
    return {k: torch.cat(v) for k, v in got.items() if v}


def _diff(a, b) -> float:
    return max_rel_diff(a.detach().cpu(), b.detach().cpu())


def _ints(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------------------------ small kernels
def test_layer_norm_without_bias_depth_average_and_clamped_gate():
    from vllm_oxide_b200 import kernels
    torch.manual_seed(0)
    for h in (42, 64, 300):
        resid, delta = torch.randn(5, h, device=DEV) * 3, torch.randn(5, h, device=DEV) * 2 + 0.7
        w = torch.randn(h, device=DEV)
        want = resid.double() + plain.layer_norm(delta.double(), w.double(), 1e-5)
        kernels.layernorm_add(resid, delta, w, None, 1e-5)
        assert _diff(resid, want) < 2e-6
        out = torch.empty(5, h, device=DEV)
        kernels.layernorm_rows(resid, w, None, 1e-5, out)
        assert _diff(out, plain.layer_norm(resid.double(), w.double(), 1e-5)) < 2e-6
    # the stream as a weighted sum over depth: slot 0 is filed, then each result is filed and the sum handed on
    T, h, slots = 7, 42, 4
    stack = torch.full((T, slots, h), float("nan"), device=DEV)
    x0 = torch.randn(T, h, device=DEV)
    x = x0.clone()
    kernels.depth_average(stack, x, None, 0)
    assert torch.equal(x, x0) and torch.equal(stack[:, 0], x0)
    results = [x0.double()]
    for n in (1, 2, 3):
        new = torch.randn(T, h, device=DEV)
        w = torch.randn(n + 1, device=DEV)
        x.copy_(new)
        kernels.depth_average(stack, x, w, n)
        results.append(new.double())
        want = sum(w[j].double() * results[j] for j in range(n + 1))
        assert _diff(x, want) < 2e-6 and torch.equal(stack[:, n], new)
    # the same sum, and a convolution's state moved on, done by the norm behind a sub-layer on its way
    for dt in (torch.float32, torch.bfloat16):
        for h in (42, 64):
            T, slots, taps = 9, 3, 3
            stack = torch.randn(T, slots, h, device=DEV)
            stack2 = stack.clone()
            resid, delta = torch.randn(T, h, device=DEV), torch.randn(T, h, device=DEV).to(dt)
            resid2 = resid.clone()
            w, dw = torch.randn(h, device=DEV), torch.randn(3, device=DEV)
            cx = torch.randn(T, h, device=DEV).to(dt)
            state = torch.randn(4, taps - 1, h, device=DEV)
            state2 = state.clone()
            pos, row_seq, starts, slots_ = _ints([5, 6, 7, 0, 3, 4, 5, 6, -1]), _ints([0, 0, 0, 1, 2, 2, 2, 2, 0]), _ints([0, 3, 4, 8]), _ints([2, 0, 3])
            kernels.layernorm_add(resid, delta, w, None, 1e-5, depth=(stack, dw, 2), conv=(cx, state, row_seq, starts, slots_, pos))
            kernels.layernorm_add(resid2, delta, w, None, 1e-5)
            kernels.depth_average(stack2, resid2, dw, 2)
            kernels.conv_state_update(cx, 0, state2, starts, slots_, 3)
            assert torch.equal(resid, resid2) and torch.equal(stack, stack2) and torch.equal(state, state2)
    # the clamped gate: values beyond the limit on both sides of both halves
    for dt in (torch.float32, torch.bfloat16):
        gu = (torch.randn(6, 2 * 30 + 8, device=DEV) * 3).to(dt)
        out = torch.empty(6, 30, dtype=dt, device=DEV)
        kernels.glu_clamped(gu[:, :60], out, 1.25)
        g, u = gu[:, :30].double().clamp(max=1.25), gu[:, 30:60].double().clamp(-1.25, 1.25)
        assert _diff(out, g * torch.sigmoid(1.702 * g) * (u + 1)) < (1e-6 if dt == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,residual,act", [(3, True, "none"), (4, False, "silu"), (2, True, "none"), (1, True, "none")])
def test_causal_convolution_with_its_state_over_short_portions(dtype, taps, residual, act):
    """Two requests in slots 2 and 0, cut into portions of 1, 2, 5 ... tokens: every row equals the convolution over the
    whole sequence, and the state a finished request leaves does not reach the request that takes its slot."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(taps)
    C, spare = 37, 3
    w, bias = torch.randn(C, taps, device=DEV), (torch.randn(C, device=DEV) if act == "silu" else None)
    xs = {0: torch.randn(23, C).to(dtype), 1: torch.randn(9, C).to(dtype)}
    state = torch.full((3, max(taps - 1, 1), C), float("nan"), device=DEV)[:, :taps - 1] if taps > 1 else None
    if state is not None:
        state = state.contiguous()
        state[2].zero_(), state[0].zero_()
    slots = {0: 2, 1: 0}
    at = {0: 0, 1: 0}
    got = {0: [], 1: []}
    for step in ([(0, 1)], [(0, 2), (1, 1)], [(1, 1), (0, 5)], [(0, 1), (1, 2)], [(0, 14), (1, 5)]):
        rows = torch.cat([xs[r][at[r]:at[r] + n] for r, n in step])
        wide = torch.full((rows.shape[0], C + spare), float("nan"), dtype=dtype, device=DEV)
        wide[:, :C] = rows.to(DEV)
        pos = _ints([p for r, n in step for p in range(at[r], at[r] + n)])
        row_seq = _ints([i for i, (r, n) in enumerate(step) for _ in range(n)])
        starts = _ints([0] + torch.tensor([n for _, n in step]).cumsum(0).tolist())
        ss = _ints([slots[r] for r, _ in step])
        out = torch.empty(rows.shape[0], C, dtype=torch.float32, device=DEV)
        kernels.causal_conv(wide[:, :C], w.t().contiguous(), bias, state, pos, row_seq, starts, ss, len(step), out, residual=residual, act=act)
        if state is not None:
            kernels.conv_state_update(wide, 0, state, starts, ss, len(step))
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n])
            at[r] += n
            o += n
    for r in xs:
        x = xs[r].double()
        want = plain.causal_conv(x, w.double().cpu(), bias.double().cpu() if bias is not None else None) + (x if residual else 0)
        if act == "silu":
            want = plain.silu(want)
        assert _diff(torch.cat(got[r]), want) < 3e-6, r
    if state is not None:
        # a step in which every request brings one token: the kernel moves the state on itself, bit for bit as the two kernels do
        for width in (C, 40):       # channels one by one, and 16 bytes a thread
            st_a = torch.randn(3, taps - 1, width, device=DEV)
            st_b = st_a.clone()
            x = torch.randn(2, width).to(dtype).to(DEV)
            wt = torch.randn(taps, width, device=DEV)
            b2 = torch.randn(width, device=DEV) if bias is not None else None
            args = (_ints([7, 3]), _ints([0, 1]), _ints([0, 1, 2]), _ints([2, 0]), 2)
            out_a, out_b = (torch.empty(2, width, dtype=dtype, device=DEV) for _ in range(2))
            kernels.causal_conv(x, wt, b2, st_a, *args, out_a, residual=residual, act=act)
            kernels.conv_state_update(x, 0, st_a, args[2], args[3], 2)
            kernels.causal_conv(x, wt, b2, st_b, *args, out_b, residual=residual, act=act, single=True)
            assert torch.equal(out_a, out_b) and torch.equal(st_a, st_b)
    if state is not None:       # a new request in slot 0 starts from zeros
        state[0].zero_()
        x = torch.randn(2, C).to(dtype)
        out = torch.empty(2, C, dtype=torch.float32, device=DEV)
        kernels.causal_conv(x.to(DEV), w.t().contiguous(), bias, state, _ints([0, 1]), _ints([0, 0]), _ints([0, 2]), _ints([0]), 1, out, residual=residual, act=act)
        want = plain.causal_conv(x.double(), w.double().cpu(), bias.double().cpu() if bias is not None else None) + (x.double() if residual else 0)
        assert _diff(out, plain.silu(want) if act == "silu" else want) < 3e-6


# ------------------------------------------------------------------------------------ attention with pooled blocks
def _paged(total, page, heads_widths, dtype, spare=3):
    """Block tables over scattered pages for requests of `total` tokens; cache tensors full of NaN."""
    pages_per = [-(-t // page) for t in total]
    n = sum(pages_per) + spare
    perm = torch.randperm(n)
    tables = torch.full((len(total), max(pages_per) + 2), -1, dtype=torch.int32)
    at = 0
    for s, pp in enumerate(pages_per):
        tables[s, :pp] = perm[at:at + pp].to(torch.int32)
        at += pp
    caches = [torch.full((n, h, page, w), float("nan"), dtype=dtype, device=DEV) for h, w in heads_widths]
    return tables, caches


def _fill(cache, tables, s, x, page, first=0):
    idx = torch.arange(first, x.shape[0])
    pg, off = tables[s, idx // page].long(), idx % page
    cache[pg.to(DEV), :, off.to(DEV)] = x[first:].to(device=DEV, dtype=cache.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,DV,window,pool,cap", [(4, 2, 24, 40, 10, 4, 6.0), (3, 3, 10, 6, 5, 8, 0.0), (2, 1, 16, 8, 9, 0, 10.0),
                                                       (2, 2, 8, 8, 1, 1, 2.0), (8, 2, 96, 80, 24, 8, 20.0), (2, 1, 64, 64, 7, 3, 0.0)])
def test_pooled_window_attention_with_one_key_that_stands_out(dtype, H, G, D, DV, window, pool, cap):
    """Rows at many positions of a request of 150 tokens over scattered pages of 16. For each tested row one key is
    scaled so that its score stands out, placed in turn: at the window's oldest token and just outside it, inside the
    newest block that is seen (where it counts with a pool-th of its weight) and in the block that is not seen yet (it
    must not count at all), in block 0 far back, at a page's last slot, and at position 0."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(H * 100 + D)
    total, page, scale = 150, 16, 0.3
    tables, (kc, vc) = _paged([total, 40], page, [(G, D), (G, DV)], dtype)
    k0, v = torch.randn(total, G, D) * 0.3, torch.randn(total, G, DV)
    rows = [0, 1, window - 1, window, window + pool - 1, window + pool, 31, 32, 77, 149]
    for i in rows:
        n_seen = max(0, (i - window + 1) // pool) if pool else 0
        marks = {0, max(0, i - window + 1), max(0, i - window), 15, 16}
        if n_seen:
            marks |= {n_seen * pool - 1, (n_seen - 1) * pool}
        if pool:
            marks.add(min(i, n_seen * pool))                    # the first token of the block that is not seen yet
        for mark in sorted(m for m in marks if m <= i):
            k = k0.clone()
            q = torch.randn(1, H, D)
            k[mark] = q[0].reshape(G, H // G, D)[:, 0] * 4      # one key that answers the first head of every group
            k, vv, q = k.to(dtype), v.to(dtype), q.to(dtype)
            _fill(kc, tables, 0, k, page)
            _fill(vc, tables, 0, vv, page)
            out = torch.empty(1, H * DV, dtype=dtype, device=DEV)
            kernels.flex_attention(q.reshape(1, -1).to(DEV), out, kc, vc, tables.to(DEV), _ints([0]), _ints([i]), H, G, D, DV, scale,
                                   window, None, None, 1.0, 0, cap, None, pool)
            want = plain.pooled_window_attention(torch.cat([torch.zeros(i, H, D, dtype=torch.float64), q.double()]), k.double()[:i + 1],
                                                 vv.double()[:i + 1], scale, cap, window, pool, rows=[i])[i].reshape(1, -1)
            assert _diff(out, want) < (3e-6 if dtype == torch.float32 else 2e-2), (i, mark)
            if dtype == torch.bfloat16 and pool and D % 8 == 0 and DV % 8 == 0:
                # the same row on the tensor cores, over pooled entries that `pool_blocks` leaves beside the caches
                kp, vp = torch.full_like(kc, float("nan")), torch.full_like(vc, float("nan"))
                kernels.pool_blocks(kc, vc, kp, vp, tables.to(DEV), _ints([0] * (i + 1)), _ints(list(range(i + 1))), pool)
                out2 = torch.empty(1, H * DV, dtype=dtype, device=DEV)
                kernels.attn_prefill_mma_any(q.reshape(1, -1).to(DEV), out2, kc, vc, tables.to(DEV), _ints([0, 1]), _ints([i]), 1, 1, H, G, D, DV,
                                             scale, window, None, None, 1.0, softcap=cap, pooled=(kp, vp, pool))
                assert _diff(out2, want) < 3e-2, (i, mark, "tensor cores")
    if dtype == torch.bfloat16 and pool and D % 8 == 0 and DV % 8 == 0:
        # a portion of 70 rows behind 80 cached tokens, and the same rows one by one: every row against the plain function
        k, vv = k0.to(dtype), v.to(dtype)
        q = (torch.randn(total, H, D) * 2).to(dtype)
        _fill(kc, tables, 0, k, page)
        _fill(vc, tables, 0, vv, page)
        kp, vp = torch.full_like(kc, float("nan")), torch.full_like(vc, float("nan"))
        kernels.pool_blocks(kc, vc, kp, vp, tables.to(DEV), _ints([0] * total), _ints(list(range(total))), pool)
        want = plain.pooled_window_attention(q.double(), k.double(), vv.double(), scale, cap, window, pool, rows=range(80, total))[80:].reshape(70, -1)
        out = torch.empty(70, H * DV, dtype=dtype, device=DEV)
        kernels.attn_prefill_mma_any(q[80:].reshape(70, -1).to(DEV), out, kc, vc, tables.to(DEV), _ints([0, 70]), _ints([80]), 1, 70, H, G, D, DV,
                                     scale, window, None, None, 1.0, softcap=cap, pooled=(kp, vp, pool))
        assert _diff(out, want) < 3e-2
        for i in (80, 95, 96, 149):
            one = torch.empty(1, H * DV, dtype=dtype, device=DEV)
            kernels.attn_prefill_mma_any(q[i].reshape(1, -1).to(DEV), one, kc, vc, tables.to(DEV), _ints([0, 1]), _ints([i]), 1, 1, H, G, D, DV,
                                         scale, window, None, None, 1.0, softcap=cap, pooled=(kp, vp, pool))
            assert _diff(one, want[i - 80:i - 79]) < 3e-2, i


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_the_whole_projection_before_the_rotation(dtype):
    """q and k are divided by the root mean square of ALL their heads' features and multiplied by a weight per feature, then
    rotated; a layer without keys prepares its queries only."""
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.parts.rotary import rotary_inv_freq
    torch.manual_seed(3)
    H, G, D, DV, rot, page, T, eps = 3, 1, 24, 8, 8, 8, 6, 1e-5
    nq, nk, nv = H * D, G * D, G * DV
    proj = torch.randn(T, nq + nk + nv + 5).to(dtype)
    qw, kw = torch.rand(nq) + 0.5, torch.rand(nk) + 0.5
    pos = [3, 4, 5, 0, 1, 17]
    inv = torch.from_numpy(rotary_inv_freq(rot, 100.0).copy())
    tables, (kc, vc) = _paged([24], page, [(G, D), (G, DV)], dtype)
    slots = [int(tables[0, p // page]) * page + p % page for p in pos]
    q = torch.empty(T, nq, dtype=dtype, device=DEV)
    kernels.flex_prep(proj.to(DEV), 0, nq, nq + nk, _ints(pos), _ints(slots), inv.to(DEV), rot, False, eps, None, None, None, 0, q, kc, vc,
                      H, G, D, DV, None, None, qw.to(DEV), kw.to(DEV))
    p64 = proj.double()
    want_q = plain.rotate_half((plain.rms(p64[:, :nq], eps) * qw.double()).reshape(T, H, D), torch.tensor(pos), rot, 100.0).reshape(T, -1)
    want_k = plain.rotate_half((plain.rms(p64[:, nq:nq + nk], eps) * kw.double()).reshape(T, G, D), torch.tensor(pos), rot, 100.0)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    assert _diff(q, want_q) < tol
    got_k = torch.stack([kc[s // page, :, s % page] for s in slots])
    assert _diff(got_k, want_k) < tol
    q2 = torch.empty(T, nq, dtype=dtype, device=DEV)
    kernels.flex_prep(proj.to(DEV), 0, 0, 0, _ints(pos), None, inv.to(DEV), rot, False, eps, None, None, None, 0, q2, None, None,
                      H, G, D, DV, None, None, qw.to(DEV), None)
    assert torch.equal(q2, q)


# ------------------------------------------------------------------------------------ the mixers as parts, one request in portions
def _step_ctx(runner_like, positions, row_seq, starts, slots, tables, slot_map, dtype, max_new, decode_only):
    from vllm_oxide_b200.parts.base import StepContext, Workspace
    n, s = len(positions), len(slots)
    return StepContext(rows=n, seqs=s, dtype=dtype, tokens=_ints([0] * n), positions=_ints(positions), row_seq=_ints(row_seq),
                       seq_starts=_ints(starts), context_lens=_ints([0] * s), seq_lens=_ints([0] * s), state_slots=_ints(slots),
                       logit_rows=_ints([0]), slot_mapping=[_ints(slot_map)] if slot_map is not None else [],
                       block_tables=[tables.to(DEV)] if tables is not None else [], workspace=Workspace(64 << 20, DEV),
                       max_new=max_new, decode_only=decode_only)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G,NG,taps", [(4, 16, 8, 2, 1, 3), (3, 8, 12, 3, 3, 2), (2, 12, 5, 1, 2, 1), (6, 32, 32, 2, 2, 4)])
def test_state_space_mixer_in_portions_and_token_by_token(dtype, H, P, N, G, NG, taps):
    """One request whole, then in portions of 1, 2, 7 ... tokens, then token by token in a slot that was used before: the
    state and the convolution's last inputs carry over exactly."""
    from vllm_oxide_b200.parts.recurrent import StateSpace
    torch.manual_seed(H + taps)
    width, T = 40, 29
    inner, chans = H * P, H * P + 2 * G * N
    t = {"in": torch.randn(2 * inner + 2 * G * N + H, width) * 0.3, "conv": torch.randn(chans, taps) * 0.5, "conv.b": torch.randn(chans) * 0.3,
         "dt_bias": torch.randn(H), "A_log": torch.rand(H) * 2 - 2, "D": torch.randn(H), "norm": torch.rand(inner) + 0.5,
         "o": torch.randn(width, inner) * 0.2}
    t = {k: v.bfloat16() for k, v in t.items()}
    mixer = StateSpace(t["in"], t["conv"], t["conv.b"], t["dt_bias"], t["A_log"], t["D"], t["norm"], t["o"], H, P, N, G, NG, 1e-5, dtype, DEV)
    x = torch.randn(T, width).to(dtype)
    m = {"heads": H, "vdim": P, "state": N, "groups": G, "norm_groups": NG, "conv": taps}
    want = plain.mamba2_mixer(x.double(), {k: v.double() for k, v in t.items()}, "", m, 1e-5)
    specs = mixer.state_spec()
    state = tuple(torch.full((3,) + tuple(s.shape), float("nan"), device=DEV) for s in specs)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for slot, cuts in ((1, [T]), (2, [1, 2, 7, 1, 1, 17]), (1, [1] * T)):
        for s in state:
            s[slot].zero_()
        got, at = [], 0
        for n in cuts:
            ctx = _step_ctx(None, list(range(at, at + n)), [0] * n, [0, n], [slot], None, None, dtype, n, n == 1)
            got.append(mixer.forward(x[at:at + n].to(DEV), ctx, None, state).clone())
            at += n
        assert _diff(torch.cat(got), want) < tol, cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,V,L,window", [(3, 16, 8, 24, 32, 13), (2, 10, 6, 6, 20, 0), (4, 32, 16, 16, 48, 20), (6, 32, 16, 32, 64, 33)])
def test_latent_attention_in_a_window_with_a_key_just_inside_and_just_outside(dtype, H, D, R, V, L, window):
    """One request of 70 tokens through the mixer: whole (portions on the tensor cores where the sizes allow), in portions,
    token by token. The token `window` behind row 60 is given a latent that answers row 60's query many times over: it
    must not count; the one just inside the window does."""
    from vllm_oxide_b200.parts.base import LayerCache
    from vllm_oxide_b200.parts.latent_attention import LatentAttention
    torch.manual_seed(H + L)
    width, T, page = 40, 70, 8
    t = {"q": torch.randn(H * (D + R), width) * 0.3, "dkv": torch.randn(L + R, width) * 0.3, "dkv.norm": torch.rand(L) + 0.5,
         "uk": torch.randn(H * D, L) * 0.3, "uv": torch.randn(H * V, L) * 0.3, "o": torch.randn(width, H * V) * 0.2}
    t = {k: v.bfloat16() for k, v in t.items()}
    mixer = LatentAttention(t["q"], t["dkv"], t["dkv.norm"], t["uk"], t["uv"], t["o"], H, D, R, V, L, 0.4, 500.0, 1e-5, dtype, DEV,
                            window=window, pairing="interleaved")
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": L, "scale": 0.4, "rot": {"base": 500.0, "dims": R}}
    if window:
        m["mask"] = {"size": window}
    t64 = {k: v.double() for k, v in t.items()}
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    for case in ("inside", "outside") if window else ("inside",):
        x = torch.randn(T, width)
        mark = 60 - window + (1 if case == "inside" else 0) if window else 3
        x[mark] = x[60] * 3                                    # a token much like row 60's own: a large score from there
        x = x.to(dtype)
        want = plain.latent_mixer(x.double(), t64, "", m, 1e-5)
        if window:      # the plain model itself tells a window that is one token off
            other = dict(m, mask={"size": window + (1 if case == "outside" else -1)})
            assert _diff(plain.latent_mixer(x.double(), t64, "", other, 1e-5), want) > 1e-2
        for cuts in ([T], [5, 2, 33, 1, 29], [40] + [1] * 30):
            tables, caches = _paged([T], page, [(1, L), (1, R)], dtype)
            cache = LayerCache(tensors=tuple(caches), group=0, write=True)
            got, at = [], 0
            for n in cuts:
                pos = list(range(at, at + n))
                slot_map = [int(tables[0, p // page]) * page + p % page for p in pos]
                ctx = _step_ctx(None, pos, [0] * n, [0, n], [0], tables, slot_map, dtype, n, n == 1)
                got.append(mixer.forward(x[at:at + n].to(DEV), ctx, cache, None).clone())
                at += n
            assert _diff(torch.cat(got), want) < tol, (case, cuts)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,width,ff,E,top,shared", [(9, 48, 24, 6, 2, 40), (70, 42, 20, 5, 1, 0), (33, 64, 16, 5, 3, 8), (600, 64, 32, 4, 2, 16)])
def test_clamped_experts_with_a_shared_expert(dtype, T, width, ff, E, top, shared):
    """The routed feed-forward against every chosen expert done plainly: logits far apart (no close calls), gate and up
    values on both sides of their limits, the shared expert behind its sigmoid."""
    from vllm_oxide_b200.parts.moe import RoutedExperts
    torch.manual_seed(T)
    t = {"router": torch.randn(E, width) * 3}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"] = torch.randn(ff, width) * 0.4, torch.randn(ff, width) * 0.4, torch.randn(width, ff) * 0.3
    if shared:
        t["shared.gate"], t["shared.up"] = torch.randn(shared, width) * 0.4, torch.randn(shared, width) * 0.4
        t["shared.down"], t["shared.sg"] = torch.randn(width, shared) * 0.3, torch.randn(1, width)
    t = {k: v.bfloat16() for k, v in t.items()}
    sh = (t["shared.gate"], t["shared.up"], t["shared.down"], t["shared.sg"], 0.8) if shared else None
    part = RoutedExperts(t["router"], [t[f"e{e}.gate"] for e in range(E)], [t[f"e{e}.up"] for e in range(E)],
                         [t[f"e{e}.down"] for e in range(E)], top, renormalize=True, dtype=dtype, device=DEV, activation="clamped_swish",
                         limit=1.1, shared=sh)
    x = torch.randn(T, width).to(dtype)
    m = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 1.1}}
    if shared:
        m["shared"] = {"ff": shared, "limit": 0.8}
    want = plain.moe(x.double(), {k: v.double() for k, v in t.items()}, "", m)
    ctx = _step_ctx(None, list(range(T)), [0] * T, [0, T], [0], None, None, dtype, T, False)
    got = part.forward(x.to(DEV), ctx)
    if dtype == torch.float32:
        assert _diff(got, want) < 1e-5
    else:
        err = _row_errors(got, want)
        assert float(err.median()) < 2e-2 and float(err.quantile(0.9)) < 6e-2


# ------------------------------------------------------------------------------------ models in the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "mamba2", "latent", "moe"])
def test_each_mechanism_alone_whole_prompt_and_token_by_token(tmp_path, name, dtype):
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    toks = _tokens(45, 50, 5)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype)
    _poison(runner)
    s = TraceSession(runner)
    whole = _replay(s, {"a": toks}, [[("a", 45)]])["a"]
    assert _close(whole, want, dtype)
    _poison(runner)
    single = _replay(s, {"b": toks}, [[("b", 19)]] + [[("b", 1)]] * 26, first_step=10)["b"]
    assert _close(single, want, dtype)
    if dtype == "float32":
        assert _diff(single, whole) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "T"])
def test_portions_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Four requests of unequal length in a pool that cannot hold them all at once: portions from 2 tokens up beside single
    tokens, portions that end inside a page, a window and a pooled block, a request that sits out a step, a fourth request
    that takes over a slot and pages that were given back in the middle. Every row equals the plain model's."""
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    vocab = _configs()[name].vocab
    reqs = {"a": _tokens(61, vocab, 1), "b": _tokens(23, vocab, 2), "c": _tokens(3, vocab, 3), "d": _tokens(34, vocab, 4)}
    want = {k: _plain_logits(d, v) for k, v in reqs.items()}
    runner = _runner(d, dtype, page=8, pages=16, max_seqs=3)        # 128 tokens of cache for 121, three slots for four requests
    _poison(runner)
    s = TraceSession(runner)
    schedule = [[("a", 2), ("b", 17)], [("a", 30), ("c", 2), ("b", 1)], [("b", 1), ("c", 1)], [("a", 7), ("b", 2)],
                [("d", 9), ("a", 1), ("b", 2)], [("a", 1), ("d", 2)], [("d", 1), ("a", 19)], [("d", 22), ("a", 1)]]
    got = _replay(s, reqs, schedule)
    for k in reqs:
        assert got[k].shape[0] == len(reqs[k])
        assert _close(got[k], want[k], dtype), k
    assert runner.manager.num_free_slots() == 3 and runner.manager.check_invariants() == ""
    for k in reqs:
        alone = _replay(s, {k: reqs[k]}, [[(k, len(reqs[k]))]], first_step=100)[k]
        if dtype == "float32":
            assert _diff(alone, got[k]) < 5e-6, k
        else:
            err = _row_errors(got[k], alone)
            assert float(err.median()) < 1.5e-2 and float(err.quantile(0.9)) < 6e-2, (k, float(err.median()), float(err.quantile(0.9)))


def test_the_norm_behind_a_sub_layer_doing_more_on_its_way_changes_nothing(tmp_path):
    """`TUNING.norm_tail`: the convolutions' state and the sum over depth done by the norm kernel itself, bit for bit what
    the separate kernels give, over portions, single tokens and a slot that is used again."""
    from vllm_oxide_b200.replay.trace import TraceSession
    from vllm_oxide_b200.tuning import TUNING
    d = _model_dir(tmp_path, "A")
    reqs = {"a": _tokens(40, 97, 1), "b": _tokens(9, 97, 2), "c": _tokens(17, 97, 3)}
    schedule = [[("a", 2), ("b", 7)], [("a", 1), ("b", 2)], [("c", 3), ("a", 30)], [("a", 7), ("c", 14)]]
    got = {}
    before = TUNING.norm_tail
    try:
        for mode in (0, 1):
            TUNING.norm_tail = mode
            runner = _runner(d, "float32", page=8, pages=16, max_seqs=2)
            got[mode] = _replay(TraceSession(runner), reqs, schedule)
    finally:
        TUNING.norm_tail = before
    for k in reqs:
        assert torch.equal(got[0][k], got[1][k]), k
        assert _close(got[1][k], _plain_logits(d, reqs[k]), "float32"), k


def test_the_shared_expert_beside_the_routed_ones_changes_nothing(tmp_path):
    """`TUNING.moe_side_stream`: in steps of single tokens the shared expert runs on a second stream; the same bits, with
    decode steps launched one by one and replayed from CUDA graphs."""
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.sampling import SamplingParams
    from vllm_oxide_b200.tuning import TUNING
    d = _model_dir(tmp_path, "A")
    prompts = [_tokens(n, 97, 60 + n) for n in (11, 4, 23)]
    got = {}
    before = TUNING.moe_side_stream
    try:
        for mode in (0, 1):
            for graphs in (False, True):
                TUNING.moe_side_stream = mode
                eng = EngineConfig(max_batch_tokens=64, max_seqs=3, max_model_len=64, block_size=8, num_pages=24, dtype="bfloat16", cuda_graphs=graphs)
                llm = LLM(ModelRunner.from_dir(d, eng))
                got[(mode, graphs)] = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_new_tokens=16, stop_token_ids=()))]
                if graphs:
                    assert llm.runner.decode_graphs and llm.runner._graphs
    finally:
        TUNING.moe_side_stream = before
    assert got[(0, False)] == got[(1, False)] == got[(0, True)] == got[(1, True)]


def test_the_stream_after_every_layer(tmp_path):
    """Layer by layer in float32: the stream that the engine's blocks hand on (the weighted sum over depth) equals the plain model's."""
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, "A")
    toks = _tokens(50, 97, 8)
    layers = []
    _plain_logits(d, toks, layers)
    runner = _runner(d, "float32")
    seen = []
    runner.after_block = lambda i, resid, pending: seen.append(resid[:len(toks)].clone())
    _replay(TraceSession(runner), {"a": toks}, [[("a", len(toks))]])
    assert len(seen) == len(layers)
    for i, (got, want) in enumerate(zip(seen, layers[:len(seen)])):
        assert _diff(got.cpu(), want) < 1e-5, i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_long_decoding_over_page_borders_windows_and_blocks(tmp_path, name, dtype):
    """150 tokens, all but six of them one by one: windows of 7 to 40 pass over decoded tokens, pooled blocks of 3, 4 and 8
    come into sight one after the other, the window groups give their pages back on the way, and the state-space layers'
    state is carried through 144 steps."""
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    toks = _tokens(150, _configs()[name].vocab, 9)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype, page=8, pages=20, max_seqs=2)
    _poison(runner)
    got = _replay(TraceSession(runner), {"a": toks}, [[("a", 6)]] + [[("a", 1)]] * 144)["a"]
    assert _close(got, want, dtype)


def test_a_window_one_token_off_or_a_mechanism_left_out_would_show(tmp_path):
    """The plain model with every window one token longer, blocks one token longer, without the cap, the convolutions, the
    depth weights, the shared expert or the skip differs from itself by far more than the tolerance: the tests above can tell."""
    d = _model_dir(tmp_path, "A")
    from safetensors.torch import load_file
    toks = _tokens(60, 97, 1)
    tensors = load_file(os.path.join(d, "model.safetensors"))

    def run(change):
        cfg = json.load(open(os.path.join(d, "config.json")))
        t = dict(tensors)
        change(cfg, t)
        return plain.forward(cfg, t, toks, torch.float64)
    want = run(lambda c, t: None)

    def mixers(c, kind):
        return [x["mixer"] for x in c["layers"] if x["type"] == kind]

    def longer_window(c, t):
        for m in mixers(c, "attention"):
            m["mask"]["size"] += 1

    def longer_latent_window(c, t):
        for m in mixers(c, "latent_attention"):
            m["mask"]["size"] += 1

    def longer_blocks(c, t):
        for m in mixers(c, "attention"):
            m["mask"]["pool"] += 1

    def no_blocks(c, t):
        for m in mixers(c, "attention"):
            m["mask"].pop("pool")

    def no_cap(c, t):
        for m in mixers(c, "attention"):
            m.pop("softcap", None)

    def zero(suffix):
        def change(c, t):
            for n in t:
                if n.endswith(suffix):
                    t[n] = torch.zeros_like(t[n])
        return change

    def flat_depth(c, t):
        for n in t:
            if n.endswith(".dwa"):
                t[n] = torch.cat([torch.zeros_like(t[n][:-1]), torch.ones_like(t[n][-1:])])
    for change in (longer_window, longer_latent_window, longer_blocks, no_blocks, no_cap, zero(".canon1"), zero(".canon2"), zero(".mix.D"),
                   zero(".shared.down"), zero(".conv.b"), flat_depth):
        assert _diff(run(change), want) > 1e-3, getattr(change, "__name__", change)


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(tmp_path, graphs):
    """More requests than state slots and a pool that forces preemption and recomputation: every generated token is the
    plain model's argmax given what came before. With CUDA graphs the decode steps are recorded and replayed."""
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.sampling import SamplingParams
    d = _model_dir(tmp_path, "A")
    eng = EngineConfig(max_batch_tokens=64, max_seqs=3, max_model_len=64, block_size=8, num_pages=9, dtype="float32", cuda_graphs=graphs)
    llm = LLM(ModelRunner.from_dir(d, eng))
    prompts = [_tokens(n, 97, 20 + n) for n in (14, 9, 17, 5, 2)]
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=12, stop_token_ids=()))
    for prompt, o in zip(prompts, outs):
        assert len(o.token_ids) == 12
        logits = _plain_logits(d, list(prompt) + o.token_ids)
        for i, tok in enumerate(o.token_ids):
            row = logits[len(prompt) - 1 + i]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(row.abs().max()):          # a near tie may fall either way
                assert tok == int(row.argmax()), (i, tok)
    assert llm.runner.manager.num_free_slots() == 3 and llm.runner.manager.check_invariants() == ""
    if graphs:
        assert llm.runner.decode_graphs and llm.runner._graphs


def test_greedy_generation_in_bfloat16_with_graphs(tmp_path):
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.sampling import SamplingParams
    d = _model_dir(tmp_path, "T")
    prompts = [_tokens(n, 77, 40 + n) for n in (33, 6, 50)]
    eng = EngineConfig(max_batch_tokens=128, max_seqs=4, max_model_len=128, block_size=16, num_pages=24, dtype="bfloat16", cuda_graphs=True)
    llm = LLM(ModelRunner.from_dir(d, eng))
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=20, stop_token_ids=()))
    for prompt, o in zip(prompts, outs):
        assert len(o.token_ids) == 20
        logits = _plain_logits(d, list(prompt) + o.token_ids)
        for i, tok in enumerate(o.token_ids):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.08 * float(row.abs().max()), (i, tok)
    assert llm.runner.decode_graphs and llm.runner._graphs


def test_command_line_generates_from_a_pironex_folder(tmp_path):
    import subprocess
    import sys
    d = _model_dir(tmp_path, "B")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "vllm_oxide_b200", "generate", d, "--prompt-ids", "5,9,2,44", "--max-new", "6", "--dtype", "float32",
                        "--max-model-len", "64", "--max-batch-tokens", "64", "--max-seqs", "2", "--num-pages", "16"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(x) for x in r.stdout.split()]
    toks = [5, 9, 2, 44]
    assert len(got) == 6
    logits = _plain_logits(d, toks + got)
    assert got[0] == int(logits[3].argmax())


def test_trace_program_replays_a_pironex_folder(tmp_path):
    """bin/trace_run on a model folder: a prompt in two portions and two single tokens, logits of chosen places."""
    import subprocess
    import numpy as np
    d = _model_dir(tmp_path, "B")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = _tokens(30, 131, 77)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:11], "want": [10]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[11:28], "want": [0, 16]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[28:29], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": toks[29:], "want": [0]}], "end": ["x"]}]
    out = os.path.join(str(tmp_path), "trace_out")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    want = _plain_logits(d, toks)
    assert not os.path.exists(os.path.join(out, "2.f32"))
    for step, places in ((0, [10]), (1, [11, 27]), (3, [29])):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(len(places), 131))
        assert _diff(got, want[places]) < TOL["float32"]
