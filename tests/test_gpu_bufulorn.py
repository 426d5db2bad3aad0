"""The Bufulorn decoder in the engine against the plain implementation (tests/plain/bufulorn_plain.py): small
configurations made here, random weights, float32 and bfloat16. Each mechanism alone (the kernels on inputs made so
that a fault shows: one key far back in the block, at a page's border, the first key of the block and, with a weight
that would swamp the row, the last key of the block before; scores beyond the cap; a distance bias that decides; an
expert that is best but sits in a group that is not kept), models of one layer, whole prompts against tokens one by
one, portions down to two tokens, unequal requests side by side against each alone, pages and state slots that are
given back and used again, long decoding over block edges, and greedy generation through `LLM` and the command line."""
import json
import os
import random

import pytest
import torch

from tests.plain import bufulorn_plain as plain
from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _configs():
    from vllm_oxide_b200.config import (BufulornConfig as C, BufulornLayer as L, ChunkAttentionConfig as AT, FeedForwardConfig as FF,
                                        HeadDecayDeltaConfig as GD)
    att = AT(heads=4, kv_heads=2, dim=24, vdim=40, scale=0.2, softcap=6.0, chunk=21)
    att_reader = AT(heads=6, kv_heads=2, dim=24, vdim=40, scale=0.3, softcap=3.0, chunk=21, kv_from=0)      # other head count, scale, cap
    att_small = AT(heads=3, kv_heads=3, dim=10, vdim=6, scale=0.35, chunk=5)                               # no cap; sizes no vector load takes
    att_all = AT(heads=2, kv_heads=1, dim=16, vdim=8, scale=0.25, softcap=10.0)                             # no blocks: every earlier key
    att_other = AT(heads=2, kv_heads=1, dim=16, vdim=8, scale=0.5, chunk=13, kv_from=1)                     # a block length its source has not
    att_one = AT(heads=1, kv_heads=1, dim=8, vdim=8, scale=0.4, softcap=2.0, chunk=1)                       # sees itself only
    att_tc = AT(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.1, softcap=8.0, chunk=48)                     # sizes of the tensor-core kernels
    att_tc_reader = AT(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.12, softcap=5.0, chunk=48, kv_from=0)
    att_96 = AT(heads=2, kv_heads=1, dim=96, vdim=32, scale=0.08, softcap=20.0, chunk=70)
    delta = GD(heads=4, kv_heads=2, dim=16, vdim=24, conv=3)
    delta_wide = GD(heads=2, kv_heads=2, dim=40, vdim=8, conv=4)
    delta_one = GD(heads=3, kv_heads=1, dim=8, vdim=12, conv=1)                                            # no convolution state at all
    dense = FF("dense", 96)
    moe = FF("moe", 24, experts=8, top=2, groups=4, keep=3)
    moe_plain = FF("moe", 20, experts=5, top=1)                                                            # no groups, one choice
    moe_all = FF("moe", 16, experts=6, top=3, groups=2, keep=2)                                            # every group kept
    return {
        "A": C(vocab=97, width=64, norm_eps=1e-5, max_positions=160, layers=(
            L("attention", attention=att, mlp=dense), L("delta", delta=delta, mlp=moe), L("attention", attention=att_reader, mlp=moe_all),
            L("delta", delta=delta_wide, mlp=None), L("attention", attention=att, mlp=dense))),
        # a width that is no multiple of 4 or 8, a delta layer first, a reader whose block length differs from its source's
        # (the cache keeps everything), a layer without feed-forward in the middle
        "B": C(vocab=131, width=42, norm_eps=1e-6, max_positions=200, layers=(
            L("delta", delta=delta_one, mlp=moe_plain), L("attention", attention=att_all, mlp=None),
            L("attention", attention=att_small, mlp=FF("dense", 50)), L("attention", attention=att_other, mlp=moe_plain),
            L("attention", attention=att_one, mlp=None))),
        "T": C(vocab=77, width=96, norm_eps=1e-5, max_positions=256, layers=(
            L("attention", attention=att_tc, mlp=dense), L("attention", attention=att_tc_reader, mlp=moe),
            L("delta", delta=delta, mlp=dense), L("attention", attention=att_96, mlp=moe))),
        "attention": C(vocab=50, width=48, norm_eps=1e-5, max_positions=64, layers=(L("attention", attention=att, mlp=None),)),
        "delta": C(vocab=50, width=48, norm_eps=1e-5, max_positions=64, layers=(L("delta", delta=delta, mlp=None),)),
        "dense": C(vocab=50, width=48, norm_eps=1e-5, max_positions=64, layers=(L("attention", attention=att_one, mlp=dense),)),
        "moe": C(vocab=50, width=48, norm_eps=1e-5, max_positions=64, layers=(L("attention", attention=att_one, mlp=moe),)),
    }


def _model_dir(tmp_path, name, seed=11):
    """Random weights; the distance bias, the activation's two numbers and the router are made large enough to matter."""
    from vllm_oxide_b200.models import bufulorn_manifest
    from vllm_oxide_b200.weights import random_tensors
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    from vllm_oxide_b200.config.model_config import write_config_json
    d = os.path.join(str(tmp_path), f"bufulorn_{name}_{seed}")
    if os.path.exists(os.path.join(d, "model.safetensors")):
        return d
    cfg = _configs()[name]
    tensors = random_tensors(bufulorn_manifest(cfg), seed, 0.25, torch.bfloat16, "cpu", norm_jitter=0.3)
    g = torch.Generator().manual_seed(seed)
    for n in list(tensors):
        if n.endswith(".r1") or n.endswith(".r2"):
            tensors[n] = (torch.rand(tensors[n].shape, generator=g) * 1.5 + 0.05).bfloat16()
        elif n.endswith(".router"):
            tensors[n] = (tensors[n].float() * 6).bfloat16()
        elif n.endswith("norm1.b") or n.endswith("norm2.b") or n.endswith("final.norm.b"):
            tensors[n] = (torch.randn(tensors[n].shape, generator=g) * 0.2).bfloat16()
        elif n.endswith(".act"):
            tensors[n] = torch.tensor([0.4, -0.7]).bfloat16()
    os.makedirs(d, exist_ok=True)
    write_config_json(d, cfg.to_dict())
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


def _plain_logits(model_dir, tokens, layers_out=None):
    from safetensors.torch import load_file
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    tensors = load_file(os.path.join(model_dir, "model.safetensors"))
    want = plain.forward(cfg, tensors, tokens, torch.float64, layers_out)
    # what float32 rounding alone does to each row, measured on the plain model itself: a row where it loses digits
    # (a router's softmax near a tie, a small variance under a norm) is judged by that
    low = plain.forward(cfg, tensors, tokens, torch.float32).double()
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


def _close(got, want, dtype) -> bool:
    """float32: every logit within TOL of the largest, plus twice what float32 rounding does to that row of the plain
    model (a key that is left out moves a row by a thousand times that). bfloat16: the typical row tight (root mean square of a row's
    error against that of its logits: the median over the rows under 4 %, and seven rows in ten under 10 %).
    A row whose router's choice is a close call may go to another expert in bfloat16 than in float64 (the routers of these
    models are made sharp, and where one expert in five is chosen the whole feed-forward changes with it), so single rows
    are judged in float32 only; a key that is skipped, a wrong page, a block one token off or a lost state moves all
    later rows by far more."""
    if dtype == "float32":
        spread = getattr(want, "spread", None)
        if spread is None:
            return max_rel_diff(got, want) < TOL[dtype]
        rows = (got.double().cpu() - want).abs().amax(-1) / want.abs().max()
        return bool((rows < TOL[dtype] + 2 * spread).all())
    err = _row_errors(got, want)
    return float(err.median()) < 4e-2 and float(err.quantile(0.7)) < 1e-1


def _row_errors(got, want):
    """Per row: the root mean square of the difference over that of `want`."""
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


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


# ------------------------------------------------------------------------------------ small kernels
def test_learned_positions_layer_norm_and_xielu():
    from vllm_oxide_b200 import kernels
    torch.manual_seed(0)
    table, ptab = torch.randn(20, 42, device=DEV).bfloat16(), torch.randn(9, 42, device=DEV).bfloat16()
    toks = torch.tensor([3, 19, 0, 5], dtype=torch.int32, device=DEV)
    pos = torch.tensor([8, 0, 3, -1], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 42, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embed(table, toks, out, flag, 1.0, ptab, pos)
    assert torch.equal(out[:3], table[toks[:3].long()].float() + ptab[pos[:3].long()].float())
    assert torch.equal(out[3], table[5].float()) and int(flag) == 0           # a padding row gets no position vector
    kernels.embed(table, toks, out, flag, 1.0, ptab, torch.tensor([8, 9, 3, 0], dtype=torch.int32, device=DEV))
    assert int(flag) == 1                                                      # a position beyond the table is reported
    for h in (42, 64, 300, 2052):           # single features, four at a time, and more than one turn of four a thread
        for dt in (torch.float32, torch.bfloat16):
            resid, delta = torch.randn(5, h, device=DEV) * 3, (torch.randn(5, h, device=DEV) * 2 + 0.7).to(dt)
            w, b = torch.randn(h, device=DEV), torch.randn(h, device=DEV)
            want = resid.double() + plain.layer_norm(delta.double(), w.double(), b.double(), 1e-5)
            copy = torch.empty(5, h, dtype=dt, device=DEV)
            kernels.layernorm_add(resid, delta, w, b, 1e-5, copy)
            assert max_rel_diff(resid, want) < 2e-6
            assert torch.equal(copy, resid.to(dt))
            rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
            picked = torch.empty(2, h, dtype=dt, device=DEV)
            before = resid.clone()
            kernels.layernorm_rows(resid, w, b, 1e-5, picked, rows)            # looked at only: the residual stays
            assert torch.equal(resid, before)
            assert max_rel_diff(picked, plain.layer_norm(before.double(), w.double(), b.double(), 1e-5)[[4, 1]]) < (2e-6 if dt == torch.float32 else 1e-2)
            rounded = torch.empty(5, h, dtype=dt, device=DEV)
            kernels.cast_rows(resid, rounded)
            assert torch.equal(rounded, resid.to(dt))
    # a row whose entries are large and nearly equal: the variance is the mean of the squared deviations, not E[x^2] - mean^2
    resid, delta = torch.zeros(1, 64, device=DEV), (1000.0 + torch.randn(1, 64, device=DEV) * 0.01)
    w, b = torch.ones(64, device=DEV), torch.zeros(64, device=DEV)
    kernels.layernorm_add(resid, delta, w, b, 1e-5)
    # (float32 holds the mean of such a row to half a unit in its last place, 3e-5 here, a few thousandths of the deviations)
    assert max_rel_diff(resid, plain.layer_norm(delta.double(), w.double(), b.double(), 1e-5)) < 1e-2
    p, q = torch.tensor(0.3), torch.tensor(-0.8)
    params = torch.tensor([float(plain.softplus(p)), 0.5 + float(plain.softplus(q))], device=DEV)
    for cols, spare in ((30, 3), (300, 3), (300, 4), (2056, 8), (2056, 0)):    # rows read feature by feature, and 16 bytes at a time
        for dt in (torch.float32, torch.bfloat16):
            z = (torch.randn(4, cols + spare, device=DEV) * 3).to(dt)
            act = torch.empty(4, cols, dtype=dt, device=DEV)
            kernels.activation(z[:, :cols], act, "xielu", params)
            want = plain.xielu(z[:, :cols].double(), p.double(), q.double())
            assert max_rel_diff(act, want) < (1e-6 if dt == torch.float32 else 5e-3)
            if spare == 0:
                kernels.activation(z, z, "xielu", params)                     # in place
                assert torch.equal(z, act)


# ------------------------------------------------------------------------------------ attention kernels
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
    """x [tokens, heads, width] of request s into its pages, from position `first` on (what lies before stays NaN)."""
    idx = torch.arange(first, x.shape[0])
    pg, off = tables[s, idx // page].long(), idx % page
    cache[pg.to(DEV), :, off.to(DEV)] = x[first:].to(device=DEV, dtype=cache.dtype)


def _chunk_attention_plain(q, k, v, first_pos, chunk, scale, cap, r1, r2):
    """q [n, H, D] at positions first_pos ..; k, v [total, G, .]: the rows' results [n, H * DV] and weights [H, n, total]."""
    n, H, _ = q.shape
    total, G, _ = k.shape
    kx, vx = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kx) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    i, j = torch.arange(first_pos, first_pos + n)[:, None], torch.arange(total)[None, :]
    if r1 is not None:
        s = s - r1[:, None, None] * torch.log1p(r2[:, None, None] * (i - j).clamp(min=0).double())
    vis = j <= i
    if chunk:
        vis = vis & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    w = torch.softmax(s.masked_fill(~vis, float("-inf")), dim=-1)
    return torch.einsum("hij,jhd->ihd", w, vx).reshape(n, -1), w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,DV,chunk,cap,bias", [
    (4, 2, 24, 40, 21, 6.0, True), (3, 3, 10, 6, 5, 0.0, True), (8, 4, 64, 64, 48, 8.0, True), (2, 1, 96, 32, 70, 20.0, False),
    (2, 2, 16, 8, 0, 4.0, True), (1, 1, 8, 8, 1, 2.0, False), (6, 2, 128, 128, 100, 0.0, False), (4, 4, 32, 48, 64, 3.0, True)])
def test_block_attention_far_key_page_borders_block_edges_cap_and_distance(dtype, H, G, D, DV, chunk, cap, bias):
    """Two requests in one batch over scattered pages: a portion of rows behind a context that is in the cache, and a
    single decoded token far into its context. One row looks at the first key of its block (far back in it) with a
    score that only the cap keeps finite in weight, another at a key at a page's last slot; the key just before the
    block (the last one of the block before) would outweigh everything if it were seen, and its pages hold NaN where
    the block's own keys do not reach. The distance bias of one head is strong enough to move the weight to the
    nearest keys."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(3)
    page, scale = 8, 0.3
    ctxs, lens = (150, 320), (70, 1)
    total = [c + n for c, n in zip(ctxs, lens)]
    tables, (kc, vc) = _paged(total, page, [(G, D), (G, DV)], dtype)
    k = [torch.randn(t, G, D) * 0.5 for t in total]
    v = [torch.randn(t, G, DV) for t in total]
    T = sum(lens)
    q = torch.randn(T, H, D) * 0.5
    group = H // G

    def aim(row, s, pos_key, weight):
        for a in range(H):
            kk = k[s][pos_key, a // group]
            q[row, a] = weight * kk / kk.norm() ** 2 / scale
    far_row = 60                                                  # request 0, position 210
    pos0, pos1 = ctxs[0] + far_row, total[1] - 1
    first0 = pos0 // chunk * chunk if chunk else 0
    first1 = pos1 // chunk * chunk if chunk else 0
    if chunk != 1:
        aim(far_row, 0, first0 if chunk else 3, 14.0)             # the first key of the block (or one far back)
        aim(T - 1, 1, (pos1 // page) * page - 1 if first1 <= (pos1 // page) * page - 1 else first1, 14.0)   # a page's last slot
    if chunk:
        # the last key of the block before: seen, it would take the whole row
        if first0 > 0:
            k[0][first0 - 1] = 40.0 * q[far_row, 0] / q[far_row, 0].norm() ** 2 / scale
        if first1 > 0:
            k[1][first1 - 1] = 40.0 * q[T - 1, 0] / q[T - 1, 0].norm() ** 2 / scale
    # what no row of this step may read stays NaN in the cache: everything before the first block that a row of the request lies in
    lo = [(ctxs[s] // chunk * chunk if chunk else 0) for s in range(2)]
    for s in range(2):
        _fill(kc, tables, s, k[s], page, first=lo[s])
        _fill(vc, tables, s, v[s], page, first=lo[s])
    r1 = r2 = None
    if bias:
        r1, r2 = torch.rand(H) * 1.5 + 0.05, torch.rand(H) * 2 + 0.05
        r1[H - 1], r2[H - 1] = 9.0, 3.0                           # the last head all but forgets what is not near
    positions = torch.cat([torch.arange(ctxs[s], total[s]) for s in range(2)]).to(device=DEV, dtype=torch.int32)
    row_seq = torch.cat([torch.full((lens[s],), s) for s in range(2)]).to(device=DEV, dtype=torch.int32)
    qd = q.reshape(T, H * D).to(device=DEV, dtype=dtype)
    g = torch.randn(T, H * DV)
    gd = g.to(device=DEV, dtype=dtype)
    wide = torch.full((T, H * DV + 8), float("nan"), dtype=dtype, device=DEV)
    out = wide[:, 8:]
    rd = (r1.to(DEV), r2.to(DEV)) if bias else None
    kernels.flex_attention(qd, out, kc, vc, tables.to(DEV), row_seq, positions, H, G, D, DV, scale, 0, None, gd, 1.0, chunk, cap, rd)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    shaped = bool(chunk or cap or bias)
    if dtype == torch.bfloat16 and shaped and kernels.attn_prefill_mma_any_supported(H, G, D, DV, page):
        # the tensor-core portion kernel in its build for shaped scores: the same mixed step, the same answer
        wide2 = torch.full((T, H * DV + 8), float("nan"), dtype=dtype, device=DEV)
        starts = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
        kernels.attn_prefill_mma_any(qd, wide2[:, 8:], kc, vc, tables.to(DEV), starts, torch.tensor(ctxs, dtype=torch.int32, device=DEV),
                                     2, max(lens), H, G, D, DV, scale, 0, None, gd, 1.0, chunk, cap, rd)
        assert bool(torch.isnan(wide2[:, :8]).all()) and not bool(torch.isnan(wide2[:, 8:]).any())
        assert max_rel_diff(wide2[:, 8:], out) < tol
        if D == DV and D in (64, 128):
            # and the split-key decode kernel on each request's last row, alone and shared out over a cluster
            last = torch.tensor([lens[0] - 1, T - 1], device=DEV)
            for splits in (1, 3, 8):
                o2 = torch.full((2, H * DV), float("nan"), dtype=dtype, device=DEV)
                kernels.attn_decode_mma(qd[last].contiguous(), o2, kc, vc, tables.to(DEV), positions[last].contiguous(), H, G, D, scale, 0,
                                        splits, None, None, None, gd[last].contiguous(), 1.0, chunk, cap, rd)
                assert max_rel_diff(o2, out[last]) < tol, splits
    r0 = 0
    for s in range(2):
        kk, vv = k[s].to(dtype).double(), v[s].to(dtype).double()
        kk[:lo[s]], vv[:lo[s]] = 0.0, 0.0                         # masked anyway; the plain form must not see the NaN story at all
        qq = qd[r0:r0 + lens[s]].cpu().double().reshape(lens[s], H, D)
        want, w = _chunk_attention_plain(qq, kk, vv, ctxs[s], chunk, scale, cap, r1.double() if bias else None, r2.double() if bias else None)
        want = want * torch.sigmoid(gd[r0:r0 + lens[s]].cpu().double())
        got = out[r0:r0 + lens[s]].cpu()
        assert not bool(torch.isnan(got).any()), s
        assert max_rel_diff(got, want) < tol, s
        if dtype == torch.bfloat16 and shaped and kernels.attn_prefill_mma_any_supported(H, G, D, DV, page):
            assert max_rel_diff(wide2[r0:r0 + lens[s], 8:].cpu(), want) < tol, s
        if s == 0 and chunk != 1 and not bias:
            assert float(w[0, far_row, first0 if chunk else 3]) > 0.5          # the far key is what the row is made of
        if s == 0 and chunk and first0 > 0:
            assert float(w[:, far_row, first0 - 1].max()) == 0.0
        if bias and s == 0 and chunk != 1:
            near = w[H - 1, far_row, max(first0, pos0 - 2):pos0 + 1].sum()
            assert float(near) > 0.9
        r0 += lens[s]
    assert bool(torch.isnan(wide[:, :8]).all())


def test_a_score_beyond_the_cap_counts_as_the_cap():
    """Two keys whose raw scores are 40 and 400: with a cap of 5 they weigh the same to four digits."""
    from vllm_oxide_b200 import kernels
    D, page = 16, 8
    tables, (kc, vc) = _paged([3], page, [(1, D), (1, D)], torch.float32)
    k = torch.zeros(3, 1, D)
    k[0, 0, 0], k[1, 0, 0], k[2, 0, 0] = 40.0, 400.0, -400.0
    v = torch.zeros(3, 1, D)
    v[0, 0, 0], v[1, 0, 1], v[2, 0, 2] = 1.0, 1.0, 1.0
    _fill(kc, tables, 0, k, page)
    _fill(vc, tables, 0, v, page)
    q = torch.zeros(1, D, device=DEV)
    q[0, 0] = 1.0
    out = torch.empty(1, D, device=DEV)
    one = torch.tensor([2], dtype=torch.int32, device=DEV)
    kernels.flex_attention(q, out, kc, vc, tables.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV), one, 1, 1, D, D, 1.0, 0, None,
                           None, 1.0, 0, 5.0, None)
    a, b, c = (float(out[0, i]) for i in range(3))
    assert abs(a - b) < 1e-4 and abs(a + b + c - 1.0) < 1e-5 and c < 1e-4 and a > 0.49


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_preparation_shared_norm_weights_and_a_layer_without_keys(dtype):
    """q and k divided by their root mean square per head and multiplied by a weight that all heads share; k and v go
    to their cache slots; a layer that reads another layer's cache prepares q only and touches no cache."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(2)
    T, H, G, D, DV, page, eps = 7, 4, 2, 24, 40, 8, 1e-5
    nq, nk, nv = H * D, G * D, G * DV
    proj = (torch.randn(T, 3 + nq + nk + nv + 5, device=DEV) * 2).to(dtype)
    wq, wk = torch.randn(D, device=DEV) + 1.0, torch.randn(D, device=DEV) - 0.5
    positions = torch.arange(30, 30 + T, dtype=torch.int32, device=DEV)
    slots = torch.tensor([17, 3, 40, 41, 8, 0, 25], dtype=torch.int32, device=DEV)
    kc = torch.full((6, G, page, D), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((6, G, page, DV), float("nan"), dtype=dtype, device=DEV)
    q = torch.empty(T, nq, dtype=dtype, device=DEV)
    kernels.flex_prep(proj, 3, 3 + nq, 3 + nq + nk, positions, slots, None, 0, True, eps, None, None, None, 0, q, kc, vc, H, G, D, DV, wq, wk)
    p = proj.double().cpu()
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    want_q = plain.rms(p[:, 3:3 + nq].reshape(T, H, D), eps) * wq.double().cpu()
    want_k = plain.rms(p[:, 3 + nq:3 + nq + nk].reshape(T, G, D), eps) * wk.double().cpu()
    want_v = p[:, 3 + nq + nk:3 + nq + nk + nv].reshape(T, G, DV)
    assert max_rel_diff(q.cpu(), want_q.reshape(T, nq)) < tol
    for r in range(T):
        s = int(slots[r])
        assert max_rel_diff(kc[s // page, :, s % page].cpu(), want_k[r]) < tol
        assert torch.equal(vc[s // page, :, s % page].cpu().double(), want_v[r])
    assert int(torch.isnan(kc).sum()) == (6 * page - T) * G * D               # nothing else was written
    q2 = torch.empty(T, nq, dtype=dtype, device=DEV)
    only_q = proj[:, :3 + nq]
    kernels.flex_prep(only_q, 3, 0, 0, positions, None, None, 0, True, eps, None, None, None, 0, q2, None, None, H, G, D, DV, wq, None)
    assert torch.equal(q2, q)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,K,V,taps", [(4, 2, 16, 24, 3), (2, 2, 40, 8, 4), (3, 1, 8, 12, 1), (6, 3, 24, 32, 2), (1, 1, 136, 16, 5)])
def test_gated_delta_with_one_decay_per_head_portions_state_and_slots(dtype, H, G, K, V, taps):
    """Preparation and scan over two requests cut into portions of 1, 2, 3 and more tokens (shorter than the convolution,
    too) in slots that are not their order, against the whole sequences done plainly; then the slots are zeroed and used
    again for the other request. The decay is one number per head, read from columns of the first product."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(5)
    C = 2 * G * K + H * V
    n = (23, 9)
    # q | k | v | decay inputs (heads) | 2 spare columns | strengths (heads)
    x = [torch.randn(t, C + H + 2 + H).to(dtype) for t in n]
    a_off, b_off = C, C + H + 2
    cw = torch.randn(C, taps) * 0.5
    a_log, dt_bias = torch.randn(H) * 0.5 - 1.0, torch.randn(H)

    def want(s):
        xs, t = x[s].double(), n[s]
        q = plain.causal_conv_silu(xs[:, :G * K], cw[:G * K].double()).reshape(t, G, K)
        k = plain.causal_conv_silu(xs[:, G * K:2 * G * K], cw[G * K:2 * G * K].double()).reshape(t, G, K)
        v = plain.causal_conv_silu(xs[:, 2 * G * K:C], cw[2 * G * K:].double()).reshape(t, H, V).to(dtype).double()
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * K ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
        beta = torch.sigmoid(xs[:, b_off:b_off + H])
        g = torch.exp(-torch.exp(a_log.double()) * plain.softplus(xs[:, a_off:a_off + H] + dt_bias.double()))
        S = torch.zeros(H, K, V, dtype=torch.float64)
        o = torch.zeros(t, H, V, dtype=torch.float64)
        for i in range(t):
            S = g[i][:, None, None] * S
            u = beta[i][:, None] * (v[i] - torch.einsum("hkv,hk->hv", S, k[i]))
            S = S + k[i][:, :, None] * u[:, None, :]
            o[i] = torch.einsum("hkv,hk->hv", S, q[i])
        return o.reshape(t, H * V), S
    state = torch.full((4, H, K, V), float("nan"), device=DEV)
    cstate = torch.full((4, max(taps - 1, 0), C), float("nan"), device=DEV) if taps > 1 else None
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for slots in ((2, 0), (1, 2)):
        for sl in slots:
            state[sl].zero_()
            if cstate is not None:
                cstate[sl].zero_()
        cuts = [[(0, 2), (1, 1)], [(0, 1), (1, 3)], [(1, 2)], [(0, 3), (1, 1)], [(0, 1)], [(0, 16), (1, 2)]]
        at, got = [0, 0], [[], []]
        for step in cuts:
            rows = torch.cat([x[s][at[s]:at[s] + c] for s, c in step]).to(DEV)
            T = rows.shape[0]
            starts = torch.tensor([0] + torch.tensor([c for _, c in step]).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
            rs = torch.cat([torch.full((c,), i) for i, (_, c) in enumerate(step)]).to(device=DEV, dtype=torch.int32)
            pos = torch.cat([torch.arange(at[s], at[s] + c) for s, c in step]).to(device=DEV, dtype=torch.int32)
            sl = torch.tensor([slots[s] for s, _ in step], dtype=torch.int32, device=DEV)
            q, k = torch.empty(T, G * K, device=DEV), torch.empty(T, G * K, device=DEV)
            v = torch.empty(T, H * V, dtype=dtype, device=DEV)
            decay, beta, o = torch.empty(T, H * K, device=DEV), torch.empty(T, H, device=DEV), torch.empty(T, H * V, device=DEV)
            kernels.gated_delta_prep(rows, 0, b_off, rows, a_off, cw.to(DEV), cstate, a_log.to(DEV), dt_bias.to(DEV), pos, rs, starts, sl,
                                     len(step), H, G, K, V, q, k, v, decay, beta, True)
            d3 = decay.reshape(T, H, K)
            assert torch.equal(d3, d3[:, :, :1].expand(T, H, K))              # one decay for all of a head's key channels
            kernels.recurrence_scan(2, q, k, v, decay, beta, None, state, starts, sl, len(step), H, o, rk_heads=G,
                                    conv_x=rows[:, :C] if cstate is not None else None, conv_state=cstate)
            r = 0
            for s, c in step:
                got[s].append(o[r:r + c].cpu())
                at[s] += c
                r += c
        for s in range(2):
            o_want, S_want = want(s)
            assert at[s] == n[s]
            assert max_rel_diff(torch.cat(got[s]), o_want) < tol, (slots, s)
            assert max_rel_diff(state[slots[s]].cpu(), S_want) < tol
    assert bool(torch.isnan(state[3]).all())              # a slot nobody held was never touched


def test_gated_delta_result_normed_per_head_times_a_silu_gate():
    from vllm_oxide_b200 import kernels
    torch.manual_seed(1)
    T, H, V = 5, 3, 20
    o, gate, w = torch.randn(T, H * V, device=DEV), torch.randn(T, H * V + 4, device=DEV) * 2, torch.randn(V, device=DEV)
    wide = torch.full((T, 7 + H * V), float("nan"), device=DEV)
    kernels.recurrence_post(o, gate[:, 4:], w.repeat(H).contiguous(), "silu", 1e-5, H, wide[:, 7:], 1.0)
    want = plain.rms(o.double().reshape(T, H, V), 1e-5) * w.double() * plain.silu(gate[:, 4:].double()).reshape(T, H, V)
    assert max_rel_diff(wide[:, 7:], want.reshape(T, H * V)) < 1e-5 and bool(torch.isnan(wide[:, :7]).all())


# ------------------------------------------------------------------------------------ routed experts
def _route_plain(logits, top, groups, keep):
    """The plain election on given logits: the router is the unit matrix."""
    r = {"experts": logits.shape[1], "top": top}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    return plain.route(logits, {"router": torch.eye(logits.shape[1], dtype=logits.dtype)}, "", r)


def test_election_among_the_best_groups():
    """Router logits written directly (x is a unit vector per token, the router's columns are the logits). Token 0: the
    third best expert of all sits in a group that is not kept, so a far weaker one of a kept group is chosen instead.
    Token 1: no groups would have chosen otherwise. Weights are the softmax scores over ALL experts, not renormalized.
    A row of negative position (padding) chooses nothing."""
    from vllm_oxide_b200 import kernels
    E, width = 6, 10
    logits = torch.tensor([[3.0, -2.0, 2.5, -1.5, 2.2, 2.0],          # groups of 2: best 3.0, 2.5, 2.2 -> kept 0 and 1
                           [0.1, 0.2, 0.3, 0.4, 0.5, 0.6],
                           [1.0, 5.0, 4.9, -3.0, 4.8, 4.7],
                           [2.0, 2.0, 2.0, 2.0, 2.0, 2.5]])
    T = logits.shape[0]
    x = torch.zeros(T, width, device=DEV)
    w_router = torch.zeros(E, width, device=DEV)
    for t in range(T):
        x[t, t + 2] = 1.0
        w_router[:, t + 2] = logits[t]
    pos = torch.tensor([4, 0, 9, -1], dtype=torch.int32, device=DEV)
    s = torch.softmax(logits.double(), -1)
    for top, groups, keep in ((3, 3, 2), (3, 0, 0), (2, 2, 1), (1, 6, 1), (4, 3, 2), (3, 3, 3)):
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        w = torch.empty(T, top, device=DEV)
        kernels.moe_route(x, w_router, pos, top, groups, keep, False, idx, w)
        want_idx, want_w = _route_plain(logits.double(), top, groups, keep)
        for t in range(T - 1):
            got = sorted(idx[t].tolist())
            assert got == sorted(want_idx[t].tolist()), (top, groups, keep, t)
            assert len(set(got)) == top
            for j in range(top):
                assert abs(float(w[t, j]) - float(s[t, int(idx[t, j])])) < 1e-6
        assert idx[T - 1].tolist() == [-1] * top
        if (top, groups, keep) == (3, 3, 2):
            assert sorted(idx[0].tolist()) == [0, 2, 3]               # 3 (-1.5) stands in for 4 (2.2) and 5 (2.0)
            assert float(w[0].sum()) < 0.8                            # and the weights are not made to sum to one
        if (top, groups, keep) == (3, 0, 0):
            assert sorted(idx[0].tolist()) == [0, 2, 4]
        kernels.moe_route(x, w_router, pos, top, groups, keep, True, idx, w)
        assert max_rel_diff(w[:T - 1].sum(-1).cpu(), torch.ones(T - 1)) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,width,ff,E,top,groups,keep", [(1, 48, 24, 8, 2, 4, 3), (37, 42, 20, 5, 1, 0, 0), (300, 64, 16, 6, 3, 2, 2),
                                                          (70, 96, 88, 10, 3, 5, 2), (5, 40, 136, 16, 4, 4, 2), (700, 72, 104, 4, 2, 0, 0),
                                                          (9, 2048, 72, 6, 2, 3, 2)])
def test_routed_experts_against_every_expert_done_plainly(dtype, T, width, ff, E, top, groups, keep):
    """Election, ordering by expert, both grouped products and the weighted sum, with an expert nobody chooses and rows
    of padding, against the plain sum over all experts. In bfloat16 with rows that 16-byte copies can fetch, tiles of
    128 pairs give bit for bit what tiles of 32 give."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(T + E)
    x = torch.randn(T, width).to(dtype)
    wr = torch.randn(E, width) * 1.5
    wr[E - 1] = 0.0
    wr[E - 1, 0] = -1.0e3 * float(x[:, 0].abs().max() + 1)         # never the best... unless x[., 0] is negative:
    x[:, 0] = x[:, 0].abs() + 0.5                                  # so it is not
    wg, wu, wd = (torch.randn(E, ff, width) * 0.3).to(dtype), (torch.randn(E, ff, width) * 0.3).to(dtype), (torch.randn(E, width, ff) * 0.3).to(dtype)
    pos = torch.arange(T, dtype=torch.int32)
    if T > 4:
        pos[3] = -1
    xd = x.to(DEV)
    idx, w = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    kernels.moe_route(xd, wr.to(DEV), pos.to(DEV), top, groups, keep, False, idx, w)
    P = T * top
    tc = dtype == torch.bfloat16
    outs = []
    for tile in (kernels.MOE_TILE_ROWS, kernels.MOE_LARGE_TILE_ROWS):
        if tile != kernels.MOE_TILE_ROWS and not (tc and width % 8 == 0 and ff % 8 == 0):
            continue
        cap = kernels.moe_sorted_rows(P, E, tile)
        order = torch.empty(cap, dtype=torch.int32, device=DEV)
        tile_expert = torch.empty(cap // tile, dtype=torch.int32, device=DEV)
        meta = torch.zeros(4, dtype=torch.int32, device=DEV)
        kernels.moe_align(idx, E, order, tile_expert, meta, tile)
        listed = sorted(p for p in order.tolist() if p >= 0)
        assert listed == [p for p in range(P) if int(idx.reshape(-1)[p]) >= 0]     # every live pair once
        h = torch.full((P, ff), float("nan"), dtype=dtype, device=DEV)
        kernels.moe_gate_up(xd, torch.cat([wg, wu], 1).contiguous().to(DEV), order, tile_expert, top, h, tc, tile)
        y = torch.full((P, width), float("nan"), device=DEV)
        kernels.moe_down(h, wd.to(DEV), order, tile_expert, w, y, tc, tile)
        out = torch.empty(T, width, dtype=dtype, device=DEV)
        kernels.moe_combine(y, idx, out)
        outs.append(out)
    if len(outs) == 2:
        assert torch.equal(outs[0], outs[1])
    t = {"router": wr.double()}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"] = wg[e].double(), wu[e].double(), wd[e].double()
    r = {"experts": E, "top": top}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    want = plain.moe_ff(x.double(), t, "", {"router": r})
    live = pos >= 0
    assert not bool((idx[live.to(DEV)] == E - 1).any())
    assert max_rel_diff(out[live.to(DEV)].cpu(), want[live]) < (2e-5 if dtype == torch.float32 else 2e-2)
    assert float(out[~live.to(DEV)].abs().max()) == 0.0 if T > 4 else True


# ------------------------------------------------------------------------------------ models in the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "delta", "dense", "moe"])
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
    # most of it at once, the rest one by one, in the slot and the pages that were just given back
    _poison(runner)
    single = _replay(s, {"b": toks}, [[("b", 19)]] + [[("b", 1)]] * 26, first_step=10)["b"]
    assert _close(single, want, dtype)
    if dtype == "float32":
        assert max_rel_diff(single, whole) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "T"])
def test_portions_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Four requests of unequal length in a pool that cannot hold them all at once: portions from 2 tokens up beside
    single tokens, portions that end inside a page and inside a block of positions, a request that sits out a step, a
    fourth request that takes over a slot and pages that were given back in the middle. Every row equals the plain
    model's."""
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
    # each alone, whole: what a row gives does not depend on the cut or the batch, beyond rounding (in bfloat16 a portion,
    # a single token and a whole prompt take different kernels)
    for k in reqs:
        alone = _replay(s, {k: reqs[k]}, [[(k, len(reqs[k]))]], first_step=100)[k]
        if dtype == "float32":
            assert max_rel_diff(alone, got[k]) < 5e-6, k
        else:
            err = _row_errors(got[k], alone)
            assert float(err.median()) < 1.5e-2 and float(err.quantile(0.9)) < 6e-2, (k, float(err.median()), float(err.quantile(0.9)))


def test_the_residual_after_every_layer(tmp_path):
    """Layer by layer in float32: the residual stream that the engine's blocks leave equals the plain model's."""
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
    for i, (got, want) in enumerate(zip(seen, layers)):
        assert max_rel_diff(got.cpu(), want) < 1e-5, i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_long_decoding_over_page_borders_and_block_edges(tmp_path, name, dtype):
    """150 tokens, all but six of them one by one: the blocks (21, 48 and 70 positions) end and begin under decoded
    tokens several times, the block groups give their pages back on the way, and the delta rule's state is carried
    through 144 steps."""
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    toks = _tokens(150, _configs()[name].vocab, 9)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype, page=8, pages=20, max_seqs=2)
    _poison(runner)
    got = _replay(TraceSession(runner), {"a": toks}, [[("a", 6)]] + [[("a", 1)]] * 144)["a"]
    assert _close(got, want, dtype)


def test_a_block_one_token_off_or_a_bias_left_out_would_show(tmp_path):
    """The plain model with every block one position longer, or without the distance bias, or without the cap, differs
    from itself by far more than the tolerance: the tests above can tell."""
    d = _model_dir(tmp_path, "A")
    from safetensors.torch import load_file
    toks = _tokens(60, 97, 1)
    tensors = load_file(os.path.join(d, "model.safetensors"))

    def run(change):
        cfg = json.load(open(os.path.join(d, "config.json")))
        t = dict(tensors)
        change(cfg, t)
        return plain.forward(cfg, t, toks)
    want = run(lambda c, t: None)

    def longer(c, t):
        for layer in c["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["mask"]["size"] += 1

    def no_bias(c, t):
        for n in t:
            if n.endswith(".r1"):
                t[n] = torch.zeros_like(t[n])

    def no_cap(c, t):
        for layer in c["layers"]:
            if layer["type"] == "attention":
                layer["mixer"].pop("softcap", None)

    def renormed(c, t):
        for n in t:
            if n.endswith(".router"):
                t[n] = t[n] * 0
    for change in (longer, no_bias, no_cap, renormed):
        assert max_rel_diff(run(change), want) > 1e-3, change.__name__


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(tmp_path, graphs):
    """More requests than state slots and a pool that forces preemption and recomputation: every generated token is the
    plain model's argmax given what came before. With CUDA graphs the decode steps are recorded and replayed (nothing in
    these parts reads device data on the host: the experts' counts stay on the device)."""
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
    """bfloat16, decode steps replayed from graphs, generation that runs over block edges: every generated token is the
    plain model's best, or as good as the best within what bfloat16 can tell apart."""
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


def test_a_prompt_longer_than_the_position_table_is_refused(tmp_path):
    """Learned positions end where their table ends: the engine's longest sequence is the table's length at most."""
    d = _model_dir(tmp_path, "attention")                         # 64 positions
    runner = _runner(d, "float32", page=8, pages=24)
    assert runner.max_model_len == 64


def test_command_line_generates_from_a_bufulorn_folder(tmp_path):
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


def test_trace_program_replays_a_bufulorn_folder(tmp_path):
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
        assert max_rel_diff(got, want[places]) < TOL["float32"]
