"""Dumizen on the GPU: each new kernel beside its plain reference or the plain function of its mechanism (keys planted
far back, at page borders, just inside and just outside the window, blocks that are just seen and not yet, in prompts
and in decoding, on the tensor-core tiles and row by row, with forced splits), and the whole model under every cut,
in long decoding and in generation, beside the plain implementation."""
import json
import math
import os
import random
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_dumizen as P
import tiny_dumizen as tiny
import traces
from flint_b200.cache.manager import CacheView, KVSpec
from flint_b200.engine.engine import Engine
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.engine.step import Tiling
from flint_b200.sampling.params import SamplingParams
from kernel_refs import RefOps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = (1, 2, 9, 37, 70, 130)


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


def paged_cache(lengths, G, d, dv, P_, pool, dtype, seed=0, spread=1.0):
    """Random keys and values of several requests in pages that lie in a shuffled order, with room for the means of
    blocks; on the CPU."""
    g = torch.Generator().manual_seed(seed)
    rnd = random.Random(seed)
    n_pages = sum(-(-n // P_) for n in lengths) + 3
    order = list(range(n_pages))
    rnd.shuffle(order)
    E = -(-P_ // pool) if pool else 0
    kc, vc = torch.zeros(n_pages, G, P_, d, dtype=dtype), torch.zeros(n_pages, G, P_, dv, dtype=dtype)
    bt = torch.full((len(lengths), max(-(-n // P_) for n in lengths) + 1), -1, dtype=torch.int32)
    for s, n in enumerate(lengths):
        for lp in range(-(-n // P_)):
            bt[s, lp] = order.pop()
            m = min(P_, n - lp * P_)
            kc[bt[s, lp], :, :m] = (spread * torch.randn(G, m, d, generator=g)).to(dtype)
            vc[bt[s, lp], :, :m] = torch.randn(G, m, dv, generator=g).to(dtype)
    pk = torch.full((n_pages, G, max(E, 1), d), 7.0, dtype=dtype) if pool else None       # stale numbers where nothing was written
    pv = torch.full((n_pages, G, max(E, 1), dv), -7.0, dtype=dtype) if pool else None
    return CacheView(kc, vc, bt, P_, KVSpec(G, d, 0, dv, pool=pool), pool_k=pk, pool_v=pv, pool_slots=E)


def on_device(view):
    mv = lambda t: t.to(DEV) if t is not None else None
    return CacheView(mv(view.k), mv(view.v), mv(view.block_table), view.page_size, view.spec, pool_k=mv(view.pool_k),
                     pool_v=mv(view.pool_v), pool_slots=view.pool_slots)


def step_of(pos, slot, n_entries, device=DEV):
    pos = torch.tensor(pos, dtype=torch.int32, device=device)
    return SimpleNamespace(pos=pos, slot=torch.tensor(slot, dtype=torch.int32, device=device), max_kv_len=int(pos.max()) + 1,
                           entries=[None] * n_entries, n_tokens=pos.numel(), status=torch.zeros(1, dtype=torch.int32, device=device))


def tiling_of(portions):
    tiles, others, row = [], [], 0
    for s_, p0, c in portions:
        if c < 16:
            others += range(row, row + c)
        else:
            for r in range(0, c, 64):
                tiles.append([row + r, min(64, c - r), s_, p0 + r])
        row += c
    tiles.sort(key=lambda t: -(t[3] + t[1]))
    return Tiling(torch.tensor(tiles, dtype=torch.int32, device=DEV).reshape(-1, 4), len(tiles),
                  torch.tensor(others, dtype=torch.int32, device=DEV), len(others))


def fill_block_means(ops, view, dev_view, lengths, pool, cuts=(5, 64, 1, 2, 40, 300)):
    """The means of all complete blocks, written on the device by steps that cut the requests anywhere, and on the
    CPU by the reference in one go."""
    G, d, dv = view.k.shape[1], view.k.shape[3], view.v.shape[3]
    done = [0] * len(lengths)
    k = 0
    while any(done[s] < n for s, n in enumerate(lengths)):
        pos, slot = [], []
        for s, n in enumerate(lengths):
            c = min(cuts[k % len(cuts)], n - done[s])
            k += 1
            pos += range(done[s], done[s] + c)
            slot += [s] * c
            done[s] += c
        ops.pool_write(dev_view, step_of(pos, slot, len(lengths)), G, d, dv, pool)
    pos = [p for n in lengths for p in range(n)]
    slot = [s for s, n in enumerate(lengths) for _ in range(n)]
    RefOps(F64).pool_write(view, step_of(pos, slot, len(lengths), "cpu"), G, d, dv, pool)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("G,d,dv,P_,pool", [(2, 24, 10, 16, 3), (1, 16, 16, 16, 16), (2, 64, 48, 64, 12), (3, 7, 33, 16, 40), (2, 32, 32, 32, 1)])
def test_block_means_are_written_once_whatever_the_cut(ops, dtype, G, d, dv, P_, pool):
    lengths = [203, 77]
    view = paged_cache(lengths, G, d, dv, P_, pool, dtype, seed=pool)
    dev = on_device(view)
    fill_block_means(ops, view, dev, lengths, pool)
    for got, want in ((dev.pool_k, view.pool_k), (dev.pool_v, view.pool_v)):
        err = (got.cpu().double() - want.double()).abs().max().item()
        assert err < (1e-6 if dtype == torch.float32 else 2e-2), err      # also where nothing was to be written


def pooled_rows(lengths, window, pool, P_):
    """(slot, position, planted key or block) rows around every edge: the row's own key, the first and last of the
    window, the position that has just left it, page borders, the block that is just seen and the one not yet."""
    rows = []
    for s, n in enumerate(lengths):
        for p in sorted({n - 1, n - 2, n // 2, window + pool - 1, window + pool - 2, window + pool, window - 1, window, 2 * P_, 2 * P_ - 1, 1, 0}):
            if not 0 <= p < n:
                continue
            nb = max(0, (p - window + 1) // pool)
            for j in {p, p - 1, p - window + 1, (p // P_) * P_, (p // P_) * P_ - 1}:
                if max(0, p - window + 1) <= j <= p:
                    rows.append((s, p, ("key", j)))
            for b in {0, nb - 1, nb // 2}:
                if 0 <= b < nb:
                    rows.append((s, p, ("block", b)))
            rows.append((s, p, ("none", 0)))
    return rows


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,P_", [(6, 2, 32, 16, 16), (4, 4, 64, 48, 64), (3, 1, 7, 33, 16)])
@pytest.mark.parametrize("window,pool", [(7, 3), (72, 12), (16, 16), (5, 1), (21, 40)])
def test_pooled_window_attention_finds_planted_keys_and_blocks(ops, dtype, H, G, d, dv, P_, window, pool):
    """A row's query is made to point at one key of its window, or at the mean of one block behind it, so that this
    one score stands far above the rest: a key or block that the kernel misses, or one too many, shows at once.
    Single rows with and without forced splits, against the plain reference over the same cache."""
    lengths = [333, 150]
    view = paged_cache(lengths, G, d, dv, P_, pool, dtype, seed=window + pool)
    dev = on_device(view)
    fill_block_means(ops, view, dev, lengths, pool)
    rows = pooled_rows(lengths, window, pool, P_)
    g = torch.Generator().manual_seed(H + d + window)
    q = torch.randn(len(rows), H, d, generator=g, dtype=F64)
    E = view.pool_slots
    for r, (s, p, (what, at)) in enumerate(rows):
        h = r % H
        if what == "key":
            target = view.k[view.block_table[s, at // P_], h // (H // G), at % P_].double()
        elif what == "block":
            target = view.pool_k[view.block_table[s, at // E], h // (H // G), at % E].double()
        else:
            continue
        q[r, h] = 12.0 * target / target.norm() * math.sqrt(d) / max(target.norm().item() / math.sqrt(d), 0.2)
    q = q.to(dtype)
    pos, slot = [p for _, p, _ in rows], [s for s, _, _ in rows]
    scale = d ** -0.5
    want = torch.zeros(len(rows), H * dv, dtype=F64)
    RefOps(F64).sink_attention(q.reshape(len(rows), H * d), view, step_of(pos, slot, len(rows), "cpu"), want, H, G, d, dv, window, 0,
                               None, scale, pool=pool)
    for splits in (None, (32, -(-(window + max(pos) // pool + 1) // 32))):
        out = torch.zeros(len(rows), H * dv, dtype=dtype, device=DEV)
        ops.sink_attention(q.reshape(len(rows), H * d).to(DEV), dev, step_of(pos, slot, len(rows)), out, H, G, d, dv, window, 0, None,
                           scale, splits=splits, pool=pool)
        err = (out.cpu().double() - want).abs().max(-1).values
        assert err.max().item() < (3e-5 if dtype == torch.float32 else 4e-2), (rows[int(err.argmax())], splits, err.max().item())


@pytest.mark.parametrize("H,G,d,dv,P_", [(4, 2, 32, 16, 16), (6, 2, 64, 48, 64), (2, 1, 16, 64, 16)])
@pytest.mark.parametrize("window,pool", [(7, 3), (72, 12), (16, 16), (5, 1), (100, 40)])
def test_pooled_window_attention_tiles_on_the_tensor_cores(ops, H, G, d, dv, P_, window, pool):
    """Portions of prompts as tiles of up to 64 rows (whole tiles, a ragged last one, a portion that starts in the
    middle of a request, of a page and of a block) beside single rows, two requests, peaked scores: the tensor-core
    kernel and the row kernel together against the plain reference."""
    lengths = [333, 150]
    view = paged_cache(lengths, G, d, dv, P_, pool, torch.bfloat16, seed=window * pool, spread=2.0)
    dev = on_device(view)
    fill_block_means(ops, view, dev, lengths, pool)
    portions = [(0, 0, 150), (1, 0, 64), (0, 150, 17), (1, 64, 3), (0, 167, 166), (1, 67, 1), (1, 68, 82)]
    pos = [p0 + i for s_, p0, c in portions for i in range(c)]
    slot = [s_ for s_, p0, c in portions for i in range(c)]
    T = len(pos)
    g = torch.Generator().manual_seed(H + d)
    q = (2.0 * torch.randn(T, H * d, generator=g, dtype=F64)).to(torch.bfloat16)
    scale = d ** -0.5
    want = torch.zeros(T, H * dv, dtype=F64)
    RefOps(F64).sink_attention(q, view, step_of(pos, slot, len(portions), "cpu"), want, H, G, d, dv, window, 0, None, scale, pool=pool)
    out = torch.zeros(T, H * dv, dtype=torch.bfloat16, device=DEV)
    ops.sink_attention(q.to(DEV), dev, step_of(pos, slot, len(portions)), out, H, G, d, dv, window, 0, None, scale,
                       tiling=tiling_of(portions), pool=pool)
    err = (out.cpu().double() - want).abs().max(-1).values
    assert err.max().item() < 4e-2, (int(err.argmax()), pos[int(err.argmax())], err.max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,cap", [(4, 2, 32, 16, 20.0), (6, 2, 64, 64, 0.0), (3, 1, 7, 33, 3.0)])
def test_sigmoid_weight_attention_rows_and_tiles(ops, dtype, H, G, d, dv, cap):
    """Weights that are sigmoids of capped scores less a distance penalty, not normalised: single rows (with forced
    splits) and, in bfloat16, tiles, against the plain reference; one key a row planted far back among hundreds."""
    lengths, P_ = [333, 150], 16
    view = paged_cache(lengths, G, d, dv, P_, 0, dtype, seed=int(cap) + H)
    dev = on_device(view)
    g = torch.Generator().manual_seed(d)
    r1, r2, pb = 0.2 + torch.rand(H, generator=g), 0.05 + 0.4 * torch.rand(H, generator=g), -3.0 + torch.randn(H, generator=g)
    portions = [(0, 0, 150), (1, 0, 64), (0, 150, 17), (1, 64, 3), (0, 167, 166), (1, 67, 1), (1, 68, 82)]
    pos = [p0 + i for s_, p0, c in portions for i in range(c)]
    slot = [s_ for s_, p0, c in portions for i in range(c)]
    T = len(pos)
    q = torch.randn(T, H, d, generator=g, dtype=F64)
    for t in range(0, T, 3):          # a far key: position p // 7 of the row's request, aligned with one query head
        j, h = pos[t] // 7, t % H
        target = view.k[view.block_table[slot[t], j // P_], h // (H // G), j % P_].double()
        q[t, h] = 10.0 * target / target.norm() * math.sqrt(d)
    q = q.reshape(T, H * d).to(dtype)
    scale = d ** -0.5
    sig_cpu, sig_dev = (cap, r1, r2, pb), (cap, r1.to(DEV), r2.to(DEV), pb.to(DEV))
    want = torch.zeros(T, H * dv, dtype=F64)
    RefOps(F64).sink_attention(q, view, step_of(pos, slot, len(portions), "cpu"), want, H, G, d, dv, 0, 0, None, scale, sigmoid=sig_cpu)
    tol = 3e-5 if dtype == torch.float32 else 6e-2
    for kw in ({}, {"splits": (32, -(-(max(pos) + 1) // 32))}, {"tiling": tiling_of(portions)}):
        if "tiling" in kw and (dtype != torch.bfloat16 or d % 16 or dv % 16):
            continue
        out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
        ops.sink_attention(q.to(DEV), dev, step_of(pos, slot, len(portions)), out, H, G, d, dv, 0, 0, None, scale, sigmoid=sig_dev, **kw)
        err = (out.cpu().double() - want).abs().max(-1).values
        assert err.max().item() < tol * max(1.0, want.abs().max().item()), (list(kw), int(err.argmax()), err.max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("whole,v_from_k,q_temp,rot", [(True, True, None, 24), (False, False, (0.7, 5), 0), (False, False, None, 12),
                                                        (True, False, (0.5, 64), 8)])
def test_the_norm_and_rotation_kernel_in_its_new_forms(ops, dtype, whole, v_from_k, q_temp, rot):
    H, G, d, P_, T = 6, 2, 24, 16, 41
    dv = d if v_from_k else 10
    g = torch.Generator().manual_seed(rot + 3)
    W = (H + G) * d + (0 if v_from_k else G * dv)
    y = torch.randn(T, W + 5, generator=g)[:, :W]              # strided rows
    pos = torch.tensor([(5 * t) % 61 + (64 if t % 2 else 0) for t in range(T)], dtype=torch.int32)
    slot = torch.tensor([t % 2 for t in range(T)], dtype=torch.int32)
    half = max(rot // 2, 1)
    ang = torch.arange(130, dtype=F64)[:, None] * 300.0 ** (-2.0 * torch.arange(half, dtype=F64) / max(rot, 1))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    qw = 1 + 0.1 * torch.randn(H * d if whole else d, generator=g)
    kw = 1 + 0.1 * torch.randn(G * d if whole else d, generator=g)
    views = []
    for device in ("cpu", DEV):
        bt = torch.arange(2 * 9, dtype=torch.int32).reshape(2, 9)
        view = CacheView(torch.zeros(18, G, P_, d, dtype=dtype), torch.zeros(18, G, P_, dv, dtype=dtype), bt, P_, KVSpec(G, d, 0, dv))
        view = on_device(view) if device == DEV else view
        q_out = torch.zeros(T, H * d, dtype=dtype if device == DEV else F64, device=device)
        o = ops if device == DEV else RefOps(F64)
        mv = lambda t: t.to(device)
        o.qk_norm_write(mv(y), mv(qw), mv(kw), 1e-5, mv(pos), mv(slot), mv(cos), mv(sin), rot, "half", None, None, "half", q_out,
                        view, H, G, d, dv, torch.zeros(1, dtype=torch.int32, device=device), whole=whole, v_from_k=v_from_k,
                        q_temp=q_temp)
        views.append((q_out, view))
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    (q_ref, c_ref), (q_dev, c_dev) = views
    assert (q_dev.cpu().double() - q_ref).abs().max() < tol * max(1.0, float(q_ref.abs().max()))
    assert (c_dev.k.cpu().double() - c_ref.k.double()).abs().max() < tol and (c_dev.v.cpu().double() - c_ref.v.double()).abs().max() < tol


def _sum_norm_add_case(ops, ref, g, T, W):
    parts = [torch.randn(3, T, W, generator=g), torch.randn(1, T, W, generator=g)]
    bias = torch.randn(W, generator=g)
    y, gates = torch.randn(3 * T, W, generator=g), torch.rand(T, 3, generator=g)
    row_of = torch.randperm(3 * T, generator=g).to(torch.int32).reshape(T, 3)
    gamma = 1 + 0.1 * torch.randn(W, generator=g)
    for kw_cpu in (dict(branches=[(parts[0], bias), (parts[1], None)], scales=(1.2, 0.5), gamma=gamma, eps=1e-5),
                   dict(branches=[(parts[0], None)], scales=(1.0,), expert_rows=(y, row_of, gates), gamma=gamma, eps=1e-6),
                   dict(expert_rows=(y, row_of, gates), gamma=gamma, eps=1e-6),
                   dict(branches=[(parts[0], bias), (parts[1], None)], scales=(0.3, -2.0), accumulate=False)):
        dev = lambda v: v.to(DEV) if isinstance(v, torch.Tensor) else ([(a.to(DEV), b.to(DEV) if b is not None else None) for a, b in v]
                                                                      if isinstance(v, list) else
                                                                      (tuple(x.to(DEV) for x in v) if isinstance(v, tuple) and isinstance(v[0], torch.Tensor) else v))
        x = torch.randn(T, W, generator=g)
        a, b = x.clone().double(), x.clone().to(DEV)
        ref.sum_norm_add(a, **kw_cpu)
        ops.sum_norm_add(b, **{k: dev(v) for k, v in kw_cpu.items()})
        assert (b.cpu().double() - a).abs().max() < 2e-5


def test_the_small_kernels_beside_their_references(ops):
    g = torch.Generator().manual_seed(5)
    ref = RefOps(F64)
    # weighted sums of branches and expert rows, normed and added (rows of whole 16-byte units and not, a wide row)
    for T, W in ((37, 200), (37, 203), (5, 4096)):
        _sum_norm_add_case(ops, ref, g, T, W)
    # retention's rotated q and k, its constant decays and step sizes
    H, D, T = 3, 10, 29
    proj = torch.randn(T, 2 * H * D + 17, generator=g)
    pos = torch.randint(0, 90, (T,), generator=g).to(torch.int32)
    ang = torch.arange(90, dtype=F64)[:, None] * 50.0 ** (-2.0 * torch.arange(3, dtype=F64) / 6)[None, :]
    cos, sin, decay_h = torch.cos(ang).float(), torch.sin(ang).float(), torch.tensor([0.9, 0.97, 0.999])
    outs = []
    for device, o in (("cpu", ref), (DEV, ops)):
        qk, dec, dt = (torch.zeros(T, n, device=device) for n in (2 * H * D, H, H))
        o.retention_prepare(proj.to(device), pos.to(device), cos.to(device), sin.to(device), 6, "half", decay_h.to(device), D ** -0.5,
                            qk, dec, dt, H, D)
        outs.append((qk.cpu(), dec.cpu(), dt.cpu()))
    for a, b in zip(*outs):
        assert (a - b).abs().max() < 1e-5
    # the output gate number by number
    attn, gate = torch.randn(T, 4 * 6, generator=g), torch.randn(T, 4 * 6, generator=g)
    a, b = torch.zeros(T, 24, dtype=F64), torch.zeros(T, 24, device=DEV)
    ref.head_finish(attn.double(), pos, None, None, "half", gate, a, 4, 6)
    ops.head_finish(attn.to(DEV), pos.to(DEV), None, None, "half", gate.to(DEV), b, 4, 6)
    assert (b.cpu().double() - a).abs().max() < 1e-5


@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 2, 1), (6, 2, 3, 2), (4, 3, 1, 1), (64, 6, 8, 3), (3, 1, 3, 2), (256, 8, 64, 5), (8, 2, 8, 3)])
def test_the_grouped_sigmoid_router_beside_its_reference(ops, E, top, groups, keep):
    g = torch.Generator().manual_seed(E + top)
    T, W = 203, 72
    x = torch.randn(T, W, generator=g)
    wr = (2.5 * torch.randn(E, W, generator=g) / math.sqrt(W)).to(torch.bfloat16)
    for corr, normalize, scale in ((0.3 * torch.randn(E, generator=g), True, 2.5), (None, False, 1.0), (-2.0 + torch.randn(E, generator=g), True, 0.7)):
        ids_r, gates_r = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top)
        RefOps(torch.float32).router_sigmoid_grouped(x, wr, corr, top, groups, keep, normalize, scale, ids_r, gates_r)
        ids, gates = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
        logits = torch.zeros(T, E, device=DEV)
        ops.router_sigmoid_grouped(x.to(DEV), wr.to(DEV), corr.to(DEV) if corr is not None else None, top, groups, keep, normalize, scale,
                                   ids, gates, logits)
        # the rule applied to the kernel's own logits gives the kernel's choice exactly; against the reference's logits
        # only near-ties may fall the other way
        s = torch.sigmoid(logits.cpu().double())
        c = s + corr.double() if corr is not None else s.clone()
        per = E // groups
        if keep < groups:
            gs = c.view(T, groups, per).topk(min(2, per), -1).values.sum(-1)
            kept = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep], True)
            c = c.masked_fill(~kept[:, :, None].expand(T, groups, per).reshape(T, E), -math.inf)
        own = torch.sort(c, dim=-1, descending=True, stable=True).indices[:, :top]
        same = (own == ids.cpu().long()).all(-1)
        assert int((~same).sum()) <= 2, int((~same).sum())           # float32 sigmoids against float64 ones: a tie at most
        agree = (ids.cpu() == ids_r).all(-1)
        assert int((~agree).sum()) <= 0.02 * T + 1
        assert (gates.cpu()[agree] - gates_r[agree]).abs().max() < 1e-4


# ------------------------------------------------------------------------------------------------ the whole model
@pytest.fixture(scope="module", params=["D1", "D2", "D3"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("dumizen") / which, cfg, seed=3)
    reqs = traces.make_requests(cfg["vocab"], LENGTHS, seed=7)
    plain = {rid: P.forward(cfg, w, t)[0] for rid, t in reqs.items()}
    return which, cfg, folder, w, reqs, plain


def replay(folder, steps, dtype, page_size=64, record=False):
    rp = Replayer(folder, dtype=dtype, max_tokens=traces.max_tokens_needed(steps), page_size=page_size, max_requests=4, device=DEV)
    out, recs = {}, {}
    for s in steps:
        rec = {} if record else None
        lg = rp.run_step(s["entries"], s["end"], record=rec)
        if lg is not None:
            out[s["step"]] = lg
        recs[s["step"]] = rec
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, recs, rp


def followed(cfg, w, reqs, folder, dtype):
    """The plain implementation run with the experts the engine chose for the whole prompts (in bfloat16 a near-tie of
    two choice scores may fall the other way), and how many (row, run) choices differ from the plain router's own."""
    steps = traces.whole(reqs)
    _, recs, _ = replay(folder, steps, dtype, record=True)
    routed = [n for n, (i, _) in enumerate(P.run_order(cfg)) if cfg["layers"][i].get("mlp")]
    out, flips = {}, 0
    for s in steps:
        rid = s["entries"][0]["id"]
        ex = recs[s["step"]]["experts"]
        forced = {n: ex[k].cpu() for k, n in enumerate(routed)}
        own = P.forward(cfg, w, reqs[rid])[2]
        out[rid] = P.forward(cfg, w, reqs[rid], forced=[forced.get(n) for n in range(len(P.run_order(cfg)))])[0]
        flips += sum(int((own[n].sort(-1).values != forced[n].long().sort(-1).values).any(-1).sum()) for n in routed)
    return out, flips


def rel_err(got, want):
    d = got.double() - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp(min=1e-6))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_matches_plain_under_every_cut(setup, dtype):
    which, cfg, folder, w, reqs, plain = setup
    if dtype == "bfloat16":
        base, flips = followed(cfg, w, reqs, folder, dtype)
        assert flips <= 0.2 * sum(LENGTHS) * tiny.run_count(cfg)
    else:
        base = plain
    limit = 1e-4 if dtype == "float32" else 6e-2
    cuts = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, tail=40), "portions": traces.portions,
            "twos": lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3, 128)), "mixed": lambda r: traces.mixed(r, seed=3)}
    for name, cut in cuts.items():
        steps = cut(reqs)
        out, _, rp = replay(folder, steps, dtype, page_size=16 if name == "mixed" else 64)
        exp = traces.expected_rows(steps, base)
        assert set(out) == set(exp)
        errs = torch.cat([rel_err(out[k], torch.stack(rows)) for k, rows in exp.items()])
        bad = int((errs > limit).sum())
        assert bad <= (0 if dtype == "float32" else 0.1 * len(errs)), f"{name}: {bad} of {len(errs)} rows, worst {float(errs.max()):.3g}"
        if name == "mixed":
            assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2


def test_a_cut_changes_float32_logits_by_rounding_only(setup):
    which, cfg, folder, w, reqs, plain = setup
    one = {"r5": reqs["r5"]}
    a, _, _ = replay(folder, traces.whole(one), "float32")
    steps = traces.portions(one, sizes=(3, 2, 17, 64, 2, 1, 5))
    b, _, _ = replay(folder, steps, "float32", page_size=16)
    got = torch.cat([b[s["step"]] for s in steps if s["step"] in b])
    assert float(rel_err(got, a[0].double()).max()) < 2e-5


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16, 17, 18])
def test_configurations_drawn_at_random(seed, tmp_path):
    cfg = tiny.random_config(seed)
    folder, w = tiny.write_model(tmp_path / "m", cfg, seed=seed)
    reqs = traces.make_requests(cfg["vocab"], (1, 2, 23, 50, 85, 170), seed=seed)
    plain = {rid: P.forward(cfg, w, t)[0] for rid, t in reqs.items()}
    for cut in (traces.whole, lambda r: traces.tail_decoded(r, tail=45), lambda r: traces.portions(r, sizes=(2, 3, 16, 1, 2, 64)),
                lambda r: traces.mixed(r, seed=seed)):
        steps = cut(reqs)
        out, _, _ = replay(folder, steps, "float32", page_size=16)
        exp = traces.expected_rows(steps, plain)
        errs = torch.cat([rel_err(out[k], torch.stack(rows)) for k, rows in exp.items()])
        assert float(errs.max()) < 1e-4, (cfg, float(errs.max()))


def test_long_decoding_token_by_token(setup):
    """Two requests decoded side by side, one token a step each, over several pages, past every window and over many
    blocks, after prompts of unequal length: the captured decode step is replayed many times, and the retention's
    state and the means of blocks are carried through all of them."""
    which, cfg, folder, w, reqs, plain = setup
    a, b = reqs["r5"], reqs["r4"]
    rp = Replayer(folder, dtype="float32", max_tokens=512, page_size=16, max_requests=2, device=DEV)
    rp.run_step([{"id": "a", "tokens": a[:40], "want": []}, {"id": "b", "tokens": b[:3], "want": []}])
    worst = 0.0
    for i in range(66):
        out = rp.run_step([{"id": "a", "tokens": [a[40 + i]], "want": [0]}, {"id": "b", "tokens": [b[3 + i]], "want": [0]}])
        worst = max(worst, float(rel_err(out, torch.stack([plain["r5"][40 + i], plain["r4"][3 + i]])).max()))
    assert worst < 1e-4
    assert len(rp.model._graphs) >= 1


def test_greedy_generation_through_the_entry_point(setup):
    which, cfg, folder, w, reqs, plain = setup
    prompts = [reqs["r2"], reqs["r3"][:14], reqs["r0"]]
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(12):
            t = int(torch.argmax(P.forward(cfg, w, toks)[0][-1]))
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages in (16, 3):
        m = load_model(folder, dtype="float32", device=DEV, page_size=16, n_pages=n_pages, max_slots=4, max_step_tokens=24,
                       max_context=256)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        assert eng.generate(prompts, 12) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_program(setup, tmp_path, dtype):
    """bin/trace_run in a process of its own, fed a mixed trace over standard input."""
    which, cfg, folder, w, reqs, plain = setup
    steps = traces.mixed(reqs, seed=5)
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, f"{REPO}/bin/trace_run", "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(traces.max_tokens_needed(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l] == [f"done {s['step']}" for s in steps]
    exp = traces.expected_rows(steps, plain)
    errs = []
    for s in steps:
        f = out_dir / f"{s['step']}.f32"
        n = sum(len(e["want"]) for e in s["entries"])
        assert f.exists() == (n > 0)
        if n:
            got = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(n, cfg["vocab"]))
            errs.append(rel_err(got, torch.stack(exp[s["step"]])))
    errs = torch.cat(errs)
    if dtype == "float32":
        assert float(errs.max()) < 1e-4
    else:       # a near-tie of two choice scores may fall the other way at some rows
        assert float(errs.median()) < 4e-2


@pytest.mark.parametrize("T,W", [(1, 192), (8, 2048), (16, 4096), (300, 200), (2048, 1024), (40, 72)])
@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 2, 1), (64, 6, 8, 3), (16, 2, 4, 2)])
def test_the_grouped_sigmoid_router_rides_on_the_norm(ops, T, W, E, top, groups, keep):
    """The norm's kernel (a block a row, a cluster a row, many rows) chooses while it has the normalised row: its
    choice is exactly the rule applied to the logits it reports, and those agree with the plain product.  Rows narrower
    than twice the experts go to the norm and the stand-alone router one after the other."""
    from flint_b200.parts.base import RouterRequest
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g)
    gamma = 1 + 0.1 * torch.randn(W, generator=g)
    wr = (2.5 * torch.randn(E, W, generator=g) / math.sqrt(W)).to(torch.bfloat16)
    corr = 0.3 * torch.randn(E, generator=g)
    req = RouterRequest(wr.to(DEV), 0.0, torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV),
                        logits=torch.zeros(T, E, device=DEV), top=top, groups=groups, keep=keep, scale=2.5, rule="sigmoid_grouped",
                        correction=corr.to(DEV), normalize=True)
    out = torch.zeros(T, W, dtype=torch.bfloat16, device=DEV)
    ops.row_norm(x.to(DEV), gamma.to(DEV), None, 1e-6, "rms", out_bf16=out, router=req)
    normed = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6) * gamma.double()
    assert (req.logits.cpu().double() - normed @ wr.double().T).abs().max() < 1e-4
    ids_r, gates_r = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top, dtype=F64)
    # the rule on the kernel's own logits: x = logits, the router's matrix the identity
    RefOps(F64).router_sigmoid_grouped(req.logits.cpu().double(), torch.eye(E, dtype=F64), corr, top, groups, keep, True, 2.5, ids_r, gates_r)
    same = (ids_r == req.expert_ids.cpu()).all(-1)
    assert int((~same).sum()) <= max(1, T // 500)
    assert (gates_r[same] - req.gates.cpu().double()[same]).abs().max() < 1e-5


def test_chat_program_with_random_weights(tmp_path):
    """bin/flint_chat with ``--random-config FILE --seed N``, token ids in and out, greedy: the tokens of the folder
    that the random-weights mode writes for that configuration and seed, under the plain implementation."""
    from flint_b200.engine.loading import write_random_model
    from flint_b200.weights.safetensors_io import SafetensorsFile
    seed, cfg = 4, tiny.D1
    folder = write_random_model(tmp_path / "model", cfg, seed=seed)
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.read(n).double() for n in f.names()}
    prompt = [3, 50, 50, 7, 80, 0, 12, 13, 14, 15, 16]
    cfg_file = tmp_path / "only_config.json"
    cfg_file.write_text(json.dumps(cfg))
    proc = subprocess.run([sys.executable, f"{REPO}/bin/flint_chat", "--random-config", str(cfg_file), "--prompt", " ".join(map(str, prompt)),
                           "--max-tokens", "8", "--temperature", "0", "--seed", str(seed), "--dtype", "float32", "--ctx-size", "128"],
                          capture_output=True, text=True, timeout=600, env={**os.environ, "VERIFY_IDS": "1"})
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(x) for x in proc.stdout.split()]
    toks, want = list(prompt), []
    for _ in range(8):
        t = int(torch.argmax(P.forward(cfg, w, toks)[0][-1]))
        want.append(t)
        toks.append(t)
    assert got == want
