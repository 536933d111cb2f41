"""Tefovik on the GPU: each new kernel beside the plain function of its mechanism (keys planted at both ends of a
run of positions, just before it, far back and at page borders, in prompts and in decoding; the convolution and both
recurrences cut anywhere; the norms, gates and sums around them), and the whole model under every cut, in long
decoding and in generation, beside the plain implementation."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_tefovik as P
import tiny_tefovik as tiny
import traces
from flint_b200.cache.manager import CacheView, KVSpec
from flint_b200.engine.engine import Engine
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.sampling.params import SamplingParams
from test_gepadra_gpu import paged_kv, step_of

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = (1, 2, 9, 37, 70, 130)


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


def run_attention(q, dense, pos, slot, H, G, scale, chunk):
    """Softmax attention row by row over the keys of the row's own run of ``chunk`` positions."""
    out = []
    for t in range(q.shape[0]):
        p = int(pos[t])
        k, v = dense[int(slot[t])]
        lo = (p // chunk) * chunk if chunk else 0
        k, v = k[lo:p + 1], v[lo:p + 1]
        heads = []
        for h in range(H):
            s = (k[:, h // (H // G)] @ q[t, h].double()) * scale
            heads.append(torch.softmax(s, 0) @ v[:, h // (H // G)])
        out.append(torch.stack(heads))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv", [(6, 2, 12, 10), (8, 4, 32, 16), (3, 1, 10, 34), (8, 1, 64, 64)])
@pytest.mark.parametrize("chunk", [9, 16, 40, 100])
def test_chunked_attention_finds_planted_keys(ops, dtype, H, G, d, dv, chunk):
    """One key a row is made to stand out: the first key of the row's run, the last key of the run before it (which
    the row must not see, however large its score), a key many runs back, keys on both sides of page borders, the
    row's own.  Single rows as in decoding, two requests, with and without forced splits of the key range."""
    g = torch.Generator().manual_seed(H * 1000 + d + chunk)
    n, P_ = [333, 150], 16
    keys = [torch.randn(m, G, d, generator=g, dtype=F64) for m in n]
    values = [torch.randn(m, G, dv, generator=g, dtype=F64) for m in n]
    rows = []          # (slot, position, planted key)
    for s, m in enumerate(n):
        for p in (m - 1, m - 2, ((m - 1) // chunk) * chunk, ((m - 1) // chunk) * chunk - 1, chunk, chunk - 1, 17, 16, 15, 1, 0):
            lo = (p // chunk) * chunk
            for j in {0, lo, lo - 1, lo + 1, p - 1, p, (p // P_) * P_, (p // P_) * P_ - 1, lo - chunk, 31, 32}:
                if 0 <= j <= p:
                    rows.append((s, p, j))
    unit = torch.nn.functional.normalize(torch.randn(len(rows), d, generator=g, dtype=F64), dim=-1)
    q = torch.randn(len(rows), H, d, generator=g, dtype=F64)
    for r in range(len(rows)):
        q[r, r % H] = 8.0 * unit[r] * math.sqrt(d)
    by_key = {}
    for r, (s, p, j) in enumerate(rows):
        by_key.setdefault((s, j), []).append(r)
    scale = d ** -0.5
    hidden = 0
    for (s, j), rs in by_key.items():
        kk = [k.clone() for k in keys]
        kk[s][j, (rs[0] % H) // (H // G)] = 3.0 * unit[rs[0]] * math.sqrt(d)
        view, dense = paged_kv(kk, values, P_, dtype, seed=j)
        qs = q[rs].to(dtype)
        pos, slot = [rows[r][1] for r in rs], [rows[r][0] for r in rs]
        hidden += sum(j < (p // chunk) * chunk for p in pos)
        want = run_attention(qs, dense, pos, slot, H, G, scale, chunk)
        for splits in (None, (8, -(-min(max(pos) + 1, chunk) // 8))):
            out = torch.zeros(len(rs), H * dv, dtype=dtype, device=DEV)
            ops.sink_attention(qs.reshape(len(rs), H * d).to(DEV), view, step_of(pos, slot, len(rs)), out, H, G, d, dv, 0, 0,
                               None, scale, splits=splits, chunk=chunk)
            err = (out.cpu().double().view(len(rs), H, dv) - want).abs().max().item()
            assert err < (2e-5 if dtype == torch.float32 else 3e-2), (s, j, splits, err)
    assert hidden > 10          # rows whose planted key lies before their run were among them


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 32, 16), (8, 8, 128, 48), (6, 2, 64, 128), (2, 1, 16, 64)])
@pytest.mark.parametrize("chunk", [9, 16, 40, 100, 200])
def test_chunked_attention_tiles_on_the_tensor_cores(ops, H, G, d, dv, chunk):
    """Portions of prompts as tiles of up to 64 rows (whole tiles, a ragged last one, portions that start in the
    middle of a run and of a page, tiles that hold several runs) beside single rows, two requests: the tensor-core
    kernel and the row kernel together against the plain mechanism, with peaked scores."""
    from flint_b200.engine.step import Tiling
    g = torch.Generator().manual_seed(H + d + chunk)
    n, P_ = [333, 150], 16
    keys = [2.0 * torch.randn(m, G, d, generator=g, dtype=F64) for m in n]
    values = [torch.randn(m, G, dv, generator=g, dtype=F64) for m in n]
    view, dense = paged_kv(keys, values, P_, torch.bfloat16, seed=3)
    portions = [(0, 0, 150), (1, 0, 64), (0, 150, 17), (1, 64, 3), (0, 167, 166), (1, 67, 1), (1, 68, 82)]    # (slot, first position, count)
    pos = [p0 + i for s_, p0, c in portions for i in range(c)]
    slot = [s_ for s_, p0, c in portions for i in range(c)]
    T = len(pos)
    q = (2.0 * torch.randn(T, H, d, generator=g, dtype=F64)).to(torch.bfloat16)
    scale = d ** -0.5
    tiles, others, row = [], [], 0
    for s_, p0, c in portions:
        if c < 16:
            others += range(row, row + c)
        else:
            for r in range(0, c, 64):
                tiles.append([row + r, min(64, c - r), s_, p0 + r])
        row += c
    tiles.sort(key=lambda t: -(t[3] + t[1]))
    tiling = Tiling(torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles), torch.tensor(others, dtype=torch.int32, device=DEV), len(others))
    want = run_attention(q, dense, pos, slot, H, G, scale, chunk)
    out = torch.zeros(T, H * dv, dtype=torch.bfloat16, device=DEV)
    ops.sink_attention(q.reshape(T, H * d).to(DEV), view, step_of(pos, slot, len(portions)), out, H, G, d, dv, 0, 0, None, scale,
                       tiling=tiling, chunk=chunk)
    err = (out.cpu().double().view(T, H, dv) - want).abs()
    assert err.max().item() < 4e-2, (int(err.view(T, -1).max(-1).values.argmax()), err.max().item())
    plain = torch.zeros_like(out)
    ops.sink_attention(q.reshape(T, H * d).to(DEV), view, step_of(pos, slot, len(portions)), plain, H, G, d, dv, 0, 0, None, scale,
                       chunk=chunk)
    assert (plain.float() - out.float()).abs().max().item() < 4e-2


def batches_of(pieces, starts, slots_of):
    """pieces: list of batches, a batch a list of (request, first token, count) -> per batch (rows of the flat
    arrays, positions, slots, where each request's rows start, whether every request brings one token)."""
    for batch in pieces:
        rows = [starts[r] + a + i for r, a, c in batch for i in range(c)]
        pos = [a + i for r, a, c in batch for i in range(c)]
        slot = [slots_of[r] for r, a, c in batch for _ in range(c)]
        seq = [0]
        for r, a, c in batch:
            seq.append(seq[-1] + c)
        yield rows, pos, slot, seq, all(c == 1 for _, _, c in batch)


LENS = [23, 1, 40]
STARTS = [0, 23, 24]
SLOTS = [3, 0, 2]
CUTS = {
    "whole": [[(0, 0, 23), (1, 0, 1), (2, 0, 40)]],
    "cut": [[(0, 0, 2), (2, 0, 17)], [(2, 17, 1), (0, 2, 1), (1, 0, 1)], [(0, 3, 20), (2, 18, 2)], [(2, 20, 19)], [(2, 39, 1)]],
    "sixes": [[(0, 0, 6), (2, 0, 7)], [(0, 6, 6), (2, 7, 6)], [(0, 12, 11), (2, 13, 12), (1, 0, 1)], [(2, 25, 15)]],
    "ones": [[(0, i, 1), (2, i, 1)] + ([(1, 0, 1)] if i == 0 else []) for i in range(23)] + [[(2, i, 1)] for i in range(23, 40)],
}


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("C,col0,act,bias", [(37, 0, "none", False), (96, 5, "silu", True), (1300, 64, "silu", False)])
def test_short_convolution_carries_its_last_inputs_however_the_tokens_are_cut(ops, taps, C, col0, act, bias):
    """Three requests against the plain convolution of each whole sequence: in one batch, in portions (also
    portions longer than twice the taps), token by token, in slots whose state an earlier request left behind."""
    g = torch.Generator().manual_seed(taps * 100 + C)
    T = sum(LENS)
    u = torch.randn(T, col0 + C + 3, generator=g)
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    want = torch.cat([P.causal_conv(u[s:s + n, col0:col0 + C].double(), w.double(), b.double() if bias else None)
                      for s, n in zip(STARTS, LENS)])
    if act == "silu":
        want = P.silu(want)
    width = max(taps - 1, 1) * C
    for name, pieces in CUTS.items():
        state = torch.full((5, width + 2), 7.0, device=DEV)
        for s in SLOTS:
            state[s, :width].zero_()
        out = torch.zeros(T, C, dtype=F64)
        for rows, pos, slot, seq, single in batches_of(pieces, STARTS, SLOTS):
            y = torch.zeros(len(rows), C, device=DEV)
            ops.short_conv(u[rows].to(DEV), col0, w.to(DEV), b.to(DEV) if bias else None, act,
                           torch.tensor(pos, dtype=torch.int32, device=DEV), torch.tensor(slot, dtype=torch.int32, device=DEV),
                           state[:, :width] if taps > 1 else None, y)
            out[rows] = y.cpu().double()
        assert (out - want).abs().max() < 2e-5 * max(1.0, float(want.abs().max())), name
        assert float(state[4].min()) == 7.0 and float(state[:, width:].min()) == 7.0      # nothing else was touched


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 20, 6), (3, 3, 40, 12), (2, 1, 64, 48), (2, 2, 130, 33), (4, 4, 32, 32), (2, 1, 144, 64)])
def test_delta_rule_kernels_follow_the_recurrence_however_the_tokens_are_cut(ops, H, G, D, V):
    g = torch.Generator().manual_seed(H + D + V)
    T = sum(LENS)
    y = torch.randn(T, 2 * G * D + H * V + 3, generator=g)          # q | k | v as the convolution leaves them
    braw = torch.randn(T, H + 2, generator=g)[:, 1:1 + H] * 2.0
    a = torch.randn(T, H * D, generator=g) * 2.0
    dt_bias, a_log = torch.randn(H * D, generator=g) - 1.0, -3.0 + 3.0 * torch.rand(H, generator=g)
    q = P.unit_length(y[:, :G * D].double().view(T, G, D), 1e-6) * D ** -0.5
    k = P.unit_length(y[:, G * D:2 * G * D].double().view(T, G, D), 1e-6)
    v = y[:, 2 * G * D:2 * G * D + H * V].double().view(T, H, V)
    beta = torch.sigmoid(braw.double())
    decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * P.softplus(a.double() + dt_bias.double()).view(T, H, D))
    want = torch.zeros(T, H, V, dtype=F64)
    for s, n in zip(STARTS, LENS):
        for h in range(H):
            S = torch.zeros(D, V, dtype=F64)
            for t in range(s, s + n):
                S, want[t, h] = P.delta_rule_step(S, q[t, h // (H // G)], k[t, h // (H // G)], v[t, h], decay[t, h], beta[t, h])
    scale = max(1.0, float(want.abs().max()))
    for name, pieces in CUTS.items():
        state = torch.full((5, H * D * V + 4), 7.0, device=DEV)
        for s in SLOTS:
            state[s, :H * D * V].zero_()
        out = torch.zeros(T, H, V, dtype=F64)
        for rows, pos, slot, seq, single in batches_of(pieces, STARTS, SLOTS):
            n = len(rows)
            yy, bb, aa = y[rows].to(DEV), braw[rows].to(DEV), a[rows].contiguous().to(DEV)
            qk, dec, be = torch.zeros(n, 2 * G * D, device=DEV), torch.zeros(n, H * D, device=DEV), torch.zeros(n, H, device=DEV)
            ops.delta_prepare(yy, bb, aa, dt_bias.to(DEV), a_log.to(DEV), qk, dec, be, H, G, D, 1e-6)
            assert (dec.cpu().double().view(n, H, D) - decay[rows]).abs().max() < 1e-6
            assert (qk.cpu().double() - torch.cat([q[rows].reshape(n, -1), k[rows].reshape(n, -1)], 1)).abs().max() < 1e-6
            o = torch.zeros(n, H * V, device=DEV)
            ops.recurrence_scan(qk[:, :G * D], qk[:, G * D:], yy[:, 2 * G * D:2 * G * D + H * V], dec, True, be, None, None,
                                torch.tensor(slot, dtype=torch.int32, device=DEV),
                                None if single else torch.tensor(seq, dtype=torch.int32, device=DEV), len(seq) - 1,
                                state[:, :H * D * V], o, H, G, D, V)
            out[rows] = o.cpu().double().view(n, H, V)
        assert (out - want).abs().max() < 2e-5 * scale, name
        assert float(state[4].min()) == 7.0 and float(state[:, H * D * V:].min()) == 7.0


@pytest.mark.parametrize("H,G,N,V", [(3, 1, 7, 10), (4, 2, 40, 6), (8, 2, 32, 16), (2, 1, 144, 64), (2, 2, 128, 64)])
def test_state_space_kernels_follow_the_recurrence_however_the_tokens_are_cut(ops, H, G, N, V):
    g = torch.Generator().manual_seed(H + N + V)
    T = sum(LENS)
    y = torch.randn(T, H * V + 2 * G * N, generator=g)              # x | B | C as the convolution leaves them
    raw = torch.randn(T, H + 3, generator=g)[:, 3:] * 2.0
    dt_bias, a_log, skip = torch.randn(H, generator=g) - 1.0, -2.0 + 2.5 * torch.rand(H, generator=g), torch.randn(H, generator=g)
    x = y[:, :H * V].double().view(T, H, V)
    B = y[:, H * V:H * V + G * N].double().view(T, G, N)
    C = y[:, H * V + G * N:].double().view(T, G, N)
    dt = P.softplus(raw.double() + dt_bias.double())
    want = torch.zeros(T, H, V, dtype=F64)
    for s, n in zip(STARTS, LENS):
        for h in range(H):
            S = torch.zeros(N, V, dtype=F64)
            for t in range(s, s + n):
                S, want[t, h] = P.state_space_step(S, x[t, h], B[t, h // (H // G)], C[t, h // (H // G)], float(dt[t, h]),
                                                   float(torch.exp(a_log[h].double())), skip[h].double())
    scale = max(1.0, float(want.abs().max()))
    for name, pieces in CUTS.items():
        state = torch.full((5, H * N * V + 4), 7.0, device=DEV)
        for s in SLOTS:
            state[s, :H * N * V].zero_()
        out = torch.zeros(T, H, V, dtype=F64)
        for rows, pos, slot, seq, single in batches_of(pieces, STARTS, SLOTS):
            n = len(rows)
            yy = y[rows].to(DEV)
            d1, dec = torch.zeros(n, H, device=DEV), torch.zeros(n, H, device=DEV)
            ops.ssd_prepare(raw[rows].to(DEV), dt_bias.to(DEV), a_log.to(DEV), d1, dec)
            assert (d1.cpu().double() - dt[rows]).abs().max() < 1e-5
            o = torch.zeros(n, H * V, device=DEV)
            ops.recurrence_scan(yy[:, H * V + G * N:], yy[:, H * V:H * V + G * N], yy[:, :H * V], dec, False, None, d1, skip.to(DEV),
                                torch.tensor(slot, dtype=torch.int32, device=DEV),
                                None if single else torch.tensor(seq, dtype=torch.int32, device=DEV), len(seq) - 1,
                                state[:, :H * N * V], o, H, G, N, V)
            out[rows] = o.cpu().double().view(n, H, V)
        assert (out - want).abs().max() < 2e-5 * scale, name
        assert float(state[4].min()) == 7.0 and float(state[:, H * N * V:].min()) == 7.0


def tables(pos_max, dims, base):
    half = max(dims // 2, 1)
    ang = torch.arange(pos_max + 1, dtype=F64)[:, None] * base ** (-2.0 * torch.arange(half, dtype=F64) / max(dims, 1))[None, :]
    return torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)


def turn_halves(x, pos, base, dims, sign=1.0):
    """dims i and i + dims/2 turn together: the plain rotation of pairs on a permuted copy."""
    d = x.shape[-1]
    perm = [j for i in range(dims // 2) for j in (i, i + dims // 2)] + list(range(dims, d))
    inv = [perm.index(i) for i in range(d)]
    return P.turn_pairs(x[..., perm], pos, base, dims, sign)[..., inv]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style,rot,normed", [("interleaved", 8, True), ("interleaved", 12, True), ("half", 12, False),
                                              ("interleaved", 0, True), ("half", 4, True)])
def test_q_and_k_are_normed_and_turned_values_turned_and_the_sums_turned_back(ops, dtype, style, rot, normed):
    H, G, d, dv, P_, T = 6, 2, 12, 10, 16, 37
    g = torch.Generator().manual_seed(rot + 1)
    W = (H + G) * d + G * dv
    y = torch.randn(T, W + 4, generator=g)
    pos = torch.tensor([(5 * t) % 61 for t in range(T)], dtype=torch.int32)
    slot = torch.tensor([t % 2 for t in range(T)], dtype=torch.int32)
    pos[1::2] += 64          # no two rows of a slot share a position
    base, eps = 300.0, 1e-5
    qn, kn = 1.0 + 0.3 * torch.randn(d, generator=g), 1.0 + 0.3 * torch.randn(d, generator=g)
    turn = P.turn_pairs if style == "interleaved" else turn_halves
    x = y.double()
    q, k = x[:, :H * d].view(T, H, d), x[:, H * d:(H + G) * d].view(T, G, d)
    v = x[:, (H + G) * d:W].view(T, G, dv)
    if normed:
        q, k = P.unit_rms(q, eps) * qn.double(), P.unit_rms(k, eps) * kn.double()
    q, k, v = turn(q, pos, base, rot), turn(k, pos, base, rot), turn(v, pos, base, dv)
    cos, sin = tables(int(pos.max()), rot, base)
    vcos, vsin = tables(int(pos.max()), dv, base)
    n_pages = 2 * 9
    view = CacheView(torch.zeros(n_pages, G, P_, d, dtype=dtype, device=DEV), torch.zeros(n_pages, G, P_, dv, dtype=dtype, device=DEV),
                     torch.arange(n_pages, dtype=torch.int32).view(2, 9).to(DEV), P_, KVSpec(G, d, 0, dv))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_out = torch.zeros(T, H * d, dtype=dtype, device=DEV)
    ops.qk_norm_write(y.to(DEV), qn.to(DEV) if normed else None, kn.to(DEV) if normed else None, eps, pos.to(DEV), slot.to(DEV),
                      cos, sin, rot, style, vcos, vsin, style, q_out, view, H, G, d, dv, status)
    tol = 4e-5 if dtype == torch.float32 else 4e-2
    assert (q_out.cpu().double().view(T, H, d) - q).abs().max() < tol
    page = view.block_table.cpu()[slot.long(), (pos // P_).long()].long()
    assert (view.k.cpu()[page, :, (pos % P_).long()].double() - k).abs().max() < tol
    assert (view.v.cpu()[page, :, (pos % P_).long()].double() - v).abs().max() < tol
    assert int(status.item()) == 0
    # the heads' sums: turned back by the row's position, times the sigmoid of one number a head
    attn = torch.randn(T, H * dv, generator=g).to(dtype)
    gate = torch.randn(T, H + 3, generator=g)[:, 2:2 + H] * 2.0
    out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
    ops.head_finish(attn.to(DEV), pos.to(DEV), vcos, vsin, style, gate.to(DEV), out, H, dv)
    want = turn(attn.double().view(T, H, dv), pos, base, dv, sign=-1.0) * torch.sigmoid(gate.double())[:, :, None]
    assert (out.cpu().double().view(T, H, dv) - want).abs().max() < tol
    ops.head_finish(attn.to(DEV), pos.to(DEV), None, None, style, None, out, H, dv)
    assert torch.equal(out.cpu(), attn)


@pytest.mark.parametrize("T,W", [(41, 40), (7, 256), (300, 2048), (3, 5000)])
def test_the_norm_after_the_sum_the_mean_of_branches_the_sum_over_depth_and_the_cap(ops, T, W):
    g = torch.Generator().manual_seed(T + W)
    eps = 1e-5
    x = torch.randn(T, W, generator=g) * 3.0 + 0.5
    parts = torch.randn(3, T, W, generator=g)
    bias, s = torch.randn(W, generator=g), 1.0 + 0.3 * torch.randn(W, generator=g)
    gamma = 1.0 + 0.1 * torch.randn(W, generator=g)
    want = P.layer_norm(2.5 * x.double() + s.double() * (parts.double().sum(0) + bias.double()), gamma.double(), eps)
    for copy_dtype in (None, torch.bfloat16):
        xx = x.clone().to(DEV)
        copy = torch.zeros(T, W, dtype=copy_dtype, device=DEV) if copy_dtype else None
        ops.post_norm(xx, parts.to(DEV), bias.to(DEV), s.to(DEV), 2.5, gamma.to(DEV), None, eps, "layer", out_copy=copy)
        assert (xx.cpu().double() - want).abs().max() < 2e-5 * float(want.abs().max())
        if copy is not None:
            assert torch.equal(copy.cpu(), xx.cpu().to(torch.bfloat16))
    xx = x.clone().to(DEV)
    ops.post_norm(xx, parts[:1].to(DEV), None, None, 1.0, gamma.to(DEV), None, eps, "rms")
    want = P.unit_rms(x.double() + parts[0].double(), eps) * gamma.double()
    assert (xx.cpu().double() - want).abs().max() < 2e-5 * float(want.abs().max())
    # the mean of branches, each divided by its own root mean square
    a, b = torch.randn(2, T, W, generator=g) * 5.0, torch.randn(1, T, W, generator=g) * 0.1
    wa, wb = 1.0 + 0.2 * torch.randn(W, generator=g), 1.0 + 0.2 * torch.randn(W, generator=g)
    out = torch.zeros(T, W, device=DEV)
    ops.branch_mean([(a.to(DEV), bias.to(DEV)), (b.to(DEV), None)], [wa.to(DEV), wb.to(DEV)], eps, out)
    want = 0.5 * (P.unit_rms(a.double().sum(0) + bias.double(), eps) * wa.double() + P.unit_rms(b.double()[0], eps) * wb.double())
    assert (out.cpu().double() - want).abs().max() < 2e-5 * float(want.abs().max())
    # the weighted sum over depth
    hist = torch.randn(5, T, W, generator=g)
    w = torch.randn(6, generator=g)
    h = torch.randn(T, W, generator=g)
    hh, hd = h.clone().to(DEV), hist.clone().to(DEV)
    copy = torch.zeros(T, W, dtype=torch.bfloat16, device=DEV)
    ops.depth_mix(hd, 4, w.to(DEV), hh, out_copy=copy)
    want = sum(w[j].double() * hist[j].double() for j in range(3)) + w[3].double() * h.double()
    assert (hh.cpu().double() - want).abs().max() < 2e-5 * float(want.abs().max())
    assert torch.equal(hd[3].cpu(), h) and torch.equal(hd[4].cpu(), hist[4]) and torch.equal(copy.cpu(), hh.cpu().to(torch.bfloat16))
    # the cap, and the cast
    z = (torch.randn(T, W, generator=g) * 20.0).to(DEV)
    want = 15.0 * torch.tanh(z.cpu().double() / 15.0)
    ops.softcap(z, 15.0)
    assert (z.cpu().double() - want).abs().max() < 1e-5
    c = torch.zeros(T, W, dtype=torch.bfloat16, device=DEV)
    ops.cast_rows(x.to(DEV), c)
    assert torch.equal(c.cpu(), x.to(torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,V,groups,per_head,first,act", [(4, 6, 4, True, False, "sigmoid"), (3, 10, 3, False, True, "silu"),
                                                            (8, 16, 1, False, True, "silu"), (2, 64, 2, True, False, "sigmoid"),
                                                            (32, 64, 8, False, True, "silu")])
def test_heads_outputs_are_normed_in_parts_and_gated(ops, dtype, H, V, groups, per_head, first, act):
    g = torch.Generator().manual_seed(H + V)
    T, N, eps = 19, H * V, 1e-5
    o = torch.randn(T, N, generator=g) * 4.0
    gate = torch.randn(T, N + 7, generator=g)[:, 3:3 + N] * 2.0
    w = 1.0 + 0.2 * torch.randn(V if per_head else N, generator=g)
    gd = gate.double()
    gv = P.silu(gd) if act == "silu" else torch.sigmoid(gd)
    x = o.double() * gv if first else o.double()
    x = P.unit_rms(x.view(T, groups, N // groups), eps).reshape(T, N) * (w.double().repeat(H) if per_head else w.double())
    want = x if first else x * gv
    out = torch.zeros(T, N, dtype=dtype, device=DEV)
    ops.gated_norm(o.to(DEV), gate.to(DEV), act, first, w.to(DEV), eps, groups, out)
    assert (out.cpu().double() - want).abs().max() < (2e-5 if dtype == torch.float32 else 2e-2) * float(want.abs().max())


def test_the_squared_relu(ops):
    g = torch.Generator().manual_seed(1)
    parts = torch.randn(2, 33, 70, generator=g)
    out = torch.zeros(33, 70, device=DEV)
    ops.row_act(parts.to(DEV), out, "relu2")
    assert (out.cpu().double() - P.relu_squared(parts.double().sum(0))).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------- the whole model
@pytest.fixture(scope="module", params=["T1", "T2"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("tefovik") / which, cfg, seed=3, ranks=tiny.RANKS[which])
    reqs = traces.make_requests(cfg["vocab"], LENGTHS, seed=7)
    plain = {rid: P.forward(cfg, w, t) for rid, t in reqs.items()}
    return which, cfg, folder, w, reqs, plain


def replay(folder, steps, dtype, page_size=64):
    rp = Replayer(folder, dtype=dtype, max_tokens=traces.max_tokens_needed(steps), page_size=page_size, max_requests=4, device=DEV)
    out = {}
    for s in steps:
        lg = rp.run_step(s["entries"], s["end"])
        if lg is not None:
            out[s["step"]] = lg
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, rp


def rel_err(got, want):
    d = got.double() - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp(min=1e-6))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_matches_plain_under_every_cut(setup, dtype):
    which, cfg, folder, w, reqs, plain = setup
    limit = 1e-4 if dtype == "float32" else 5e-2
    cuts = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, tail=24), "portions": traces.portions,
            "twos": lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3, 128)), "mixed": lambda r: traces.mixed(r, seed=3)}
    for name, cut in cuts.items():
        steps = cut(reqs)
        out, rp = replay(folder, steps, dtype, page_size=16 if name == "mixed" else 64)
        exp = traces.expected_rows(steps, plain)
        assert set(out) == set(exp)
        errs = torch.cat([rel_err(out[k], torch.stack(rows)) for k, rows in exp.items()])
        assert float(errs.max()) < limit, f"{name}: worst {float(errs.max()):.3g}, median {float(errs.median()):.3g}"
        if name == "mixed":
            assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2


@pytest.mark.parametrize("seed", [2, 7, 23, 41])
def test_configurations_drawn_at_random_match_plain_in_float32(seed, tmp_path):
    """Sizes, constants and orders of layers that no other test has, whole and under three cuts."""
    cfg, ranks = tiny.random_config(seed)
    folder, w = tiny.write_model(tmp_path / "m", cfg, seed=seed, ranks=ranks)
    reqs = traces.make_requests(cfg["vocab"], (1, 2, 9, 37, 70, 150), seed=seed)
    plain = {rid: P.forward(cfg, w, t) for rid, t in reqs.items()}
    cuts = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, tail=24),
            "twos": lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3, 128)), "mixed": lambda r: traces.mixed(r, seed=3)}
    for name, cut in cuts.items():
        steps = cut(reqs)
        out, _ = replay(folder, steps, "float32", page_size=16 if name == "mixed" else 64)
        exp = traces.expected_rows(steps, plain)
        assert set(out) == set(exp)
        errs = torch.cat([rel_err(out[k], torch.stack(rows)) for k, rows in exp.items()])
        assert float(errs.max()) < 1e-4, f"{name}: worst {float(errs.max()):.3g} for {cfg}"


def test_a_cut_changes_float32_logits_by_rounding_only(setup):
    """The same request whole, in twos and token by token: the recurrences and the convolutions walk the tokens in
    the same order whatever the cut, so the logits agree far below the distance to the plain implementation."""
    which, cfg, folder, w, reqs, plain = setup
    one = {"r4": reqs["r4"]}
    base, _ = replay(folder, traces.whole(one), "float32")
    ref = base[0]
    for steps in (traces.portions(one, sizes=(2,)), traces.portions(one, sizes=(1,)), traces.portions(one, sizes=(33, 5, 9))):
        out, _ = replay(folder, steps, "float32", page_size=16)
        got = torch.cat([out[s["step"]] for s in steps])
        assert float(rel_err(got, ref.double()).max()) < 2e-5


def test_long_decoding_token_by_token(setup):
    """Two requests decoded side by side, one token a step each, over several pages and runs of positions, after
    prompts of unequal length: the captured decode step is replayed many times and every state is carried through."""
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
            lg = P.forward(cfg, w, toks)[-1]
            t = int(torch.argmax(lg))
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
    assert float(torch.cat(errs).max()) < (1e-4 if dtype == "float32" else 5e-2)


def test_chat_program_with_random_weights(tmp_path):
    """bin/flint_chat with ``--random-config FILE --seed N``, token ids in and out, greedy: the tokens of the folder
    that the random-weights mode writes for that configuration and seed, under the plain implementation."""
    from flint_b200.engine.loading import write_random_model
    from flint_b200.weights.safetensors_io import SafetensorsFile
    seed, cfg = 4, tiny.T1
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
        t = int(torch.argmax(P.forward(cfg, w, toks)[-1]))
        want.append(t)
        toks.append(t)
    assert got == want
