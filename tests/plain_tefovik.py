"""Tefovik written out plainly in float64, one function per mechanism, token loops where the design has a recurrence.

Nothing here is shared with the package: it reads the nested configuration as a dict and the weights by their stored
names.  Notation: h [T, W] are the rows a sublayer reads, p the positions 0 .. T - 1 of one sequence.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------- small pieces
def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def unit_length(x, eps):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def relu_squared(x):
    return torch.clamp(x, min=0) ** 2


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), with zeros before the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y if bias is None else y + bias


def turn_pairs(x, pos, base, dims, sign=1.0):
    """x [T, heads, d]: of every head's first ``dims`` dims, dim 2i and dim 2i + 1 turn together by the angle
    sign * pos * base^(-2i / dims); the other dims stay."""
    out = x.clone()
    for i in range(dims // 2):
        ang = sign * pos.to(F64) * base ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def chunk_visible(T, size):
    """[T, T] bool: query i sees key j when j <= i and both lie in the same run of ``size`` positions counted from 0
    (size 0: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok = ok & ((i // size) == (j // size))
    return ok


# ------------------------------------------------------------------------------------------------- mixers
def chunk_attention(h, w, p, m, eps):
    """The attention branch: conv -> per-head RMS norm of q, k -> rotation; values turned by their own position and
    the heads' sums turned back by the query's; softmax inside a run of positions; a sigmoid gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = causal_conv(h @ w[p + "q"].T, w[p + "q.conv"]).view(T, H, d)
    k = causal_conv(h @ w[p + "k"].T, w[p + "k.conv"]).view(T, G, d)
    v = causal_conv(h @ w[p + "v"].T, w[p + "v.conv"]).view(T, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q, k = turn_pairs(q, pos, base, dims), turn_pairs(k, pos, base, dims)
    v = turn_pairs(v, pos, base, dv)
    seen = chunk_visible(T, m.get("mask", {}).get("size", 0) if m.get("mask") else 0)
    heads = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        score = (q[:, a] @ k[:, g].T) * m["scale"]
        score = score.masked_fill(~seen, -math.inf)
        heads[:, a] = torch.softmax(score, -1) @ v[:, g]
    heads = turn_pairs(heads, pos, base, dv, sign=-1.0)
    heads = heads * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return heads.reshape(T, H * dv) @ w[p + "o"].T


def delta_rule_step(S, q, k, v, g, beta):
    """One token of one head.  S [d, dv]; g [d] the decay of the key channels.  Returns the new S and the read-out,
    which already sees this token's write."""
    S = g[:, None] * S
    u = beta * (v - S.T @ k)
    S = S + torch.outer(k, u)
    return S, S.T @ q


def gated_delta(h, w, p, m, eps, unit_eps=1e-6):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = unit_length(q, unit_eps) * d ** -0.5
    k = unit_length(k, unit_eps)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        kh = a // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S, o[t, a] = delta_rule_step(S, q[t, kh], k[t, kh], v[t, a], g[t, a], beta[t, a])
    o = unit_rms(o, eps) * w[p + "norm"]
    o = o * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def state_space_step(S, x, B, C, dt, rate, skip):
    """One token of one head.  S [N, dv]: S <- exp(-rate dt) S + dt B x^T; y = S^T C + skip x."""
    S = math.exp(-rate * dt) * S + dt * torch.outer(B, x)
    return S, S.T @ C + skip * x


def state_space(h, w, p, m, eps):
    T = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    y = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(N, dv, dtype=F64)
        for t in range(T):
            S, y[t, a] = state_space_step(S, x[t, a], B[t, g], C[t, g], float(dt[t, a]), float(rate[a]), w[p + "D"][a])
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def two_branches(h, w, p, m, eps):
    """Half the sum of the two branches, each first RMS-normed over the width and scaled by its own weight."""
    a = chunk_attention(h, w, p + "left.", m["left"], eps)
    b = gated_delta(h, w, p + "right.", m["right"], eps)
    return 0.5 * (unit_rms(a, eps) * w[p + "left.out"] + unit_rms(b, eps) * w[p + "right.out"])


def dense_ff(h, w, p):
    return relu_squared(h @ w[p + "up"].T) @ w[p + "down"].T


# ------------------------------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, keep=None):
    """Logits [T, vocab] of one sequence.  ``keep``: a dict that receives ``layers``, what every layer hands on."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = layer_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    results = [x]
    handed_on = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "parallel":
            mix = two_branches(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "mamba2":
            mix = state_space(x, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = layer_norm(alpha * x + w[p + "ls1"] * mix, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = layer_norm(alpha * x + w[p + "ls2"] * dense_ff(x, w, p + "mlp."), w[p + "norm2"], eps)
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        handed_on.append(x)
    if keep is not None:
        keep["layers"] = handed_on
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg["logit_softcap"]
    return cap * torch.tanh(logits / cap)
