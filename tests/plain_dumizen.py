"""Dumizen, plainly: one function per mechanism, whole sequences from position 0, float64, slow.

Nothing here is shared with the package: the tests compare the engine against these functions.  ``cfg`` is the
parsed config.json (a dict), ``w`` maps tensor names to float64 tensors.

A layer is  x <- x + n1b(mixer(n1(x)));  x <- x + n2b(ff(n2(x)))  with RMS norms n(x) = x / sqrt(mean(x^2) + eps) * g.
Layers ``loop.start .. loop.stop - 1`` run ``loop.times`` times with the same weights; before every pass
x <- W_in [x; x0] + step[t] with x0 the embedded rows.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, g, eps):
    return rms(x, eps) * g


# ------------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """(frequencies [dims/2], factor on cos and sin) of a ``rot`` section; YaRN if it has ``scaling``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(t):
        return dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1


def rotate(x, pos, rot):
    """x [T, heads, dim]: the first rot.dims dims of every head turn by the row's position, dim i with i + dims/2."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = pos.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def expand_kv(t, heads):
    """[T, G, d] -> [T, heads, d]: query head h reads key/value head floor(h / (heads / G))."""
    return t.repeat_interleave(heads // t.shape[1], dim=1)


# ------------------------------------------------------------------------------------------------ mixers
def pooled_window_attention(h, w, pre, m, eps):
    """Softmax attention over the last mask.size positions and, behind them, one mean key and value per block of
    mask.pool positions that lies wholly before the window."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, V)
    q = rotate(rms(q, eps) * w[pre + "q.norm"], pos, m.get("rot"))
    k = rotate(rms(k, eps) * w[pre + "k.norm"], pos, m.get("rot"))
    mask = m.get("mask")
    i, j = pos[:, None], pos[None, :]
    if mask:
        size, P = int(mask["size"]), int(mask.get("pool") or 0)
        seen = (i - j >= 0) & (i - j < size)
        nb = T // P if P else 0            # without a block size: the window alone
        P = P or 1
        kp = k[:nb * P].view(nb, P, G, D).mean(1)
        vp = v[:nb * P].view(nb, P, G, V).mean(1)
        b = torch.arange(nb)[None, :]
        seen_p = b * P + P - 1 <= i - size
    else:
        seen = i >= j
        kp, vp, seen_p = k[:0], v[:0], torch.zeros((T, 0), dtype=torch.bool)
    kk, vv = expand_kv(torch.cat([k, kp], 0), H), expand_kv(torch.cat([v, vp], 0), H)
    s = torch.einsum("thd,jhd->htj", q, kk) * float(m["scale"])
    s = s.masked_fill(~torch.cat([seen, seen_p], 1)[None], -math.inf)
    p = torch.softmax(s, -1)
    o = torch.einsum("htj,jhd->thd", p, vv).reshape(T, H * V)
    return o @ w[pre + "o"].T


def sink_gated_attention(h, w, pre, m, eps):
    """Causal attention whose values are the keys as projected, q and k normed over the whole projection, one added
    to the softmax's denominator, and a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q, k = h @ w[pre + "q"].T, h @ w[pre + "k"].T
    v = k.view(T, G, V)
    q = rotate((rms(q, eps) * w[pre + "q.norm"]).view(T, H, D), pos, m.get("rot"))
    k = rotate((rms(k, eps) * w[pre + "k.norm"]).view(T, G, D), pos, m.get("rot"))
    s = torch.einsum("thd,jhd->htj", q, expand_kv(k, H)) * float(m["scale"])
    s = s.masked_fill((pos[:, None] < pos[None, :])[None], -math.inf)
    e = torch.exp(s - s.max(-1, keepdim=True).values.clamp(min=0))
    p = e / (torch.exp(-s.max(-1, keepdim=True).values.clamp(min=0)) + e.sum(-1, keepdim=True))
    o = torch.einsum("htj,jhd->thd", p, expand_kv(v, H)).reshape(T, H * V)
    return (o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def retention(h, w, pre, m, eps):
    """S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, token by token; then a unit-RMS norm per head, a
    silu gate and the output projection."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = rotate((h @ w[pre + "q"].T).view(T, H, D), pos, m.get("rot"))
    k = rotate((h @ w[pre + "k"].T).view(T, H, D), pos, m.get("rot")) * D ** -0.5
    v = (h @ w[pre + "v"].T).view(T, H, V)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=F64)
    S = torch.zeros((H, D, V), dtype=F64)
    o = torch.zeros((T, H, V), dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    g = h @ w[pre + "g"].T
    return (rms(o, eps).reshape(T, H * V) * (g * torch.sigmoid(g))) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    return (float(m["left_scale"]) * sink_gated_attention(h, w, pre + "left.", m["left"], eps)
            + float(m["right_scale"]) * retention(h, w, pre + "right.", m["right"], eps))


def sigmoid_attention(h, w, pre, m, eps):
    """Causal attention without rotation and without a softmax: a query temperature that grows with the position,
    capped scores, a logarithmic distance penalty per head, and sigmoid weights that are not normalised."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, V)
    qt = m.get("q_temp")
    if qt:
        temp = 1 + float(qt["coef"]) * torch.log(torch.floor((pos.to(F64) + 1) / int(qt["every"])) + 1)
        q = q * temp[:, None, None]
    s = torch.einsum("thd,jhd->htj", q, expand_kv(k, H)) * float(m["scale"])
    cap = float(m.get("softcap") or 0)
    if cap:
        s = cap * torch.tanh(s / cap)
    dist = (pos[:, None] - pos[None, :]).clamp(min=0).to(F64)
    s = s - w[pre + "r1"][:, None, None] * torch.log(1 + w[pre + "r2"][:, None, None] * dist[None])
    p = torch.sigmoid(s + w[pre + "pb"][:, None, None]) * (pos[:, None] >= pos[None, :])[None]
    o = torch.einsum("htj,jhd->thd", p, expand_kv(v, H)).reshape(T, H * V)
    return o @ w[pre + "o"].T + w[pre + "o.b"]


MIXERS = {"attention": pooled_window_attention, "parallel": parallel_mixer, "attention_2": sigmoid_attention}


# ------------------------------------------------------------------------------------------------ feed-forward
def route(h, w, pre, f):
    """(chosen experts [T, top], their weights [T, top]) by the grouped sigmoid rule."""
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    s = torch.sigmoid(h @ w[pre + "router"].T)
    choice = s + w[pre + "correction"] if pre + "correction" in w else s.clone()
    per = E // count
    grouped = choice.view(-1, count, per)
    gscore = grouped.topk(min(2, per), -1).values.sum(-1)
    kept = torch.zeros_like(gscore, dtype=torch.bool)
    order = torch.sort(gscore, dim=-1, descending=True, stable=True).indices[:, :keep]
    kept.scatter_(1, order, True)
    allowed = kept[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = choice.masked_fill(~allowed, -math.inf)
    ids = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :top]
    chosen = s.gather(1, ids)
    return ids, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))


def expert(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def moe(h, w, pre, f, forced=None):
    """``forced``: experts [T, top] to use instead of the rule's own choice (their weights still follow the rule's
    formula over the forced set)."""
    ids, weights = route(h, w, pre, f)
    if forced is not None:
        ids = forced.to(torch.long)
        s = torch.sigmoid(h @ w[pre + "router"].T).gather(1, ids)
        weights = s / (s.sum(-1, keepdim=True) + 1e-20) * float(f["router"].get("scale", 1.0))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), weights[t]):
            out[t] += g * expert(h[t:t + 1], w[f"{pre}e{e}.up"], w[f"{pre}e{e}.down"])[0]
    if f.get("shared"):
        out = out + expert(h, w[pre + "shared.up"], w[pre + "shared.down"])
    return out, ids


# ------------------------------------------------------------------------------------------------ the model
def run_order(cfg):
    """[(layer, pass number or None if the layer's run does not open a pass)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    out = [(i, None) for i in range(start)]
    for t in range(times):
        out += [(i, t if i == start else None) for i in range(start, stop)]
    return out + [(i, None) for i in range(stop, n)]


def forward(cfg, w, tokens, forced=None):
    """logits [T, vocab], the rows after every layer run [runs, T, width], the experts chosen in every run."""
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    after, chosen = [], []
    for n, (i, opens) in enumerate(run_order(cfg)):
        layer, pre = cfg["layers"][i], f"l{i}."
        if opens is not None:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T + w["loop.step"][opens]
        y = MIXERS[layer["type"]](norm(x, w[pre + "norm1"], eps), w, pre + "mix.", layer["mixer"], eps)
        x = x + norm(y, w[pre + "norm1b"], eps)
        if layer.get("mlp"):
            y, ids = moe(norm(x, w[pre + "norm2"], eps), w, pre + "mlp.", layer["mlp"],
                         forced[n] if forced is not None else None)
            chosen.append(ids)
            x = x + norm(y, w[pre + "norm2b"], eps)
        else:
            chosen.append(None)
        after.append(x.clone())
    logits = norm(x, w["final.norm"], eps) @ w["embed"].T
    return logits, torch.stack(after), chosen
