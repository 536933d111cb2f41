"""Tiny Dumizen configurations that differ in every size, constant and in the order of layers, and a writer of model
folders whose random weights are large enough that every mechanism shows in the logits (attention is peaked, the
unit sink takes a real share, retention keeps memory over many tokens, router scores and corrections are spread so
that groups matter, the distance penalty and the cap of the sigmoid attention bite)."""
from __future__ import annotations

import math
import random

import torch

from tiny_puledra import write_model as _write_folder


def _rot(dims, base=10000.0, yarn=None):
    r = {"dims": dims, "base": base}
    if yarn:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    return r


def _pooled(heads, kv, dim, vdim, size=None, pool=None, rot=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if size:
        m["mask"] = {"size": size, "pool": pool}
    if rot:
        m["rot"] = rot
    return m


def _sigmoid(heads, kv, dim, vdim, cap=0.0, temp=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if cap:
        m["softcap"] = cap
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def _parallel(left, right, ls, rs):
    heads, kv, dim, lrot, lscale = left
    rheads, rdim, rvdim, decay, rrot = right
    lm = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": lscale}
    if lrot:
        lm["rot"] = lrot
    rm = {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": list(decay)}
    if rrot:
        rm["rot"] = rrot
    return {"left": lm, "right": rm, "left_scale": ls, "right_scale": rs}


def _moe(ff, experts, top, count=1, keep=1, scale=1.0, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale,
                                                         "groups": {"count": count, "keep": keep}}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


# D1: sizes that are no multiples of 8 (rows read element by element, products on the float32 pipes), three query
# heads a key head, values wider and narrower than keys, a window shorter than a page with blocks of 3 and of 5
# positions, a window longer than a page with blocks longer than a page, blocks of 1, a layer that sees everything, a
# partly and a fully rotated head with and without YaRN, the parallel mixer first in the loop, a layer without a
# feed-forward, one to three experts a token from one, two and three groups, a mixture without a shared expert, a
# loop of three passes that starts at layer 0 and ends at the last layer.
D1 = {
    "architecture": "Dumizen", "vocab": 83, "width": 40, "norm": {"eps": 1e-5},
    "loop": {"start": 0, "stop": 5, "times": 3},
    "layers": [
        {"type": "parallel", "mixer": _parallel((6, 2, 12, _rot(12, 5000.0, (3.0, 16, 8.0, 2.0)), 0.35),
                                                (3, 10, 6, (0.9, 0.97, 0.995), _rot(6, 300.0)), 0.8, 1.5),
         "mlp": _moe(12, 6, 2, count=3, keep=2, scale=1.7, shared=20)},
        {"type": "attention", "mixer": _pooled(6, 2, 10, 14, size=7, pool=3, rot=_rot(4, 100.0)), "mlp": None},
        {"type": "attention_2", "mixer": _sigmoid(3, 1, 9, 5, cap=4.0, temp=(0.7, 5)), "mlp": _moe(8, 4, 3, shared=None)},
        {"type": "attention", "mixer": _pooled(2, 2, 6, 4, size=21, pool=19, rot=_rot(6, 20.0, (2.0, 24, 4.0, 1.0)), scale=0.5),
         "mlp": _moe(16, 6, 1, count=2, keep=1, scale=0.6, shared=8)},
        {"type": "attention", "mixer": _pooled(4, 1, 8, 8, size=5, pool=1), "mlp": _moe(8, 3, 1, count=3, keep=2)},
    ],
}

# D2: sizes in multiples of 16 (every product on the tensor cores in bfloat16), no loop entry that starts at 0: a layer
# before and one after the loop, the sigmoid attention without a cap and without a temperature, one query head a key
# head, a window of exactly one page, blocks that divide a page and blocks that do not, the parallel mixer last in the
# loop, a pooled layer without a mask.
D2 = {
    "architecture": "Dumizen", "vocab": 160, "width": 64, "norm": {"eps": 1e-6},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "attention", "mixer": _pooled(4, 2, 32, 16, size=16, pool=4, rot=_rot(16, 10000.0, (4.0, 32, 16.0, 1.0))),
         "mlp": _moe(32, 8, 2, count=4, keep=2, scale=2.5, shared=48)},
        {"type": "attention_2", "mixer": _sigmoid(4, 4, 16, 16), "mlp": _moe(16, 4, 2, count=2, keep=1, scale=1.0, shared=16)},
        {"type": "parallel", "mixer": _parallel((4, 2, 32, _rot(32, 500000.0, (2.0, 64, 32.0, 1.0)), 0.18),
                                                (2, 32, 16, (0.95, 0.999), _rot(32, 1000000.0)), 1.2, 0.5),
         "mlp": _moe(32, 8, 3, count=2, keep=1, scale=2.0, shared=32)},
        {"type": "attention", "mixer": _pooled(8, 2, 16, 32, size=24, pool=7, rot=_rot(8)), "mlp": None},
        {"type": "attention", "mixer": _pooled(2, 1, 16, 16), "mlp": _moe(16, 4, 1, shared=16)},
    ],
}

# D3: no loop at all, and one layer of each kind
D3 = {
    "architecture": "Dumizen", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention_2", "mixer": _sigmoid(2, 1, 16, 16, cap=10.0, temp=(0.5, 8)), "mlp": _moe(16, 4, 2, count=2, keep=1, scale=2.0)},
        {"type": "parallel", "mixer": _parallel((2, 1, 16, _rot(8), 0.25), (2, 16, 16, (0.9, 0.99), None), 1.0, 1.0), "mlp": None},
        {"type": "attention", "mixer": _pooled(2, 1, 16, 16, size=10, pool=4, rot=_rot(16)), "mlp": _moe(16, 2, 1, shared=16)},
    ],
}

CONFIGS = {"D1": D1, "D2": D2, "D3": D3}


def run_count(cfg):
    loop = cfg.get("loop")
    return len(cfg["layers"]) + ((loop["times"] - 1) * (loop["stop"] - loop["start"]) if loop else 0)


def tensor_shapes(cfg):
    """Every tensor of a checkpoint by name, written down here independently of the package."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W)}
    if cfg.get("loop"):
        out.update({"loop.in": (W, 2 * W), "loop.step": (cfg["loop"]["times"], W)})
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out.update({p + "norm1": (W,), p + "norm1b": (W,)})
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                        p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                        p + "mix.o": (W, H * dv)})
        elif layer["type"] == "attention_2":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                        p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.r1": (H,), p + "mix.r2": (H,),
                        p + "mix.pb": (H,), p + "mix.o": (W, H * dv), p + "mix.o.b": (W,)})
        else:
            l, r = m["left"], m["right"]
            H, G, d = l["heads"], l["kv_heads"], l["dim"]
            out.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.q.norm": (H * d,),
                        p + "mix.left.k.norm": (G * d,), p + "mix.left.g": (H * d, W), p + "mix.left.o": (W, H * d)})
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            out.update({p + "mix.right.q": (H * d, W), p + "mix.right.k": (H * d, W), p + "mix.right.v": (H * dv, W),
                        p + "mix.right.g": (H * dv, W), p + "mix.right.o": (W, H * dv)})
        f = layer.get("mlp")
        if f:
            out.update({p + "norm2": (W,), p + "norm2b": (W,)})
            E = f["router"]["experts"]
            out.update({p + "mlp.router": (E, W), p + "mlp.correction": (E,)})
            for e in range(E):
                out[p + f"mlp.e{e}.up"] = (f["expert"]["ff"], W)
                out[p + f"mlp.e{e}.down"] = (W, f["expert"]["ff"])
            if f.get("shared"):
                out.update({p + "mlp.shared.up": (f["shared"]["ff"], W), p + "mlp.shared.down": (W, f["shared"]["ff"])})
    out["final.norm"] = (W,)
    return out


def random_weights(cfg, seed=0):
    """bfloat16 tensors: matrices N(0, g^2 / fan_in) with g = 2.5 for queries, keys, routers and gates, norm scales
    1 + N(0, 0.1), corrections N(0, 0.3) (so that choice scores go negative and groups change the choice), distance
    penalties r1 in (0.2, 1) and r2 in (0.05, 0.5), weight biases N(-1, 0.5), other vectors N(0, 0.5)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith((".norm1", ".norm2", ".norm1b", ".norm2b", "final.norm", ".q.norm", ".k.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(".correction"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith(".r1"):
            t = 0.2 + 0.8 * torch.rand(shape, generator=g)
        elif name.endswith(".r2"):
            t = 0.05 + 0.45 * torch.rand(shape, generator=g)
        elif name.endswith(".pb"):
            t = -1.0 + 0.5 * torch.randn(shape, generator=g)
        elif name == "loop.step" or len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name == "loop.in":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1] / 2)
        else:
            gain = 2.5 if name.endswith((".q", ".k", ".router", ".g", ".up")) else 1.0
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[1])
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(folder, cfg, seed=0, weights=None):
    return _write_folder(folder, cfg, seed, weights if weights is not None else random_weights(cfg, seed))


def random_config(seed):
    """A configuration drawn at random: one to five layers in any order, odd head sizes, windows and blocks of 1 to 40
    positions, with and without a loop."""
    r = random.Random(seed)
    W = r.choice([24, 32, 40, 48])
    layers = []
    for _ in range(r.randint(1, 5)):
        kind = r.choice(["attention", "attention_2", "parallel"])
        kv = r.choice([1, 2])
        heads = kv * r.choice([1, 2, 3])
        dim = r.choice([6, 8, 10, 16, 24])
        if kind == "attention":
            rot = _rot(r.choice([2, 4, dim]), r.choice([50.0, 10000.0]), r.choice([None, (2.0, 16, 8.0, 1.0)]))
            size = r.choice([None, 1, 2, 5, 16, 17, 40])
            m = _pooled(heads, kv, dim, r.choice([4, 7, 16]), size=size, pool=r.choice([1, 2, 3, 16, 40]), rot=r.choice([None, rot]))
        elif kind == "attention_2":
            m = _sigmoid(heads, kv, dim, r.choice([4, 7, 16]), cap=r.choice([0.0, 3.0, 20.0]), temp=r.choice([None, (0.5, 3), (1.0, 64)]))
        else:
            rh = r.choice([1, 2, 3])
            m = _parallel((heads, kv, dim, r.choice([None, _rot(dim, 1000.0, (4.0, 8, 4.0, 1.0))]), dim ** -0.5),
                          (rh, r.choice([4, 10, 16]), r.choice([4, 6, 16]), [r.uniform(0.8, 0.999) for _ in range(rh)],
                           r.choice([None, _rot(4, 100.0)])), r.uniform(0.5, 1.5), r.uniform(0.5, 1.5))
        count = r.choice([1, 2, 3])
        per = r.choice([1, 2, 3])
        keep = r.randint(1, count)
        f = r.choice([None, _moe(r.choice([8, 12]), count * per, r.randint(1, keep * per), count=count, keep=keep,
                                 scale=r.choice([1.0, 2.5]), shared=r.choice([None, 8]))])
        layers.append({"type": kind, "mixer": m, "mlp": f})
    cfg = {"architecture": "Dumizen", "vocab": r.choice([50, 97]), "width": W, "norm": {"eps": r.choice([1e-5, 1e-6])},
           "layers": layers}
    if r.random() < 0.7:
        start = r.randrange(len(layers))
        cfg["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": r.randint(1, 3)}
    return cfg
