"""Tiny Tefovik configurations that differ in every size, constant and in the order of layers, and a writer of model
folders whose random weights are large enough that every mechanism shows in the logits (attention is peaked, the
recurrent states keep memory over many tokens, the layer scales and depth weights are far from 0 and 1, the cap on
the logits bites)."""
from __future__ import annotations

import math

import torch

from tiny_puledra import write_model as _write_folder


def _left(heads, kv, dim, vdim, scale, taps, chunk, rot, base=10000.0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "conv": taps,
         "rot": {"dims": rot, "base": base}}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def _right(heads, kv, dim, vdim, taps):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}


def _par(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _ssm(heads, vdim, state, groups, norm_groups, taps, ff):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": taps},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


# T1: sizes that are no multiples of 8 (rows read element by element, products on the float32 pipes); a state-space
# layer first, and one with a feed-forward; three query heads to a key head; values wider and narrower than keys;
# runs shorter than a page of 16 and runs that cross a page's border; heads rotated partly, fully and not at all;
# a layer that sees every earlier position; convolutions of 1, 2, 3, 4 and 5 taps; a delta rule whose heads share
# keys two by two and one with 40 key dims (two lanes a column); state-space heads in groups; a norm in three parts.
T1 = {
    "architecture": "Tefovik", "vocab": 83, "width": 40, "norm": {"eps": 1e-5}, "postln_alpha": 2.0, "logit_softcap": 8.0,
    "layers": [
        _ssm(3, 10, 7, 1, 3, 3, ff=24),
        _par(_left(6, 2, 12, 10, 0.4, 2, 9, 8, base=100.0), _right(4, 2, 20, 6, 5), ff=None),
        _par(_left(2, 2, 8, 18, 0.5, 4, 24, 8), _right(3, 3, 40, 12, 3), ff=56),
        _ssm(4, 6, 40, 2, 1, 4, ff=None),
        _par(_left(3, 1, 10, 4, 0.35, 1, None, 0), _right(2, 1, 6, 14, 2), ff=16),
    ],
}

# T2: sizes in multiples of 16 (every product on the tensor cores in bfloat16, attention in tiles); two parallel
# layers side by side and two state-space layers side by side; a run as long as a page of 16 and one of 40; one
# and two query heads a key head; 64 key dims (two lanes a column) and a state of 144 (eight lanes a column).
T2 = {
    "architecture": "Tefovik", "vocab": 160, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 3.5, "logit_softcap": 20.0,
    "layers": [
        _par(_left(8, 4, 32, 16, 0.2, 4, 40, 16, base=500000.0), _right(4, 2, 64, 32, 4), ff=96),
        _par(_left(4, 4, 16, 32, 0.3, 3, 16, 16), _right(2, 1, 32, 48, 2), ff=64),
        _ssm(8, 16, 32, 2, 4, 4, ff=128),
        _ssm(2, 64, 144, 1, 2, 2, ff=None),
    ],
}

CONFIGS = {"T1": T1, "T2": T2}
RANKS = {"T1": (3, 5), "T2": (8, 4)}          # of the delta rule's two low-rank pairs (decay, gate)


def tensor_shapes(cfg, ranks=(3, 5)):
    """Every tensor of a checkpoint by name, written down here independently of the package."""
    W = cfg["width"]
    ra, rg = ranks
    out = {"embed": (cfg["vocab"], W), "embed.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out.update({p + "norm1": (W,), p + "ls1": (W,), p + "dwa": (i + 2,)})
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d, dv, t = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
            q = p + "mix.left."
            out.update({q + "q": (H * d, W), q + "k": (G * d, W), q + "v": (G * dv, W), q + "q.norm": (d,), q + "k.norm": (d,),
                        q + "q.conv": (H * d, t), q + "k.conv": (G * d, t), q + "v.conv": (G * dv, t), q + "g": (H, W),
                        q + "o": (W, H * dv), q + "out": (W,)})
            H, G, d, dv, t = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            q = p + "mix.right."
            out.update({q + "q": (G * d, W), q + "q.conv": (G * d, t), q + "k": (G * d, W), q + "k.conv": (G * d, t),
                        q + "v": (H * dv, W), q + "v.conv": (H * dv, t), q + "b": (H, W), q + "A_log": (H,), q + "norm": (dv,),
                        q + "a1": (ra, W), q + "a2": (H * d, ra), q + "dt_bias": (H * d,), q + "g1": (rg, W),
                        q + "g2": (H * dv, rg), q + "o": (W, H * dv), q + "out": (W,)})
        else:
            H, dv, N, G, t = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * dv, H * dv + 2 * G * N
            q = p + "mix."
            out.update({q + "in": (2 * inner + 2 * G * N + H, W), q + "conv": (ch, t), q + "conv.b": (ch,), q + "dt_bias": (H,),
                        q + "A_log": (H,), q + "D": (H,), q + "norm": (inner,), q + "o": (W, inner)})
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "ls2": (W,), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    out.update({"final.norm": (W,), "head": (cfg["vocab"], W)})
    return out


def random_weights(cfg, seed=0, ranks=(3, 5)):
    """bfloat16 tensors.  Matrices N(0, g^2 / fan_in), g = 2 for what feeds gates and decays; q and k norm scales
    near 1.5 (peaked attention); convolutions N(0, 0.5^2); decay rates exp(A_log) in (0.05, 1) with step biases
    N(-1, 1) (memory over tens of tokens); layer scales 1 + N(0, 0.3^2); depth weights N(0, 0.3^2) with one more on
    the newest rows; the head N(0, 6^2 / W) so that the cap bites."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        rnd = lambda s=1.0: s * torch.randn(shape, generator=g)
        if name.endswith(".dwa"):
            t = rnd(0.3)
            t[-1] += 1.0
        elif name.endswith((".ls1", ".ls2")):
            t = 1.0 + rnd(0.3)
        elif name.endswith((".q.norm", ".k.norm")):
            t = 1.5 + rnd(0.2)
        elif name.endswith(".conv"):
            t = rnd(0.5)
        elif name.endswith(".A_log"):
            t = -3.0 + 3.0 * torch.rand(shape, generator=g)
        elif name.endswith(".dt_bias"):
            t = -1.0 + rnd()
        elif name.endswith((".conv.b", ".D")):
            t = rnd()
        elif len(shape) == 1:
            t = 1.0 + rnd(0.1 if "norm" in name else 0.2)
        elif name == "embed":
            t = rnd()
        elif name == "head":
            t = rnd(6.0 / math.sqrt(shape[1]))
        else:
            gain = 2.0 if name.endswith((".b", ".g", ".a2", ".g2", ".up", ".in")) else 1.0
            t = rnd(gain / math.sqrt(shape[1]))
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(folder, cfg, seed=0, weights=None, ranks=(3, 5)):
    return _write_folder(folder, cfg, seed, weights if weights is not None else random_weights(cfg, seed, ranks))


def random_config(seed):
    """A configuration drawn at random: one to five layers in any order, with or without a feed-forward, head counts,
    head sizes (also odd ones, 130 and 256 key dims, states of 7 to 256), rotated dims, runs of 1 to 1,000 positions or
    none, one to five taps, norm parts and constants.  Returns (config, ranks of the delta rule's low-rank pairs)."""
    import random
    r = random.Random(1000 + seed)
    layers = []
    for _ in range(r.randint(1, 5)):
        ff = r.choice([None, 16, 56, 96, 128])
        if r.random() < 0.55:
            kv = r.choice([1, 2, 3, 4])
            d = r.choice([8, 10, 16, 32, 64, 48])
            left = _left(kv * r.choice([1, 2, 3]), kv, d, r.choice([4, 10, 16, 32, 64, 18]), r.choice([0.1, 0.3, d ** -0.5]),
                         r.randint(1, 5), r.choice([None, 1, 3, 16, 17, 64, 100, 200, 1000]), r.choice([0, d, d // 4 * 2, 2]),
                         base=r.choice([100.0, 1e4, 5e5]))
            g = r.choice([1, 2, 3])
            right = _right(g * r.choice([1, 2]), g, r.choice([6, 20, 32, 40, 64, 128, 130, 256]),
                           r.choice([6, 12, 32, 33, 48, 64]), r.randint(1, 5))
            layers.append(_par(left, right, ff))
        else:
            G = r.choice([1, 2, 4])
            H, V = G * r.choice([1, 2, 3]), r.choice([6, 10, 16, 32, 64])
            parts = r.choice([n for n in (1, 2, 3, 4, H) if (H * V) % n == 0])
            layers.append(_ssm(H, V, r.choice([7, 16, 32, 40, 48, 128, 144, 256]), G, parts, r.randint(1, 5), ff))
    cfg = {"architecture": "Tefovik", "vocab": r.choice([83, 160, 301]), "width": r.choice([24, 40, 64, 72, 96, 128]),
           "norm": {"eps": r.choice([1e-5, 1e-6])}, "postln_alpha": r.choice([1.0, 2.0, 3.5]),
           "logit_softcap": r.choice([8.0, 15.0, 30.0]), "layers": layers}
    return cfg, (r.choice([1, 3, 8]), r.choice([2, 5, 16]))
