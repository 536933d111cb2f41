"""Typed configuration of Dumizen, read from the keys of its own config.json.

The file is nested: ``vocab``, ``width``, ``norm`` (eps), ``layers`` (a list with one entry per layer: the mixer's
``type`` (``attention``, ``parallel`` or ``attention_2``), the mixer's sizes and constants (``mixer``) and the
feed-forward (``mlp``, or null for none)) and ``loop`` (``start``, ``stop``, ``times``: layers start .. stop - 1 run
that many times in a row; absent: every layer runs once).  Nothing is assumed about the number or the order of the
layers, and every size and constant comes from the file.  The design gives no limit on positions;
``DEFAULT_MAX_POSITIONS`` bounds what an engine may be built for.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from . import fields as F
from .puledra import _section

DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class Rotation:
    dims: int               # leading dims of every head that rotate
    base: float
    yarn: tuple | None      # (factor, original, fast, slow) or None


@dataclass(frozen=True)
class Heads:
    heads: int
    kv_heads: int
    dim: int                # query/key dims per head
    vdim: int               # value dims per head
    scale: float
    rot: Rotation | None


@dataclass(frozen=True)
class PooledWindowAttention:
    """Softmax attention over a sliding window and, behind it, the means of whole blocks of positions."""
    h: Heads
    window: int             # 0: every earlier key is seen, no blocks
    pool: int               # positions a block


@dataclass(frozen=True)
class GatedSinkAttention:
    """The left half of a parallel mixer: causal attention whose values are its keys, with a unit sink and a gate."""
    h: Heads


@dataclass(frozen=True)
class Retention:
    """The right half of a parallel mixer."""
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Rotation | None


@dataclass(frozen=True)
class ParallelMixer:
    left: GatedSinkAttention
    right: Retention
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class SigmoidAttention:
    """Causal attention with sigmoid weights, a capped score, a distance penalty and a query temperature."""
    h: Heads
    softcap: float          # 0: none
    q_temp: tuple | None    # (coef, every) or None


@dataclass(frozen=True)
class ExpertMlp:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    scale: float
    shared_ff: int          # 0: no shared expert


@dataclass(frozen=True)
class DumizenLayer:
    type: str
    mixer: object
    mlp: ExpertMlp | None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _rotation(m, dim, where):
    rot = _section(m, "rot", optional=True)
    if rot is None:
        return None
    dims = F.get_int(rot, "dims", minimum=0)
    if dims == 0:
        return None
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}.rot.dims must be even and at most dim {dim}, got {dims}")
    sc = _section(rot, "scaling", optional=True)
    yarn = None
    if sc is not None:
        yarn = (F.get_float(sc, "factor"), F.get_float(sc, "original"), F.get_float(sc, "fast"), F.get_float(sc, "slow"))
        if min(yarn) <= 0:
            raise ConfigError(f"{where}.rot.scaling: factor, original, fast and slow must be positive")
    return Rotation(dims, F.get_float(rot, "base"), yarn)


def _heads(m, where, values_are_keys=False):
    heads, kv = F.get_int(m, "heads", minimum=1), F.get_int(m, "kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{where}.heads {heads} is not a multiple of kv_heads {kv}")
    dim = F.get_int(m, "dim", minimum=1)
    vdim = F.get_int(m, "vdim", dim if values_are_keys else F._MISSING, minimum=1)
    if values_are_keys and vdim != dim:
        raise ConfigError(f"{where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    return Heads(heads, kv, dim, vdim, F.get_float(m, "scale", dim ** -0.5), _rotation(m, dim, where))


def _mixer(kind, m, where):
    if kind == "attention":
        mask = _section(m, "mask", optional=True)
        window = F.get_int(mask, "size", minimum=1) if mask is not None else 0
        pool = F.get_int(mask, "pool", 0, minimum=0) if mask is not None else 0       # 0: a plain window
        return PooledWindowAttention(_heads(m, where), window, pool)
    if kind == "attention_2":
        qt = _section(m, "q_temp", optional=True)
        q_temp = (F.get_float(qt, "coef"), F.get_int(qt, "every", minimum=1)) if qt is not None else None
        cap = F.get_float(m, "softcap", 0.0)
        if cap < 0:
            raise ConfigError(f"{where}.softcap must not be negative, got {cap}")
        return SigmoidAttention(_heads(m, where), cap, q_temp)
    if kind == "parallel":
        left, right = _section(m, "left"), _section(m, "right")
        heads, dim = F.get_int(right, "heads", minimum=1), F.get_int(right, "dim", minimum=1)
        r = Retention(heads, dim, F.get_int(right, "vdim", minimum=1), F.get_float_list(right, "decay", length=heads),
                      _rotation(right, dim, where + ".right"))
        return ParallelMixer(GatedSinkAttention(_heads(left, where + ".left", values_are_keys=True)), r,
                             F.get_float(m, "left_scale"), F.get_float(m, "right_scale"))
    raise ConfigError(f"{where}: unknown layer type {kind!r} (known: attention, parallel, attention_2)")


def _mlp(f, where):
    kind = F.get_str(f, "kind", "moe")
    if kind != "moe":
        raise ConfigError(f"{where}: unknown kind {kind!r} (known: moe)")
    r = _section(f, "router")
    g = _section(r, "groups", optional=True)
    shared = _section(f, "shared", optional=True)
    out = ExpertMlp(ff=F.get_int(_section(f, "expert"), "ff", minimum=1), experts=F.get_int(r, "experts", minimum=1),
                    top=F.get_int(r, "top", minimum=1), groups=F.get_int(g, "count", minimum=1) if g else 1,
                    keep=F.get_int(g, "keep", minimum=1) if g else 1, scale=F.get_float(r, "scale", 1.0),
                    shared_ff=F.get_int(shared, "ff", minimum=1) if shared else 0)
    if out.top > out.experts:
        raise ConfigError(f"{where}.router.top {out.top} exceeds the {out.experts} experts")
    if out.experts % out.groups or out.keep > out.groups or out.keep * (out.experts // out.groups) < out.top:
        raise ConfigError(f"{where}.router.groups: {out.keep} of {out.groups} groups of {out.experts} experts cannot give "
                          f"{out.top} a token")
    return out


@dataclass(frozen=True)
class DumizenConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop: Loop | None
    architecture: str = "Dumizen"

    @classmethod
    def from_dict(cls, d: dict) -> "DumizenConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}] must be an object")
            kind = F.get_str(entry, "type")
            f = _section(entry, "mlp", optional=True)
            out.append(DumizenLayer(kind, _mixer(kind, _section(entry, "mixer"), f"layers[{i}].mixer"),
                                    _mlp(f, f"layers[{i}].mlp") if f is not None else None))
        lp = _section(d, "loop", optional=True)
        loop = None
        if lp is not None:
            loop = Loop(F.get_int(lp, "start", minimum=0), F.get_int(lp, "stop", minimum=0), F.get_int(lp, "times", minimum=1))
            if not loop.start < loop.stop <= len(out):
                raise ConfigError(f"loop: layers {loop.start} .. {loop.stop - 1} are not a run of the {len(out)} layers")
        return cls(vocab=F.get_int(d, "vocab", minimum=1), width=F.get_int(d, "width", minimum=1),
                   eps=F.get_float(_section(d, "norm"), "eps"), layers=tuple(out), loop=loop)
