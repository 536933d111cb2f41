"""Typed configuration of Tefovik, read from the keys of its own config.json.

The file is nested: ``vocab``, ``width``, ``norm`` (eps), ``postln_alpha``, ``logit_softcap`` and ``layers``, a list with
one entry per layer that gives the layer's ``type`` (``parallel``: an attention branch beside a delta-rule branch;
``mamba2``: a state-space mixer), the mixer's sizes and constants (``mixer``) and the feed-forward (``mlp``: ``kind``
``dense``, or null for none).  Nothing is assumed about the number or the order of the layers, and every size and
constant comes from the file.  The design gives no limit on positions; ``DEFAULT_MAX_POSITIONS`` bounds what an
engine may be built for.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from . import fields as F
from .puledra import _section

DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class ChunkAttention:
    heads: int
    kv_heads: int
    dim: int                # query/key dims per head
    vdim: int               # value dims per head
    scale: float
    taps: int               # length of the short convolution after the q, k and v projections
    chunk: int              # a position sees the earlier positions of its own run of so many (0: all earlier ones)
    rot_dims: int           # leading dims of every q and k head that rotate
    rot_base: float


@dataclass(frozen=True)
class DeltaRule:
    heads: int              # value heads
    kv_heads: int           # query/key heads
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class StateSpace:
    heads: int
    vdim: int
    state: int              # N, the state's size per head and value dim
    groups: int             # heads that share B and C
    norm_groups: int
    taps: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class TefovikLayer:
    type: str
    mixer: object           # (ChunkAttention, DeltaRule) for ``parallel``, StateSpace for ``mamba2``
    mlp: object


def _heads(m, where):
    heads, kv = F.get_int(m, "heads", minimum=1), F.get_int(m, "kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{where}.heads {heads} is not a multiple of kv_heads {kv}")
    return heads, kv


def _left(m, where):
    heads, kv = _heads(m, where)
    dim, vdim = F.get_int(m, "dim", minimum=1), F.get_int(m, "vdim", minimum=1)
    rot = _section(m, "rot")
    rot_dims = F.get_int(rot, "dims", minimum=0)
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{where}.rot.dims must be even and at most dim {dim}, got {rot_dims}")
    if vdim % 2:
        raise ConfigError(f"{where}.vdim must be even (values rotate in pairs), got {vdim}")
    mask = _section(m, "mask", optional=True)
    return ChunkAttention(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=F.get_float(m, "scale"),
                          taps=F.get_int(m, "conv", minimum=1),
                          chunk=F.get_int(mask, "size", 0, minimum=0) if mask is not None else 0,
                          rot_dims=rot_dims, rot_base=F.get_float(rot, "base"))


def _right(m, where):
    heads, kv = _heads(m, where)
    return DeltaRule(heads=heads, kv_heads=kv, dim=F.get_int(m, "dim", minimum=1), vdim=F.get_int(m, "vdim", minimum=1),
                     taps=F.get_int(m, "conv", minimum=1))


def _state_space(m, where):
    heads, groups = F.get_int(m, "heads", minimum=1), F.get_int(m, "groups", minimum=1)
    if heads % groups:
        raise ConfigError(f"{where}.heads {heads} is not a multiple of groups {groups}")
    vdim, ng = F.get_int(m, "vdim", minimum=1), F.get_int(m, "norm_groups", minimum=1)
    if (heads * vdim) % ng:
        raise ConfigError(f"{where}.norm_groups {ng} does not divide heads x vdim = {heads * vdim}")
    return StateSpace(heads=heads, vdim=vdim, state=F.get_int(m, "state", minimum=1), groups=groups, norm_groups=ng,
                      taps=F.get_int(m, "conv", minimum=1))


def _mlp(f, where):
    kind = F.get_str(f, "kind")
    if kind != "dense":
        raise ConfigError(f"{where}: unknown kind {kind!r} (known: dense)")
    return DenseMlp(ff=F.get_int(f, "ff", minimum=1))


@dataclass(frozen=True)
class TefovikConfig:
    vocab: int
    width: int
    eps: float
    alpha: float            # the residual's weight in the sum that each norm of a layer reads
    softcap: float          # logits <- softcap tanh(logits / softcap)
    layers: tuple
    architecture: str = "Tefovik"

    @classmethod
    def from_dict(cls, d: dict) -> "TefovikConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}] must be an object")
            kind = F.get_str(entry, "type")
            m = _section(entry, "mixer")
            if kind == "parallel":
                mixer = (_left(_section(m, "left"), f"layers[{i}].mixer.left"),
                         _right(_section(m, "right"), f"layers[{i}].mixer.right"))
            elif kind == "mamba2":
                mixer = _state_space(m, f"layers[{i}].mixer")
            else:
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (known: parallel, mamba2)")
            f = _section(entry, "mlp", optional=True)
            out.append(TefovikLayer(kind, mixer, _mlp(f, f"layers[{i}].mlp") if f is not None else None))
        softcap = F.get_float(d, "logit_softcap")
        if softcap <= 0:
            raise ConfigError(f"config field 'logit_softcap' must be positive, got {softcap}")
        return cls(vocab=F.get_int(d, "vocab", minimum=1), width=F.get_int(d, "width", minimum=1),
                   eps=F.get_float(_section(d, "norm"), "eps"), alpha=F.get_float(d, "postln_alpha"),
                   softcap=softcap, layers=tuple(out))
