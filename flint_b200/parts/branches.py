"""A mixer made of several mixers side by side: all read the same rows, and the result is the mean of their
outputs, each first divided by its root mean square over the width and scaled by a weight of its own,

    out = (1 / n) sum_b  w_b * y_b / sqrt(mean(y_b^2) + eps)

or, with ``combine: "weighted"``, the plain weighted sum  out = sum_b scale_b y_b  with one constant a branch
(``scales``) and no stored weights.

Each branch is any registered mixer, built from its own ``PartSpec``; its tensors live under ``<name>.`` and its
weight w_b is ``<name>.out``.  A branch may own a paged cache (at most one branch of a mixer may) and fixed-size
state; the branches' states lie side by side in one row of the cache manager's slab.  The reference has no mixer of
several branches; its hybrid family alternates mixers layer by layer
(crates/thuban_architectures/src/qwen35/state.rs:5-55).
"""
from __future__ import annotations

import torch

from ..cache.manager import StateSpec
from ..errors import ConfigError, ModelError
from ..registry import MIXERS
from .base import Mixer, Pending, vec
from .block import branch_of


@MIXERS.register("branches")
class Branches(Mixer):
    """params: hidden_size, eps, branches: ((name, PartSpec), ...), combine ("rms_mean", the default, or "weighted"
    with ``scales``, one number a branch).  tensors: every branch's own under ``<name>.``, and for the mean
    ``<name>.out`` [hidden]."""

    returns_pending = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.eps = int(params["hidden_size"]), float(params.get("eps", 0.0))
        self.combine = params.get("combine", "rms_mean")
        if self.combine not in ("rms_mean", "weighted"):
            raise ConfigError(f"branches: combine must be 'rms_mean' or 'weighted', got {self.combine!r}")
        self.scales = tuple(float(x) for x in params.get("scales", ()))
        if self.combine == "weighted" and len(self.scales) != len(params["branches"]):
            raise ConfigError("branches: a weighted sum needs one scale a branch")
        self.branches = [(name, MIXERS.get(ps.kind)(ps.params, ctx)) for name, ps in params["branches"]]
        if not 1 <= len(self.branches) <= 4:
            raise ConfigError(f"branches: {len(self.branches)} branches are not supported (1 to 4)")
        if sum(m.cache_spec() is not None for _, m in self.branches) > 1:
            raise ConfigError("branches: at most one branch may own a paged cache")
        self.graph_safe = all(m.graph_safe for _, m in self.branches)
        self.out_w = []

    def weights(self):
        w = {}
        for name, m in self.branches:
            for k, ws in m.weights().items():
                w[f"{name}.{k}"] = ws
            if self.combine == "rms_mean":
                w[f"{name}.out"] = vec(self.hidden, init="gamma")
        return w

    def fused(self):
        return {f"{name}.{k}": [f"{name}.{p}" for p in pieces] for name, m in self.branches for k, pieces in m.fused().items()}

    def load(self, t):
        self.out_w = []
        for name, m in self.branches:
            m.load({k: t[f"{name}.{k}"] for k in m.weights() if f"{name}.{k}" in t})
            if self.combine == "rms_mean":
                self.out_w.append(t[f"{name}.out"])

    def input_dtypes(self):
        return tuple({dt for _, m in self.branches for dt in m.input_dtypes()})

    def cache_spec(self):
        return next((s for s in (m.cache_spec() for _, m in self.branches) if s is not None), None)

    def _state_parts(self):
        specs = [m.state_spec() for _, m in self.branches]
        for s in specs:
            if s is not None and (len(s.shape) != 1 or s.dtype != torch.float32):
                raise ConfigError("branches: a branch's state must be one float32 row")
        return specs

    def state_spec(self):
        n = sum(s.shape[0] for s in self._state_parts() if s is not None)
        return StateSpec((n,), torch.float32) if n else None

    def step_needs(self):
        needs = [n for n in (m.step_needs() for _, m in self.branches) if n is not None]
        if len(set(needs)) > 1:
            raise ConfigError("branches: the branches ask for different tilings of the step's rows")
        return needs[0] if needs else None

    def plan_step(self, step, captured):
        return tuple(m.plan_step(step, captured) for _, m in self.branches)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        outs, at = [], 0
        for (name, m), spec in zip(self.branches, self._state_parts()):
            st = None
            if spec is not None:
                if state is None:
                    raise ModelError("branches: a branch needs state, the mixer has no slab")
                st = state[:, at:at + spec.shape[0]]
                at += spec.shape[0]
            c = cache if m.cache_spec() is not None else None
            outs.append(branch_of(m, next(iter(x.values())),
                                  lambda rows, m=m, c=c, st=st: m.forward(x, rows, step, c, st, writes_cache)))
        T = outs[0].partials.shape[1]
        out = torch.empty((1, T, self.hidden), dtype=torch.float32, device=outs[0].partials.device)
        if self.combine == "weighted":
            self.ops.sum_norm_add(out[0], [(o.partials, o.bias) for o in outs], self.scales, accumulate=False)
        else:
            self.ops.branch_mean([(o.partials, o.bias) for o in outs], self.out_w, self.eps, out[0])
        return Pending(partials=out)
