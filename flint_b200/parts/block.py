"""Arrangements of a layer's parts.

``prenorm``: h += mixer(norm1(h)); h += ffn(norm2(h)) -- the reference's decoder layer
(crates/thuban_architectures/src/transformer/forward.rs:102-440) and Phi-MoE's.
``parallel``: h += mixer(norm1(h)) + ffn(norm1(h)) with one shared norm (the feed-forward may be absent);
``parallel_two_norms``: h += mixer(norm1(h)) + ffn(norm2(h)), both of the same h.
``postnorm``: h <- norm1(a h + s1 * mixer(h)); h <- norm2(a h + s2 * ffn(h)): the parts read the rows themselves and
the norms come after the sums (a and the scales s are the norms' ``residual_scale`` and ``branch_scale``).
``sandwich``: h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h))): a norm before and one after each part, the
second applied to what the part adds (RMS norms; the second half only with a feed-forward).
An arrangement only orders parts; it does not know what they are.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..registry import BLOCKS
from .base import Pending


def run_norm(norm, residual, want, pending=None, router=None, row_index=None):
    """Run a norm; a pending addition or a routing request that the norm cannot take is served
    by separate kernels instead.  Returns (outputs, router or None if it still has to be done)."""
    if pending is not None and not norm.supports_pending:
        norm.ops.apply_pending(residual, pending)
        pending = None
    if router is not None and not norm.supports_router:
        router = None
    kw = {}
    if pending is not None:
        kw["pending"] = pending
    if router is not None:
        kw["router"] = router
    if row_index is not None:
        kw["row_index"] = row_index
    return norm.forward(residual, want, **kw), router


def settle(part, residual, pending):
    """Apply a pending addition right away (for arrangements that cannot carry it)."""
    if pending is not None:
        part.ops.apply_pending(residual, pending)


class Block:
    roles = ()

    def __init__(self, parts: dict):
        self.parts = parts

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        """Runs the layer on ``residual`` in place.  ``carry``: a Pending addition left by the
        previous layer; returns the Pending addition this layer leaves (or None)."""
        raise NotImplementedError


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    roles = ("norm1", "mixer", "norm2", "ffn")

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        mixer, ffn = p["mixer"], p["ffn"]
        x, _ = run_norm(p["norm1"], residual, mixer.input_dtypes(), carry)
        pend = mixer.forward(x, residual, step, cache, state, writes_cache)
        request = ffn.router_request(residual.shape[0]) if hasattr(ffn, "router_request") else None
        if request is not None and step.record is not None and getattr(request, "logits", 0) is None:
            # a test asked for this step's internals: the logits behind the routing come along
            request.logits = request.weight.new_empty((residual.shape[0], request.weight.shape[0]), dtype=torch.float32)
        want = ffn.input_dtypes_when_routed() if request is not None and p["norm2"].supports_router \
            else ffn.input_dtypes()
        x, routed = run_norm(p["norm2"], residual, want, pend, request)
        return ffn.forward(x, residual, step, routed=routed) if routed is not None else ffn.forward(x, residual, step)


def merge_pending(part, residual, first, second):
    """One Pending for two parts' additions: partial sums of a product from one and gated expert rows from the
    other travel together to the next norm; what cannot be merged is applied right away."""
    if first is None or second is None:
        return first if second is None else second
    for a, b in ((first, second), (second, first)):
        if a.y is None and b.partials is None and b.bias is None:
            return Pending(partials=a.partials, bias=a.bias, y=b.y, row_of=b.row_of, gates=b.gates)
    settle(part, residual, first)
    return second


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    roles = ("norm1", "mixer")        # "ffn" is optional: a layer may be a mixer alone

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        ffn = p.get("ffn")
        # a feed-forward that routes may have its routing done by the one norm, while the row is at hand
        request = ffn.router_request(residual.shape[0]) if hasattr(ffn, "router_request") else None
        routed_by_norm = request is not None and p["norm1"].supports_router
        if routed_by_norm and step.record is not None and getattr(request, "logits", 0) is None:
            request.logits = request.weight.new_empty((residual.shape[0], request.weight.shape[0]), dtype=torch.float32)
        ffn_want = () if ffn is None else (ffn.input_dtypes_when_routed() if routed_by_norm else ffn.input_dtypes())
        want = tuple(set(p["mixer"].input_dtypes()) | set(ffn_want))
        x, routed = run_norm(p["norm1"], residual, want, carry, request if routed_by_norm else None)
        mixed = p["mixer"].forward(x, residual, step, cache, state, writes_cache)
        if ffn is None:
            return mixed
        fed = ffn.forward(x, residual, step, routed=routed) if routed is not None else ffn.forward(x, residual, step)
        return merge_pending(p["mixer"], residual, mixed, fed)


@BLOCKS.register("parallel_two_norms")
class ParallelTwoNormsBlock(Block):
    """h += mixer(norm1(h)) + ffn(norm2(h)): both branches read the same rows, each through a norm of its own
    (the feed-forward with its norm may be absent).  What the layer before left pending is applied by norm1's
    kernel, so norm2 reads the finished rows; both branches' additions travel on to the next layer's norm."""
    roles = ("norm1", "mixer")

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        mixer, ffn = p["mixer"], p.get("ffn")
        x, _ = run_norm(p["norm1"], residual, mixer.input_dtypes(), carry)
        if ffn is None:
            return mixer.forward(x, residual, step, cache, state, writes_cache)
        if "norm2" not in p:
            raise ConfigError("block 'parallel_two_norms': a feed-forward needs its norm (norm2)")
        request = ffn.router_request(residual.shape[0]) if hasattr(ffn, "router_request") else None
        routed_by_norm = request is not None and p["norm2"].supports_router
        if routed_by_norm and step.record is not None and getattr(request, "logits", 0) is None:
            request.logits = request.weight.new_empty((residual.shape[0], request.weight.shape[0]), dtype=torch.float32)
        want = ffn.input_dtypes_when_routed() if routed_by_norm else ffn.input_dtypes()
        # both norms read the rows before either branch may add to them
        y, routed = run_norm(p["norm2"], residual, want, None, request if routed_by_norm else None)
        mixed = mixer.forward(x, residual, step, cache, state, writes_cache)
        fed = ffn.forward(y, residual, step, routed=routed) if routed is not None else ffn.forward(y, residual, step)
        return merge_pending(mixer, residual, mixed, fed)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """h += n1b(mixer(n1(h))); h += n2b(ffn(n2(h))).  What a part adds (partial sums of its last product, or its
    chosen experts' rows with their weights) is summed, divided by its root mean square, scaled and added into the rows
    by one kernel; nothing is left pending for the next layer."""
    roles = ("norm1", "mixer", "norm1b")

    def _run(self, part, norm_after, residual, call):
        """residual += norm_after(what the part adds).  A part that says ``returns_pending`` hands back what it adds
        (partial sums with a bias, or expert rows with their weights); any other adds into a zeroed buffer."""
        if norm_after.mode != "rms":
            raise ConfigError("block 'sandwich': the norms after the parts are RMS norms")
        pend = call(None) if getattr(part, "returns_pending", False) else branch_of(part, residual, call)
        branches = [(pend.partials, pend.bias)] if pend.partials is not None else []
        rows = (pend.y, pend.row_of, pend.gates) if pend.y is not None else None
        part.ops.sum_norm_add(residual, branches, [1.0] * len(branches), expert_rows=rows, gamma=norm_after.gamma,
                              eps=norm_after.eps)

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        mixer, ffn = p["mixer"], p.get("ffn")
        x, _ = run_norm(p["norm1"], residual, mixer.input_dtypes(), carry)
        self._run(mixer, p["norm1b"], residual, lambda rows: mixer.forward(x, rows, step, cache, state, writes_cache))
        if ffn is None:
            return None
        if "norm2" not in p or "norm2b" not in p:
            raise ConfigError("block 'sandwich': a feed-forward needs its two norms (norm2, norm2b)")
        request = ffn.router_request(residual.shape[0]) if hasattr(ffn, "router_request") else None
        routed_by_norm = request is not None and p["norm2"].supports_router
        if routed_by_norm and step.record is not None and getattr(request, "logits", 0) is None:
            request.logits = request.weight.new_empty((residual.shape[0], request.weight.shape[0]), dtype=torch.float32)
        want = ffn.input_dtypes_when_routed() if routed_by_norm else ffn.input_dtypes()
        y, routed = run_norm(p["norm2"], residual, want, None, request if routed_by_norm else None)
        self._run(ffn, p["norm2b"], residual,
                  lambda rows: ffn.forward(y, rows, step, routed=routed) if routed is not None else ffn.forward(y, rows, step))
        return None


def rows_in(part_ops, residual, step, dtypes):
    """The rows themselves in the element types a part reads: the float32 rows as they are; another type from the
    copy that the producer of the rows left in ``step.shared["rows"]`` (tensor, {type: copy}), else cast here."""
    left = step.shared.get("rows")
    copies = left[1] if left is not None and left[0] is residual else {}
    out = {}
    for dt in set(dtypes):
        if dt == residual.dtype:
            out[dt] = residual
        elif dt in copies:
            out[dt] = copies[dt]
        else:
            out[dt] = torch.empty(residual.shape, dtype=dt, device=residual.device)
            part_ops.cast_rows(residual, out[dt])
    return out


def branch_of(part, residual, run):
    """What a part adds, as a ``Pending`` of partial sums that nobody has applied.  A part that says
    ``returns_pending`` never touches the rows it is given and always returns such a ``Pending``; any other part
    adds into a zeroed float32 buffer shaped like ``residual``, which then is the one partial sum.  ``run(rows)`` calls
    the part's forward."""
    if getattr(part, "returns_pending", False):
        return run(None)
    buf = torch.zeros(residual.shape, dtype=torch.float32, device=residual.device)
    pend = run(buf)
    if pend is not None:
        part.ops.apply_pending(buf, pend)
    return Pending(partials=buf.unsqueeze(0))


@BLOCKS.register("postnorm")
class PostNormBlock(Block):
    """h <- norm1(a h + s1 * mixer(h)); h <- norm2(a h + s2 * ffn(h)), the second half only with a feed-forward.
    Both norms must be able to run after the sum (``Norm.post``)."""
    roles = ("norm1", "mixer")

    def forward(self, residual, step, cache, state, writes_cache=True, carry=None):
        p = self.parts
        mixer, ffn = p["mixer"], p.get("ffn")
        settle(mixer, residual, carry)
        act = mixer.ctx.act_dtype
        x = rows_in(mixer.ops, residual, step, mixer.input_dtypes())
        step.shared.pop("rows", None)          # the rows change below
        mixed = branch_of(mixer, residual, lambda rows: mixer.forward(x, rows, step, cache, state, writes_cache))
        if ffn is None:
            p["norm1"].post(residual, mixed)
            return None
        if "norm2" not in p:
            raise ConfigError("block 'postnorm': a feed-forward needs its norm (norm2)")
        want = set(ffn.input_dtypes())
        copy = torch.empty(residual.shape, dtype=act, device=residual.device) if act in want and act != residual.dtype else None
        p["norm1"].post(residual, mixed, copy=copy)
        if copy is not None:
            step.shared["rows"] = (residual, {act: copy})
        y = rows_in(ffn.ops, residual, step, want)
        step.shared.pop("rows", None)
        fed = branch_of(ffn, residual, lambda rows: ffn.forward(y, rows, step))
        p["norm2"].post(residual, fed)
        return None
