"""The attention mixer: grouped-query attention over the paged cache.

q/k/v projection (one product over the concatenated weights, bias in its epilogue),
rotary encoding of q and k fused with the write of k and v into the cache pages,
attention of every row over its request's cached keys (causal, optionally windowed,
scale 1/sqrt(head_dim) unless given), and the output projection accumulated into the
residual stream.  Order of operations as the reference's dense decoder
(crates/thuban_architectures/src/transformer/forward.rs:114-365).
"""
from __future__ import annotations

import math

import torch

from ..cache.manager import KVSpec, StateSpec
from ..engine.step import StepNeeds
from ..errors import ConfigError, ModelError
from ..registry import MIXERS, POSITION_ENCODINGS
from ..weights.sources import WeightSpec
from .base import Mixer, Pending, mat, matmul_dtype, vec


def shared_position_encoding(spec, ctx):
    """One position-encoding object per distinct spec in a model."""
    key = ("position", spec.kind, repr(sorted(spec.params.items(), key=lambda kv: kv[0])))
    if key not in ctx.shared:
        ctx.shared[key] = POSITION_ENCODINGS.get(spec.kind)(spec.params, ctx)
    return ctx.shared[key]


@MIXERS.register("attention")
class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = none),
    qkv_bias, out_bias, scale (optional), position (PartSpec or None).

    Further, all optional: value_dim (values of another size than keys), keep_first (with a window: the first
    so many tokens of a sequence stay visible behind it, at their true positions), sinks (a learned logit per
    query head, tensor ``sinks`` [num_heads], that joins the softmax's denominator without a key or a value),
    value_mix ("source": this layer's values, as projected, are left for later layers of the step; "blend":
    v <- (1 - a) v + a v_source with the scalar tensor ``value_mix`` = a, before v is cached; the tensor may be
    stored for a source too, which ignores it), chunk (c > 0: the sequence is cut into runs of c positions counted
    from position 0, and a position sees only the earlier positions of its own run).  A layer that uses any of
    these runs on the general attention kernels (``csrc/attention_sink.cu``).

    And what happens around the attention itself: conv_taps (n >= 1: q, k and v pass a causal convolution of n taps
    per channel right after the projection, tensors ``q_conv.weight`` / ``k_conv.weight`` / ``v_conv.weight``
    [channels, n]; the last n - 1 projected rows of a request are fixed-size state), qk_norm (q and k are divided by
    their root mean square per head, eps ``qk_norm_eps``, and scaled by ``q_norm.weight`` / ``k_norm.weight``
    [head_dim], before they rotate), value_position (a PartSpec of a rotary encoding over all value dims: the
    value of position j is cached turned by j, and every head's sum is turned back by its query's position),
    head_gate (every head's output times sigmoid(W x), one number a head, tensor ``gate_proj.weight`` [num_heads,
    hidden]).

    And: pool (P > 0, with a window: behind the window a position also sees one mean key and one mean value for every
    block of P positions that lies wholly before the window, block b if b P + P - 1 <= p - window; the means are taken
    over the cached rows and join the same softmax; such a layer keeps its pages), qk_norm "whole" (q is divided by one
    root mean square over all its heads and scaled by ``q_norm.weight`` [num_heads head_dim], k likewise), values_from_keys
    (no value projection: the values are the keys as projected, before norm and rotation), unit_sink (one is added
    to the softmax's denominator: a sink whose logit is 0), out_gate (the heads' outputs times sigmoid(W x) number by
    number, tensor ``gate_proj.weight`` [num_heads value_dim, hidden]), q_temp (coef, every: q at position p times
    1 + coef ln(floor((p + 1) / every) + 1)), weights "sigmoid" (no softmax: key j weighs sigmoid(z + b_h), not
    normalised, with z the score, capped as softcap tanh(z / softcap) if ``softcap`` > 0, less r1_h ln(1 + r2_h (p - j))
    with ``distance_bias``; tensors ``r1``, ``r2``, and with ``weight_bias`` ``pb``, one number a query head)."""

    graph_safe = True
    returns_pending = True       # the output projection always leaves as partial sums; the rows given are not touched
    # portions of at least 16 rows go to the tensor-core attention in tiles of 128 query rows, the rest row by row
    NEEDS = StepNeeds(tile_rows=128, tile_min_rows=16)
    # the general kernels' tensor-core form takes tiles of 64 rows
    NEEDS_GENERAL = StepNeeds(tile_rows=64, tile_min_rows=16)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nq, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nq % self.nkv:
            raise ConfigError("num_heads must be a multiple of num_kv_heads")
        self.vd = int(p.get("value_dim") or self.hd)
        self.window = int(p.get("window", 0) or 0)
        self.keep_first = int(p.get("keep_first", 0) or 0) if self.window else 0
        self.sinks = bool(p.get("sinks", False))
        self.value_mix = p.get("value_mix")
        if self.value_mix not in (None, "source", "blend"):
            raise ConfigError(f"value_mix must be 'source' or 'blend', got {self.value_mix!r}")
        self.chunk = int(p.get("chunk", 0) or 0)
        if self.chunk and self.window:
            raise ConfigError("attention: a window and runs of a fixed length cannot be combined")
        self.taps = int(p.get("conv_taps", 0) or 0)
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_whole = p.get("qk_norm") == "whole"
        self.pool = int(p.get("pool", 0) or 0)
        if self.pool and (not self.window or self.keep_first or self.chunk):
            raise ConfigError("attention: means of blocks need a window, and exclude kept first tokens and runs")
        self.values_from_keys = bool(p.get("values_from_keys", False))
        if self.values_from_keys and self.vd != self.hd:
            raise ConfigError("attention: values that are the keys have the keys' size")
        self.unit_sink = bool(p.get("unit_sink", False))
        self.out_gate = bool(p.get("out_gate", False))
        self.q_temp = tuple(p["q_temp"]) if p.get("q_temp") is not None else None
        self.weights_rule = p.get("weights", "softmax")
        if self.weights_rule not in ("softmax", "sigmoid"):
            raise ConfigError(f"attention: weights must be 'softmax' or 'sigmoid', got {self.weights_rule!r}")
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.distance_bias, self.weight_bias = bool(p.get("distance_bias", False)), bool(p.get("weight_bias", False))
        if self.weights_rule == "sigmoid" and (self.sinks or self.unit_sink):
            raise ConfigError("attention: weights without a softmax take no sink")
        if self.weights_rule != "sigmoid" and (self.softcap or self.distance_bias or self.weight_bias):
            raise ConfigError("attention: a cap, a distance penalty and a bias of the weights belong to weights 'sigmoid'")
        if self.sinks and self.unit_sink:
            raise ConfigError("attention: a learned sink and a unit sink exclude each other")
        self.qk_eps = float(p.get("qk_norm_eps", 1e-6))
        self.head_gate = bool(p.get("head_gate", False))
        self.value_position = (shared_position_encoding(p["value_position"], ctx)
                               if p.get("value_position") is not None else None)
        if self.value_position is not None and self.value_position.rotary_dim != self.vd:
            raise ConfigError("attention: the values' rotation must cover all value dims")
        # q, k and v take a longer way from the projection to the cache, and the heads' sums one to the output
        self.reworked = bool(self.taps or self.qk_norm or self.head_gate or self.value_position is not None or self.pool
                             or self.values_from_keys or self.out_gate or self.q_temp is not None
                             or self.weights_rule == "sigmoid")
        if self.head_gate and self.out_gate:
            raise ConfigError("attention: a gate per head and a gate per number exclude each other")
        if self.reworked and self.value_mix:
            raise ConfigError("attention: blended values cannot be combined with a convolution, q/k norms, rotated "
                              "values or a gate per head")
        self.general = bool(self.vd != self.hd or self.keep_first or self.sinks or self.unit_sink or self.value_mix
                            or self.chunk or self.reworked)
        if self.general:
            if max(self.hd, self.vd) > 256 or min(self.hd, self.vd) < 1:
                raise ConfigError(f"head sizes {self.hd} (keys) and {self.vd} (values) are not supported (1 to 256)")
        elif self.hd % 16 or self.hd > 256:
            raise ConfigError(f"head_dim {self.hd} is not supported (multiples of 16 up to 256)")
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.position = shared_position_encoding(p["position"], ctx) if p.get("position") is not None else None
        self.rot = self.position.rotary_dim if self.position is not None else 0
        self.rot_style = self.position.style if self.position is not None else "half"
        if self.rot > self.hd:
            raise ConfigError("rotary_dim exceeds head_dim")

    def weights(self):
        nq, nkv, hd, vd, H = self.nq, self.nkv, self.hd, self.vd, self.hidden
        w = {"q_proj.weight": mat(nq * hd, H), "k_proj.weight": mat(nkv * hd, H),
             "v_proj.weight": mat(nkv * vd, H), "o_proj.weight": mat(H, nq * vd)}
        if self.qkv_bias:
            w.update({"q_proj.bias": vec(nq * hd), "k_proj.bias": vec(nkv * hd), "v_proj.bias": vec(nkv * vd)})
        if self.values_from_keys:
            w.pop("v_proj.weight")
            w.pop("v_proj.bias", None)
        if self.out_bias:
            w["o_proj.bias"] = vec(H)
        if self.sinks:
            w["sinks"] = vec(nq)
        if "value_mix" in self.params:
            w["value_mix"] = WeightSpec((), role="vector", optional=self.value_mix != "blend")
        if self.taps:
            for n, rows in (("q", nq * hd), ("k", nkv * hd), ("v", nkv * vd)):
                w[f"{n}_conv.weight"] = WeightSpec((rows, self.taps), role="vector", std=0.3)
        if self.qk_norm:
            w.update({"q_norm.weight": vec(nq * hd if self.qk_whole else hd, init="gamma"),
                      "k_norm.weight": vec(nkv * hd if self.qk_whole else hd, init="gamma")})
        if self.head_gate:
            w["gate_proj.weight"] = mat(nq, H)
        if self.out_gate:
            w["gate_proj.weight"] = mat(nq * vd, H)
        if self.distance_bias:
            w.update({"r1": vec(nq), "r2": vec(nq, init="gamma")})
        if self.weight_bias:
            w["pb"] = vec(nq)
        return w

    def fused(self):
        if self.values_from_keys:
            return {}
        f = {"qkv_proj.weight": ["q_proj.weight", "k_proj.weight", "v_proj.weight"]}
        if self.qkv_bias:
            f["qkv_proj.bias"] = ["q_proj.bias", "k_proj.bias", "v_proj.bias"]
        return f

    def load(self, t):
        qkv_names = ["q_proj.weight", "k_proj.weight"] + ([] if self.values_from_keys else ["v_proj.weight"])
        gated = self.head_gate or self.out_gate
        dt = matmul_dtype(*(t[n] for n in qkv_names), *([t["gate_proj.weight"]] if gated else []))
        # one product gives q, k, v and, with a gate, its logits
        pieces = [t[n] for n in qkv_names] + ([t["gate_proj.weight"]] if gated else [])
        self.w_qkv = torch.cat([w.to(dt) for w in pieces], 0)
        self.w_conv = (torch.cat([t["q_conv.weight"], t["k_conv.weight"], t["v_conv.weight"]], 0).contiguous()
                       if self.taps else None)
        self.q_norm, self.k_norm = t.get("q_norm.weight"), t.get("k_norm.weight")
        self.v_cos, self.v_sin = self.value_position.tables() if self.value_position is not None else (None, None)
        self.b_qkv = (torch.cat([t[n.replace("weight", "bias")] for n in qkv_names], 0).contiguous()
                      if self.qkv_bias else None)
        # the same for a projection that also gives the gates' logits (which have no bias)
        self.b_qkv_all = (torch.cat([self.b_qkv, self.b_qkv.new_zeros(t["gate_proj.weight"].shape[0])])
                          if self.qkv_bias and gated else self.b_qkv)
        self.w_o = t["o_proj.weight"]
        self.b_o = t.get("o_proj.bias")
        self.sink = t.get("sinks")
        if self.unit_sink:           # a sink whose logit is 0: one more in the denominator
            self.sink = torch.zeros(self.nq, dtype=torch.float32, device=self.ctx.device)
        self.sigmoid = ((self.softcap, t.get("r1"), t.get("r2"), t.get("pb")) if self.weights_rule == "sigmoid" else None)
        # read once, when the tensors arrive: the kernels take the blend weight as a launch parameter
        self.blend = float(t["value_mix"]) if self.value_mix == "blend" else 0.0
        if self.position is not None:
            self.cos, self.sin = self.position.tables()
        else:
            self.cos = self.sin = torch.zeros((1, 1), dtype=torch.float32, device=self.ctx.device)

    def input_dtypes(self):
        return (self.w_qkv.dtype,)

    def cache_spec(self):
        if self.pool:            # the pages stay: the means of a page's blocks live beside it
            return KVSpec(self.nkv, self.hd, 0, value_dim=None if self.vd == self.hd else self.vd, pool=self.pool)
        if self.general:
            return KVSpec(self.nkv, self.hd, self.window, value_dim=None if self.vd == self.hd else self.vd,
                          keep_first=self.keep_first)
        return KVSpec(self.nkv, self.hd, self.window)

    def state_spec(self):
        if self.taps > 1:        # the last taps - 1 projected rows of q | k | v
            return StateSpec(((self.taps - 1) * ((self.nq + self.nkv) * self.hd + self.nkv * self.vd),), torch.float32)
        return None

    def step_needs(self):
        if not self.general:
            return self.NEEDS
        ok = getattr(self.ops, "sink_attention_tiles_ok", None)
        tiles = ok is not None and ok(self.ctx.act_dtype, self.ctx.act_dtype, self.hd, self.vd)
        return self.NEEDS_GENERAL if tiles else None

    def plan_step(self, step, captured):
        """How the key ranges of a batch of decoded tokens are cut.  Requests of about the same length share one
        way of cutting their keys; a ragged batch lets the kernel cut the keys of all rows into equal runs
        itself.  In a captured step the splits are chosen for a bucketed context length, so that few graphs are
        needed as requests grow: four buckets per doubling of the context, at least 256 apart."""
        if step.n_tokens != len(step.entries):
            return None
        if self.general:
            return self._plan_general(step, captured)
        lens = [e.start_pos + 1 for e in step.entries]
        step.even_lengths = min(lens) * 4 >= max(lens) * 3
        if not captured:
            return (step.even_lengths,)
        kv = max(step.max_kv_len, 1)
        gran = max(256, 1 << max(kv.bit_length() - 3, 0))
        step.max_kv_len = -(-kv // gran) * gran
        return (step.max_kv_len, step.even_lengths)

    def _plan_general(self, step, captured):
        """Decoded tokens on the general kernels: a captured step cuts its key ranges for a bucketed context
        (buckets as above), which is part of the graph's key."""
        if not captured:
            return None
        kv = max(step.max_kv_len, 1)
        gran = max(256, 1 << max(kv.bit_length() - 3, 0))
        step.max_kv_len = -(-kv // gran) * gran
        return (step.max_kv_len,)

    def _forward_reworked(self, xin, step, cache, state):
        """The general kernels with more on both sides: the projection (with the gates' logits), the convolution over
        each request's rows and its carried ones, one kernel that norms and rotates q and k, rotates the values and
        writes q and the cache rows, the attention, one kernel that turns every head's sum back and gates it, and
        the output projection as partial sums."""
        ops, nq, nkv, hd, vd = self.ops, self.nq, self.nkv, self.hd, self.vd
        T, dev = xin.shape[0], xin.device
        act = self.ctx.act_dtype if self.w_qkv.dtype == torch.bfloat16 else torch.float32
        W = (nq + nkv) * hd + (0 if self.values_from_keys else nkv * vd)
        proj = torch.empty((T, self.w_qkv.shape[0]), dtype=torch.float32, device=dev)
        ops.gemm(xin, self.w_qkv, proj, bias=self.b_qkv_all)
        if self.taps:
            if self.taps > 1 and state is None:
                raise ModelError("attention: the convolution needs a state slab")
            y = torch.empty((T, W), dtype=torch.float32, device=dev)
            ops.short_conv(proj, 0, self.w_conv, None, "none", step.pos, step.slot, state, y)
        else:
            y = proj[:, :W]
        q = torch.empty((T, nq * hd), dtype=act, device=dev)
        extra = {k: v for k, v in (("whole", self.qk_whole), ("v_from_k", self.values_from_keys), ("q_temp", self.q_temp))
                 if v}
        ops.qk_norm_write(y, self.q_norm, self.k_norm, self.qk_eps, step.pos, step.slot, self.cos, self.sin, self.rot,
                          self.rot_style, self.v_cos, self.v_sin,
                          self.value_position.style if self.value_position is not None else "half", q, cache, nq, nkv, hd,
                          vd, step.status, **extra)
        if self.pool:       # the blocks that this step completes get their mean key and value
            ops.pool_write(cache, step, nkv, hd, vd, self.pool)
        attn = torch.empty((T, nq * vd), dtype=act, device=dev)
        needs = self.step_needs()
        more = {k: v for k, v in (("pool", self.pool), ("sigmoid", self.sigmoid)) if v}
        ops.sink_attention(q, cache, step, attn, nq, nkv, hd, vd, self.window, self.keep_first, self.sink, self.scale,
                           tiling=step.tiling(needs) if needs is not None and q.dtype == torch.bfloat16 else None,
                           chunk=self.chunk, **more)
        if self.head_gate or self.out_gate or self.value_position is not None:
            out = torch.empty_like(attn)
            ops.head_finish(attn, step.pos, self.v_cos, self.v_sin,
                            self.value_position.style if self.value_position is not None else "half",
                            proj[:, W:] if self.head_gate or self.out_gate else None, out, nq, vd)
            attn = out
        return Pending(partials=ops.gemm_partials(attn, self.w_o), bias=self.b_o)

    def _forward_general(self, xin, step, cache, writes_cache, state=None):
        """Sizes and masks the fast kernels do not take: projection left as partial sums, one kernel that adds
        them with the bias, rotates, blends the values and writes q and the cache rows, one attention kernel
        with the window's kept first tokens and the sink, then the output projection as partial sums."""
        if not writes_cache:
            raise ModelError("attention: a layer on the general kernels owns its cache")
        if self.reworked:
            return self._forward_reworked(xin, step, cache, state)
        ops, nq, nkv, hd, vd = self.ops, self.nq, self.nkv, self.hd, self.vd
        T, dev = xin.shape[0], xin.device
        act = self.ctx.act_dtype if self.w_qkv.dtype == torch.bfloat16 else torch.float32
        qkv = ops.gemm_partials(xin, self.w_qkv)
        q = torch.empty((T, nq * hd), dtype=act, device=dev)
        v_keep = v_from = None
        if self.value_mix == "source":
            v_keep = step.shared["attention.value_mix"] = torch.empty((T, nkv * vd), dtype=torch.float32, device=dev)
        elif self.value_mix == "blend":
            v_from = step.shared.get("attention.value_mix")
            if v_from is None or tuple(v_from.shape) != (T, nkv * vd):
                raise ModelError("attention: values are to be blended, but no earlier layer of the step left its own "
                                 "(of the same size)")
        ops.qkv_write(qkv, self.b_qkv, step.pos, step.slot, self.cos, self.sin, self.rot, self.rot_style, q, cache,
                      nq, nkv, hd, vd, step.status, v_keep=v_keep, v_from=v_from, blend=self.blend)
        attn = torch.empty((T, nq * vd), dtype=act, device=dev)
        needs = self.step_needs()
        ops.sink_attention(q, cache, step, attn, nq, nkv, hd, vd, self.window, self.keep_first, self.sink, self.scale,
                           tiling=step.tiling(needs) if needs is not None and q.dtype == torch.bfloat16 else None,
                           chunk=self.chunk)
        return Pending(partials=ops.gemm_partials(attn, self.w_o), bias=self.b_o)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        if cache is None:
            raise ModelError("attention needs a cache")
        if self.general:
            return self._forward_general(x[self.w_qkv.dtype], step, cache, writes_cache, state)
        ops, nq, nkv, hd = self.ops, self.nq, self.nkv, self.hd
        xin = x[self.w_qkv.dtype]
        T = xin.shape[0]
        act = self.ctx.act_dtype
        q = torch.empty((T, nq * hd), dtype=act, device=xin.device)
        fused = None
        if writes_cache:
            # the projection is left as partial sums over pieces of K; the rotary kernel adds them and the bias
            qkv = ops.gemm_partials(xin, self.w_qkv)
            if T == len(step.entries) and hasattr(ops, "rope_attention_decode"):
                # decoded tokens: one kernel rotates, writes the cache pages and attends
                attn = torch.empty_like(q)
                if ops.rope_attention_decode(qkv, self.b_qkv, self.cos, self.sin, self.rot, self.rot_style, cache, step,
                                             attn, nq, nkv, hd, self.window, self.scale):
                    fused = attn
        if fused is not None:
            attn = fused
        elif writes_cache:
            ops.rope_kv_write(qkv, step.pos, step.slot, self.cos, self.sin, self.rot, q, cache, nq, nkv, hd,
                              True, step.status, bias=self.b_qkv, style=self.rot_style)
        else:   # reads another call's cache: only the queries are needed
            width, nqd = (nq + 2 * nkv) * hd, nq * hd
            qkv = torch.empty((1, T, width), dtype=torch.float32, device=xin.device)
            ops.gemm(xin, self.w_qkv[:nqd], qkv[0, :, :nqd], bias=self.b_qkv[:nqd] if self.b_qkv is not None else None)
            ops.rope_kv_write(qkv, step.pos, step.slot, self.cos, self.sin, self.rot, q, cache, nq, nkv, hd,
                              False, step.status, style=self.rot_style)
        if fused is None:
            attn = torch.empty_like(q)
            ops.attention(q, cache, step, attn, nq, nkv, hd, self.window, self.scale, tiling=step.tiling(self.NEEDS))
        # the output projection is handed to the next norm as partial sums (and its bias)
        return Pending(partials=ops.gemm_partials(attn, self.w_o), bias=self.b_o)
