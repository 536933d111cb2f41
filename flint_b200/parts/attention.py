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
    hidden])."""

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
        self.qk_eps = float(p.get("qk_norm_eps", 1e-6))
        self.head_gate = bool(p.get("head_gate", False))
        self.value_position = (shared_position_encoding(p["value_position"], ctx)
                               if p.get("value_position") is not None else None)
        if self.value_position is not None and self.value_position.rotary_dim != self.vd:
            raise ConfigError("attention: the values' rotation must cover all value dims")
        # q, k and v take a longer way from the projection to the cache, and the heads' sums one to the output
        self.reworked = bool(self.taps or self.qk_norm or self.head_gate or self.value_position is not None)
        if self.reworked and self.value_mix:
            raise ConfigError("attention: blended values cannot be combined with a convolution, q/k norms, rotated "
                              "values or a gate per head")
        self.general = bool(self.vd != self.hd or self.keep_first or self.sinks or self.value_mix or self.chunk
                            or self.reworked)
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
            w.update({"q_norm.weight": vec(hd, init="gamma"), "k_norm.weight": vec(hd, init="gamma")})
        if self.head_gate:
            w["gate_proj.weight"] = mat(nq, H)
        return w

    def fused(self):
        f = {"qkv_proj.weight": ["q_proj.weight", "k_proj.weight", "v_proj.weight"]}
        if self.qkv_bias:
            f["qkv_proj.bias"] = ["q_proj.bias", "k_proj.bias", "v_proj.bias"]
        return f

    def load(self, t):
        dt = matmul_dtype(t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"])
        # one product gives q, k, v and, with a gate per head, its logits
        pieces = [t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"]] + ([t["gate_proj.weight"]] if self.head_gate else [])
        self.w_qkv = torch.cat([w.to(dt) for w in pieces], 0)
        self.w_conv = (torch.cat([t["q_conv.weight"], t["k_conv.weight"], t["v_conv.weight"]], 0).contiguous()
                       if self.taps else None)
        self.q_norm, self.k_norm = t.get("q_norm.weight"), t.get("k_norm.weight")
        self.v_cos, self.v_sin = self.value_position.tables() if self.value_position is not None else (None, None)
        self.b_qkv = (torch.cat([t["q_proj.bias"], t["k_proj.bias"], t["v_proj.bias"]], 0).contiguous()
                      if self.qkv_bias else None)
        # the same for a projection that also gives the gates' logits (which have no bias)
        self.b_qkv_all = (torch.cat([self.b_qkv, self.b_qkv.new_zeros(self.nq)]) if self.qkv_bias and self.head_gate
                          else self.b_qkv)
        self.w_o = t["o_proj.weight"]
        self.b_o = t.get("o_proj.bias")
        self.sink = t.get("sinks")
        # read once, when the tensors arrive: the kernels take the blend weight as a launch parameter
        self.blend = float(t["value_mix"]) if self.value_mix == "blend" else 0.0
        if self.position is not None:
            self.cos, self.sin = self.position.tables()
        else:
            self.cos = self.sin = torch.zeros((1, 1), dtype=torch.float32, device=self.ctx.device)

    def input_dtypes(self):
        return (self.w_qkv.dtype,)

    def cache_spec(self):
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
        W = (nq + nkv) * hd + nkv * vd
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
        ops.qk_norm_write(y, self.q_norm, self.k_norm, self.qk_eps, step.pos, step.slot, self.cos, self.sin, self.rot,
                          self.rot_style, self.v_cos, self.v_sin,
                          self.value_position.style if self.value_position is not None else "half", q, cache, nq, nkv, hd,
                          vd, step.status)
        attn = torch.empty((T, nq * vd), dtype=act, device=dev)
        needs = self.step_needs()
        ops.sink_attention(q, cache, step, attn, nq, nkv, hd, vd, self.window, self.keep_first, self.sink, self.scale,
                           tiling=step.tiling(needs) if needs is not None and q.dtype == torch.bfloat16 else None,
                           chunk=self.chunk)
        if self.head_gate or self.value_position is not None:
            out = torch.empty_like(attn)
            ops.head_finish(attn, step.pos, self.v_cos, self.v_sin,
                            self.value_position.style if self.value_position is not None else "half",
                            proj[:, W:] if self.head_gate else None, out, nq, vd)
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
