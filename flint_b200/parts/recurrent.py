"""Two mixers that carry a matrix of state per head from token to token: the gated delta rule and a state-space
model with a scalar decay per head (the state-space duality form of Mamba-2).

A third, ``retention``, is linear attention with a fixed decay per head: S <- decay_h S + k v^T, o = S^T q, with q and
k rotated by the position; it runs the state-space form of the same kernel with the decay and the step size constant.

Both keep, per request, a float32 matrix S per head and the last ``taps - 1`` inputs of a short causal convolution
in one row of the cache manager's state slab (zeroed on admission), and both run the same recurrence kernel
(``ops.recurrence_scan``), which walks every request's rows of the step in order from the state its earlier steps
left: the result does not depend on how a prompt was cut.  With k, q of a key head (or B, C of a group), a value
row v and S [dim, value_dim]:

    gated delta rule   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    state space        S <- a S + B (dt x)^T;                                    y = S^T C + D x

``gated_delta``: q, k, v pass the convolution and SiLU; q and k become unit vectors per head (q also times
dim^(-1/2)); beta = sigmoid(W_b x); g = exp(-exp(A_log) softplus(W_a2 W_a1 x + dt_bias)) per head and key channel; each
head's o is divided by its root mean square, scaled by ``norm`` and by sigmoid(W_g2 W_g1 x), then projected.
``ssd``: W_in x = [z | x | B | C | dt]; x, B, C pass the convolution (with a bias) and SiLU; dt = softplus(dt + dt_bias),
a = exp(-exp(A_log) dt); y times silu(z) is RMS-normed in ``norm_groups`` equal parts, scaled by ``norm`` and projected.
Decays, step sizes, gates of the recurrence, unit norms and the state are float32 whatever the products run in.
The reference keeps recurrent state per sequence slot outside its paged pool in the same way
(crates/thuban_architectures/src/qwen35/state.rs:5-55).
"""
from __future__ import annotations

import torch

from ..cache.manager import StateSpec
from ..errors import ConfigError, ModelError
from ..registry import MIXERS
from ..weights.sources import WeightSpec
from .base import Mixer, Pending, mat, matmul_dtype, vec


def request_starts(step):
    """Where each request's rows start in the flattened batch (int32 on the device, one entry more than there are
    requests), or None for a batch of single tokens (row r is request r).  Uploaded once per step."""
    if step.n_tokens == len(step.entries):
        return None
    if "request_starts" not in step.plans:
        starts = torch.tensor(list(step.entry_start) + [step.n_tokens], dtype=torch.int32)
        step.plans["request_starts"] = starts.to(step.pos.device)
    return step.plans["request_starts"]


def conv_weight(channels, taps):
    return WeightSpec((channels, taps), role="vector", std=0.3)


class _Recurrent(Mixer):
    graph_safe = True
    returns_pending = True

    def plan_step(self, step, captured):
        request_starts(step)
        return None

    def _split_state(self, state, n_matrix):
        if state is None:
            raise ModelError(f"{type(self).__name__} needs a state slab")
        return state[:, :n_matrix], (state[:, n_matrix:] if state.shape[1] > n_matrix else None)


@MIXERS.register("gated_delta")
class GatedDeltaRule(_Recurrent):
    """params: hidden_size, num_heads (value heads), num_kv_heads (query/key heads), dim, value_dim, conv_taps,
    unit_eps, norm_eps.  tensors: q, k [G dim, hidden]; v [H value_dim, hidden]; q.conv, k.conv, v.conv [channels, taps];
    b [H, hidden]; a1 [r, hidden], a2 [H dim, r], dt_bias [H dim], A_log [H]; g1 [r', hidden], g2 [H value_dim, r'];
    norm [value_dim]; o [hidden, H value_dim].  The ranks r, r' are read from the tensors."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.G, self.D, self.V = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["dim"]), int(p["value_dim"])
        if self.H % self.G:
            raise ConfigError("gated_delta: num_heads must be a multiple of num_kv_heads")
        if self.D > 256:
            raise ConfigError(f"gated_delta: {self.D} key dims per head are not supported (up to 256)")
        self.taps = int(p["conv_taps"])
        self.unit_eps, self.eps = float(p["unit_eps"]), float(p["norm_eps"])
        self.rank_a = int(p.get("decay_rank", 0)) or None
        self.rank_g = int(p.get("gate_rank", 0)) or None
        self.conv_ch = 2 * self.G * self.D + self.H * self.V

    def weights(self):
        H, G, D, V, W, t = self.H, self.G, self.D, self.V, self.hidden, self.taps
        ra, rg = self.rank_a or max(W // 16, 1), self.rank_g or max(W // 16, 1)
        any_rank = lambda rows, cols: WeightSpec((rows, cols), role="matrix", free_dims=(0,))
        return {"q": mat(G * D, W), "k": mat(G * D, W), "v": mat(H * V, W), "q.conv": conv_weight(G * D, t),
                "k.conv": conv_weight(G * D, t), "v.conv": conv_weight(H * V, t), "b": mat(H, W), "a1": any_rank(ra, W),
                "a2": WeightSpec((H * D, ra), std=0.2, free_dims=(1,)), "dt_bias": vec(H * D), "A_log": vec(H),
                "g1": any_rank(rg, W), "g2": WeightSpec((H * V, rg), std=0.2, free_dims=(1,)), "norm": vec(V, init="gamma"), "o": mat(W, H * V)}

    def load(self, t):
        names = ("q", "k", "v", "b", "a1", "g1")
        dt = matmul_dtype(*(t[n] for n in names), t["o"], t["a2"], t["g2"])
        self.ra, self.rg = t["a1"].shape[0], t["g1"].shape[0]
        if t["a2"].shape[1] != self.ra or t["g2"].shape[1] != self.rg:
            raise ConfigError(f"gated_delta: the low-rank pairs disagree (a1 {tuple(t['a1'].shape)} with a2 "
                              f"{tuple(t['a2'].shape)}, g1 {tuple(t['g1'].shape)} with g2 {tuple(t['g2'].shape)})")
        # one product gives q, k, v, the write strength's logit and the two low-rank inputs
        self.w_in = torch.cat([t[n].to(dt) for n in names], 0).contiguous()
        self.w_conv = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], 0).contiguous()
        self.w_a2, self.w_g2, self.w_o = t["a2"].to(dt), t["g2"].to(dt), t["o"].to(dt)
        self.dt_bias, self.a_log, self.w_norm = t["dt_bias"], t["A_log"], t["norm"]

    def input_dtypes(self):
        return (self.w_in.dtype,)

    def state_spec(self):
        return StateSpec((self.H * self.D * self.V + (self.taps - 1) * self.conv_ch,), torch.float32)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        ops, H, G, D, V = self.ops, self.H, self.G, self.D, self.V
        S, conv_state = self._split_state(state, H * D * V)
        xin = x[self.w_in.dtype]
        T, dev = xin.shape[0], xin.device
        f32 = dict(dtype=torch.float32, device=dev)
        proj = torch.empty((T, self.w_in.shape[0]), **f32)
        ops.gemm(xin, self.w_in, proj)
        C = self.conv_ch
        y = torch.empty((T, C), **f32)
        ops.short_conv(proj, 0, self.w_conv, None, "silu", step.pos, step.slot, conv_state, y)
        # the low-rank second halves read float32 columns of the projection
        c_b, c_a, c_g = C, C + H, C + H + self.ra
        a = torch.empty((T, H * D), **f32)
        ops.gemm(proj[:, c_a:c_a + self.ra], self.w_a2, a)
        gate = torch.empty((T, H * V), **f32)
        ops.gemm(proj[:, c_g:c_g + self.rg], self.w_g2, gate)
        qk = torch.empty((T, 2 * G * D), **f32)
        decay = torch.empty((T, H * D), **f32)
        beta = torch.empty((T, H), **f32)
        ops.delta_prepare(y, proj[:, c_b:c_b + H], a, self.dt_bias, self.a_log, qk, decay, beta, H, G, D, self.unit_eps)
        o = torch.empty((T, H * V), **f32)
        ops.recurrence_scan(qk[:, :G * D], qk[:, G * D:], y[:, 2 * G * D:], decay, True, beta, None, None, step.slot,
                            request_starts(step), len(step.entries), S, o, H, G, D, V)
        act = self.ctx.act_dtype if self.w_o.dtype == torch.bfloat16 else torch.float32
        out = torch.empty((T, H * V), dtype=act, device=dev)
        ops.gated_norm(o, gate, "sigmoid", False, self.w_norm, self.eps, H, out)
        return Pending(partials=ops.gemm_partials(out, self.w_o))


@MIXERS.register("retention")
class Retention(_Recurrent):
    """Linear attention with a fixed decay per head and no softmax or denominator: per head S <- decay_h S + k v^T,
    o = S^T q, where q and k rotate by the position over their leading dims and k is scaled by dim^(-1/2); each head's o
    is divided by its root mean square (no scale), the heads side by side are multiplied by silu(W_g x) and projected.
    The state (S per head, float32) is a ``StateSpec`` slab zeroed at admission.

    params: hidden_size, num_heads, dim, value_dim, decay (one number a head), norm_eps, position (PartSpec or None).
    tensors: q, k [H dim, hidden]; v, g [H value_dim, hidden]; o [hidden, H value_dim]."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        from .attention import shared_position_encoding
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.D, self.V = int(p["num_heads"]), int(p["dim"]), int(p["value_dim"])
        if self.D > 256:
            raise ConfigError(f"retention: {self.D} key dims per head are not supported (up to 256)")
        decay = [float(x) for x in p["decay"]]
        if len(decay) != self.H:
            raise ConfigError(f"retention: {len(decay)} decays for {self.H} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=ctx.device)
        self.eps = float(p["norm_eps"])
        self.position = shared_position_encoding(p["position"], ctx) if p.get("position") is not None else None
        self.rot = self.position.rotary_dim if self.position is not None else 0
        if self.rot > self.D:
            raise ConfigError("retention: rotary_dim exceeds dim")
        self.ones = torch.ones(self.V, dtype=torch.float32, device=ctx.device)

    def weights(self):
        H, D, V, W = self.H, self.D, self.V, self.hidden
        return {"q": mat(H * D, W), "k": mat(H * D, W), "v": mat(H * V, W), "g": mat(H * V, W), "o": mat(W, H * V)}

    def load(self, t):
        names = ("q", "k", "v", "g")
        dt = matmul_dtype(*(t[n] for n in names), t["o"])
        self.w_in = torch.cat([t[n].to(dt) for n in names], 0).contiguous()      # one product gives q, k, v and the gate
        self.w_o = t["o"].to(dt)
        self.cos, self.sin = self.position.tables() if self.position is not None else (None, None)

    def input_dtypes(self):
        return (self.w_in.dtype,)

    def state_spec(self):
        return StateSpec((self.H * self.D * self.V,), torch.float32)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        ops, H, D, V = self.ops, self.H, self.D, self.V
        if state is None:
            raise ModelError("retention needs a state slab")
        xin = x[self.w_in.dtype]
        T, dev = xin.shape[0], xin.device
        f32 = dict(dtype=torch.float32, device=dev)
        proj = torch.empty((T, self.w_in.shape[0]), **f32)
        ops.gemm(xin, self.w_in, proj)
        qk = torch.empty((T, 2 * H * D), **f32)
        decay, dt = torch.empty((T, H), **f32), torch.empty((T, H), **f32)
        # the key's scale rides on the step size: S <- decay S + k (dt v)^T
        ops.retention_prepare(proj, step.pos, self.cos, self.sin, self.rot,
                              self.position.style if self.position is not None else "half", self.decay, D ** -0.5, qk, decay,
                              dt, H, D)
        o = torch.empty((T, H * V), **f32)
        ops.recurrence_scan(qk[:, :H * D], qk[:, H * D:], proj[:, 2 * H * D:2 * H * D + H * V], decay, False, None, dt, None,
                            step.slot, request_starts(step), len(step.entries), state, o, H, H, D, V)
        act = self.ctx.act_dtype if self.w_o.dtype == torch.bfloat16 else torch.float32
        out = torch.empty((T, H * V), dtype=act, device=dev)
        ops.gated_norm(o, proj[:, 2 * H * D + H * V:], "silu", False, self.ones, self.eps, H, out)
        return Pending(partials=ops.gemm_partials(out, self.w_o))


@MIXERS.register("ssd")
class StateSpaceDuality(_Recurrent):
    """params: hidden_size, num_heads, value_dim, state (N), groups, norm_groups, conv_taps, norm_eps.
    tensors: in [2 inner + 2 groups N + H, hidden] (inner = H value_dim; rows z | x | B | C | dt); conv
    [inner + 2 groups N, taps] with conv.b; dt_bias, A_log, D [H]; norm [inner]; o [hidden, inner]."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.V, self.N, self.G = int(p["num_heads"]), int(p["value_dim"]), int(p["state"]), int(p["groups"])
        self.norm_groups = int(p.get("norm_groups", 1))
        if self.H % self.G:
            raise ConfigError("ssd: num_heads must be a multiple of groups")
        if self.N > 256:
            raise ConfigError(f"ssd: a state of {self.N} per head and value dim is not supported (up to 256)")
        self.inner = self.H * self.V
        if self.inner % self.norm_groups:
            raise ConfigError("ssd: norm_groups must divide num_heads x value_dim")
        self.taps = int(p["conv_taps"])
        self.eps = float(p["norm_eps"])
        self.conv_ch = self.inner + 2 * self.G * self.N

    def weights(self):
        H, W = self.H, self.hidden
        return {"in": mat(2 * self.inner + 2 * self.G * self.N + H, W), "conv": conv_weight(self.conv_ch, self.taps),
                "conv.b": vec(self.conv_ch), "dt_bias": vec(H), "A_log": vec(H), "D": vec(H, init="gamma"),
                "norm": vec(self.inner, init="gamma"), "o": mat(W, self.inner)}

    def load(self, t):
        dt = matmul_dtype(t["in"], t["o"])
        self.w_in, self.w_o = t["in"].to(dt), t["o"].to(dt)
        self.w_conv, self.b_conv = t["conv"], t["conv.b"]
        self.dt_bias, self.a_log, self.skip, self.w_norm = t["dt_bias"], t["A_log"], t["D"], t["norm"]

    def input_dtypes(self):
        return (self.w_in.dtype,)

    def state_spec(self):
        return StateSpec((self.H * self.N * self.V + (self.taps - 1) * self.conv_ch,), torch.float32)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        ops, H, G, N, V, inner = self.ops, self.H, self.G, self.N, self.V, self.inner
        S, conv_state = self._split_state(state, H * N * V)
        xin = x[self.w_in.dtype]
        T, dev = xin.shape[0], xin.device
        f32 = dict(dtype=torch.float32, device=dev)
        proj = torch.empty((T, self.w_in.shape[0]), **f32)
        ops.gemm(xin, self.w_in, proj)
        C = self.conv_ch
        y = torch.empty((T, C), **f32)
        ops.short_conv(proj, inner, self.w_conv, self.b_conv, "silu", step.pos, step.slot, conv_state, y)
        dt = torch.empty((T, H), **f32)
        decay = torch.empty((T, H), **f32)
        ops.ssd_prepare(proj[:, inner + C:], self.dt_bias, self.a_log, dt, decay)
        o = torch.empty((T, inner), **f32)
        # C reads the state out, B writes x (times dt) into it
        ops.recurrence_scan(y[:, inner + G * N:], y[:, inner:inner + G * N], y[:, :inner], decay, False, None, dt, self.skip,
                            step.slot, request_starts(step), len(step.entries), S, o, H, G, N, V)
        act = self.ctx.act_dtype if self.w_o.dtype == torch.bfloat16 else torch.float32
        out = torch.empty((T, inner), dtype=act, device=dev)
        ops.gated_norm(o, proj[:, :inner], "silu", True, self.w_norm, self.eps, self.norm_groups, out)
        return Pending(partials=ops.gemm_partials(out, self.w_o))
