"""Feed-forward parts: a dense gated MLP, a top-2 sparsemixer mixture of experts, and a mixture whose softmax
router chooses the top k experts among the best groups of neighbouring experts.

Dense: h += (act(x Wg^T) * (x Wu^T)) Wd^T, as the reference's feed-forward
(crates/thuban_model/src/ops/mlp.rs:24-79).  Mixture of experts (no counterpart in
the reference): float32 router logits, sparsemixer top-2 selection, rows sorted by
expert, two grouped products, and the gated sum of the two experts' outputs added to
the residual stream in a fixed order.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..registry import FEED_FORWARDS
from .base import FeedForward, Pending, RouterRequest, mat, matmul_dtype, vec


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """params: hidden_size, intermediate_size, act; tensors gate_proj/up_proj [I,H], down_proj [H,I].
    act ``silu`` or ``gelu_pytorch_tanh``: act(gate) * up.  act ``swish_clamped`` with ``act_slope`` s and
    ``act_limit`` c: g = min(gate, c), u = clamp(up, -c, c), g sigmoid(s g) (u + 1)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.act = params.get("act", "silu")
        self.act_params = None
        if self.act == "swish_clamped":
            self.act_params = (float(params["act_slope"]), float(params["act_limit"]))
            if self.act_params[1] <= 0:
                raise ConfigError(f"gated_mlp: act_limit must be positive, got {self.act_params[1]}")
        elif self.act not in ("silu", "gelu_pytorch_tanh"):
            raise ConfigError(f"gated_mlp: unknown activation {self.act!r}")

    def weights(self):
        return {"gate_proj.weight": mat(self.inter, self.hidden), "up_proj.weight": mat(self.inter, self.hidden),
                "down_proj.weight": mat(self.hidden, self.inter)}

    def fused(self):
        return {"gate_up_proj.weight": ["gate_proj.weight", "up_proj.weight"]}

    def load(self, t):
        dt = matmul_dtype(*t.values())
        # gate and up rows in the layout the kernels want: one product gives both
        self.w_gate_up = self.ops.pair_gate_up(t["gate_proj.weight"].to(dt), t["up_proj.weight"].to(dt)).contiguous()
        self.w_down = t["down_proj.weight"].to(dt)

    def input_dtypes(self):
        return (self.w_gate_up.dtype,)

    def forward(self, x, residual, step):
        xin = x[self.w_gate_up.dtype]
        a = torch.empty((xin.shape[0], self.inter), dtype=self.w_gate_up.dtype, device=xin.device)
        if self.act_params is None:
            self.ops.gated_gemm(xin, self.w_gate_up, a, self.act)
        else:
            self.ops.gated_gemm(xin, self.w_gate_up, a, self.act, act_params=self.act_params)
        self.ops.gemm(a, self.w_down, residual, accumulate=True)


@FEED_FORWARDS.register("mlp")
class PlainMLP(FeedForward):
    """An ungated unit: act(x Wu^T) Wd^T.  params: hidden_size, intermediate_size, act (``relu2``: the square of
    max(z, 0); ``gelu``, ``gelu_pytorch_tanh``, ``silu``); tensors up_proj [I,H], down_proj [H,I].  The down
    product is left as partial sums for whoever applies it."""

    graph_safe = True
    returns_pending = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.act = params.get("act", "gelu")
        if self.act not in ("relu2", "gelu", "gelu_pytorch_tanh", "silu"):
            raise ConfigError(f"mlp: unknown activation {self.act!r}")

    def weights(self):
        return {"up_proj.weight": mat(self.inter, self.hidden), "down_proj.weight": mat(self.hidden, self.inter)}

    def load(self, t):
        dt = matmul_dtype(*t.values())
        self.w_up, self.w_down = t["up_proj.weight"].to(dt), t["down_proj.weight"].to(dt)

    def input_dtypes(self):
        return (self.w_up.dtype,)

    def forward(self, x, residual, step):
        xin = x[self.w_up.dtype]
        a = torch.empty((xin.shape[0], self.inter), dtype=self.w_up.dtype, device=xin.device)
        self.ops.row_act(self.ops.gemm_partials(xin, self.w_up), a, self.act)
        return Pending(partials=self.ops.gemm_partials(a, self.w_down))


@FEED_FORWARDS.register("sparsemixer_moe")
class SparseMixerMoE(FeedForward):
    """params: hidden_size, intermediate_size, num_experts, jitter_eps, act.
    tensors: gate.weight [E,H]; experts.{e}.w1 / w3 [I,H] (gate / up), w2 [H,I] (down)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.E = int(params["num_experts"])
        if not 2 <= self.E <= 256:
            raise ConfigError(f"num_experts {self.E} is not supported (2..256)")
        self.eps = float(params["jitter_eps"])
        self.act = params.get("act", "silu")

    def weights(self):
        w = {"gate.weight": mat(self.E, self.hidden)}
        for e in range(self.E):
            w[f"experts.{e}.w1.weight"] = mat(self.inter, self.hidden)
            w[f"experts.{e}.w2.weight"] = mat(self.hidden, self.inter)
            w[f"experts.{e}.w3.weight"] = mat(self.inter, self.hidden)
        return w

    def load(self, t):
        self.w_router = t["gate.weight"]
        dt = matmul_dtype(*(t[k] for k in t if k.startswith("experts.")))
        # per expert the gate rows (w1) and the up rows (w3) in the layout the kernels want: [E, rows, H]
        self.w13 = torch.stack([self.ops.pair_gate_up(t[f"experts.{e}.w1.weight"].to(dt), t[f"experts.{e}.w3.weight"].to(dt))
                                for e in range(self.E)], 0).contiguous()
        self.w2 = torch.stack([t[f"experts.{e}.w2.weight"].to(dt) for e in range(self.E)], 0).contiguous()

    def input_dtypes(self):
        return (torch.float32, self.w13.dtype)

    def router_request(self, n_rows):
        """Routing can ride on the norm before this part (the normalised row is in registers there)."""
        dev = self.w_router.device
        return RouterRequest(self.w_router, self.eps, torch.empty((n_rows, 2), dtype=torch.int32, device=dev),
                             torch.empty((n_rows, 2), dtype=torch.float32, device=dev))

    def input_dtypes_when_routed(self):
        return (self.w13.dtype,)

    def forward(self, x, residual, step, routed=None):
        ops = self.ops
        xa = x[self.w13.dtype]
        T = xa.shape[0]
        dev = xa.device
        if routed is not None:
            ids, gates, logits = routed.expert_ids, routed.gates, routed.logits
        else:
            ids = torch.empty((T, 2), dtype=torch.int32, device=dev)
            gates = torch.empty((T, 2), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_sparsemixer(x[torch.float32], self.w_router, self.eps, ids, gates, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w13.dtype), xa)
        a = torch.empty((2 * T, self.inter), dtype=self.w13.dtype, device=dev)
        ops.gated_gemm(xs, self.w13, a, self.act, plan)
        y = torch.empty((2 * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w2, y, plan, plan_ready=True)     # the gate/up product ran over the same plan
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(gates)
            if logits is not None:
                step.record.setdefault("router_logits", []).append(logits)
        # the gated sum of the two experts' rows is added by the next norm's kernel
        return Pending(y=y, row_of=plan.row_of, gates=gates)


@FEED_FORWARDS.register("grouped_topk_moe")
class GroupedTopKMoE(FeedForward):
    """A mixture of gated experts with a softmax router: scores s = softmax(W_router x) in float32; the experts
    form ``groups`` equal groups of neighbours, a group scores as its best member, only members of the
    ``keep_groups`` best groups may be chosen, and the ``top`` best of those are; an expert's weight is its score
    over the sum of the chosen scores (+ 1e-20), times ``router_scale``.  The output is the weighted sum of the
    chosen experts' down(act(gate x) * (up x)).  (No counterpart in the reference, whose feed-forward is dense:
    crates/thuban_model/src/ops/mlp.rs:24-79.)

    params: hidden_size, intermediate_size, num_experts, top, groups, keep_groups, router_scale, act.
    tensors: router [E, H]; e{i}.gate / e{i}.up [I, H], e{i}.down [H, I]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.E, self.top = int(p["num_experts"]), int(p["top"])
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep_groups", 1))
        self.router_scale = float(p.get("router_scale", 1.0))
        self.act = p.get("act", "silu")
        if not 1 <= self.E <= 256:
            raise ConfigError(f"num_experts {self.E} is not supported (1..256)")
        if not 1 <= self.top <= min(self.E, 16):
            raise ConfigError(f"{self.top} experts a token of {self.E} is not supported (1..16)")
        if self.groups < 1 or self.groups > 64 or self.E % self.groups:
            raise ConfigError(f"{self.E} experts do not form {self.groups} equal groups (up to 64)")
        if not 1 <= self.keep <= self.groups or self.keep * (self.E // self.groups) < self.top:
            raise ConfigError(f"{self.keep} of {self.groups} groups cannot give {self.top} experts a token")

    def weights(self):
        w = {"router": mat(self.E, self.hidden)}
        for e in range(self.E):
            w[f"e{e}.gate"] = mat(self.inter, self.hidden)
            w[f"e{e}.up"] = mat(self.inter, self.hidden)
            w[f"e{e}.down"] = mat(self.hidden, self.inter)
        return w

    def load(self, t):
        self.w_router = t["router"]
        dt = matmul_dtype(*(v for k, v in t.items() if k != "router"))
        self.w13 = torch.stack([self.ops.pair_gate_up(t[f"e{e}.gate"].to(dt), t[f"e{e}.up"].to(dt))
                                for e in range(self.E)], 0).contiguous()
        self.w2 = torch.stack([t[f"e{e}.down"].to(dt) for e in range(self.E)], 0).contiguous()

    def input_dtypes(self):
        return (torch.float32, self.w13.dtype)       # the router reads the float32 rows

    def router_request(self, n_rows):
        """Routing can ride on the norm before this part (the normalised row is in registers there)."""
        dev = self.w_router.device
        return RouterRequest(self.w_router, 0.0, torch.empty((n_rows, self.top), dtype=torch.int32, device=dev),
                             torch.empty((n_rows, self.top), dtype=torch.float32, device=dev), top=self.top,
                             groups=self.groups, keep=self.keep, scale=self.router_scale)

    def input_dtypes_when_routed(self):
        return (self.w13.dtype,)

    def forward(self, x, residual, step, routed=None):
        ops = self.ops
        xa = x[self.w13.dtype]
        T, dev, k = xa.shape[0], xa.device, self.top
        if routed is not None:
            ids, gates, logits = routed.expert_ids, routed.gates, routed.logits
        else:
            ids = torch.empty((T, k), dtype=torch.int32, device=dev)
            gates = torch.empty((T, k), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_topk(x[torch.float32], self.w_router, k, self.groups, self.keep, self.router_scale, ids, gates, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w13.dtype, k), xa)
        a = torch.empty((k * T, self.inter), dtype=self.w13.dtype, device=dev)
        ops.gated_gemm(xs, self.w13, a, self.act, plan)
        y = torch.empty((k * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w2, y, plan, plan_ready=True)
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(gates)
            if logits is not None:
                step.record.setdefault("router_logits", []).append(logits)
        # the weighted sum of the chosen experts' rows is added by the next norm's kernel
        return Pending(y=y, row_of=plan.row_of, gates=gates)


@FEED_FORWARDS.register("sigmoid_topk_moe")
class SigmoidTopKMoE(FeedForward):
    """A mixture of small ungated experts, expert(x) = W_down act(W_up x), with a sigmoid router: scores
    s = sigmoid(W_router x) in float32; the ``top`` experts with the largest scores are chosen (the lower index
    among equals) and their scores are used as they are.  A score scales the expert's INPUT: the output is
    sum_e expert_e(s_e x).  Since W_up is linear, act(W_up (s x)) = act(s (W_up x)): the score is applied to the
    up product's float32 sums, before the activation.  An optional shared expert of the same form runs on every
    token and is weighted by sigmoid(w_sg . x), one number a token; it rides along as one more row per token of
    the experts' pending rows.  (No counterpart in the reference, whose feed-forward is dense:
    crates/thuban_model/src/ops/mlp.rs:24-79.)

    With ``weighting: "output"`` the chosen experts' OUTPUTS are weighted instead, and the choice may follow the
    grouped rule: choice scores s + ``correction`` (a stored offset per expert); the experts form ``groups`` equal
    groups of neighbours, a group scores as the sum of its two largest choice scores, only members of the
    ``keep_groups`` best groups can be chosen, the ``top`` largest choice scores among them are; the weights are the
    chosen experts' s, over their sum (+ 1e-20) if ``normalize``, times ``router_scale``.  ``shared_gate: False``: the
    shared expert is added as it is (no gate tensor).

    params: hidden_size, intermediate_size, num_experts, top, shared_intermediate_size (0: none), act ("gelu",
    the erf form, or "gelu_pytorch_tanh", "silu", "relu2"); weighting ("input", the default, or "output"), groups,
    keep_groups, correction, normalize, router_scale, shared_gate (default true).
    tensors: router [E, H]; e{i}.up [I, H], e{i}.down [H, I]; shared.up [Is, H], shared.down [H, Is], shared.sg [1, H];
    correction [E]."""

    graph_safe = True
    returns_pending = True        # the rows given are never touched: what the experts add goes back as a Pending

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.E, self.top = int(p["num_experts"]), int(p["top"])
        self.shared = int(p.get("shared_intermediate_size", 0) or 0)
        self.act = p.get("act", "gelu")
        if not 1 <= self.E <= 256:
            raise ConfigError(f"num_experts {self.E} is not supported (1..256)")
        if not 1 <= self.top <= min(self.E, 16):
            raise ConfigError(f"{self.top} experts a token of {self.E} is not supported (1..16)")
        self.weighting = p.get("weighting", "input")
        if self.weighting not in ("input", "output"):
            raise ConfigError(f"sigmoid_topk_moe: weighting must be 'input' or 'output', got {self.weighting!r}")
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep_groups", 1))
        self.correction = bool(p.get("correction", False))
        self.normalize = bool(p.get("normalize", False))
        self.router_scale = float(p.get("router_scale", 1.0))
        self.shared_gate = bool(p.get("shared_gate", True))
        if self.weighting == "input" and (self.groups > 1 or self.correction or self.normalize or self.router_scale != 1.0
                                          or not self.shared_gate):
            raise ConfigError("sigmoid_topk_moe: groups, a correction, normalised or scaled weights and an ungated shared "
                              "expert go with weighting 'output'")
        if self.groups < 1 or self.groups > 64 or self.E % self.groups:
            raise ConfigError(f"{self.E} experts do not form {self.groups} equal groups (up to 64)")
        if not 1 <= self.keep <= self.groups or self.keep * (self.E // self.groups) < self.top:
            raise ConfigError(f"{self.keep} of {self.groups} groups cannot give {self.top} experts a token")
        if self.act not in ("gelu", "gelu_pytorch_tanh", "silu", "relu2"):
            raise ConfigError(f"sigmoid_topk_moe: unknown activation {self.act!r}")
        if self.weighting == "input" and self.act == "relu2":
            raise ConfigError("sigmoid_topk_moe: act 'relu2' goes with weighting 'output'")

    def weights(self):
        w = {"router": mat(self.E, self.hidden)}
        for e in range(self.E):
            w[f"e{e}.up"] = mat(self.inter, self.hidden)
            w[f"e{e}.down"] = mat(self.hidden, self.inter)
        if self.shared:
            w.update({"shared.up": mat(self.shared, self.hidden), "shared.down": mat(self.hidden, self.shared)})
            if self.shared_gate:
                w["shared.sg"] = mat(1, self.hidden)
        if self.correction:
            w["correction"] = vec(self.E)
        return w

    def load(self, t):
        # the shared expert's gate is one more row of the router's matrix: its logit comes with the experts'
        self.w_router = torch.cat([t["router"], t["shared.sg"].to(t["router"].dtype)], 0).contiguous() \
            if self.shared and self.shared_gate else t["router"]
        self.w_correction = t.get("correction")
        dt = matmul_dtype(*(v for k, v in t.items() if k not in ("router", "shared.sg", "correction")))
        self.w_up = torch.stack([t[f"e{e}.up"].to(dt) for e in range(self.E)], 0).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down"].to(dt) for e in range(self.E)], 0).contiguous()
        if self.shared:
            self.w_sup, self.w_sdown = t["shared.up"].to(dt), t["shared.down"].to(dt)

    def input_dtypes(self):
        return (torch.float32, self.w_up.dtype)       # the router reads the float32 rows

    def router_request(self, n_rows):
        """Routing can ride on the norm before this part (the normalised row is in registers there)."""
        if self.weighting == "output":
            dev, k = self.w_router.device, self.top
            return RouterRequest(self.w_router, 0.0, torch.empty((n_rows, k), dtype=torch.int32, device=dev),
                                 torch.empty((n_rows, k), dtype=torch.float32, device=dev), top=k, groups=self.groups,
                                 keep=self.keep, scale=self.router_scale, rule="sigmoid_grouped",
                                 correction=self.w_correction, normalize=self.normalize)
        dev, k, extra = self.w_router.device, self.top, 1 if self.shared else 0
        return RouterRequest(self.w_router, 0.0, torch.empty((n_rows, k), dtype=torch.int32, device=dev),
                             torch.empty((n_rows, k), dtype=torch.float32, device=dev), top=k, rule="sigmoid", extra=extra,
                             weights=torch.empty((n_rows, k + extra), dtype=torch.float32, device=dev))

    def input_dtypes_when_routed(self):
        return (self.w_up.dtype,)

    def forward(self, x, residual, step, routed=None):
        ops = self.ops
        xa = x[self.w_up.dtype]
        T, dev, k, extra = xa.shape[0], xa.device, self.top, 1 if self.shared else 0
        if self.weighting == "output":
            return self._forward_output_weighted(x, xa, step, routed)
        if routed is not None:
            # what the pending rows are weighted by when they are added: 1 for the experts (their score went into
            # their input), the sigmoid gate for the shared expert
            ids, scores, weights, logits = routed.expert_ids, routed.gates, routed.weights, routed.logits
        else:
            ids = torch.empty((T, k), dtype=torch.int32, device=dev)
            scores = torch.empty((T, k), dtype=torch.float32, device=dev)
            weights = torch.empty((T, k + extra), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E + extra), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_sigmoid(x[torch.float32], self.w_router, self.E, k, ids, scores, weights, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w_up.dtype, k), xa)
        a = torch.empty((k * T, self.inter), dtype=self.w_up.dtype, device=dev)
        ops.row_act(ops.gemm_partials(xs, self.w_up, plan=plan), a, self.act, row_of=plan.row_of, row_scale=scores)
        y = torch.empty(((k + extra) * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w_down, y[:k * T], plan, plan_ready=True)
        row_of = plan.row_of
        if self.shared:
            b = torch.empty((T, self.shared), dtype=self.w_up.dtype, device=dev)
            ops.row_act(ops.gemm_partials(xa, self.w_sup), b, self.act)
            ops.gemm(b, self.w_sdown, y[k * T:])
            own = torch.arange(k * T, (k + 1) * T, dtype=torch.int32, device=dev)
            row_of = torch.cat([row_of, own[:, None]], 1)
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(scores)
            step.record.setdefault("router_logits", []).append(logits)
        return Pending(y=y, row_of=row_of, gates=weights)

    def _forward_output_weighted(self, x, xa, step, routed=None):
        """The chosen experts' outputs as rows with their weights, and the shared expert's output as the partial sums
        of its down product: whoever adds them (the kernel after the part) adds both."""
        ops = self.ops
        T, dev, k, extra = xa.shape[0], xa.device, self.top, 1 if self.shared else 0
        if routed is not None:          # the norm before this part chose while it had the row
            ids, gates, logits = routed.expert_ids, routed.gates, routed.logits
        else:
            ids = torch.empty((T, k), dtype=torch.int32, device=dev)
            gates = torch.empty((T, k), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_sigmoid_grouped(x[torch.float32], self.w_router, self.w_correction, k, self.groups, self.keep,
                                       self.normalize, self.router_scale, ids, gates, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w_up.dtype, k), xa)
        a = torch.empty((k * T, self.inter), dtype=self.w_up.dtype, device=dev)
        ops.row_act(ops.gemm_partials(xs, self.w_up, plan=plan), a, self.act)
        y = torch.empty((k * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w_down, y, plan, plan_ready=True)
        shared = None
        if self.shared:          # added as it is: its down product travels as partial sums beside the experts' rows
            b = torch.empty((T, self.shared), dtype=self.w_up.dtype, device=dev)
            ops.row_act(ops.gemm_partials(xa, self.w_sup), b, self.act)
            shared = ops.gemm_partials(b, self.w_sdown)
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(gates)
            step.record.setdefault("router_logits", []).append(logits)
        return Pending(partials=shared, y=y, row_of=plan.row_of, gates=gates)
