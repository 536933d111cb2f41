"""Norm parts: LayerNorm (with or without bias) and RMSNorm.

LayerNorm: y = (x - mean) * rsqrt(var + eps) * gamma + beta with var = mean((x-mean)^2);
RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gamma; with ``weight_offset`` c the stored scale w is an offset,
gamma = c + w (formed once, in float32, when the tensors are loaded).  Statistics are float32.  With
``branch_scale`` the norm also stores a scale s per channel for what a block adds before it, and ``post`` runs the
norm after the sum: x <- norm(a x + s * branch) with a = ``residual_scale``, in place.  The
reference's norm shader has both as modes (crates/thuban_kernel/wgsl/norm.wgsl:66-83,
112-121) and picks by config key (crates/thuban_architectures/src/phi.rs:55-63).
"""
from __future__ import annotations

import torch

from ..registry import NORMS
from .base import Norm, vec


class _RowNorm(Norm):
    mode = "layer"
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.has_bias = bool(params.get("bias", False))
        # a scale stored as an offset: the row is multiplied by weight_offset + w (0: by w itself)
        self.weight_offset = float(params.get("weight_offset", 0.0))
        # for a block that norms after the sum: the residual's weight, and whether a scale of the branch is stored
        self.residual_scale = float(params.get("residual_scale", 1.0))
        self.has_branch_scale = bool(params.get("branch_scale", False))
        self.gamma = self.beta = self.branch_scale = None

    def weights(self):
        w = {"weight": vec(self.width, init="normal" if self.weight_offset else "gamma")}
        if self.has_bias:
            w["bias"] = vec(self.width)
        if self.has_branch_scale:
            w["branch_scale"] = vec(self.width, init="gamma")
        return w

    def load(self, tensors):
        self.gamma = tensors["weight"]
        if self.weight_offset:
            self.gamma = (self.gamma.to(torch.float32) + self.weight_offset).contiguous()
        self.beta = tensors.get("bias")
        self.branch_scale = tensors.get("branch_scale")

    supports_pending = True
    supports_router = True

    def post(self, x, branch, copy=None):
        """x <- norm(residual_scale x + branch_scale * branch) in place; ``branch``: a ``Pending`` of partial sums
        (and a bias).  ``copy``: a tensor of another element type that receives the result too."""
        self.ops.post_norm(x, branch.partials, branch.bias, self.branch_scale, self.residual_scale, self.gamma, self.beta,
                           self.eps, self.mode, out_copy=copy)

    def forward(self, x, want, row_index=None, pending=None, router=None, out=None):
        """``out``: {element type: tensor} to write into instead of new tensors (then ``want`` is ignored)."""
        rows = row_index.numel() if row_index is not None else x.shape[0]
        if out is None:
            out = {}
            for dt in set(want):
                out[dt] = torch.empty((rows, self.width), dtype=dt, device=x.device)
        self.ops.row_norm(x, self.gamma, self.beta, self.eps, self.mode, out_f32=out.get(torch.float32),
                          out_bf16=out.get(torch.bfloat16), row_index=row_index, pending=pending, router=router)
        return out


@NORMS.register("layernorm")
class LayerNorm(_RowNorm):
    mode = "layer"


@NORMS.register("rmsnorm")
class RMSNorm(_RowNorm):
    mode = "rms"

    def __init__(self, params, ctx):
        super().__init__({**params, "bias": False}, ctx)
