"""Tefovik as a ``ModelSpec``.

The embedded rows pass a LayerNorm.  Every layer is a ``postnorm`` block: x <- norm1(alpha x + s1 * mixer(x)), then
x <- norm2(alpha x + s2 * ff(x)) (LayerNorms with a scale and no bias; s1, s2 learned per channel; the second half is
absent in a layer without a feed-forward).  What a layer hands on is a learned weighted sum of the embedded rows
and the results of all layers so far (``depth_mix``).  A ``parallel`` layer's mixer is the mean of two branches, each
RMS-normed over the width (``branches``): grouped-query attention whose q, k and v pass a short causal convolution,
with a per-head RMS norm of q and k, a partial interleaved rotation, values rotated by their own position and the
heads' sums rotated back by the query's, a mask that cuts the sequence into runs of a fixed length, and a sigmoid
gate per head (``attention`` with these options); and a gated delta rule with a decay per key channel
(``gated_delta``).  A ``mamba2`` layer's mixer is a state-space model with a scalar decay per head (``ssd``).  The
feed-forward is an ungated unit with a squared ReLU (``mlp``).  The logits are capped by a tanh.  Checkpoints name
tensors ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.ls1``, ``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm`` and ``head``.  The reference registers its families in one table keyed by the checkpoint's
architecture string (crates/thuban_architectures/src/loader.rs:39-60).
"""
from __future__ import annotations

from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.tefovik import DEFAULT_MAX_POSITIONS, TefovikConfig
from ..registry import ARCHITECTURES

UNIT_NORM_EPS = 1e-6      # the design fixes the constant under the root of the delta rule's unit norms


@ARCHITECTURES.register("Tefovik")
class TefovikArchitecture:
    config_class = TefovikConfig

    @staticmethod
    def parse_config(d: dict) -> TefovikConfig:
        return TefovikConfig.from_dict(d)

    @staticmethod
    def model_spec(cfg: TefovikConfig) -> ModelSpec:
        W = cfg.width
        plain_norm = PartSpec("layernorm", {"width": W, "eps": cfg.eps})
        post_norm = PartSpec("layernorm", {"width": W, "eps": cfg.eps, "branch_scale": True, "residual_scale": cfg.alpha})
        layers, order, stored = [], [], {}
        for i, layer in enumerate(cfg.layers):
            pre = f"l{i}."
            if layer.type == "parallel":
                a, d = layer.mixer
                position = PartSpec("rope", {"rotary_dim": a.rot_dims, "theta": a.rot_base, "style": "interleaved",
                                             "max_positions": DEFAULT_MAX_POSITIONS}) if a.rot_dims else None
                value_position = PartSpec("rope", {"rotary_dim": a.vdim, "theta": a.rot_base, "style": "interleaved",
                                                   "max_positions": DEFAULT_MAX_POSITIONS})
                left = PartSpec("attention", {
                    "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                    "value_dim": a.vdim, "scale": a.scale, "position": position, "conv_taps": a.taps, "qk_norm": True,
                    "qk_norm_eps": cfg.eps, "chunk": a.chunk, "value_position": value_position, "head_gate": True})
                right = PartSpec("gated_delta", {
                    "hidden_size": W, "num_heads": d.heads, "num_kv_heads": d.kv_heads, "dim": d.dim, "value_dim": d.vdim,
                    "conv_taps": d.taps, "unit_eps": UNIT_NORM_EPS, "norm_eps": cfg.eps})
                mixer = PartSpec("branches", {"hidden_size": W, "eps": cfg.eps,
                                              "branches": (("left", left), ("right", right))})
                for ours, theirs in (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"),
                                     ("o_proj.weight", "o"), ("q_conv.weight", "q.conv"), ("k_conv.weight", "k.conv"),
                                     ("v_conv.weight", "v.conv"), ("q_norm.weight", "q.norm"), ("k_norm.weight", "k.norm"),
                                     ("gate_proj.weight", "g")):
                    stored[f"{pre}mix.left.{ours}"] = f"{pre}mix.left.{theirs}"
            else:
                s = layer.mixer
                mixer = PartSpec("ssd", {"hidden_size": W, "num_heads": s.heads, "value_dim": s.vdim, "state": s.state,
                                         "groups": s.groups, "norm_groups": s.norm_groups, "conv_taps": s.taps,
                                         "norm_eps": cfg.eps})
            parts = {"norm1": post_norm, "mixer": mixer}
            names = {"norm1": "norm1.", "mixer": "mix.", "norm2": "norm2.", "ffn": "mlp."}
            stored[f"{pre}norm1.weight"] = f"{pre}norm1"
            stored[f"{pre}norm1.branch_scale"] = f"{pre}ls1"
            if layer.mlp is not None:
                parts["norm2"] = post_norm
                stored[f"{pre}norm2.weight"] = f"{pre}norm2"
                stored[f"{pre}norm2.branch_scale"] = f"{pre}ls2"
                parts["ffn"] = PartSpec("mlp", {"hidden_size": W, "intermediate_size": layer.mlp.ff, "act": "relu2"})
                stored[f"{pre}mlp.up_proj.weight"] = f"{pre}mlp.up"
                stored[f"{pre}mlp.down_proj.weight"] = f"{pre}mlp.down"
            layers.append(LayerSpec("postnorm", parts, pre, names))
            order.append(LayerCall(i))
        stored.update({"embed.weight": "embed", "embed.norm.weight": "embed.norm", "final.norm.weight": "final.norm",
                       "head.weight": "head"})
        return ModelSpec(
            architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, max_positions=DEFAULT_MAX_POSITIONS,
            layers=tuple(layers), order=tuple(order), final_norm=plain_norm, embed_name="embed.",
            final_norm_name="final.norm.", head_name="head.", embed_norm=plain_norm, embed_norm_name="embed.norm.",
            depth_mix=True, logit_softcap=cfg.softcap, stored_names=stored)
