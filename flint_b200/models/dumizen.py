"""Dumizen as a ``ModelSpec``.

Every layer is a ``sandwich`` block, x <- x + n1b(mixer(n1(x))); x <- x + n2b(ff(n2(x))), with RMS norms before and
after each part.  The mixer is one of: grouped-query attention with biases, a norm of q and k per head, a partial
rotation with YaRN frequencies, and a sliding window behind which every whole block of positions is seen through its
mean key and value (``attention`` with ``pool``); two mixers side by side (``branches`` with ``combine: weighted``):
causal attention whose values are its keys as projected, with q and k normed over the whole projection, one added to
the softmax's denominator and a sigmoid gate on the heads' outputs, beside a retention (``retention``: linear attention
with a fixed decay per head, state in a slab of the cache manager); or causal attention without rotation whose weights
are sigmoids of capped scores less a logarithmic distance penalty, with a query temperature that grows with the
position (``attention`` with ``weights: sigmoid``).  The feed-forward is a mixture of ungated squared-ReLU experts
chosen by a sigmoid router with a correction, limited to the best groups, beside a shared expert
(``sigmoid_topk_moe`` with ``weighting: output``).  Layers ``loop.start .. loop.stop - 1`` run ``loop.times`` times
with the same weights (each run a call of the run order with a cache and state of its own); every pass opens with
x <- W_in [x; x0] + step[t] (``PassInput``).  The output head is the embedding table.  Checkpoints name tensors
``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1`` .. ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*`` and
``final.norm``.  The reference registers its families in one table keyed by the checkpoint's architecture string
(crates/thuban_architectures/src/loader.rs:39-60).
"""
from __future__ import annotations

from ..config.dumizen import DEFAULT_MAX_POSITIONS, DumizenConfig, PooledWindowAttention, SigmoidAttention
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec, PassInput
from ..registry import ARCHITECTURES

ATTENTION_NAMES = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"),
                   ("q_proj.bias", "q.b"), ("k_proj.bias", "k.b"), ("v_proj.bias", "v.b"), ("o_proj.bias", "o.b"),
                   ("q_norm.weight", "q.norm"), ("k_norm.weight", "k.norm"), ("gate_proj.weight", "g"))


def _position(rot):
    if rot is None:
        return None
    params = {"rotary_dim": rot.dims, "theta": rot.base, "style": "half", "max_positions": DEFAULT_MAX_POSITIONS}
    if rot.yarn is not None:
        params["yarn"] = dict(zip(("factor", "original", "fast", "slow"), rot.yarn))
    return PartSpec("rope", params)


def _heads(cfg, h):
    return {"hidden_size": cfg.width, "num_heads": h.heads, "num_kv_heads": h.kv_heads, "head_dim": h.dim,
            "value_dim": h.vdim, "scale": h.scale, "position": _position(h.rot), "qk_norm_eps": cfg.eps}


@ARCHITECTURES.register("Dumizen")
class DumizenArchitecture:
    config_class = DumizenConfig

    @staticmethod
    def parse_config(d: dict) -> DumizenConfig:
        return DumizenConfig.from_dict(d)

    @staticmethod
    def model_spec(cfg: DumizenConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps})
        layers, stored = [], {}
        for i, layer in enumerate(cfg.layers):
            m, pre = layer.mixer, f"l{i}."
            if isinstance(m, PooledWindowAttention):
                mixer = PartSpec("attention", {**_heads(cfg, m.h), "qkv_bias": True, "qk_norm": "head",
                                               "window": m.window, "pool": m.pool if m.window else 0})
                renames = [("mix.", ATTENTION_NAMES)]
            elif isinstance(m, SigmoidAttention):
                mixer = PartSpec("attention", {**_heads(cfg, m.h), "qkv_bias": True, "out_bias": True, "weights": "sigmoid",
                                               "softcap": m.softcap, "distance_bias": True, "weight_bias": True,
                                               "q_temp": m.q_temp})
                renames = [("mix.", ATTENTION_NAMES)]
            else:
                left = PartSpec("attention", {**_heads(cfg, m.left.h), "qk_norm": "whole", "values_from_keys": True,
                                              "unit_sink": True, "out_gate": True})
                r = m.right
                right = PartSpec("retention", {"hidden_size": cfg.width, "num_heads": r.heads, "dim": r.dim,
                                               "value_dim": r.vdim, "decay": r.decay, "norm_eps": cfg.eps,
                                               "position": _position(r.rot)})
                mixer = PartSpec("branches", {"hidden_size": cfg.width, "combine": "weighted",
                                              "scales": (m.left_scale, m.right_scale),
                                              "branches": (("left", left), ("right", right))})
                renames = [("mix.left.", ATTENTION_NAMES)]
            for sub, names in renames:
                for ours, theirs in names:
                    stored[f"{pre}{sub}{ours}"] = f"{pre}{sub}{theirs}"
            parts = {"norm1": norm, "mixer": mixer, "norm1b": norm}
            names = {"norm1": "norm1.", "norm1b": "norm1b.", "mixer": "mix.", "norm2": "norm2.", "norm2b": "norm2b.",
                     "ffn": "mlp."}
            for n in ("norm1", "norm1b"):
                stored[f"{pre}{n}.weight"] = f"{pre}{n}"
            f = layer.mlp
            if f is not None:
                parts.update({"norm2": norm, "norm2b": norm})
                for n in ("norm2", "norm2b"):
                    stored[f"{pre}{n}.weight"] = f"{pre}{n}"
                parts["ffn"] = PartSpec("sigmoid_topk_moe", {
                    "hidden_size": cfg.width, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
                    "shared_intermediate_size": f.shared_ff, "act": "relu2", "weighting": "output", "groups": f.groups,
                    "keep_groups": f.keep, "correction": True, "normalize": True, "router_scale": f.scale,
                    "shared_gate": False})
            layers.append(LayerSpec("sandwich", parts, pre, names))
        n = len(cfg.layers)
        order, passes = [], []
        if cfg.loop is None:
            order = [LayerCall(i) for i in range(n)]
        else:
            lp = cfg.loop
            order = [LayerCall(i) for i in range(lp.start)]
            for t in range(lp.times):
                passes.append(PassInput(call=len(order), row=t))
                order += [LayerCall(i) for i in range(lp.start, lp.stop)]
            order += [LayerCall(i) for i in range(lp.stop, n)]
        stored.update({"embed.weight": "embed", "final.norm.weight": "final.norm"})
        return ModelSpec(
            architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
            max_positions=DEFAULT_MAX_POSITIONS, layers=tuple(layers), order=tuple(order), final_norm=norm,
            embed_name="embed.", final_norm_name="final.norm.", tie_word_embeddings=True, stored_names=stored,
            pass_inputs=tuple(passes), pass_input_name="loop.")
