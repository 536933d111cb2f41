"""The generic model: parts built from a ``ModelSpec``, tensors loaded by name, and the
step function.

``Model.step(entries)`` runs exactly the tokens it is given, as one batch, against the
cache that earlier steps left, and returns float32 logits ``[wanted, vocab]`` for the
wanted places, in the order of the entries and of each entry's ``want``.  It is the
counterpart of the reference's ``LanguageModel::forward``
(crates/thuban_model/src/traits.rs:29-46,
crates/thuban_architectures/src/transformer/forward.rs:51-508), with two differences:
positions come with the batch, and the wanted rows are gathered *before* the final
norm and the output head, so that the head runs on the wanted rows only.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..cache.manager import CacheManager
from ..config.spec import ModelSpec
from ..errors import ConfigError, ModelError
from ..parts.base import BuildContext, matmul_dtype
from ..parts.block import run_norm
from ..registry import ARCHITECTURES, BLOCKS, EMBED_ADDITIONS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from ..weights.loader import load_tensors
from ..weights.sources import RenamedSource, SafetensorsSource, WeightSpec
from .step import StepEntry, StepStaging

def registry_for_role(role: str):
    if role.startswith("norm"):
        return NORMS
    if role.startswith("mixer"):
        return MIXERS
    if role.startswith("ffn"):
        return FEED_FORWARDS
    raise ConfigError(f"no part registry for role {role!r}")


class Layer:
    def __init__(self, spec, ctx):
        self.spec = spec
        self.ctx = ctx
        self.parts = {role: registry_for_role(role).get(ps.kind)(ps.params, ctx) for role, ps in spec.parts.items()}
        self.block = BLOCKS.get(spec.block)(self.parts)
        missing = [r for r in self.block.roles if r not in self.parts]
        if missing:
            raise ConfigError(f"block {spec.block!r} needs parts {missing}")

    def weights(self):
        out = {}
        for role, part in self.parts.items():
            for name, ws in part.weights().items():
                out[self.spec.prefix + self.spec.names[role] + name] = ws
        return out

    def fused(self):
        out = {}
        for role, part in self.parts.items():
            pre = self.spec.prefix + self.spec.names[role]
            for name, pieces in part.fused().items():
                out[pre + name] = [pre + p for p in pieces]
        return out

    def load(self, tensors):
        for role, part in self.parts.items():
            pre = self.spec.prefix + self.spec.names[role]
            part.load({name: tensors[pre + name] for name in part.weights() if pre + name in tensors})


def build_embed_additions(spec: ModelSpec, ctx) -> list:
    """[(part, tensor-name prefix)] for ``spec.embed_additions``."""
    return [(EMBED_ADDITIONS.get(ps.kind)(ps.params, ctx), prefix) for ps, prefix in spec.embed_additions]


def embed_norm_of(spec: ModelSpec, ctx):
    """The norm of the embedded rows that ``spec`` names, or None."""
    return NORMS.get(spec.embed_norm.kind)(spec.embed_norm.params, ctx) if spec.embed_norm is not None else None


def depth_mix_names(spec: ModelSpec) -> list:
    """The tensor of every call of the run order that holds its weights over the rows so far ([] without depth mix)."""
    if not spec.depth_mix:
        return []
    return [spec.layers[call.layer].prefix + spec.depth_mix_name for call in spec.order]


def expected_tensors(spec: ModelSpec, layers, final_norm, embed_position=None, embed_additions=()) -> dict:
    """Every tensor name the model reads, with its shape and role."""
    exp = {spec.embed_name + "weight": WeightSpec((spec.vocab_size, spec.hidden_size))}
    if spec.embed_norm is not None:
        ctx = layers[0].ctx if layers else None
        for name, ws in embed_norm_of(spec, ctx).weights().items():
            exp[spec.embed_norm_name + name] = ws
    names = depth_mix_names(spec)
    if len(set(names)) != len(names):
        raise ConfigError("depth mix: a layer that is called twice cannot store one set of weights per call")
    for i, name in enumerate(names):
        exp[name] = WeightSpec((i + 2,), role="vector", init="gamma")
    if spec.pass_inputs:
        exp[spec.pass_input_name + "in"] = WeightSpec((spec.hidden_size, 2 * spec.hidden_size))
        exp[spec.pass_input_name + "step"] = WeightSpec((max(p.row for p in spec.pass_inputs) + 1, spec.hidden_size),
                                                        role="vector")
    if embed_position is not None:
        for name, ws in embed_position.weights().items():
            exp[spec.embed_position_name + name] = ws
    for part, prefix in embed_additions:
        for name, ws in part.weights().items():
            exp[prefix + name] = ws
    for layer in layers:
        exp.update(layer.weights())
    for name, ws in final_norm.weights().items():
        exp[spec.final_norm_name + name] = ws
    if not spec.tie_word_embeddings:
        exp[spec.head_name + "weight"] = WeightSpec((spec.vocab_size, spec.hidden_size))
    if spec.head_bias:
        exp[spec.head_name + "bias"] = WeightSpec((spec.vocab_size,), role="vector")
    return exp


def fused_tensors(layers) -> dict:
    """Fused tensor name -> the expected tensors a checkpoint may store stacked in it."""
    out = {}
    for layer in layers:
        out.update(layer.fused())
    return out


class Model:
    """Parts + tensors + cache + step function for one model on one device."""

    def __init__(self, spec: ModelSpec, source, *, dtype="bfloat16", device="cuda:0", ops=None,
                 page_size=64, n_pages=None, max_slots=8, max_context=None, max_step_tokens=8192,
                 use_graphs=True):
        if dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}")
        self.spec = spec
        self.compute = dtype
        self.device = torch.device(device)
        if ops is None:
            from ..csrc.ops import get_ops
            ops = get_ops(self.device)
        self.ops = ops
        self.max_context = int(max_context or spec.max_positions)
        if self.max_context > spec.max_positions:
            raise ConfigError(f"max_context {self.max_context} exceeds the model's {spec.max_positions} positions")
        self.ctx = BuildContext(ops=ops, device=self.device, compute=dtype, max_context=self.max_context)
        self.layers = [Layer(ls, self.ctx) for ls in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, self.ctx)
        self.embed_position = None
        if spec.embed_position is not None:
            self.embed_position = POSITION_ENCODINGS.get(spec.embed_position.kind)(spec.embed_position.params, self.ctx)
            if not hasattr(self.embed_position, "after_embedding"):
                raise ConfigError(f"position encoding {spec.embed_position.kind!r} cannot act on the embedded rows "
                                  f"(it has no after_embedding)")

        self.embed_additions = build_embed_additions(spec, self.ctx)
        expected = expected_tensors(spec, self.layers, self.final_norm, self.embed_position, self.embed_additions)
        self.expected = expected
        tensors = load_tensors(source, expected, dtype, self.device, fused_tensors(self.layers))
        self.embed_table = tensors[spec.embed_name + "weight"]
        self.head_weight = self.embed_table if spec.tie_word_embeddings else tensors[spec.head_name + "weight"]
        self.head_bias = tensors.get(spec.head_name + "bias")
        self.final_norm.load({n: tensors[spec.final_norm_name + n] for n in self.final_norm.weights()})
        self.embed_norm = embed_norm_of(spec, self.ctx)
        if self.embed_norm is not None:
            self.embed_norm.load({n: tensors[spec.embed_norm_name + n] for n in self.embed_norm.weights()})
        self.depth_weights = [tensors[n] for n in depth_mix_names(spec)]
        # x <- W [x; x0] + b[row] before some calls: the two halves of W's columns as matrices of their own
        self.pass_inputs = {}
        if spec.pass_inputs:
            w_in, w_step, W = tensors[spec.pass_input_name + "in"], tensors[spec.pass_input_name + "step"], spec.hidden_size
            self.pass_w = (w_in[:, :W].contiguous(), w_in[:, W:].contiguous())
            for p in spec.pass_inputs:
                if not 0 <= p.call < len(spec.order) or p.call in self.pass_inputs:
                    raise ConfigError(f"pass input: call {p.call} is not an entry of the run order, or named twice")
                self.pass_inputs[p.call] = w_step[p.row].contiguous()
        if self.embed_position is not None:
            self.embed_position.load({n: tensors[spec.embed_position_name + n] for n in self.embed_position.weights()})
        for part, prefix in self.embed_additions:
            part.load({n: tensors[prefix + n] for n in part.weights()})
        for layer in self.layers:
            layer.load(tensors)
        del tensors

        # ---- the run order and who owns which cache
        self.order = list(spec.order)
        kv_calls, state_calls = {}, {}
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order names layer {call.layer}, the model has {len(self.layers)}")
            mixer = self.layers[call.layer].parts.get("mixer")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < i or self.order[call.cache_of].cache_of is not None:
                    raise ConfigError(f"call {i} must read the cache of an earlier call that owns one")
                continue
            if mixer is None:
                continue
            ks = mixer.cache_spec()
            if ks is not None:
                kv_calls[i] = ks
            ss = mixer.state_spec()
            if ss is not None:
                state_calls[i] = ss
        for k, (part, _) in enumerate(self.embed_additions):       # state of the additions to the embedded rows
            ss = part.state_spec()
            if ss is not None:
                state_calls[("embed", k)] = ss
        if n_pages is None:
            n_pages = max_slots * -(-self.max_context // page_size)
        cache_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        self.cache = CacheManager(kv_calls, state_calls, page_size=page_size, n_pages=n_pages, max_slots=max_slots,
                                  max_context=self.max_context, dtype=cache_dtype, device=self.device)
        # one mixer of each kind plans the step, and the step carries a tiling for every distinct declaration
        self.planners = list({type(m): m for m in (layer.parts.get("mixer") for layer in self.layers)
                              if m is not None}.values())
        needs = [n for n in (m.step_needs() for layer in self.layers for m in [layer.parts.get("mixer")] if m is not None)
                 if n is not None]
        self.staging = StepStaging(max_step_tokens, self.device, status=getattr(ops, "page_error", None), needs=needs)
        self.max_step_tokens = max_step_tokens
        # where the sampler leaves its tokens on the device, if the kernel set has such a place: an entry may
        # take its token from there (StepEntry.feed) instead of from the host
        self.fed_from = getattr(ops, "token_out", None)
        # decode steps (one token per entry) are captured once per batch size and mixers' plan (the attention's
        # key-range split), and replayed: their hundreds of small launches would otherwise be bound by the host
        self.use_graphs = (use_graphs and self.device.type == "cuda" and self.final_norm.graph_safe
                           and (self.embed_norm is None or self.embed_norm.graph_safe)
                           and (self.embed_position is None or self.embed_position.graph_safe)
                           and all(part.graph_safe for part, _ in self.embed_additions)
                           and all(p.graph_safe for layer in self.layers for p in layer.parts.values()))
        self._graphs = {}
        self._graph_pool = None         # one memory pool for all captured steps: only one of them runs at a time
        self.graph_max_batch = 256
        # Captured graphs are kept by (batch size, the mixers' plans); a long-running engine with
        # varying batches would collect thousands, so only the most recently used ones are kept.
        self.graph_max_kept = 64

    # ------------------------------------------------------------------ facts
    @property
    def vocab_size(self):
        return self.spec.vocab_size

    @property
    def eos_token_ids(self):
        return tuple(self.spec.eos_token_ids)

    def _parts_with_tensors(self):
        for part, _ in self.embed_additions:
            yield part
        for layer in self.layers:
            yield from layer.parts.values()

    def weight_bytes(self):
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embed_table); add(self.head_weight); add(self.head_bias)
        for part in self._parts_with_tensors():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    add(v)
        return total

    # ------------------------------------------------------------------ the step function
    def step(self, entries, record=None, attention_splits=None) -> torch.Tensor:
        """Run one batch.  ``entries``: list of StepEntry.  Pages for every entry must
        have been made by ``cache.ensure``.  Returns logits [wanted, vocab] float32."""
        for e in entries:
            for g in self.cache.groups:
                t = g.pages.tables[e.slot]
                if len(t.pages) * g.pages.page_size < e.start_pos + len(e.tokens):
                    raise ModelError(f"slot {e.slot}: pages do not cover positions up to "
                                     f"{e.start_pos + len(e.tokens) - 1}")
        self.cache.sync()
        step = self.staging.pack(entries, self.spec.vocab_size, self.max_context)
        if step.n_fed and self.fed_from is None:
            raise ModelError("an entry's token is fed from the sampler's output, but this kernel set keeps none")
        step.record = record
        step.attention_splits = attention_splits
        captured = (self.use_graphs and attention_splits is None
                    and step.n_tokens == len(entries) <= self.graph_max_batch and step.n_want == step.n_tokens)
        plans = tuple(m.plan_step(step, captured) for m in self.planners)
        if captured:
            return self._graphed_decode(step, plans)
        return self.forward(step)

    def _graphed_decode(self, step, plans):
        key = (step.n_tokens, plans)      # the batch size and what the mixers' plans say shapes their launches
        entry = self._graphs.pop(key, None)
        if entry is None:
            # The first step of its kind runs eagerly (which also loads modules and warms the allocator) and its
            # result is the step's result; the capture that follows executes nothing, so a part with state of
            # its own advances once.
            logits = self.forward(step)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = self.ops.launches
            wanted, step.record = step.record, {}     # internals are recorded as references to the
            with torch.cuda.graph(graph, pool=self._graph_pool):   # graph's own tensors, refreshed by every replay
                graph_logits = self.forward(step)
            self._graphs[key] = (graph, graph_logits, self.ops.launches - before, step.record)
            step.record = wanted
            while len(self._graphs) > self.graph_max_kept:       # the least recently used goes
                self._graphs.pop(next(iter(self._graphs)))
            return logits
        self._graphs[key] = entry         # most recently used last
        graph, logits, n, internals = entry
        graph.replay()
        self.ops.launches += n
        if step.record is not None:
            step.record.update(internals)
        return logits

    def forward(self, step) -> torch.Tensor:
        ops, spec = self.ops, self.spec
        T = step.n_tokens
        h = torch.empty((T, spec.hidden_size), dtype=torch.float32, device=self.device)
        if self.fed_from is not None:
            ops.embed(step.ids, self.embed_table, h, spec.embed_scale, fed_rows=step.fed_rows, fed_from=self.fed_from)
        else:
            ops.embed(step.ids, self.embed_table, h, spec.embed_scale)
        if self.embed_position is not None:
            self.embed_position.after_embedding(h, step)
        for k, (part, _) in enumerate(self.embed_additions):
            part.forward(h, step, self.cache.state_of(("embed", k)), fed_from=self.fed_from)
        # a copy of the rows in the activations' type, for parts that read the rows themselves (no norm before them)
        copy = (torch.empty((T, spec.hidden_size), dtype=self.ctx.act_dtype, device=self.device)
                if self.ctx.act_dtype != torch.float32 and (self.embed_norm is not None or spec.depth_mix) else None)
        history = None
        if spec.depth_mix:       # the embedded rows and every call's result: what a call hands on is a weighted sum of them
            history = torch.empty((len(self.order) + 1, T, spec.hidden_size), dtype=torch.float32, device=self.device)
        if self.embed_norm is not None:
            normed = history[0] if history is not None else torch.empty_like(h)
            self.embed_norm.forward(h, (), out={torch.float32: normed, **({copy.dtype: copy} if copy is not None else {})})
            if history is not None:
                h.copy_(normed)
            else:
                h = normed
            if copy is not None:
                step.shared["rows"] = (h, {copy.dtype: copy})
        elif history is not None:
            history[0].copy_(h)
        carry = None     # an addition to h that a layer left for the next norm to apply
        x0 = None        # the embedded rows in the type the pass inputs' product reads
        if self.pass_inputs:
            wdt = self.pass_w[0].dtype
            x0 = torch.empty((T, spec.hidden_size), dtype=wdt, device=self.device)
            ops.cast_rows(h, x0)
        for i, call in enumerate(self.order):
            if i in self.pass_inputs:         # h <- W [h; x0] + b: two products into new rows, the residual sum in float32
                if carry is not None:
                    ops.apply_pending(h, carry)
                    carry = None
                hx = torch.empty_like(x0)
                ops.cast_rows(h, hx)
                h = torch.empty_like(h)
                ops.gemm(hx, self.pass_w[0], h, bias=self.pass_inputs[i])
                ops.gemm(x0, self.pass_w[1], h, accumulate=True)
            layer = self.layers[call.layer]
            owner = i if call.cache_of is None else call.cache_of
            carry = layer.block.forward(h, step, self.cache.view(owner), self.cache.state_of(i),
                                        writes_cache=call.cache_of is None, carry=carry)
            if step.record is not None and carry is None and history is None:
                step.record.setdefault("rows_after", []).append(h.clone())      # the rows as this call leaves them
            if history is not None:
                if carry is not None:
                    ops.apply_pending(h, carry)
                    carry = None
                # history[i + 1] <- h, then h <- sum_j w[j] history[j] over the i + 2 sets of rows so far
                ops.depth_mix(history, i + 2, self.depth_weights[i], h, out_copy=copy)
                if step.record is not None:
                    step.record.setdefault("handed_on", []).append(h.clone())
                if copy is not None:
                    step.shared["rows"] = (h, {copy.dtype: copy})
        R = step.n_want
        logits = torch.empty((R, spec.vocab_size), dtype=torch.float32, device=self.device)
        if R:
            wdt = self.head_weight.dtype
            x, _ = run_norm(self.final_norm, h, (wdt,), carry, row_index=step.want_rows)
            ops.gemm(x[wdt], self.head_weight, logits, bias=self.head_bias)
            if spec.logit_softcap:
                ops.softcap(logits, spec.logit_softcap)
        return logits

    def check_status(self, flags=None):
        """Raise if a kernel met a position without a page or gave up a bounded wait.  ``flags``: the two
        flags (tensor-core error, page error) if the caller has read them already; else they are read here
        (which synchronises)."""
        tc = getattr(self.ops, "tc_error", None)
        if flags is None:
            flags = (int(tc.item()) if tc is not None else 0, int(self.staging.status.item()))
        if flags[1]:
            self.staging.status.zero_()
            raise ModelError("a kernel met a position whose page was not allocated")
        if flags[0]:
            tc.zero_()
            counters = getattr(self.ops, "attention_arrivals", None)
            if counters is not None:
                counters.zero_()          # a kernel that gave up may have left an arrival uncounted
            raise ModelError("a tensor-core kernel gave up waiting for its operands")


# ---------------------------------------------------------------------- loading by config.json

def read_config(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} not found")
    try:
        return json.loads(path.read_text())
    except ValueError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None


def architecture_of(config: dict):
    """The architecture class a config.json names: the first entry of ``architectures``, or the string under
    ``architecture``."""
    archs = config.get("architectures")
    if archs is None and isinstance(config.get("architecture"), str):
        archs = [config["architecture"]]
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json names no architecture ('architectures' or 'architecture'); registered: "
                          + ", ".join(ARCHITECTURES.names()))
    return ARCHITECTURES.get(archs[0])


def load_model(model_dir, **kw) -> Model:
    """Build the model that config.json names and load its tensors from the folder."""
    from .. import models  # noqa: F401  (registers the built-in architectures)
    cfg = read_config(model_dir)
    arch = architecture_of(cfg)
    spec = arch.model_spec(arch.parse_config(cfg))
    source = SafetensorsSource(model_dir)
    return Model(spec, RenamedSource(source, spec.stored_names) if spec.stored_names else source, **kw)
