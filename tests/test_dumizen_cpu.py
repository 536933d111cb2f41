"""Dumizen through the engine's plumbing on the CPU (the kernels replaced by their plain references): the
configuration reader, tensor names, the run order of a looped model, the plain mechanisms' invariants, the means of
blocks in the pages of the cache, state across steps and slots, and replay under every cut against the plain
implementation."""
import copy
import math

import pytest
import torch

import plain_dumizen as P
import tiny_dumizen as tiny
import traces
from flint_b200.engine.engine import Engine
from flint_b200.engine.loading import expected_from_config, write_random_model
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.errors import ConfigError, WeightError
from flint_b200.sampling.params import SamplingParams
from kernel_refs import RefOps

LENGTHS = (1, 2, 9, 37, 70, 130)
F64 = torch.float64


@pytest.fixture(scope="module", params=["D1", "D2", "D3"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("dumizen") / which, cfg, seed=3)
    reqs = traces.make_requests(cfg["vocab"], LENGTHS, seed=7)
    plain = {rid: P.forward(cfg, w, t)[0] for rid, t in reqs.items()}
    return which, cfg, folder, w, reqs, plain


def replay(folder, steps, page_size=16, record=False):
    n = traces.max_tokens_needed(steps)
    rp = Replayer(folder, dtype="float32", max_tokens=n, page_size=page_size, max_requests=4, device="cpu", ops=RefOps())
    out, recs = {}, {}
    for s in steps:
        rec = {} if record else None
        lg = rp.run_step(s["entries"], s["end"], record=rec)
        if lg is not None:
            out[s["step"]] = lg
        recs[s["step"]] = rec
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, recs, rp


def compare(out, steps, plain, tol=3e-4):
    exp = traces.expected_rows(steps, plain)
    assert set(out) == set(exp)
    for k, rows in exp.items():
        want = torch.stack(rows)
        err = (out[k].double() - want).abs().max().item()
        assert err < tol * max(1.0, float(want.abs().max())), f"step {k}: max error {err:.2e}"


# ------------------------------------------------------------------------------------------------ the plain mechanisms
def one_layer(kind, mixer, width=16):
    return {"architecture": "Dumizen", "vocab": 11, "width": width, "norm": {"eps": 1e-6},
            "layers": [{"type": kind, "mixer": mixer, "mlp": None}]}


def test_the_plain_mechanisms_hold_their_invariants():
    g = torch.Generator().manual_seed(1)
    # YaRN: frequencies below the ramp stay, those above it are divided by the factor; without scaling nothing changes
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 32, "fast": 16.0, "slow": 1.0}}
    f, mag = P.rotary_frequencies(rot)
    plain_f, one = P.rotary_frequencies({"dims": 8, "base": 100.0})
    assert one == 1.0 and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12
    assert torch.all(f <= plain_f + 1e-15) and torch.all(f >= plain_f / 4 - 1e-15) and f[0] == plain_f[0]
    x = torch.randn(5, 3, 12, generator=g, dtype=F64)
    y = P.rotate(x, torch.arange(5), {"dims": 8, "base": 100.0})
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[2, 1, 0] ** 2 + y[2, 1, 4] ** 2, x[2, 1, 0] ** 2 + x[2, 1, 4] ** 2)     # dim i turns with i + dims/2
    # the pooled window: with one block of 3 and a window of 2, position 4 sees positions 3, 4 and the mean of 0..2;
    # position 3 sees 2, 3 and no block (the block's last position 2 is still inside the window)
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.0, "mask": {"size": 2, "pool": 3}}
    W = 4
    w = {"p.q": torch.zeros(4, W, dtype=F64), "p.k": torch.zeros(4, W, dtype=F64), "p.v": torch.eye(4, dtype=F64),
         "p.q.b": torch.zeros(4, dtype=F64), "p.k.b": torch.zeros(4, dtype=F64), "p.v.b": torch.zeros(4, dtype=F64),
         "p.q.norm": torch.ones(4, dtype=F64), "p.k.norm": torch.ones(4, dtype=F64), "p.o": torch.eye(4, dtype=F64)}
    h = torch.randn(6, W, generator=g, dtype=F64)
    o = P.pooled_window_attention(h, w, "p.", m, 1e-6)          # scale 0: every seen key weighs the same
    assert torch.allclose(o[4], (h[3] + h[4] + h[:3].mean(0)) / 3)
    assert torch.allclose(o[3], (h[2] + h[3]) / 2)
    assert torch.allclose(o[5], (h[4] + h[5] + h[:3].mean(0)) / 3)       # position 3 is seen by nobody after it left
    # the unit sink: with scores of 0, n keys share n / (n + 1) of the weight
    lm = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.0}
    lw = {"l.q": torch.zeros(4, W, dtype=F64), "l.k": torch.eye(4, dtype=F64), "l.q.norm": torch.ones(4, dtype=F64),
          "l.k.norm": torch.ones(4, dtype=F64), "l.g": torch.zeros(4, W, dtype=F64), "l.o": torch.eye(4, dtype=F64)}
    o = P.sink_gated_attention(h, lw, "l.", lm, 1e-6)            # values are the keys as projected; the gate is 1/2
    assert torch.allclose(o[2], 0.5 * h[:3].sum(0) / 4)
    # retention: o_t = sum_j decay^(t - j) (q_t . k_j / sqrt(dim)) v_j before the norm; one head, no rotation
    rm = {"heads": 1, "dim": 4, "vdim": 4, "decay": [0.5]}
    rw = {"r.q": torch.eye(4, dtype=F64), "r.k": torch.eye(4, dtype=F64), "r.v": torch.eye(4, dtype=F64),
          "r.g": torch.eye(4, dtype=F64), "r.o": torch.eye(4, dtype=F64)}
    o = P.retention(h, rw, "r.", rm, 1e-6)
    raw = sum(0.5 ** (3 - j) * (h[3] @ h[j]) / 2.0 * h[j] for j in range(4))
    assert torch.allclose(o[3], P.rms(raw, 1e-6) * h[3] * torch.sigmoid(h[3]))
    # sigmoid attention: weights are not normalised, and the penalty grows with the distance
    sm = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.0}
    sw = {"s.q": torch.zeros(4, W, dtype=F64), "s.k": torch.zeros(4, W, dtype=F64), "s.v": torch.eye(4, dtype=F64),
          "s.q.b": torch.zeros(4, dtype=F64), "s.k.b": torch.zeros(4, dtype=F64), "s.v.b": torch.zeros(4, dtype=F64),
          "s.r1": torch.tensor([1.0], dtype=F64), "s.r2": torch.tensor([1.0], dtype=F64), "s.pb": torch.tensor([0.0], dtype=F64),
          "s.o": torch.eye(4, dtype=F64), "s.o.b": torch.zeros(4, dtype=F64)}
    o = P.sigmoid_attention(h, sw, "s.", sm, 1e-6)
    want = sum(torch.sigmoid(torch.tensor(-math.log(1 + 2 - j), dtype=F64)) * h[j] for j in range(3))
    assert torch.allclose(o[2], want)
    # the router: a correction changes the choice and not the weights; a group that is not kept gives no expert
    f = {"router": {"experts": 4, "top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}}}
    mw = {"m.router": torch.tensor([[3.0], [-3.0], [1.0], [0.9]], dtype=F64), "m.correction": torch.tensor([0.0, 0.0, 0.0, 0.0], dtype=F64)}
    ids, weights = P.route(torch.ones(1, 1, dtype=F64), mw, "m.", f)
    assert sorted(ids[0].tolist()) == [2, 3]          # group 1 (0.73 + 0.71) beats group 0 (0.95 + 0.05) although expert 0 is best
    assert abs(float(weights.sum()) - 2.0) < 1e-9
    mw["m.correction"] = torch.tensor([0.0, 0.6, 0.0, 0.0], dtype=F64)
    ids, weights = P.route(torch.ones(1, 1, dtype=F64), mw, "m.", f)
    assert sorted(ids[0].tolist()) == [0, 1]
    s = torch.sigmoid(torch.tensor([3.0, -3.0], dtype=F64))
    assert torch.allclose(weights[0].sort().values, (s / s.sum() * 2.0).sort().values)


def test_the_run_order_of_a_looped_model():
    assert P.run_order(tiny.D2) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None), (4, None)]
    assert P.run_order(tiny.D3) == [(0, None), (1, None), (2, None)]
    spec, _ = expected_from_config(tiny.D2)
    assert [c.layer for c in spec.order] == [0, 1, 2, 1, 2, 3, 4]
    assert [(p.call, p.row) for p in spec.pass_inputs] == [(1, 0), (3, 1)]
    spec, _ = expected_from_config(tiny.D1)
    assert [c.layer for c in spec.order] == [0, 1, 2, 3, 4] * 3 and [p.call for p in spec.pass_inputs] == [0, 5, 10]
    assert expected_from_config(tiny.D3)[0].pass_inputs == ()


# ------------------------------------------------------------------------------------------------ configuration and tensors
def test_config_names_every_size_and_refuses_what_it_cannot_read():
    for which, cfg in tiny.CONFIGS.items():
        spec, expected = expected_from_config(cfg)
        stored = {spec.stored_names.get(n, n): tuple(ws.shape) for n, ws in expected.items()}
        assert stored == tiny.tensor_shapes(cfg)
        assert spec.tie_word_embeddings and all(l.block == "sandwich" for l in spec.layers)
    spec, _ = expected_from_config(tiny.D1)
    assert "norm2" not in spec.layers[1].parts and "ffn" not in spec.layers[1].parts
    assert spec.layers[1].parts["mixer"].params["pool"] == 3 and spec.layers[1].parts["mixer"].params["window"] == 7
    for key, value, message in ((("layers", 0, "type"), "conv", "unknown layer type"),
                                (("layers", 1, "mixer", "kv_heads"), 4, "multiple of kv_heads"),
                                (("layers", 1, "mixer", "rot", "dims"), 26, "at most dim"),
                                (("layers", 0, "mixer", "right", "decay"), [0.5], "3 entries"),
                                (("layers", 0, "mixer", "left", "vdim"), 7, "values are the keys"),
                                (("layers", 2, "mlp", "router", "top"), 6, "exceeds"),
                                (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
                                (("layers", 0, "mlp", "kind"), "dense", "unknown kind"),
                                (("loop", "stop"), 9, "not a run"),
                                (("layers", 2, "mixer", "softcap"), -1.0, "softcap")):
        bad = copy.deepcopy(tiny.D1)
        d = bad
        for k in key[:-1]:
            d = d[k]
        d[key[-1]] = value
        with pytest.raises(ConfigError, match=message):
            expected_from_config(bad)
    bad = copy.deepcopy(tiny.D1)
    del bad["layers"][3]["mixer"]["vdim"]
    with pytest.raises(ConfigError, match="vdim"):
        expected_from_config(bad)


def test_a_missing_or_misshaped_tensor_is_named(tmp_path):
    w = tiny.random_weights(tiny.D1, 1)
    del w["l0.mix.right.g"]
    w["l2.mix.r1"] = w["l2.mix.r1"][:2]
    w["loop.step"] = w["loop.step"][:2]
    folder, _ = tiny.write_model(tmp_path / "m", tiny.D1, weights=w)
    with pytest.raises(WeightError) as e:
        load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=4, max_slots=2, max_context=64)
    assert all(n in str(e.value) for n in ("l0.mix.right.g", "l2.mix.r1", "loop.step"))


def test_random_weights_mode_writes_the_design_s_own_names(tmp_path):
    folder = write_random_model(tmp_path / "m", tiny.D2, seed=5)
    from flint_b200.weights.safetensors_io import SafetensorsFile
    names = set(SafetensorsFile(folder / "model.safetensors").names())
    assert names == set(tiny.tensor_shapes(tiny.D2))
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=8, max_slots=2, max_context=128)
    # seven calls: every call of a looped layer has a cache (and the parallel mixer a state) of its own
    assert m.spec.architecture == "Dumizen" and len(m.order) == 7 and len(m.cache.state) == 2
    assert sum(len(g.calls) for g in m.cache.groups) == 7


# ------------------------------------------------------------------------------------------------ the engine against the plain model
def test_every_layer_run_hands_on_what_the_plain_model_does(setup):
    which, cfg, folder, w, reqs, plain = setup
    t = reqs["r3"]
    _, after, _ = P.forward(cfg, w, t)
    steps = traces.whole({"r3": t})
    _, recs, _ = replay(folder, steps, record=True)
    rows = recs[0]["rows_after"]
    assert len(rows) == tiny.run_count(cfg) == after.shape[0]
    for i, r in enumerate(rows):
        assert (r.double() - after[i]).abs().max() < 3e-4 * float(after[i].abs().max()), f"run {i}"


def test_replay_matches_plain_whole_and_cut(setup):
    which, cfg, folder, w, reqs, plain = setup
    for cut in (traces.whole, lambda r: traces.tail_decoded(r, tail=40), traces.portions,
                lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3, 128))):
        steps = cut(reqs)
        out, _, _ = replay(folder, steps)
        compare(out, steps, plain)


def test_replay_matches_plain_in_mixed_batches_with_slots_and_pages_used_again(setup):
    which, cfg, folder, w, reqs, plain = setup
    more = dict(reqs)
    more.update({f"x{k}": v for k, v in traces.make_requests(cfg["vocab"], (33, 5, 64, 17), seed=11).items()})
    full = dict(plain)
    full.update({rid: P.forward(cfg, w, t)[0] for rid, t in more.items() if rid not in full})
    for seed in (3, 4):
        steps = traces.mixed(more, seed=seed)
        out, _, rp = replay(folder, steps)
        compare(out, steps, full)
        assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2      # pages were used again


def test_state_and_block_means_start_anew_in_a_slot_that_was_used(setup):
    """One slot, three requests one after the other: each must see the state of a new sequence, and no mean of a
    block that an earlier request left in a page."""
    which, cfg, folder, w, reqs, plain = setup
    rp = Replayer(folder, dtype="float32", max_tokens=192, page_size=16, max_requests=1, device="cpu", ops=RefOps())
    for rid in ("r4", "r3", "r4"):
        t = reqs[rid]
        a = rp.run_step([{"id": rid, "tokens": t[:5], "want": [4]}])
        b = rp.run_step([{"id": rid, "tokens": t[5:], "want": [len(t) - 6]}], end=[rid])
        got = torch.cat([a, b]).double()
        want = torch.stack([plain[rid][4], plain[rid][-1]])
        assert (got - want).abs().max() < 3e-4 * float(want.abs().max())


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_configurations_drawn_at_random(seed, tmp_path):
    cfg = tiny.random_config(seed)
    folder, w = tiny.write_model(tmp_path / "m", cfg, seed=seed)
    reqs = traces.make_requests(cfg["vocab"], (1, 2, 23, 50, 85), seed=seed)
    plain = {rid: P.forward(cfg, w, t)[0] for rid, t in reqs.items()}
    for cut in (traces.whole, lambda r: traces.tail_decoded(r, tail=45), lambda r: traces.portions(r, sizes=(2, 3, 16, 1, 2, 64)),
                lambda r: traces.mixed(r, seed=seed)):
        steps = cut(reqs)
        out, _, _ = replay(folder, steps)
        compare(out, steps, plain)


def test_greedy_generation_through_the_engine_with_preemption(setup):
    which, cfg, folder, w, reqs, plain = setup
    prompts = [reqs["r2"], reqs["r3"][:14], reqs["r0"]]
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(10):
            t = int(torch.argmax(P.forward(cfg, w, toks)[0][-1]))
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages in (16, 3):
        m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=n_pages, max_slots=4,
                       max_step_tokens=24, max_context=256, use_graphs=False)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        assert eng.generate(prompts, 10) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0


def test_a_window_without_blocks_gives_its_pages_back(tmp_path):
    """A mask that names no block size is a plain window: nothing behind it is seen, and the pages behind it go
    back to the pool while the request runs."""
    cfg = copy.deepcopy(tiny.D3)
    cfg["layers"] = [cfg["layers"][2]]
    del cfg["layers"][0]["mixer"]["mask"]["pool"]
    folder, w = tiny.write_model(tmp_path / "m", cfg, seed=3)
    reqs = traces.make_requests(cfg["vocab"], (70, 9), seed=7)
    plain = {rid: P.forward(cfg, w, t)[0] for rid, t in reqs.items()}
    steps = traces.portions(reqs, sizes=(7, 2, 13, 3))
    out, _, rp = replay(folder, steps)
    compare(out, steps, plain)
    spec = rp.model.cache.groups[0].spec
    assert spec.window == 10 and spec.pool == 0
    rp2 = Replayer(folder, dtype="float32", max_tokens=128, page_size=16, max_requests=1, device="cpu", ops=RefOps())
    rp2.run_step([{"id": "a", "tokens": reqs["r0"][:60], "want": []}])
    assert rp2.model.cache.groups[0].pages.pool.used_pages <= 2        # 60 positions would hold four pages of 16
