"""Tefovik through the engine's plumbing on the CPU (the kernels replaced by their plain references): the
configuration reader, tensor names, the norm after the sum, the weighted sum over depth, the convolution's and the
recurrences' state across steps and slots, runs of positions across pages, and replay under every cut against the
plain implementation."""
import copy

import pytest
import torch

import plain_tefovik as P
import tiny_tefovik as tiny
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


@pytest.fixture(scope="module", params=["T1", "T2"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("tefovik") / which, cfg, seed=3, ranks=tiny.RANKS[which])
    reqs = traces.make_requests(cfg["vocab"], LENGTHS, seed=7)
    plain = {rid: P.forward(cfg, w, t) for rid, t in reqs.items()}
    return which, cfg, folder, w, reqs, plain


def replay(folder, steps, page_size=16):
    n = traces.max_tokens_needed(steps)
    rp = Replayer(folder, dtype="float32", max_tokens=n, page_size=page_size, max_requests=4, device="cpu", ops=RefOps())
    out = {}
    for s in steps:
        lg = rp.run_step(s["entries"], s["end"])
        if lg is not None:
            out[s["step"]] = lg
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, rp


def compare(out, steps, plain, tol=3e-4):
    exp = traces.expected_rows(steps, plain)
    assert set(out) == set(exp)
    for k, rows in exp.items():
        want = torch.stack(rows)
        err = (out[k].double() - want).abs().max().item()
        assert err < tol * max(1.0, float(want.abs().max())), f"step {k}: max error {err:.2e}"


def test_the_plain_mechanisms_hold_their_invariants():
    # the convolution's last column weighs the current token, and nothing comes from before the sequence
    u = torch.arange(1.0, 6.0, dtype=F64)[:, None]
    wc = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64)
    assert P.causal_conv(u, wc).flatten().tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    # runs of positions are counted from 0
    seen = P.chunk_visible(12, 5)
    assert seen[9].nonzero().flatten().tolist() == [5, 6, 7, 8, 9] and seen[10].nonzero().flatten().tolist() == [10]
    assert seen[4].nonzero().flatten().tolist() == [0, 1, 2, 3, 4] and P.chunk_visible(4, 0)[3].all()
    # a rotation keeps each pair's length, leaves the other dims and position 0 alone, and turns back
    x = torch.randn(5, 3, 12, dtype=F64)
    pos = torch.arange(5)
    y = P.turn_pairs(x, pos, 100.0, 8)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[2, 1, 2] ** 2 + y[2, 1, 3] ** 2, x[2, 1, 2] ** 2 + x[2, 1, 3] ** 2)     # dim 2i turns with 2i + 1
    assert torch.allclose(P.turn_pairs(y, pos, 100.0, 8, sign=-1.0), x)
    # values turned by their own position and sums turned back by the query's: weights of relative positions
    v = torch.randn(4, 1, 6, dtype=F64)
    turned = P.turn_pairs(v, torch.arange(4), 50.0, 6)
    back = P.turn_pairs(turned[1:2].expand(4, 1, 6).clone(), torch.arange(4), 50.0, 6, sign=-1.0)
    assert torch.allclose(back[3], P.turn_pairs(v[1:2], torch.tensor([-2]), 50.0, 6)[0])
    # the delta rule: with no decay and beta = 1 the state returns the value it was just given for a unit key
    k = torch.tensor([0.6, 0.8, 0.0], dtype=F64)
    S, o = P.delta_rule_step(torch.randn(3, 2, dtype=F64), k, k, torch.tensor([3.0, -1.0], dtype=F64), torch.ones(3, dtype=F64), 1.0)
    assert torch.allclose(o, torch.tensor([3.0, -1.0], dtype=F64))
    # the decay acts on the rows of the key channels, before the write
    S0 = torch.ones(3, 2, dtype=F64)
    S, _ = P.delta_rule_step(S0, k, torch.zeros(3, dtype=F64), torch.zeros(2, dtype=F64), torch.tensor([0.5, 1.0, 0.25], dtype=F64), 0.0)
    assert torch.allclose(S, torch.tensor([[0.5, 0.5], [1.0, 1.0], [0.25, 0.25]], dtype=F64))
    # the state-space step: decay exp(-rate dt), write dt B x^T, skip D x
    S, yv = P.state_space_step(torch.zeros(2, 2, dtype=F64), torch.tensor([1.0, 2.0], dtype=F64), torch.tensor([1.0, 0.0], dtype=F64),
                               torch.tensor([1.0, 1.0], dtype=F64), 0.5, 2.0, 3.0)
    assert torch.allclose(yv, torch.tensor([0.5 + 3.0, 1.0 + 6.0], dtype=F64))
    S, _ = P.state_space_step(S, torch.zeros(2, dtype=F64), torch.zeros(2, dtype=F64), torch.zeros(2, dtype=F64), 0.5, 2.0, 0.0)
    assert torch.allclose(S[0], torch.tensor([0.5, 1.0], dtype=F64) * torch.exp(torch.tensor(-1.0, dtype=F64)))
    assert float(P.relu_squared(torch.tensor(-2.0))) == 0.0 and float(P.relu_squared(torch.tensor(3.0))) == 9.0


def _with_free_dims(shapes, expected, stored):
    """``shapes`` with the extents that the checkpoint decides replaced by those the package would draw."""
    out = dict(shapes)
    for n, ws in expected.items():
        s = stored.get(n, n)
        if ws.free_dims and s in out:
            out[s] = tuple(ws.shape[i] if i in ws.free_dims else e for i, e in enumerate(out[s]))
    return out


def test_config_names_every_size_and_refuses_what_it_cannot_read():
    for which, cfg in tiny.CONFIGS.items():
        spec, expected = expected_from_config(cfg)
        stored = {spec.stored_names.get(n, n): tuple(ws.shape) for n, ws in expected.items()}
        assert stored == _with_free_dims(tiny.tensor_shapes(cfg, tiny.RANKS[which]), expected, spec.stored_names)
        assert not spec.tie_word_embeddings and [c.layer for c in spec.order] == list(range(len(cfg["layers"])))
        assert spec.depth_mix and spec.logit_softcap == cfg["logit_softcap"] and spec.embed_norm is not None
    spec, _ = expected_from_config(tiny.T1)
    assert [l.parts["mixer"].kind for l in spec.layers] == ["ssd", "branches", "branches", "ssd", "branches"]
    assert "ffn" in spec.layers[0].parts and "ffn" not in spec.layers[1].parts and "norm2" not in spec.layers[3].parts
    left = dict(spec.layers[4].parts["mixer"].params["branches"])["left"].params
    assert left["chunk"] == 0 and left["position"] is None and left["conv_taps"] == 1
    assert spec.layers[2].parts["norm1"].params["residual_scale"] == 2.0
    for key, value, message in ((("layers", 0, "type"), "conv", "unknown layer type"),
                                (("layers", 1, "mixer", "left", "kv_heads"), 4, "multiple of kv_heads"),
                                (("layers", 1, "mixer", "left", "rot", "dims"), 14, "at most dim"),
                                (("layers", 1, "mixer", "left", "vdim"), 9, "must be even"),
                                (("layers", 1, "mixer", "right", "kv_heads"), 3, "multiple of kv_heads"),
                                (("layers", 0, "mixer", "norm_groups"), 4, "does not divide"),
                                (("layers", 3, "mixer", "groups"), 3, "multiple of groups"),
                                (("logit_softcap",), 0.0, "positive"),
                                (("layers", 0, "mlp", "kind"), "conv", "unknown kind")):
        bad = copy.deepcopy(tiny.T1)
        d = bad
        for k in key[:-1]:
            d = d[k]
        d[key[-1]] = value
        with pytest.raises(ConfigError, match=message):
            expected_from_config(bad)
    for path in (("layers", 3, "mixer", "state"), ("layers", 2, "mixer", "right", "conv"), ("postln_alpha",), ("norm",)):
        bad = copy.deepcopy(tiny.T1)
        d = bad
        for k in path[:-1]:
            d = d[k]
        del d[path[-1]]
        with pytest.raises(ConfigError, match=path[-1]):
            expected_from_config(bad)


def test_a_missing_or_misshaped_tensor_is_named(tmp_path):
    w = tiny.random_weights(tiny.T1, 1)
    del w["l1.mix.right.dt_bias"]
    w["l0.mix.conv"] = w["l0.mix.conv"][:, :2]
    w["l2.dwa"] = w["l2.dwa"][:3]
    w["l1.mix.right.a2"] = torch.cat([w["l1.mix.right.a2"], w["l1.mix.right.a2"][:, :1]], 1)      # ranks that disagree
    folder, _ = tiny.write_model(tmp_path / "m", tiny.T1, weights=w)
    with pytest.raises((WeightError, ConfigError)) as e:
        load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=4, max_slots=2, max_context=64)
    assert all(n in str(e.value) for n in ("l1.mix.right.dt_bias", "l0.mix.conv", "l2.dwa"))
    w = tiny.random_weights(tiny.T1, 1)
    w["l1.mix.right.a2"] = torch.cat([w["l1.mix.right.a2"], w["l1.mix.right.a2"][:, :1]], 1)
    folder, _ = tiny.write_model(tmp_path / "n", tiny.T1, weights=w)
    with pytest.raises(ConfigError, match="low-rank pairs disagree"):
        load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=4, max_slots=2, max_context=64)


def test_what_every_layer_hands_on(setup):
    """The rows after every layer (the weighted sum over depth included), not only the logits."""
    which, cfg, folder, w, reqs, plain = setup
    keep = {}
    P.forward(cfg, w, reqs["r3"], keep)
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=8, max_slots=2, max_context=128)
    rp = Replayer(folder, dtype="float32", max_tokens=128, model=m)
    rec = {}
    rp.run_step([{"id": "a", "tokens": reqs["r3"], "want": [0]}], record=rec)
    assert len(rec["handed_on"]) == len(cfg["layers"])
    for got, want in zip(rec["handed_on"], keep["layers"]):
        assert (got.double() - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_replay_matches_plain_whole_and_cut(setup):
    which, cfg, folder, w, reqs, plain = setup
    for steps in (traces.whole(reqs), traces.tail_decoded(reqs, tail=24), traces.portions(reqs),
                  traces.portions(reqs, sizes=(2, 2, 1, 2, 3, 128))):
        out, _ = replay(folder, steps)
        compare(out, steps, plain)


def test_replay_matches_plain_in_mixed_batches_with_slots_and_pages_used_again(setup):
    which, cfg, folder, w, reqs, plain = setup
    more = dict(reqs)
    more.update({f"s{i}": t for i, t in enumerate(traces.make_requests(cfg["vocab"], (5, 33, 18), seed=11).values())})
    plain = dict(plain)
    for rid in ("s0", "s1", "s2"):
        plain[rid] = P.forward(cfg, w, more[rid])
    for seed in (0, 3):
        steps = traces.mixed(more, seed=seed)
        out, rp = replay(folder, steps)
        compare(out, steps, plain)
        assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2


@pytest.mark.parametrize("seed", [2, 23])
def test_configurations_drawn_at_random_match_plain(seed, tmp_path):
    """Sizes, constants and orders of layers that no other test has, whole, in twos and in a mixed batch."""
    cfg, ranks = tiny.random_config(seed)
    folder, w = tiny.write_model(tmp_path / "m", cfg, seed=seed, ranks=ranks)
    reqs = traces.make_requests(cfg["vocab"], (1, 2, 9, 37), seed=seed)
    plain = {rid: P.forward(cfg, w, t) for rid, t in reqs.items()}
    for steps in (traces.whole(reqs), traces.portions(reqs, sizes=(2, 2, 1, 2, 3, 128)), traces.mixed(reqs, seed=3)):
        out, _ = replay(folder, steps)
        compare(out, steps, plain)


def test_every_state_starts_from_zero_in_a_slot_that_was_used(setup):
    """One slot, three requests one after the other: each must see the state of a new sequence (the matrices of
    the recurrences and the convolutions' last inputs alike)."""
    which, cfg, folder, w, reqs, plain = setup
    rp = Replayer(folder, dtype="float32", max_tokens=192, page_size=16, max_requests=1, device="cpu", ops=RefOps())
    for rid in ("r3", "r2", "r3"):
        t = reqs[rid]
        a = rp.run_step([{"id": rid, "tokens": t[:5], "want": [4]}])
        b = rp.run_step([{"id": rid, "tokens": t[5:], "want": [len(t) - 6]}], end=[rid])
        got = torch.cat([a, b]).double()
        want = torch.stack([plain[rid][4], plain[rid][-1]])
        assert (got - want).abs().max() < 3e-4 * float(want.abs().max())


def test_random_weights_mode_writes_the_design_s_own_names(tmp_path):
    folder = write_random_model(tmp_path / "m", tiny.T2, seed=5)
    from flint_b200.weights.safetensors_io import SafetensorsFile
    names = set(SafetensorsFile(folder / "model.safetensors").names())
    assert names == set(tiny.tensor_shapes(tiny.T2))
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=8, max_slots=2, max_context=128)
    # two attention branches with different head sizes: two page groups; a state slab for every layer
    assert m.spec.architecture == "Tefovik" and len(m.cache.groups) == 2 and len(m.cache.state) == 4


def test_greedy_generation_through_the_engine_with_preemption(setup):
    which, cfg, folder, w, reqs, plain = setup
    prompts = [reqs["r2"], reqs["r3"][:14], reqs["r0"]]
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(10):
            t = int(torch.argmax(P.forward(cfg, w, toks)[-1]))
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages, ahead in ((16, True), (16, False), (3, True)):
        m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=n_pages, max_slots=4,
                       max_step_tokens=24, max_context=256, use_graphs=False)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16, run_ahead=ahead)
        assert eng.generate(prompts, 10) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0
