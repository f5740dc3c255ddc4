"""Kikerax without a GPU: config.json is read into a typed configuration and
back, the model description names the tensors, parts and caches that the plain
implementation's weights ask for, bad configurations are refused, and the plain
implementation itself has the properties the engine is held to (a position
depends on its prefix alone; chunks, the two maps, the gates, the recurrence
and the router behave as their equations say on inputs made to show it)."""
import json
import math

import numpy as np
import pytest

import plain_kikerax as plain
import tiny_kikerax as tiny
from alofa_b200.config.registry import get_architecture, read_model_config
from alofa_b200.errors import AlofaError
from alofa_b200.parts.base import PagedKV, Runtime, SlotState
from alofa_b200.parts.model import Model, expected_tensors


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("kikerax")
    return {name: tiny.write(base / name, name, seed=i) for i, name in enumerate(tiny.CONFIGS)}


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_config_is_read_and_written_back(folders, name):
    arch, cfg = read_model_config(folders[name])
    assert arch.name == "Kikerax"
    assert arch.to_json(cfg) == json.loads(json.dumps(tiny.CONFIGS[name]))
    assert cfg.width == tiny.CONFIGS[name]["width"] and [l.type for l in cfg.layers] == [l["type"] for l in tiny.CONFIGS[name]["layers"]]


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_the_description_names_the_tensors_parts_and_caches(folders, name):
    import torch

    raw = tiny.CONFIGS[name]
    arch, cfg = read_model_config(folders[name])
    spec = arch.build_spec(cfg)
    want = tiny.tensor_shapes(raw)
    got = {n: tuple(t.shape) for n, t in expected_tensors(spec).items()}
    assert got == want
    assert [e.layer for e in spec.run] == list(range(len(raw["layers"])))
    assert all(spec.layers[e.layer].block.kind == "postnorm_residual" for e in spec.run)
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32))
    plan = model.cache_plan()
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            # keys and values of the same size (the values are the keys before their norm), every key kept; the state, then the convolution's last inputs
            assert plan[i] == (PagedKV(a["kv_heads"], a["dim"], None, a["dim"]), SlotState((r["width"] * r["conv"],)))
        else:
            # two keys a key head, one value; a chunk's pages are given back like a window's
            assert plan[i] == PagedKV(2 * m["kv_heads"], m["dim"], m.get("mask", {}).get("size"), m["vdim"], m["kv_heads"])
    head = spec.head.params
    assert head["tied_to"] == "embed" and head["softcap"] == raw.get("logit_softcap")


@pytest.mark.parametrize("broken", [
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"].pop("diff"),
    lambda c: c["layers"][0]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][0]["mlp"].update(kind="routed"),
    lambda c: c["layers"][1]["mixer"]["left"].update(vdim=8),
    lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4),
    lambda c: c["layers"][1]["mixer"]["right"].update(blocks=5),
    lambda c: c["layers"][1]["mixer"]["left"]["q_temp"].update(every=0),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=7),
    lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4),
    lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=0),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=5),  # two groups of two experts hold four
    lambda c: c.update(logit_softcap=0.0),
    lambda c: c.update(layers=[]),
    lambda c: c.pop("norm"),
    lambda c: c.pop("width"),
])
def test_bad_configs_are_refused(broken):
    raw = json.loads(json.dumps(tiny.CONFIGS["A"]))
    broken(raw)
    with pytest.raises(AlofaError) as err:
        get_architecture("Kikerax").read_config(raw, "test")
    assert err.value.code == "parse"


def test_keys_that_switch_a_mechanism_on_may_be_absent():
    raw = json.loads(json.dumps(tiny.CONFIGS["B"]))
    arch = get_architecture("Kikerax")
    cfg = arch.read_config(raw, "test")
    assert cfg.logit_softcap is None and cfg.layers[0].mixer.left.softcap is None and cfg.layers[0].mixer.left.q_temp is None
    assert cfg.layers[1].mixer.rot is None and cfg.layers[1].mixer.chunk is None
    assert cfg.layers[0].mlp.groups is None and cfg.layers[0].mlp.shared_ff == 0
    spec = arch.build_spec(cfg)
    assert not any("shared" in n for n in expected_tensors(spec) if n.startswith("l0."))


def test_random_model_folder(tmp_path):
    """The package's seeded random mode writes a folder of this architecture that the plain reader takes."""
    from alofa_b200.weights.random_init import write_random_model

    arch = get_architecture("Kikerax")
    folder = write_random_model(tmp_path / "m", "Kikerax", arch.read_config(tiny.CONFIGS["A"], "test"), seed=3)
    w, cfg = plain.load(folder)
    want = tiny.tensor_shapes(tiny.CONFIGS["A"])
    assert {n: v.shape for n, v in w.items()} == want
    assert np.isfinite(plain.forward(w, cfg, tiny.tokens("A", 9))).all()


# ---- the plain implementation's own properties ---------------------------------------------------------------
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_plain_positions_depend_on_their_prefix_alone(folders, name):
    w, cfg = plain.load(folders[name])
    ids = tiny.tokens(name, 45)
    whole = plain.forward(w, cfg, ids)
    np.testing.assert_allclose(plain.forward(w, cfg, ids[:27]), whole[:27], rtol=1e-9, atol=1e-9)
    cap = cfg.get("logit_softcap")
    assert cap is None or np.abs(whole).max() < cap


def test_plain_chunks_are_counted_from_the_start():
    m = plain.chunk_mask(10, 4)
    assert m[3, :4].all() and not m[4, :4].any() and m[4, 4] and m[7, 4:8].all() and not m[7, 8:].any() and m[9, 8:10].all() and not m[9, :8].any()
    assert (plain.chunk_mask(6, 100) == plain.causal_mask(6)).all()
    assert (plain.chunk_mask(5, 1) == np.eye(5, dtype=bool)).all()


def _attention_weights(rng, width, m):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": rng.standard_normal((H * 2 * d, width)), "k": rng.standard_normal((G * 2 * d, width)), "v": rng.standard_normal((G * dv, width)),
         "q.b": rng.standard_normal(H * 2 * d), "k.b": rng.standard_normal(G * 2 * d), "v.b": rng.standard_normal(G * dv), "q.norm": np.ones(d), "k.norm": np.ones(d),
         "lq1": np.zeros(d), "lk1": np.zeros(d), "lq2": np.zeros(d), "lk2": np.zeros(d), "g": np.zeros((H, width)), "o": np.eye(H * dv, H * dv)[: H * dv], "o.b": np.zeros(H * dv)}
    return {"a." + n: v for n, v in w.items()}


def test_plain_two_maps_are_subtracted_and_normed():
    rng = np.random.default_rng(0)
    width, m = 12, {"heads": 2, "kv_heads": 1, "dim": 6, "vdim": 6, "scale": 0.7, "diff": 0.25}
    w = _attention_weights(rng, width, m)
    w["a.o"] = np.eye(12)
    h = rng.standard_normal((7, width))
    out = plain.differential_attention(w, "a.", m, h, 1e-6).reshape(7, 2, 6)
    # lambda = e^0 - e^0 + diff; after the norm every head has root mean square (1 - diff); the gate is sigmoid(0) = 1/2
    assert plain.difference_weight(w, "a.", 0.25) == pytest.approx(0.25)
    np.testing.assert_allclose(np.sqrt((out ** 2).mean(axis=-1)), 0.5 * 0.75, rtol=1e-4)
    # the first token sees itself alone in both maps: o = (1 - lambda) v, whatever q and k are
    v0 = h[0] @ w["a.v"].T + w["a.v.b"]
    np.testing.assert_allclose(out[0, 0], 0.5 * 0.75 * v0 / np.sqrt((v0 ** 2).mean() + 1e-6 / 0.75 ** 2), rtol=1e-6)
    # equal maps and lambda = 1 would give zero: with lq1 . lk1 = ln 2 lambda grows by one
    w2 = dict(w)
    w2["a.lq1"], w2["a.lk1"] = np.full(6, math.log(2.0) / 6), np.ones(6)
    assert plain.difference_weight(w2, "a.", 0.25) == pytest.approx(1.25)


def test_plain_values_are_the_keys_before_their_norm():
    rng = np.random.default_rng(1)
    width, m = 8, {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 1.0}
    w = {"a.q": rng.standard_normal((8, width)), "a.k": rng.standard_normal((8, width)), "a.q.norm": np.ones(4), "a.k.norm": 3.0 * np.ones(4), "a.g": np.zeros((2, width)),
         "a.o": np.eye(8)}
    h = rng.standard_normal((5, width))
    out = plain.keyed_attention(w, "a.", m, h, 1e-6)
    # the first token: its own key as projected (not normed, not times the norm's weight), times the gate 1/2
    np.testing.assert_allclose(out[0], 0.5 * (h[0] @ w["a.k"].T), rtol=1e-9)
    # temperature: at position p the query is multiplied by 1 + coef ln(floor((p + 1) / every) + 1): nothing before position every - 1
    m2 = dict(m, q_temp={"coef": 0.5, "every": 3})
    warm = plain.keyed_attention(w, "a.", m2, h, 1e-6)
    np.testing.assert_allclose(warm[:2], out[:2], rtol=1e-12)
    assert not np.allclose(warm[2], out[2])
    # a cap far above the scores changes nothing, a small one flattens the softmax towards the mean of the values
    np.testing.assert_allclose(plain.keyed_attention(w, "a.", dict(m, softcap=1e6), h, 1e-6), out, rtol=1e-6)
    flat = plain.keyed_attention(w, "a.", dict(m, softcap=1e-6), h, 1e-6)
    np.testing.assert_allclose(flat[4], 0.5 * (h @ w["a.k"].T).mean(axis=0), rtol=1e-4)


def test_plain_recurrent_unit_written_as_a_carried_state():
    rng = np.random.default_rng(2)
    width, W, B, K = 6, 8, 2, 3
    m = {"width": W, "blocks": B, "conv": K}
    w = {"r.y": rng.standard_normal((W, width)), "r.y.b": rng.standard_normal(W), "r.x": rng.standard_normal((W, width)), "r.x.b": rng.standard_normal(W),
         "r.conv": rng.standard_normal((W, K)), "r.conv.b": rng.standard_normal(W), "r.ra": rng.standard_normal((B, 4, 4)), "r.ra.b": rng.standard_normal((B, 4)),
         "r.ri": rng.standard_normal((B, 4, 4)), "r.ri.b": rng.standard_normal((B, 4)), "r.lam": rng.uniform(-4, 0, W), "r.o": np.eye(W)}
    h = rng.standard_normal((9, width))
    out = plain.gated_recurrent_unit(w, "r.", m, h)
    np.testing.assert_allclose(plain.gated_recurrent_unit(w, "r.", m, h[:5]), out[:5], rtol=1e-12)
    # by hand for the first two tokens: zeros before the start in the convolution, S = 0 before the first token (which is no special case)
    x = h @ w["r.x"].T + w["r.x.b"]
    u0 = w["r.conv"][:, 2] * x[0] + w["r.conv.b"]
    u1 = w["r.conv"][:, 2] * x[1] + w["r.conv"][:, 1] * x[0] + w["r.conv.b"]
    S, outs = np.zeros(W), []
    for t, u in enumerate((u0, u1)):
        r = np.concatenate([plain.sigmoid(w["r.ra"][b] @ u[4 * b : 4 * b + 4] + w["r.ra.b"][b]) for b in range(B)])  # block b reads its own channels only
        i = np.concatenate([plain.sigmoid(w["r.ri"][b] @ u[4 * b : 4 * b + 4] + w["r.ri.b"][b]) for b in range(B)])
        a = np.exp(-8.0 * r * np.log1p(np.exp(w["r.lam"])))
        S = a * S + np.sqrt(1 - a * a) * i * u
        outs.append(S * plain.gelu_tanh(h[t] @ w["r.y"].T + w["r.y.b"]))
    np.testing.assert_allclose(out[:2], outs, rtol=1e-9)


def test_plain_router_takes_the_best_groups_by_their_two_largest():
    width = 4
    h = np.eye(width)[:1] * 0.0  # logits 0: every score 1/2, so the correction alone decides
    w = {"m.router": np.zeros((6, width)), "m.correction": np.array([0.9, -5.0, 0.5, 0.45, 0.4, 0.42])}
    r = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    # groups (0, 1), (2, 3), (4, 5): sums of the two largest choice scores are -3.1, 1.95, 1.82: only experts 2 and 3 can be chosen, although expert 0 is the largest
    chosen, weights, margin = plain.route(w, "m.", r, h)
    assert sorted(chosen[0]) == [2, 3]
    np.testing.assert_allclose(weights[0], [1.5, 1.5])  # the scores themselves (1/2 each), over their sum, times the scale
    assert margin[0] == pytest.approx(1.95 - 1.82)
    # with every group kept the largest two win
    chosen, _, _ = plain.route(w, "m.", dict(r, groups={"count": 3, "keep": 3}), h)
    assert sorted(chosen[0]) == [0, 2]
    # negative choice scores: an expert outside the kept groups is never taken, although 0 would beat them
    w["m.correction"] = np.array([-0.6, -0.7, -5.0, -6.0, -5.5, -5.6])
    chosen, _, _ = plain.route(w, "m.", dict(r, top=2), h)
    assert sorted(chosen[0]) == [0, 1]
