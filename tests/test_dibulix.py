"""Dibulix without a GPU: config.json is read into a typed configuration and
back, the model description names the tensors, parts and caches that the plain
implementation's weights ask for, bad configurations are refused, and the plain
implementation itself has the properties the engine is held to (a position
depends on its prefix alone; windows, the sink and the recurrences behave as
their equations say on inputs made to show it)."""
import json
import math

import numpy as np
import pytest

import plain_dibulix as plain
import tiny_dibulix as tiny
from alofa_b200.config.registry import get_architecture, read_model_config
from alofa_b200.errors import AlofaError
from alofa_b200.parts.base import PagedKV, PagedRows, Runtime, SlotState
from alofa_b200.parts.model import Model, expected_tensors
from alofa_b200.weights.loader import shape_fits


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("dibulix")
    return {name: tiny.write(base / name, name, seed=i) for i, name in enumerate(tiny.CONFIGS)}


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_config_is_read_and_written_back(folders, name):
    arch, cfg = read_model_config(folders[name])
    assert arch.name == "Dibulix"
    assert arch.to_json(cfg) == json.loads(json.dumps(tiny.CONFIGS[name]))
    assert cfg.width == tiny.CONFIGS[name]["width"] and [l.type for l in cfg.layers] == [l["type"] for l in tiny.CONFIGS[name]["layers"]]


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_the_description_names_the_tensors_parts_and_caches(folders, name):
    import torch

    raw = tiny.CONFIGS[name]
    arch, cfg = read_model_config(folders[name])
    spec = arch.build_spec(cfg)
    want = tiny.tensor_shapes(raw)
    got = expected_tensors(spec)
    assert set(got) == set(want)
    assert all(shape_fits(want[n], got[n].shape) for n in want), [n for n in want if not shape_fits(want[n], got[n].shape)]
    assert [e.layer for e in spec.run] == list(range(len(raw["layers"])))
    assert all(spec.layers[e.layer].block.kind == "hyper_residual" for e in spec.run)
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32))
    assert model.stream_copies == raw["streams"]
    plan = model.cache_plan()
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "parallel":
            a = m["left"]
            assert plan[i] == (PagedKV(a["kv_heads"], a["dim"], a["mask"]["size"], a["vdim"]), SlotState((m["right"]["width"],)))
        elif layer["type"] == "channel_delta":
            words = m["heads"] * m["vdim"] * m["dim"] + (m["conv"] - 1) * (2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])
            assert plan[i] == SlotState((words,))
        else:
            assert plan[i] == PagedRows(m["kv_rank"] + m["rot_dim"], m["mask"]["size"])


@pytest.mark.parametrize("broken", [
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][1]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][2]["mixer"]["left"].update(kv_heads=4),
    lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=5),
    lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][0]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][0]["mlp"].update(kind="routed"),
    lambda c: c.update(streams=9),
    lambda c: c.update(layers=[]),
    lambda c: c.pop("norm"),
    lambda c: c.pop("width"),
])
def test_bad_configs_are_refused(broken):
    raw = json.loads(json.dumps(tiny.CONFIGS["A"]))
    broken(raw)
    with pytest.raises(AlofaError) as err:
        get_architecture("Dibulix").read_config(raw, "test")
    assert err.value.code == "parse"


def test_a_config_without_streams_is_one_plain_residual():
    raw = json.loads(json.dumps(tiny.CONFIGS["B"]))
    del raw["streams"]
    arch = get_architecture("Dibulix")
    spec = arch.build_spec(arch.read_config(raw, "test"))
    assert not any(".hc" in n for n in expected_tensors(spec))
    # one stream whose connection weights are all 1 is the same function
    w = {n: v.double().numpy() for n, v in tiny.weights(tiny.CONFIGS["B"], 3).items()}
    ones = {n: np.ones_like(v) if ".hc" in n else v for n, v in w.items()}
    ids = tiny.tokens("B", 20)
    np.testing.assert_allclose(plain.forward(ones, tiny.CONFIGS["B"], ids), plain.forward(w_without_connections(ones), raw, ids), rtol=1e-10, atol=1e-10)


def w_without_connections(w):
    return {n: v for n, v in w.items() if ".hc" not in n}


def test_random_model_folder(tmp_path):
    """The package's seeded random mode writes a folder of this architecture
    that the plain reader takes, its stream-mixing matrices near the identity."""
    from alofa_b200.weights.random_init import write_random_model

    arch = get_architecture("Dibulix")
    folder = write_random_model(tmp_path / "m", "Dibulix", arch.read_config(tiny.CONFIGS["A"], "test"), seed=3)
    w, cfg = plain.load(folder)
    want = tiny.tensor_shapes(tiny.CONFIGS["A"])
    free = ("a1", "a2", "g1", "g2")  # their inner size is the file's own; the random mode picks one
    assert set(w) == set(want) and all(w[n].shape == want[n] for n in want if n.split(".")[-1] not in free)
    assert w["l1.mix.a1"].shape[0] == w["l1.mix.a2"].shape[1] and w["l1.mix.g1"].shape[0] == w["l1.mix.g2"].shape[1]
    assert np.abs(w["l0.hc1.mix"] - np.eye(2)).max() < 0.1
    assert np.isfinite(plain.forward(w, cfg, tiny.tokens("A", 9))).all()


# ---- the plain implementation's own properties ---------------------------------------------------------------
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_plain_positions_depend_on_their_prefix_alone(folders, name):
    w, cfg = plain.load(folders[name])
    ids = tiny.tokens(name, 45, seed=3)
    whole = plain.forward(w, cfg, ids)
    for n in (1, 2, 17, 44):
        assert np.abs(plain.forward(w, cfg, ids[:n]) - whole[:n]).max() < 1e-9


def test_plain_window_holds_itself_and_the_tokens_before_it():
    """One value stands out at position 3: with a window of 4 it is seen up to position 6, not at 7."""
    T, window = 12, 4
    q, k = np.zeros((T, 1, 2)), np.zeros((T, 1, 2))
    v = np.zeros((T, 1, 1))
    v[3] = 1.0
    out = plain.attend(q, k, v, 1.0, window, sink=False)[:, 0, 0]
    np.testing.assert_allclose(out[3:7], [1 / 4] * 4)
    assert out[7] == 0 and (out[:3] == 0).all()
    out = plain.attend(q, k, v, 1.0, None, sink=False)[:, 0, 0]
    np.testing.assert_allclose(out[3:], 1 / np.arange(4, T + 1))


def test_plain_sink_adds_one_to_the_denominator():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((5, 2, 3)), rng.standard_normal((5, 1, 3)), rng.standard_normal((5, 1, 4))
    with_sink, without = plain.attend(q, k, v, 0.7, None, sink=True), plain.attend(q, k, v, 0.7, None, sink=False)
    for i in range(5):
        for h in range(2):
            total = np.exp(k[: i + 1, 0] @ q[i, h] * 0.7).sum()
            np.testing.assert_allclose(with_sink[i, h], without[i, h] * total / (1.0 + total))
    # the first token alone: its weight is e^s / (1 + e^s), not 1
    s = float(k[0, 0] @ q[0, 0]) * 0.7
    np.testing.assert_allclose(with_sink[0, 0], v[0, 0] * math.exp(s) / (1 + math.exp(s)))


def test_plain_rotation_layouts_and_scaled_frequencies():
    x = np.arange(8, dtype=np.float64).reshape(1, 1, 8) + 1
    pairs = plain.rotate(x, [3], 4, 100.0, "pairs")
    halves = plain.rotate(x, [3], 4, 100.0, "halves")
    f = 100.0 ** (-2.0 * np.arange(2) / 4)
    c, s = np.cos(3 * f), np.sin(3 * f)
    np.testing.assert_allclose(pairs[0, 0], [1 * c[0] - 2 * s[0], 2 * c[0] + 1 * s[0], 3 * c[1] - 4 * s[1], 4 * c[1] + 3 * s[1], 5, 6, 7, 8])
    np.testing.assert_allclose(halves[0, 0], [1 * c[0] - 3 * s[0], 2 * c[1] - 4 * s[1], 3 * c[0] + 1 * s[0], 4 * c[1] + 2 * s[1], 5, 6, 7, 8])
    # scaled: the fastest pairs keep their frequency, the slowest are divided by the factor, both cos and sin grow by 0.1 ln(factor) + 1
    f, mag = plain.rotary_frequencies(32, 10000.0, {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0})
    plain_f = 10000.0 ** (-2.0 * np.arange(16) / 32)
    assert mag == pytest.approx(0.1 * math.log(8.0) + 1.0)
    assert f[0] == plain_f[0] and f[-1] == pytest.approx(plain_f[-1] / 8.0)
    ratio = plain_f / f
    assert (np.diff(ratio) >= -1e-12).all() and 1.0 < ratio[3] < 8.0


def test_plain_recurrences_written_as_a_carried_state():
    rng = np.random.default_rng(1)
    T, H, N, P = 9, 2, 5, 3
    q, k, v = rng.standard_normal((T, H, N)), rng.standard_normal((T, H, N)), rng.standard_normal((T, H, P))
    beta, g = rng.uniform(0.1, 0.9, (T, H)), rng.uniform(0.5, 1.0, (T, H, N))
    whole = plain.delta_rule(q, k, v, beta, g)
    # a prefix and the rest from the prefix's state: by hand for the first token after a cut
    np.testing.assert_allclose(plain.delta_rule(q[:4], k[:4], v[:4], beta[:4], g[:4]), whole[:4])
    # with beta = 1 and a unit key, the token's own value is read back exactly: S^T k = v
    k1 = plain.unit_vectors(k)
    back = plain.delta_rule(k1, k1, v, np.ones((T, H)), g)
    np.testing.assert_allclose(back, v, atol=1e-4)  # the unit norm's 1e-6 keeps |k|^2 a little under 1
    # minGRU: z = 1 replaces the state by the candidate, z = 0 keeps it
    u = np.array([[-2.0, 0.0, 3.0]])
    np.testing.assert_allclose(plain.min_gru_recurrence(np.full((1, 3), 50.0), u, np.full((1, 3), 50.0)) / 50.0, [[plain.sigmoid(-2.0), 0.5, 3.5]], rtol=1e-9)
    kept = plain.min_gru_recurrence(np.array([[50.0], [-50.0], [-50.0]]), np.array([[1.0], [7.0], [-7.0]]), np.full((3, 1), 50.0)) / 50.0
    np.testing.assert_allclose(kept[:, 0], [1.5, 1.5, 1.5], rtol=1e-9)
    # the convolution's last column is the token's own; before the start there are zeros
    x, taps = rng.standard_normal((6, 4)), rng.standard_normal((4, 3))
    conv = plain.short_convolution(x, taps)
    np.testing.assert_allclose(conv[0], plain.silu(taps[:, 2] * x[0]))
    np.testing.assert_allclose(conv[4], plain.silu(taps[:, 2] * x[4] + taps[:, 1] * x[3] + taps[:, 0] * x[2]))


def test_plain_connections_move_every_stream_from_the_old_ones():
    rng = np.random.default_rng(2)
    xs = [rng.standard_normal((3, 4)) for _ in range(3)]
    y, mix, out = rng.standard_normal((3, 4)), rng.standard_normal((3, 3)), rng.standard_normal(3)
    new = plain.connect(xs, y, mix, out)
    for t in range(3):
        np.testing.assert_allclose(new[t], mix[0, t] * xs[0] + mix[1, t] * xs[1] + mix[2, t] * xs[2] + out[t] * y)
    assert not np.allclose(new[1], plain.connect(xs, y, mix.T, out)[1])  # [from, to], not [to, from]
