"""Punolix without a GPU: configuration, plan and schedule, what the cache is asked for, and the plain implementation's
own mechanisms against closed forms."""
import copy

import numpy as np
import pytest

import plain_punolix as pp
import punolix_helpers as ph
import questwend_b200  # noqa: F401
from questwend_b200.config import ConfigError
from questwend_b200.config.registry import config_from_dict, get_architecture
from questwend_b200.parts.base import KVSpec, StateSpec


def shaped(cfgd, w):
    return config_from_dict(cfgd).with_tensor_shapes({k: v.shape for k, v in w.items()})


def test_config_reads_every_size_and_round_trips():
    cfg = config_from_dict(ph.MIXED)
    assert cfg.architecture == "Punolix" and cfg.width == 64 and cfg.vocab == 96 and cfg.loop == (1, 4, 3)
    assert cfg.embedding_scale == 3.0 and cfg.residual_mult == 0.6
    assert cfg.layers[1]["mixer"]["left"]["mask"] == {"size": 20} and cfg.layers[2]["mlp"] is None
    assert cfg.layers[1]["mixer"]["left"]["rot"]["scaling"] == {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}
    assert cfg.layers[0]["mixer"]["softcap"] == 6.0 and cfg.layers[4]["mixer"]["softcap"] == 0.0
    assert config_from_dict(cfg.to_dict()) == cfg
    ones = config_from_dict(ph.ONES)
    assert ones.embedding_scale == 1.0 and ones.residual_mult == 1.0 and ones.layers[2]["mixer"]["left"]["mask"] is None
    assert ones.layers[2]["mixer"]["left"]["conv"] == 0
    with_rank = shaped(ph.MIXED, ph.draw_weights(ph.MIXED, rank=7))
    assert with_rank.layers[1]["mixer"]["right"]["rank"] == 7 and "rank" not in cfg.layers[1]["mixer"]["right"]


def test_schedule_repeats_the_looped_run_and_opens_every_pass():
    assert [i for i, _ in config_from_dict(ph.MIXED).passes()] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert config_from_dict(ph.MIXED).passes() == pp.runs(ph.MIXED)
    assert config_from_dict(ph.ONES).passes() == [(0, 0), (1, None), (2, None)]
    no_loop = copy.deepcopy(ph.MIXED)
    del no_loop["loop"]
    assert config_from_dict(no_loop).passes() == [(i, None) for i in range(5)]
    plan = get_architecture("Punolix").plan(config_from_dict(ph.MIXED))
    assert [r.layer for r in plan.schedule] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    opens = [(i, r.before.params["row"], r.before.params["add_embedding"]) for i, r in enumerate(plan.schedule) if r.before is not None]
    assert opens == [(1, 0, False), (4, 1, True), (7, 2, True)]
    assert all(r.before.params["scale"] == 3.0 and r.before.params["rows"] == 3 for r in plan.schedule if r.before is not None)
    assert "loop.step" not in {t.name for t in get_architecture("Punolix").plan(config_from_dict(no_loop)).manifest()}


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "conv", "'type'"), (("layers", 0, "mixer", "kv_heads"), 3, "'heads'"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "'dims'"), (("layers", 0, "mixer", "rot", "dims"), 32, "'dims'"),
    (("layers", 0, "mixer", "vdim"), 264, "value sizes"), (("layers", 1, "mixer", "left", "conv"), 17, "taps"),
    (("layers", 1, "mixer", "left", "dim"), 300, "key sizes"), (("layers", 1, "mixer", "right", "dim"), 600, "rows"),
    (("layers", 1, "mixer", "right", "tau"), 0.0, "'tau'"), (("layers", 0, "mixer", "diff"), 1.0, "'diff'"),
    (("layers", 0, "mixer", "softcap"), -2.0, "'softcap'"), (("layers", 1, "mixer", "left", "mask", "size"), 0, "'size'"),
    (("layers", 1, "mixer", "left", "rot", "scaling", "high"), 1.0, "'high'"),
    (("loop", "stop"), 6, "loop"), (("loop", "times"), 0, "'times'"), (("layers", 0, "mlp", "kind"), "moe", "'kind'")])
def test_config_refuses_with_the_keys_name(path, value, word):
    bad = copy.deepcopy(ph.MIXED)
    at = bad
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    assert word in str(e.value)


def test_manifest_names_and_shapes():
    for cfgd in (ph.MIXED, ph.ONES):
        w = ph.draw_weights(cfgd)
        plan = get_architecture("Punolix").plan(shaped(cfgd, w))
        shapes = {t.name: tuple(t.shape) for t in plan.manifest() if not t.ignored}
        assert shapes == {k: v.shape for k, v in w.items()}


def test_what_the_cache_is_asked_for():
    import torch
    from questwend_b200.engine.model import Model
    from questwend_b200.parts.base import Runtime
    w = ph.draw_weights(ph.MIXED)
    model = Model(get_architecture("Punolix").plan(shaped(ph.MIXED, w)), Runtime(torch.device("cpu"), torch.bfloat16))
    units = model.cache_units()
    assert len(units) == 11
    kv, state, cache_of = units[0]
    assert kv == KVSpec(2, 2 * 16, 0, value_dim=24) and state is None and cache_of is None      # both maps of a key head in one row
    kv, state, _ = units[1]
    assert kv == KVSpec(2, 24, 0, value_dim=16)
    channels = 4 * 24 + 2 * 24 + 2 * 16
    assert state == (StateSpec((2, channels), torch.float32), StateSpec((2, 24, 16), torch.float32))
    assert units[4][:2] == units[1][:2] and units[7][:2] == units[1][:2]                          # a pass has a cache and state of its own
    ones = Model(get_architecture("Punolix").plan(shaped(ph.ONES, ph.draw_weights(ph.ONES))), Runtime(torch.device("cpu"), torch.float32))
    assert ones.cache_units()[2][1] == StateSpec((2, 8, 8), torch.float32)                        # no convolution: the matrix only


def test_random_weights_folder_round_trips(tmp_path):
    import questwend_b200 as qw
    from questwend_b200.config.registry import load_config
    cfg = config_from_dict(ph.MIXED)
    qw.write_model_folder(str(tmp_path), cfg, seed=3, dtype="bfloat16")
    again = load_config(str(tmp_path))
    assert again.layers[1]["mixer"]["right"]["rank"] == 16 and again.loop == cfg.loop


# ----------------------------------------------------------------------------- the plain implementation's mechanisms
def test_plain_rotation_layouts_and_bands():
    x = np.random.default_rng(0).standard_normal((5, 3, 12))
    f = pp.frequencies(100.0, 8)
    assert np.allclose(f, [1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75])
    for layout, pairs in (("interleaved", [(0, 1), (2, 3), (4, 5), (6, 7)]), ("halves", [(0, 4), (1, 5), (2, 6), (3, 7)])):
        y = pp.rotate(x, np.arange(5), f, 8, layout)
        assert np.array_equal(y[..., 8:], x[..., 8:]) and np.allclose(y[0], x[0])
        for i, (a, b) in enumerate(pairs):
            ang = 3 * f[i]
            assert np.allclose(y[3, :, a], x[3, :, a] * np.cos(ang) - x[3, :, b] * np.sin(ang))
            assert np.allclose(y[3, :, b], x[3, :, b] * np.cos(ang) + x[3, :, a] * np.sin(ang))
    scaled = pp.frequencies(10000.0, 8, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
    plain = pp.frequencies(10000.0, 8)
    assert scaled[0] == plain[0] and scaled[3] == plain[3] / 4.0 and plain[1] / 4.0 < scaled[1] < plain[1]


def test_plain_convolution_mask_and_recurrence():
    u = np.arange(12.0).reshape(6, 2)
    taps = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = pp.short_convolution(u, taps)
    assert np.array_equal(y[:, 1], u[:, 1]) and y[0, 0] == 0.0 and y[1, 0] == 200.0 and y[3, 0] == 2.0 + 40.0 + 600.0
    m = pp.visible(7, 3)
    assert m[2, 0] and m[3, 3] and not m[3, 2] and not m[2, 3] and m[5, 3] and not m[6, 5] and pp.visible(4)[3, 0]
    # gated linear attention against its sum form: o_t = sum_j (prod_{j < i <= t} alpha_i) * k_j (q_t . that) v_j
    rng = np.random.default_rng(2)
    D, mx = 6, {"heads": 1, "dim": 3, "vdim": 2, "tau": 2.0}
    w = {"q": rng.standard_normal((3, D)), "k": rng.standard_normal((3, D)), "v": rng.standard_normal((2, D)), "g": rng.standard_normal((2, D)),
         "a1": rng.standard_normal((2, D)), "a2": rng.standard_normal((3, 2)), "a2.b": rng.standard_normal(3), "norm": np.ones(2),
         "o": np.eye(2)}
    h = rng.standard_normal((5, D))
    got = pp.gated_linear_attention(h, w, "", mx, 1e-6)
    q, k, v = h @ w["q"].T / np.sqrt(3), h @ w["k"].T, h @ w["v"].T
    alpha = pp.sigmoid(h @ w["a1"].T @ w["a2"].T + w["a2.b"]) ** 0.5
    o = np.zeros((5, 2))
    for t in range(5):
        for j in range(t + 1):
            o[t] += ((q[t] * np.prod(alpha[j + 1:t + 1], axis=0)) @ k[j]) * v[j]
    assert np.allclose(got, pp.unit_rms(o, 1e-6) * pp.silu(h @ w["g"].T))
