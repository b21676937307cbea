"""Sagupel without a GPU: configuration, plan, what the cache is asked for, and the plain implementation's own
mechanisms against closed forms."""
import copy

import numpy as np
import pytest

import plain_sagupel as ps
import sagupel_helpers as sh
import questwend_b200  # noqa: F401
from questwend_b200.config import ConfigError
from questwend_b200.config.registry import config_from_dict, get_architecture
from questwend_b200.parts.base import KVSpec, StateSpec


def test_config_reads_every_size_and_round_trips():
    cfg = config_from_dict(sh.MIXED)
    assert cfg.architecture == "Sagupel" and cfg.width == 64 and cfg.vocab == 96 and cfg.canon_taps == 4
    assert cfg.postln_alpha == 1.5 and cfg.norm_eps == 2e-5
    assert cfg.layers[0]["mixer"]["decay"] == [0.875, 0.96875, 0.9921875] and cfg.layers[2]["mlp"] is None
    assert cfg.layers[1]["mixer"]["left"]["rot"] == {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0}}
    assert cfg.layers[5]["mixer"]["left"]["rot"] == {"base": 10000.0, "dims": 2} and cfg.layers[5]["mixer"]["left"]["softcap"] == 2.5
    assert cfg.layers[3]["mixer"]["mask"] == {"size": 70} and cfg.layers[1]["mlp"] == {"kind": "dense", "ff": 40, "limit": 0.8}
    assert config_from_dict(cfg.to_dict()) == cfg
    ones = config_from_dict(sh.ONES)
    assert ones.postln_alpha == 1.0 and ones.canon_taps == 1 and ones.layers[0]["mixer"]["rot"] is None
    assert ones.layers[3]["mixer"]["mask"] is None and ones.layers[1]["mixer"]["left"]["softcap"] == 0.0
    assert config_from_dict(ones.to_dict()) == ones
    no_conv = copy.deepcopy(sh.MIXED)
    del no_conv["canon"]
    assert config_from_dict(no_conv).canon_taps == 0


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "conv", "'type'"), (("layers", 2, "mixer", "kv_heads"), 4, "'heads'"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "'dims'"), (("layers", 0, "mixer", "rot", "dims"), 32, "'dims'"),
    (("layers", 0, "mixer", "decay"), [0.5, 0.5], "'decay'"), (("layers", 0, "mixer", "dim"), 600, "rows"),
    (("layers", 2, "mixer", "vdim"), 16, "'vdim'"), (("layers", 2, "mixer", "dim"), 264, "'vdim'"),
    (("layers", 1, "mixer", "right", "conv"), 17, "taps"), (("layers", 1, "mixer", "right", "kv_heads"), 3, "'heads'"),
    (("layers", 1, "mixer", "left", "softcap"), -2.0, "'softcap'"), (("layers", 2, "mixer", "mask", "size"), 0, "'size'"),
    (("layers", 1, "mixer", "left", "rot", "scaling", "factor"), 0.0, "'factor'"), (("canon", "taps"), 40, "taps"),
    (("layers", 0, "mlp", "kind"), "moe", "'kind'"), (("layers", 0, "mlp", "limit"), 0.0, "'limit'")])
def test_config_refuses_with_the_keys_name(path, value, word):
    bad = copy.deepcopy(sh.MIXED)
    at = bad
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    assert word in str(e.value)


def test_manifest_names_and_shapes():
    for cfgd in (sh.MIXED, sh.ONES):
        w = sh.draw_weights(cfgd)
        plan = get_architecture("Sagupel").plan(config_from_dict(cfgd))
        shapes = {t.name: tuple(t.shape) for t in plan.manifest() if not t.ignored}
        assert shapes == {k: v.shape for k, v in w.items()}
    no_conv = copy.deepcopy(sh.MIXED)
    del no_conv["canon"]
    names = {t.name for t in get_architecture("Sagupel").plan(config_from_dict(no_conv)).manifest()}
    assert "l0.canon1" not in names and "l0.mix.q" in names


def test_what_the_cache_is_asked_for():
    import torch
    from questwend_b200.engine.model import Model
    from questwend_b200.parts.base import Runtime
    model = Model(get_architecture("Sagupel").plan(config_from_dict(sh.MIXED)), Runtime(torch.device("cpu"), torch.bfloat16))
    units = model.cache_units()
    assert len(units) == 7
    tail = StateSpec((3, 64), torch.float32)                    # every layer keeps the last inputs of its input convolution
    kv, state, cache_of = units[0]
    assert kv is None and state == (tail, StateSpec((3, 8, 16), torch.float32)) and cache_of is None
    kv, state, _ = units[1]
    assert kv == KVSpec(2, 24, 0, value_dim=24)
    assert state == (tail, StateSpec((3, 2 * 16 + 2 * 24), torch.float32), StateSpec((2, 24, 16), torch.float32))
    assert units[2][0] == KVSpec(2, 8, 20, value_dim=8) and units[2][1] == tail
    assert units[3][0] == KVSpec(3, 40, 70, value_dim=40)
    ones = Model(get_architecture("Sagupel").plan(config_from_dict(sh.ONES)), Runtime(torch.device("cpu"), torch.float32))
    units = ones.cache_units()
    assert units[0][1] == StateSpec((1, 8, 8), torch.float32)           # one tap: no tail, the matrix only
    assert units[1][1] == StateSpec((1, 8, 8), torch.float32) and units[2][1] is None and units[3][0].window == 0


def test_random_weights_folder_round_trips(tmp_path):
    import questwend_b200 as qw
    from questwend_b200.config.registry import load_config
    cfg = config_from_dict(sh.MIXED)
    qw.write_model_folder(str(tmp_path), cfg, seed=3, dtype="bfloat16")
    assert load_config(str(tmp_path)) == cfg


# ----------------------------------------------------------------------------- the plain implementation's mechanisms
def test_plain_rotation_and_convolution():
    x = np.random.default_rng(0).standard_normal((5, 3, 12))
    y = ps.rotate_halves(x, np.arange(5), 8, 100.0, 2.0)
    assert np.array_equal(y[..., 8:], x[..., 8:]) and np.allclose(y[0], x[0])
    for i in range(4):
        ang = 3 * 100.0 ** (-2.0 * i / 8) / 2.0
        assert np.allclose(y[3, :, i], x[3, :, i] * np.cos(ang) - x[3, :, i + 4] * np.sin(ang))
        assert np.allclose(y[3, :, i + 4], x[3, :, i + 4] * np.cos(ang) + x[3, :, i] * np.sin(ang))
    assert np.array_equal(ps.rotate_halves(x, np.arange(5), 0, 100.0), x)
    u = np.arange(12.0).reshape(6, 2)
    taps = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = ps.causal_conv(u, taps)
    assert np.array_equal(y[:, 1], u[:, 1]) and y[0, 0] == 0.0 and y[1, 0] == 200.0 and y[3, 0] == 2.0 + 40.0 + 600.0
    assert np.array_equal(ps.causal_conv(u, taps, plus_input=True), u + y)


def test_plain_retention_against_its_sum_form():
    """o_t = sum_j decay^(t - j) (q_t . k_j) v_j."""
    rng = np.random.default_rng(2)
    D, m = 6, {"heads": 2, "dim": 4, "vdim": 3, "decay": [0.5, 0.9], "rot": {"base": 50.0, "dims": 2}}
    w = {"q": rng.standard_normal((8, D)), "k": rng.standard_normal((8, D)), "v": rng.standard_normal((6, D)),
         "g": rng.standard_normal((6, D)), "o": np.eye(6)}
    h = rng.standard_normal((7, D))
    got = ps.retention(h, m, w, "", 1e-6)
    pos = np.arange(7)
    q = ps.rotate_halves((h @ w["q"].T).reshape(7, 2, 4), pos, 2, 50.0)
    k = ps.rotate_halves((h @ w["k"].T).reshape(7, 2, 4), pos, 2, 50.0) / 2.0
    v = (h @ w["v"].T).reshape(7, 2, 3)
    o = np.zeros((7, 2, 3))
    for hd in range(2):
        for t in range(7):
            for j in range(t + 1):
                o[t, hd] += m["decay"][hd] ** (t - j) * (q[t, hd] @ k[j, hd]) * v[j, hd]
    assert np.allclose(got, ps.unit_rms(o, 1e-6).reshape(7, 6) * ps.silu(h @ w["g"].T))


def test_plain_softmax_attention_window_sink_slopes_and_mix():
    rng = np.random.default_rng(3)
    D, m = 6, {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.7, "mask": {"size": 3}}
    w = {"q": rng.standard_normal((8, D)), "k": rng.standard_normal((4, D)), "q.norm": np.ones(4), "k.norm": np.ones(4),
         "sink": np.array([0.3, -1.0]), "o": np.eye(8)}
    h = rng.standard_normal((6, D))
    got = ps.window_attention(h, m, w, "", 1e-6).reshape(6, 2, 4)
    k_raw = h @ w["k"].T
    q, k = ps.unit_rms((h @ w["q"].T).reshape(6, 2, 4), 1e-6), ps.unit_rms(k_raw, 1e-6)
    for hd in range(2):
        slope = 2.0 ** (-8.0 * (hd + 1) / 2)
        t = 5
        e = np.array([np.exp(0.7 * q[t, hd] @ k[j] - slope * (t - j)) for j in (3, 4, 5)])
        want = (e[:, None] * k_raw[3:6]).sum(0) / (e.sum() + np.exp(w["sink"][hd]))
        assert np.allclose(got[t, hd], want)
    # a mix that is the identity, a number per head that is 1 and a huge cap change nothing; a swap of two heads' weights does
    m2 = {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.7, "softcap": 1e6, "rot": {"base": 10.0, "dims": 0}}
    w2 = {"q": w["q"], "k": rng.standard_normal((8, D)), "q.b": np.zeros(8), "k.b": np.zeros(8), "q.norm": np.ones(4),
          "k.norm": np.ones(4), "temp": np.ones(2), "talk": np.eye(2), "g": np.zeros((2, D)), "o": np.eye(8)}
    kw = dict(biases=True, rotation=True, softcap=True, temp=True, talk=True, gate=True)
    a = ps.softmax_attention(h, m2, w2, "", 1e-6, **kw)
    b = ps.softmax_attention(h, m2, w2, "", 1e-6)
    assert np.allclose(a, 0.5 * b)
    w2["talk"] = np.array([[0.0, 1.0], [1.0, 0.0]])
    c = ps.softmax_attention(h, m2, w2, "", 1e-6, **kw).reshape(6, 2, 4)
    k2 = (h @ w2["k"].T).reshape(6, 2, 4)
    q2, kn = ps.unit_rms((h @ w["q"].T).reshape(6, 2, 4), 1e-6), ps.unit_rms(k2, 1e-6)
    s = np.array([0.7 * q2[4, 1] @ kn[j, 1] for j in range(5)])
    p = np.exp(s - s.max()) / np.exp(s - s.max()).sum()
    assert np.allclose(c[4, 0], 0.5 * (p[:, None] * k2[:5, 0]).sum(0))      # head 0: head 1's weights on head 0's own values


def test_plain_delta_rule_and_feed_forward():
    rng = np.random.default_rng(4)
    D, m = 6, {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 2, "conv": 2}
    w = {k: rng.standard_normal(s) for k, s in (("q", (3, D)), ("k", (3, D)), ("v", (4, D)), ("q.conv", (3, 2)), ("k.conv", (3, 2)),
                                                ("v.conv", (4, 2)), ("a", (2, D)), ("g", (4, D)), ("A_log", 2), ("dt_bias", 2))}
    w.update({"b": np.zeros((2, D)), "norm": np.ones(2), "o": np.eye(4)})
    h = rng.standard_normal((5, D))
    got = ps.gated_delta(h, m, w, "", 1e-6)
    # one token: S = beta k v^T with beta = 1/2, o = S^T q = (k . q) v / 2
    q, k, v = (ps.silu((h[:1] @ w[n].T) * w[n + ".conv"][:, 1]) for n in "qkv")
    q, k = q / np.sqrt((q * q).sum() + 1e-6) / np.sqrt(3.0), k / np.sqrt((k * k).sum() + 1e-6)
    o = 0.5 * (k @ q.T) * v.reshape(2, 2)
    assert np.allclose(got[0], (ps.unit_rms(o, 1e-6).reshape(4) * ps.silu(h[0] @ w["g"].T)))
    mlp = {"ff": 3, "limit": 1.0}
    wf = {"gate": np.array([[5.0, 0.0], [0.5, 0.0], [-3.0, 0.0]]), "up": np.array([[0.0, 4.0], [0.0, -4.0], [0.0, 0.25]]), "down": np.eye(3)}
    y = ps.feed_forward(np.array([[1.0, 1.0]]), mlp, wf, "")
    assert np.allclose(y[0], [ps.sigmoid(1.702) * 2.0, 0.0, -3.0 * ps.sigmoid(-3.0 * 1.702) * 1.25])
