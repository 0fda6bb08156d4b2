"""Purusun without a GPU: configuration, the model description built from it
(run order of a looped stretch, cache needs, tensor names), the random-weights
writer and the loader's one error, the window's page bookkeeping with kept
first pages; the plain implementation against closed forms; and that the test
models' weights make every mechanism show."""

import copy
import json
import math
import os

import numpy as np
import pytest

import plain_purusun as pp
import purusun_models as pm


def spec_of(cfg):
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config.registry import spec_from_config_dict

    return spec_from_config_dict(cfg)


def test_config_to_model_description():
    from reflex_b200.engine.model import expected_tensors

    typed, spec = spec_of(pm.PUR_A)
    assert spec.architecture == "purusun" and spec.vocab_size == 97 and spec.hidden_size == 64
    assert spec.residual_streams == 2 and spec.tie_word_embeddings
    assert [l.block for l in spec.layers] == ["hyper_prenorm"] * 3
    assert [l.mixer.kind for l in spec.layers] == ["gqa_attention", "selective_scan", "gqa_attention"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == ["relu2", "relu2", None]
    a = spec.layers[0].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.window, a.scale) == (4, 2, 16, 20, 0.9)
    assert a.param("keep_first") == 3 and a.param("values_are_keys") and a.param("output_gate")
    assert a.position.kind == "rope_scaled" and a.position.rotary_dim == 8 and dict(a.position.params)["factor"] == 8.0
    assert spec.layers[2].mixer.position.kind == "rope_neox"
    s = spec.layers[1].mixer
    assert (s.param("inner"), s.param("state"), s.param("dt_rank"), s.param("taps")) == (48, 8, 4, 3)
    assert spec.layers[0].mixer_norm.weight_offset == 1.0 and spec.final_norm.weight_offset == 1.0
    assert a.qk_norm.weight_offset == 0.0
    # layers 0 and 1 twice, then layer 2; a cache entry per run
    assert [(r.layer, r.cache, r.mixes_input) for r in spec.run_order] == \
        [(0, 0, False), (1, 1, False), (0, 2, False), (1, 3, False), (2, 4, False)]
    names = expected_tensors(spec)
    for n in ("embed", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.g",
              "l0.mix.o", "l0.mlp.up", "l0.mlp.down", "l0.ls1", "l0.ls2", "l0.hc1.in", "l0.hc1.out", "l0.hc1.mix",
              "l0.hc2.mix", "l1.mix.in", "l1.mix.conv", "l1.mix.conv.b", "l1.mix.x", "l1.mix.dt", "l1.mix.dt.b",
              "l1.mix.A_log", "l1.mix.D", "l1.mix.o", "l2.hc1.in", "final.norm"):
        assert n in names, n
    for n in ("l0.mix.v", "head", "l2.norm2", "l2.ls2", "l2.hc2.in", "l2.mlp.up", "l1.mix.q"):
        assert n not in names, n
    assert names["l0.mix.k"][1].shape == (32, 64) and names["l0.mix.g"][1].shape == (64, 64)
    assert names["l0.hc1.mix"][1].shape == (2, 2) and names["l0.hc2.in"][1].shape == (2,)
    assert names["l1.mix.in"][1].shape == (96, 64) and names["l1.mix.x"][1].shape == (4 + 16, 48)
    assert names["l1.mix.conv"][1].shape == (48, 3) and names["l1.mix.A_log"][1].shape == (48, 8)
    assert typed.to_dict()["loop"] == {"start": 0, "stop": 2, "times": 2} and typed.to_dict()["streams"] == 2


def test_models_without_streams_a_loop_a_window_or_a_rotation():
    from reflex_b200.cache.specs import KVSpec, StateSpec
    from reflex_b200.engine.model import CausalLM, expected_tensors
    import torch

    typed, spec = spec_of(pm.PUR_B)
    assert spec.residual_streams == 1 and len(spec.run_order) == 3 and "streams" not in typed.to_dict()
    names = expected_tensors(spec)
    assert "l0.hc1.in" not in names and "l0.ls1" in names
    a = spec.layers[0].mixer
    assert a.window is None and a.position is None and a.param("keep_first") == 0
    model = CausalLM(spec, torch.float32, "cpu")
    needs = model.cache_entry_specs()
    assert needs[0] == KVSpec(1, 8, None) and needs[2] == KVSpec(2, 32, 5, keep_first=0)
    assert needs[1] == StateSpec((24,), "float32")  # one tap: no filter inputs, one state a channel
    # one stream with its tensors
    _t, spec_c = spec_of(pm.PUR_C)
    names_c = expected_tensors(spec_c)
    assert spec_c.residual_streams == 1 and names_c["l0.hc1.mix"][1].shape == (1, 1)
    assert [(r.layer, r.cache) for r in spec_c.run_order] == [(0, 0), (1, 1), (1, 2), (1, 3), (2, 4)]
    model_a = CausalLM(spec_of(pm.PUR_A)[1], torch.float32, "cpu")
    needs_a = model_a.cache_entry_specs()
    assert needs_a[0] == KVSpec(2, 16, 20, keep_first=3) and needs_a[4] == KVSpec(1, 64, 70, keep_first=65)
    assert needs_a[1] == StateSpec((2 * 48 + 48 * 8,), "float32")


def test_config_problems_are_named_together():
    from reflex_b200.errors import CheckpointError

    cfg = copy.deepcopy(pm.PUR_A)
    del cfg["width"]
    del cfg["layers"][0]["mixer"]["kv_heads"]
    cfg["layers"][0]["mixer"]["mask"] = {"keep_first": 2}
    cfg["layers"][1]["mixer"]["state"] = "8"
    cfg["layers"][2]["type"] = "retention"
    cfg["layers"][1]["mlp"] = {"kind": "gated", "ff": 3}
    with pytest.raises(CheckpointError) as e:
        spec_of(cfg)
    for part in ("width", "layers[0].mixer.kv_heads", "layers[0].mixer.mask.size", "layers[1].mixer.state",
                 "layers[2].type='retention'", "layers[1].mlp.kind='gated'"):
        assert part in str(e.value), part
    for bad in ({"streams": 9}, {"loop": {"start": 2, "stop": 1, "times": 1}}):
        with pytest.raises(CheckpointError):
            spec_of(dict(copy.deepcopy(pm.PUR_A), **bad))
    cfg = copy.deepcopy(pm.PUR_A)
    cfg["layers"][0]["mixer"]["vdim"] = 8
    with pytest.raises(CheckpointError):
        spec_of(cfg)


def test_writer_and_loader_and_its_one_error(tmp_path):
    from reflex_b200.errors import CheckpointError
    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    from reflex_b200.weights.loader import Checkpoint, check_names_and_shapes

    d = write_random_model(pm.PUR_C, 1, str(tmp_path / "m"), "bfloat16")
    cfg, w = pp.read_model(d)
    assert cfg["architecture"] == "Purusun" and w["l0.mix.q"].shape == (120, 100)
    assert np.abs(w["l0.norm1"]).max() <= 0.101 and np.abs(w["final.norm"]).max() <= 0.101  # stored around zero
    assert 0.89 <= w["l0.mix.q.norm"].min() and 0.2 <= w["l0.hc1.mix"].min() <= w["l0.hc1.mix"].max() <= 0.8
    _typed, spec = spec_of(cfg)
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    ck.close()
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    del tensors["l1.mix.A_log"]
    tensors["l0.mix.v"] = tensors["l0.mix.k"]
    tensors["l2.hc1.in"] = tensors["l2.hc1.in"].repeat(2)
    write_safetensors(path, list(tensors.items()))
    ck = Checkpoint(d)
    with pytest.raises(CheckpointError) as e:
        check_names_and_shapes(spec, ck)
    ck.close()
    assert "l1.mix.A_log" in str(e.value) and "l0.mix.v" in str(e.value) and "l2.hc1.in" in str(e.value)


def test_a_window_with_kept_first_pages_gives_back_the_pages_between():
    from reflex_b200.cache.specs import KVSpec
    from reflex_b200.cache.store import Cache

    cache = Cache({0: KVSpec(1, 8, 70, keep_first=65), 1: KVSpec(1, 8, 70)}, 64 * 40, 1 << 20, None, None, max_slots=2)
    kept, plain = cache.kv_groups
    a = cache.take_slot()
    for n in (100, 100, 200, 1, 300):  # 701 tokens in all
        cache.reserve([(a, n)])
        cache.commit([(a, n)])
    # the last 70 positions begin in page 9; the first two pages hold the 65 kept positions
    assert plain.held_pages(a) == [9, 10] and kept.held_pages(a) == [0, 1, 9, 10]
    assert kept.pool.held_count == 4 and plain.pool.held_count == 2
    b = cache.take_slot()
    cache.reserve([(b, 30)])
    cache.commit([(b, 30)])
    assert kept.held_pages(b) == [0]
    cache.give_slot(a)
    cache.give_slot(b)
    assert kept.pool.held_count == 0 and plain.pool.held_count == 0
    c = cache.take_slot()  # every page can be taken again
    cache.reserve([(c, 64 * 40)])
    cache.commit([(c, 64 * 40)])
    assert kept.held_pages(c) == [0, 1, 38, 39]


# ------------------------------------------------------- the plain implementation
def test_scaled_frequencies_keep_slow_and_blend():
    f = pp.rotary_frequencies(8, 100.0, None)
    assert np.allclose(f, [1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75])
    g = pp.rotary_frequencies(8, 100.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
    # wavelengths 6.3, 19.9, 62.8, 198.7 against the bounds 16 and 64: kept, blended, blended, slowed
    assert g[0] == f[0] and g[3] == f[3] / 8.0 and f[1] / 8.0 < g[1] < f[1] and f[2] / 8.0 < g[2] < f[2]
    s = (64 / (2 * math.pi / f[1]) - 1.0) / 3.0
    assert np.isclose(g[1], (1 - s) * f[1] / 8.0 + s * f[1])


def test_rotation_turns_pairs_half_a_head_apart_and_keeps_dot_products_of_equal_distance():
    rng = np.random.default_rng(0)
    f = pp.rotary_frequencies(4, 10.0, None)
    t = rng.standard_normal((1, 1, 6))
    r = pp.rotate(np.repeat(t, 5, axis=0), np.arange(5), f)
    assert np.allclose(r[0], t[0]) and np.allclose(r[:, :, 4:], t[:, :, 4:])  # position 0 and the dimensions beyond
    a = 3 * f[1]
    assert np.isclose(r[3, 0, 1], t[0, 0, 1] * math.cos(a) - t[0, 0, 3] * math.sin(a))
    assert np.isclose(r[3, 0, 3], t[0, 0, 3] * math.cos(a) + t[0, 0, 1] * math.sin(a))
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    d1 = (pp.rotate(q, np.array([7]), f) * pp.rotate(k, np.array([4]), f)).sum()
    d2 = (pp.rotate(q, np.array([13]), f) * pp.rotate(k, np.array([10]), f)).sum()
    assert np.isclose(d1, d2)


def test_window_and_kept_first_tokens():
    assert [j for j in range(12) if pp.visible(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(12) if pp.visible(11, j, 4, 0)] == [8, 9, 10, 11]
    assert [j for j in range(12) if pp.visible(3, j, 4, 2)] == [0, 1, 2, 3]
    assert [j for j in range(6) if pp.visible(4, j, None, 0)] == [0, 1, 2, 3, 4]


def test_scan_with_pinned_steps_has_a_closed_form():
    """W_dt = 0 pins dt = softplus(b); a constant input x and B = C = x (one
    state): S_t = dt x^2 (1 - a^t) / (1 - a) with a = exp(dt A), y_t = S_t x + D x."""
    T, dtb, A_log, D = 7, 0.4, 0.2, 0.3
    w = {"in": np.array([[1.0], [1.0]]), "conv": np.array([[1.0]]), "conv.b": np.array([0.0]),
         "x": np.array([[0.0], [1.0], [1.0]]), "dt": np.array([[0.0]]), "dt.b": np.array([dtb]),
         "A_log": np.array([[A_log]]), "D": np.array([D]), "o": np.array([[1.0]])}
    h = np.full((T, 1), 0.8)
    out = pp.selective_scan(h, w, {"inner": 1, "state": 1, "dt_rank": 1, "conv": 1})
    x = float(pp.silu(0.8))
    dt = float(pp.softplus(dtb))
    a = math.exp(-dt * math.exp(A_log))
    want = [(dt * x * x * (1 - a ** (t + 1)) / (1 - a) * x + D * x) * float(pp.silu(0.8)) for t in range(T)]
    assert np.allclose(out[:, 0], want)


def test_scan_equals_its_recurrence_written_out():
    """One channel, two states, by hand for three tokens."""
    w = {"in": np.array([[1.0], [0.0]]), "conv": np.array([[0.5, 1.0]]), "conv.b": np.array([0.1]),
         "x": np.array([[2.0], [1.0], [-1.0], [0.5], [0.25]]), "dt": np.array([[1.0]]), "dt.b": np.array([-0.3]),
         "A_log": np.array([[0.0, math.log(2.0)]]), "D": np.array([0.4]), "o": np.array([[1.0]])}
    h = np.array([[1.0], [-2.0], [0.5]])
    w["in"] = np.array([[1.0], [1.0]])  # z = h
    out = pp.selective_scan(h, w, {"inner": 1, "state": 2, "dt_rank": 1, "conv": 2})
    xs = [pp.silu(np.array(v)) for v in (1.0 + 0.1, -2.0 + 0.5 * 1.0 + 0.1, 0.5 + 0.5 * -2.0 + 0.1)]
    S = np.zeros(2)
    want = []
    for t, x in enumerate(xs):
        dt = pp.softplus(2.0 * x - 0.3)
        B, C = np.array([1.0, -1.0]) * x, np.array([0.5, 0.25]) * x
        S = np.exp(dt * np.array([-1.0, -2.0])) * S + dt * x * B
        want.append((S @ C + 0.4 * x) * pp.silu(h[t, 0]))
    assert np.allclose(out[:, 0], want)


def test_streams_read_and_write():
    xs = np.arange(12, dtype=float).reshape(2, 2, 3)  # two streams, two tokens, width 3
    assert np.allclose(pp.hyper_read(xs, np.array([2.0, -1.0])), 2 * xs[0] - xs[1])
    y = np.ones((2, 3))
    mix = np.array([[1.0, 0.5], [0.0, 2.0]])  # [from, to]
    new = pp.hyper_write(xs, y, mix, np.array([10.0, 20.0]))
    assert np.allclose(new[0], xs[0] * 1.0 + xs[1] * 0.0 + 10.0)
    assert np.allclose(new[1], xs[0] * 0.5 + xs[1] * 2.0 + 20.0)


def test_run_order():
    assert pp.run_order(pm.PUR_A) == [0, 1, 0, 1, 2] and pp.run_order(pm.PUR_B) == [0, 1, 2]
    assert pp.run_order(pm.PUR_C) == [0, 1, 1, 1, 2] and pp.run_order(pm.PUR_D) == [0, 1]


# ------------------------------------------------- every mechanism shows in the test models
def _logits(name, cfg_change=None, weight_change=None, n=None):
    cfg, w = pp.read_model(pm.model_folder(name))
    cfg, w = copy.deepcopy(cfg), dict(w)
    if cfg_change:
        cfg_change(cfg)
    if weight_change:
        weight_change(w)
    toks = pm.tokens(n or 90, cfg["vocab"], 4)
    return pp.forward(cfg, w, toks)


def _moved(a, b):
    return float(np.abs(a - b).max() / np.abs(a).max())


def test_the_test_models_show_every_mechanism():
    base = _logits("A")

    def window(c):
        c["layers"][0]["mixer"]["mask"]["size"] += 1

    def kept(c):
        c["layers"][0]["mixer"]["mask"]["keep_first"] -= 1

    def unscaled(c):
        del c["layers"][0]["mixer"]["rot"]["scaling"]

    def rot_dims(c):
        c["layers"][0]["mixer"]["rot"]["dims"] = 16

    def once(c):
        c["loop"]["times"] = 1

    def taps(w):
        w["l1.mix.conv"] = w["l1.mix.conv"].copy()
        w["l1.mix.conv"][:, 0] = 0.0

    def scale(w):
        w["l0.ls1"] = np.ones_like(w["l0.ls1"])

    def mix(w):
        w["l0.hc1.mix"] = np.array([[0.9, 0.1], [0.7, 0.3]])

    def mix_t(w):
        w["l0.hc1.mix"] = np.array([[0.9, 0.7], [0.1, 0.3]])

    def gate(w):
        w["l0.mix.g"] = w["l0.mix.g"] * 0.0

    def decay(w):
        w["l1.mix.A_log"] = w["l1.mix.A_log"] + 0.3

    def skip(w):
        w["l1.mix.D"] = w["l1.mix.D"] * 0.0

    def one_plus(w):
        w["l0.norm2"] = w["l0.norm2"] - 1.0

    for what, kw in (("window", dict(cfg_change=window)), ("kept", dict(cfg_change=kept)),
                     ("scaling", dict(cfg_change=unscaled)),
                     ("rotated dims", dict(cfg_change=rot_dims)), ("loop", dict(cfg_change=once)),
                     ("oldest tap", dict(weight_change=taps)), ("layer scale", dict(weight_change=scale)),
                     ("gate", dict(weight_change=gate)),
                     ("decay", dict(weight_change=decay)), ("skip", dict(weight_change=skip)),
                     ("one plus", dict(weight_change=one_plus))):
        assert _moved(base, _logits("A", **kw)) > 2e-3, what  # ten times the 32-bit tests' tolerance
    # the values are the keys as projected: doubling W_k leaves the normed keys (the scores) as they
    # were and doubles the values
    def doubled(w):
        w["l0.mix.k"] = w["l0.mix.k"] * 2.0

    assert _moved(base, _logits("A", weight_change=doubled)) > 5e-3
    assert _moved(_logits("A", weight_change=mix), _logits("A", weight_change=mix_t)) > 5e-3  # [from, to]
