"""Zelinex without a GPU: configuration, the model description built from it
(run order of a looped stretch with its pass vectors, cache needs, tensor
names, the low rank taken from the checkpoint), the random-weights writer and
the loader's one error; the plain implementation against closed forms; and
that the test models' weights make every mechanism show."""

import copy
import math
import os

import numpy as np
import pytest

import plain_zelinex as pz
import zelinex_models as zm


def spec_of(cfg):
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config.registry import spec_from_config_dict

    return spec_from_config_dict(cfg)


def test_config_to_model_description():
    from reflex_b200.engine.model import expected_tensors

    typed, spec = spec_of(zm.ZEL_A)
    assert spec.architecture == "zelinex" and spec.vocab_size == 97 and spec.hidden_size == 64
    assert spec.tie_word_embeddings and spec.pass_vectors_name == "loop.step" and spec.pass_vectors == 2
    assert [l.block for l in spec.layers] == ["sandwich"] * 3
    assert [l.mixer.kind for l in spec.layers] == ["pair", "delta_rule", "pair"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == ["xielu", "moe", None]
    p = spec.layers[0].mixer
    assert p.param("combine") == "scaled_sum" and (p.param("left_scale"), p.param("right_scale")) == (0.7, 1.2)
    a, s = p.param("left"), p.param("right")
    assert a.kind == "sigmoid_attention" and s.kind == "ssd"
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.window, a.scale) == (4, 2, 16, 24, 20, 0.5)
    assert a.position.kind == "rope_neox" and a.position.rotary_dim == 8 and a.position.theta == 100.0
    assert (s.param("heads"), s.param("vdim"), s.param("state"), s.param("groups"), s.param("taps"),
            s.param("norm_groups")) == (2, 16, 8, 1, 3, 1)
    d = spec.layers[1].mixer
    assert (d.num_heads, d.head_dim) == (2, 16) and abs(d.param("rate") - math.exp(-0.5)) < 1e-15
    f = spec.layers[1].feed_forward
    assert (f.param("experts"), f.param("top"), f.param("scores"), f.param("activation"), f.param("shared_ff"),
            f.param("shared_kind")) == (4, 2, "softmax_all", "swiglu", 32, "swiglu")
    assert dict(spec.layers[0].params)["residual_mult"] == 0.8
    assert [r for r, _ in spec.layers[0].extra_norms] == ["post_mixer", "post_feed_forward"]
    assert [r for r, _ in spec.layers[2].extra_norms] == ["post_mixer"]
    # layers 0 and 1 twice, then layer 2; a cache entry per run; a pass starts with its vector,
    # the second also with the embedding output
    assert [(r.layer, r.cache, r.pass_vector, r.adds_input) for r in spec.run_order] == \
        [(0, 0, 0, False), (1, 1, None, False), (0, 2, 1, True), (1, 3, None, False), (2, 4, None, False)]
    names = expected_tensors(spec)
    for n in ("embed", "loop.step", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.left.q", "l0.mix.left.pb",
              "l0.mix.left.o", "l0.mix.right.in", "l0.mix.right.conv", "l0.mix.right.conv.b", "l0.mix.right.dt_bias",
              "l0.mix.right.A_log", "l0.mix.right.D", "l0.mix.right.norm", "l0.mix.right.o", "l0.mlp.up", "l0.mlp.act",
              "l1.mix.r", "l1.mix.a.b", "l1.mix.w1", "l1.mix.w2", "l1.mix.w0", "l1.mix.norm", "l1.mlp.router",
              "l1.mlp.e3.gate", "l1.mlp.shared.down", "l2.norm1b", "final.norm"):
        assert n in names, n
    for n in ("head", "l2.norm2", "l2.norm2b", "l2.mlp.up", "l1.mlp.e4.up", "l1.mlp.shared.sg", "l0.mix.left_out"):
        assert n not in names, n
    assert names["l0.mix.left.v"][1].shape == (48, 64) and names["l0.mix.left.o"][1].shape == (64, 96)
    assert names["l0.mix.right.in"][1].shape == (2 * 32 + 2 * 8 + 2, 64) and names["l0.mix.right.conv"][1].shape == (48, 3)
    assert names["loop.step"][1].shape == (2, 64) and names["l0.mlp.act"][1].shape == (2,)
    assert names["l1.mix.w1"][1].shape == (-1, 64) and names["l1.mix.w1"][1].fits((5, 64))
    assert not names["l1.mix.w1"][1].fits((5, 65)) and names["l1.mix.w2"][1].fits((32, 5))
    assert typed.to_dict()["loop"] == {"start": 0, "stop": 2, "times": 2} and typed.to_dict()["residual_mult"] == 0.8


def test_models_without_a_loop_a_window_a_rotation_or_a_shared_expert():
    from reflex_b200.cache.specs import KVSpec, StateSpec
    from reflex_b200.engine.model import CausalLM, expected_tensors

    _typed, spec = spec_of(zm.ZEL_B)
    assert spec.pass_vectors_name is None and "loop.step" not in expected_tensors(spec)
    assert all(r.pass_vector is None and not r.adds_input for r in spec.run_order)
    a = spec.layers[0].mixer.param("left")
    assert a.window is None and a.position is None
    assert spec.layers[1].feed_forward.param("shared_ff") == 0
    assert "l1.mlp.shared.gate" not in expected_tensors(spec)
    import torch

    model = CausalLM(spec, torch.float32, "cpu")
    specs = model.cache_entry_specs()
    assert specs[0] == (KVSpec(1, 8, None, v_head_dim=8), StateSpec((3 * 1 * 24,), "float32"))  # one tap: no filter state
    assert specs[1] == StateSpec((32 * 32,), "float32")
    _typed, spec = spec_of(zm.ZEL_C)
    model = CausalLM(spec, torch.float32, "cpu")
    kv, st = model.cache_entry_specs()[1]
    assert kv == KVSpec(3, 40, 64, v_head_dim=16) and st.shape == (4 * (96 + 160) + 2 * 40 * 48,)
    # the middle layer three times: entries 1, 2, 3 with vectors 0, 1, 2
    assert [(r.layer, r.pass_vector, r.adds_input) for r in spec.run_order] == \
        [(0, None, False), (1, 0, False), (1, 1, True), (1, 2, True), (2, None, False)]


def test_config_problems_are_named_together():
    from reflex_b200.errors import CheckpointError

    cfg = copy.deepcopy(zm.ZEL_A)
    del cfg["width"]
    del cfg["layers"][0]["mixer"]["left"]["kv_heads"]
    cfg["layers"][0]["mixer"]["left"]["mask"] = {}
    cfg["layers"][0]["mixer"]["right"]["state"] = "8"
    del cfg["layers"][0]["mixer"]["right_scale"]
    cfg["layers"][2]["type"] = "retention"
    cfg["layers"][1]["mlp"]["router"] = {"experts": 4}
    cfg["layers"][0]["mlp"] = {"kind": "gated", "ff": 3}
    with pytest.raises(CheckpointError) as e:
        spec_of(cfg)
    for part in ("width", "layers[0].mixer.left.kv_heads", "layers[0].mixer.left.mask.size",
                 "layers[0].mixer.right.state", "layers[0].mixer.right_scale", "layers[2].type='retention'",
                 "layers[1].mlp.router.top", "layers[0].mlp.kind='gated'"):
        assert part in str(e.value), part
    for bad in ({"loop": {"start": 2, "stop": 1, "times": 1}}, {"vocab": 0}):
        with pytest.raises(CheckpointError):
            spec_of(dict(copy.deepcopy(zm.ZEL_A), **bad))
    cfg = copy.deepcopy(zm.ZEL_A)
    cfg["layers"][0]["mixer"]["right"]["groups"] = 3  # does not divide the heads
    with pytest.raises(CheckpointError):
        spec_of(cfg)


def test_writer_and_loader_and_its_one_error(tmp_path):
    from reflex_b200.errors import CheckpointError
    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    from reflex_b200.weights.loader import Checkpoint, check_names_and_shapes

    d = write_random_model(zm.ZEL_C, 1, str(tmp_path / "m"), "bfloat16")
    cfg, w = pz.read_model(d)
    assert cfg["architecture"] == "Zelinex" and w["l1.mix.left.q"].shape == (120, 100)
    assert w["l0.mix.w1"].shape[1] == 100 and w["l0.mix.w1"].shape[0] == w["l0.mix.w2"].shape[1] >= 1
    assert 0.89 <= w["l0.norm1b"].min() and w["loop.step"].shape == (3, 100)
    _typed, spec = spec_of(cfg)
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    ck.close()
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    # another low rank is another checkpoint of the same model description
    tensors["l0.mix.w1"] = tensors["l0.mix.w1"][:3].contiguous()
    tensors["l0.mix.w2"] = tensors["l0.mix.w2"][:, :3].contiguous()
    write_safetensors(path, list(tensors.items()))
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    ck.close()
    del tensors["l1.mix.right.A_log"]
    tensors["l1.mix.left.out"] = tensors["l1.norm1"]
    tensors["l1.mix.left.pb"] = tensors["l1.mix.left.pb"].repeat(2)
    write_safetensors(path, list(tensors.items()))
    ck = Checkpoint(d)
    with pytest.raises(CheckpointError) as e:
        check_names_and_shapes(spec, ck)
    ck.close()
    assert "l1.mix.right.A_log" in str(e.value) and "l1.mix.left.out" in str(e.value) and "l1.mix.left.pb" in str(e.value)


# ------------------------------------------------------- the plain implementation
def test_rotation_turns_pairs_half_the_rotated_part_apart():
    t = np.zeros((3, 1, 8))
    t[:, 0, 1] = 1.0   # pairs with dimension 3 when four dimensions turn
    t[:, 0, 6] = 5.0   # beyond the rotated part
    out = pz.rotate(t, np.array([0, 1, 7]), 4, 100.0)
    f1 = 100.0 ** (-2.0 / 4)
    for r, p in enumerate([0, 1, 7]):
        assert abs(out[r, 0, 1] - math.cos(p * f1)) < 1e-12 and abs(out[r, 0, 3] - math.sin(p * f1)) < 1e-12
        assert out[r, 0, 6] == 5.0 and out[r, 0, 0] == 0.0
    # scores depend on the distance alone
    g = np.random.default_rng(0)
    q, k = g.standard_normal((1, 1, 8)), g.standard_normal((1, 1, 8))
    a = (pz.rotate(q, np.array([9]), 8, 50.0) * pz.rotate(k, np.array([4]), 8, 50.0)).sum()
    b = (pz.rotate(q, np.array([105]), 8, 50.0) * pz.rotate(k, np.array([100]), 8, 50.0)).sum()
    assert abs(a - b) < 1e-9


def test_window():
    m = pz.visible(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True] + [False] * 4
    assert pz.visible(4, None)[3].all() and not pz.visible(4, None)[0, 1]


def test_sigmoid_attention_is_not_normalised_over_the_keys():
    """With zero queries every visible key weighs sigmoid(b): the output is that
    times the sum of the visible values, so it grows with their number."""
    W, T = 8, 6
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 1.0, "mask": {"size": 4}}
    g = np.random.default_rng(1)
    w = {"q": np.zeros((8, W)), "k": g.standard_normal((4, W)), "v": g.standard_normal((3, W)),
         "pb": np.array([0.0, -1.0]), "o": np.eye(6)}
    h = g.standard_normal((T, W))
    out = pz.sigmoid_attention(h, w, m)
    v = h @ w["v"].T
    for i in range(T):
        total = v[max(0, i - 3):i + 1].sum(axis=0)
        assert np.allclose(out[i, :3], 0.5 * total) and np.allclose(out[i, 3:], pz.sigmoid(-1.0) * total)


def test_state_space_scan_with_pinned_steps_has_a_closed_form():
    T, P, N = 7, 2, 3
    g = np.random.default_rng(2)
    x, B, C = g.standard_normal((T, 1, P)), g.standard_normal((T, 1, N)), g.standard_normal((T, 1, N))
    dt = np.full((T, 1), 0.3)
    y = pz.ssd_scan(x, B, C, dt, np.array([-2.0]), np.array([0.5]), 1, 1)
    for t in range(T):
        want = 0.5 * x[t, 0]
        for s in range(t + 1):
            want = want + math.exp(-2.0 * 0.3 * (t - s)) * 0.3 * (C[t, 0] @ B[s, 0]) * x[s, 0]
        assert np.allclose(y[t, 0], want)


def test_causal_convolution_looks_back_and_starts_from_zeros():
    x = np.arange(1.0, 6.0)[:, None]
    out = pz.causal_conv(x, np.array([[100.0, 10.0, 1.0]]), np.array([0.5]))
    assert out[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]


def test_delta_rule_removes_along_the_unit_key_and_decays_per_channel():
    """One step from S = 0 writes k v^T; a second step with a = 1 and the same key
    direction removes what the first wrote along it before adding its own."""
    d = 4
    g = np.random.default_rng(3)
    k = g.standard_normal(d)
    v1, v2, r = g.standard_normal(d), g.standard_normal(d), g.standard_normal(d)
    ks = np.stack([k, 2.0 * k])[:, None, :]
    vs = np.stack([v1, v2])[:, None, :]
    rs = np.stack([r, r])[:, None, :]
    ones = np.ones((2, 1, d))
    o = pz.delta_scan(rs, ks, vs, ones, ones)
    assert np.allclose(o[0, 0], np.outer(k, v1).T @ r)
    u = k / math.sqrt(k @ k + 1e-6)
    S = np.outer(k, v1) - np.outer(u, u @ np.outer(k, v1)) + np.outer(2 * k, v2)
    assert np.allclose(o[1, 0], S.T @ r)
    # with no removal, a decay per key channel scales the rows of the old state
    w = np.stack([np.ones(d), np.array([0.5, 1.0, 0.0, 0.25])])[:, None, :]
    o = pz.delta_scan(rs, ks, vs, w, np.zeros((2, 1, d)))
    S = w[1, 0][:, None] * np.outer(k, v1) + np.outer(2 * k, v2)
    assert np.allclose(o[1, 0], S.T @ r)


def test_xielu_branches_and_routing_weights():
    z = np.array([-2.0, 0.0, 3.0])
    ap, an = pz.softplus(0.3), 0.5 + pz.softplus(-0.2)
    out = pz.xielu(z, 0.3, -0.2)
    assert np.allclose(out, [an * (math.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, ap * 9 + 1.5])
    router = np.array([[1.0, 0.0], [0.0, 1.0], [-1.0, -1.0], [0.5, 0.5]])
    ids, wts = pz.route(np.array([[2.0, 0.0], [0.0, 0.1]]), router, 2, 1.25)
    assert ids.tolist() == [[0, 3], [1, 3]]
    e = np.exp([2.0, 1.0])
    assert np.allclose(wts[0], 1.25 * e / e.sum()) and abs(wts[1].sum() - 1.25) < 1e-12


def test_run_order():
    assert pz.run_order({"layers": [0, 1, 2]}) == [(0, None, False), (1, None, False), (2, None, False)]
    cfg = {"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 2}}
    assert pz.run_order(cfg) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False),
                                 (3, None, False)]


# ------------------------------------------------- the test models show their mechanisms
def _logits(name, cfg_change=None, weight_change=None, n=90):
    cfg, w = pz.read_model(zm.model_folder(name))
    cfg, w = copy.deepcopy(cfg), dict(w)
    if cfg_change:
        cfg_change(cfg)
    if weight_change:
        weight_change(w)
    return pz.forward(cfg, w, zm.tokens(n, cfg["vocab"], 11))


def _moved(a, b):
    return np.abs(a - b).max() / np.abs(a).max()


def test_the_test_models_show_every_mechanism():
    base = _logits("A")

    def window(c):
        c["layers"][0]["mixer"]["left"]["mask"]["size"] += 1

    def rot_dims(c):
        c["layers"][0]["mixer"]["left"]["rot"]["dims"] = 16

    def once(c):
        c["loop"]["times"] = 1

    def mult(c):
        c["residual_mult"] = 0.9

    def left_scale(c):
        c["layers"][0]["mixer"]["left_scale"] = 0.8

    def norm_parts(c):
        c["layers"][2]["mixer"]["right"]["norm_groups"] = 1

    def groups(w):
        # the two groups' B rows (with their filters) change places: heads 0, 1 and 2, 3 then read the other's
        for name, axis0 in (("l2.mix.right.in", 64), ("l2.mix.right.conv", 32), ("l2.mix.right.conv.b", 32)):
            t = w[name].copy()
            t[axis0:axis0 + 16], t[axis0 + 16:axis0 + 32] = w[name][axis0 + 16:axis0 + 32], w[name][axis0:axis0 + 16]
            w[name] = t

    def router_scale(c):
        c["layers"][1]["mlp"]["router"]["scale"] = 1.2

    def bias(w):
        w["l0.mix.left.pb"] = w["l0.mix.left.pb"] * 0.0

    def taps(w):
        w["l0.mix.right.conv"] = w["l0.mix.right.conv"].copy()
        w["l0.mix.right.conv"][:, 0] = 0.0

    def decay(w):
        w["l0.mix.right.A_log"] = w["l0.mix.right.A_log"] + 0.3

    def skip(w):
        w["l0.mix.right.D"] = w["l0.mix.right.D"] * 0.0

    def step_bias(w):
        w["l0.mix.right.dt_bias"] = w["l0.mix.right.dt_bias"] + 0.3

    def post(w):
        w["l0.norm1b"] = np.ones_like(w["l0.norm1b"])

    def removal(w):
        w["l1.mix.a.b"] = w["l1.mix.a.b"] - 1.0

    def delta_decay(w):
        w["l1.mix.w0"] = w["l1.mix.w0"] + 1.0

    def delta_gate(w):
        w["l1.mix.g"] = w["l1.mix.g"] * 0.0

    def act(w):
        w["l0.mlp.act"] = w["l0.mlp.act"] + np.array([0.0, 0.5])

    def shared(w):
        w["l1.mlp.shared.down"] = w["l1.mlp.shared.down"] * 0.0

    def vector(w):
        w["loop.step"] = w["loop.step"][::-1].copy()

    for what, kw in (("window", dict(cfg_change=window)), ("rotated dims", dict(cfg_change=rot_dims)),
                     ("loop", dict(cfg_change=once)), ("multiplier", dict(cfg_change=mult)),
                     ("left scale", dict(cfg_change=left_scale)), ("norm parts", dict(cfg_change=norm_parts)),
                     ("groups", dict(weight_change=groups)), ("router scale", dict(cfg_change=router_scale)),
                     ("score bias", dict(weight_change=bias)), ("oldest tap", dict(weight_change=taps)),
                     ("decay", dict(weight_change=decay)), ("skip", dict(weight_change=skip)),
                     ("step bias", dict(weight_change=step_bias)), ("post norm", dict(weight_change=post)),
                     ("removal rate", dict(weight_change=removal)), ("delta decay", dict(weight_change=delta_decay)),
                     ("delta gate", dict(weight_change=delta_gate)), ("negative branch", dict(weight_change=act)),
                     ("shared expert", dict(weight_change=shared)), ("pass vectors", dict(weight_change=vector))):
        assert _moved(base, _logits("A", **kw)) > 2e-3, what  # ten times the 32-bit tests' tolerance
