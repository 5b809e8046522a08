"""Modadra on the host: configuration, the model as data, what the cache manager makes of a mixer of two mixers, and the
plain implementation's own mechanisms."""
import copy

import numpy as np
import pytest

from machserve_b200.cache import CacheManager
from machserve_b200.config import ConfigError, config_from_json
from machserve_b200.parts import CacheSet, DecoderModel, FixedState, PagedCache
from tests.modadra_cases import CASES
from tests.plain import modadra as plain


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_round_trip_and_tensors(name):
    raw = CASES[name]["config"]
    cfg = config_from_json(raw)
    assert type(cfg).from_json(cfg.to_json()) == cfg
    model = DecoderModel(cfg.model_spec())
    decl = {d.name: tuple(d.shape) for d in model.tensors()}
    w = raw["width"]
    assert decl["embed"] == (raw["vocab"], w) and decl["head"] == (raw["vocab"], w) and decl["final.norm"] == (w,)
    for i, layer in enumerate(raw["layers"]):
        a, d, p = layer["mixer"]["left"], layer["mixer"]["right"], f"l{i}."
        assert decl[p + "norm1"] == (w,)
        assert decl[p + "mix.left.q"] == (a["heads"] * a["dim"], w) and decl[p + "mix.left.k"] == (a["kv_heads"] * a["dim"], w)
        assert decl[p + "mix.left.v"] == (a["kv_heads"] * a["vdim"], w) and decl[p + "mix.left.g"] == (a["heads"], w)
        assert decl[p + "mix.left.o"] == (w, a["heads"] * a["vdim"])
        assert decl[p + "mix.right.q"] == (d["kv_heads"] * d["dim"], w) and decl[p + "mix.right.k"] == (d["kv_heads"] * d["dim"], w)
        assert decl[p + "mix.right.v"] == (d["heads"] * d["vdim"], w) and decl[p + "mix.right.g"] == (d["heads"] * d["vdim"], w)
        assert decl[p + "mix.right.q.conv"] == (d["kv_heads"] * d["dim"], d["conv"])
        assert decl[p + "mix.right.v.conv"] == (d["heads"] * d["vdim"], d["conv"])
        for n in ("b", "a"):
            assert decl[p + "mix.right." + n] == (d["heads"], w)
        for n in ("A_log", "dt_bias"):
            assert decl[p + "mix.right." + n] == (d["heads"],)
        assert decl[p + "mix.right.norm"] == (d["vdim"],) and decl[p + "mix.right.o"] == (w, d["heads"] * d["vdim"])
        assert decl[p + "mix.left.out"] == (w,) and decl[p + "mix.right.out"] == (w,)
        mlp = layer["mlp"]
        if mlp is None:
            assert p + "norm2" not in decl and not any(k.startswith(p + "mlp.") for k in decl)
        else:
            e = mlp["router"]["experts"]
            assert decl[p + "norm2"] == (w,) and decl[p + "mlp.router"] == (e, w) and decl[p + "mlp.correction"] == (e,)
            assert decl[f"{p}mlp.e{e - 1}.up"] == (mlp["expert"]["ff"], w) and decl[f"{p}mlp.e0.down"] == (w, mlp["expert"]["ff"])
            assert f"{p}mlp.e{e}.up" not in decl and f"{p}mlp.e0.gate" not in decl and p + "mlp.router.b" not in decl


def test_optional_keys():
    raw = copy.deepcopy(CASES["A"]["config"])
    raw.pop("residual_mult")
    raw.pop("logit_softcap")
    left, right = raw["layers"][0]["mixer"]["left"], raw["layers"][0]["mixer"]["right"]
    for key in ("rot", "mask", "kv_heads", "vdim"):
        left.pop(key)
    right.pop("kv_heads")
    right.pop("vdim")
    raw["layers"][0]["mlp"]["router"].pop("groups")
    raw["layers"][0]["mlp"]["router"].pop("scale")
    cfg = config_from_json(raw)
    a, d, m = cfg.layers[0].mixer.left, cfg.layers[0].mixer.right, cfg.layers[0].mlp
    assert (a.rot_dims, a.window, a.kv_heads, a.vdim) == (0, None, a.heads, a.dim)
    assert (d.kv_heads, d.vdim) == (d.heads, d.dim)
    assert (m.groups, m.keep, m.scale) == (1, 1, 1.0) and cfg.residual_mult == 1.0 and cfg.logit_softcap is None
    assert type(cfg).from_json(cfg.to_json()) == cfg
    spec = cfg.model_spec()
    mixer = spec.layers[0].mixer
    assert mixer["left"]["position"] is None and mixer["left"]["window"] is None and spec.head["softcap"] is None
    need = DecoderModel(spec).cache_needs()[0]
    assert isinstance(need, CacheSet) and need.needs[0].window is None


def test_a_mixer_of_two_keeps_pages_and_a_state():
    cfg = config_from_json(CASES["A"]["config"])
    needs = DecoderModel(cfg.model_spec()).cache_needs()
    assert len(needs) == 3 and all(isinstance(n, CacheSet) for n in needs)
    assert [[type(m) for m in n.needs] for n in needs] == [[PagedCache, FixedState]] * 3
    d = CASES["A"]["config"]["layers"][0]["mixer"]["right"]
    channels = 2 * d["kv_heads"] * d["dim"] + d["heads"] * d["vdim"]
    assert needs[0].needs[1].shape == (d["heads"] * d["dim"] * d["vdim"] + (d["conv"] - 1) * channels,), \
        "a slot holds the matrices and the convolution's last taps - 1 inputs"
    cache = CacheManager(needs, page_size=8, num_pages=12, num_state_slots=2)
    assert sorted(cache.state_runs) == [(0, 1), (1, 1), (2, 1)], "member 1 of every run has a state of its own"
    by_window = {g.need.window: g for g in cache.groups}
    assert set(by_window) == {12, 7, 20} and all(g.runs == [(i, 0)] for i, g in enumerate(cache.groups))
    # a request that grows token by token holds the pages that its next query's window reaches only
    cache.begin("a")
    for n in range(1, 90):
        cache.reserve("a", n)
        cache.commit("a", n)
        cache.check()
        for window, g in by_window.items():
            assert g.pool.num_held <= (window - 1 + 7) // 8 + 2
    cache.release("a")
    assert all(g.pool.num_held == 0 for g in cache.groups)
    # equal needs of several runs share a group; a window longer than the context keeps every page
    same = config_from_json(CASES["B"]["config"])
    raw = copy.deepcopy(CASES["B"]["config"])
    raw["layers"].append(copy.deepcopy(raw["layers"][0]))
    shared = CacheManager(DecoderModel(config_from_json(raw).model_spec()).cache_needs(), page_size=16, num_pages=8, num_state_slots=1)
    assert len(shared.groups) == 2 and sorted(len(g.runs) for g in shared.groups) == [1, 2]
    assert len(CacheManager(DecoderModel(same.model_spec()).cache_needs(), 16, 8, 1).groups) == 2


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "serial"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 18), "at most"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "not supported"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "more than"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 4), "equal groups"),
    (lambda c: c.pop("width"), "'width' is required"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "'scale' is required"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "'conv' is required"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c.__setitem__("layers", []), "at least one layer"),
])
def test_config_errors_name_the_key(change, message):
    raw = copy.deepcopy(CASES["A"]["config"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_json(raw)


# ------------------------------------------------------------------ the mechanisms on the host


def test_plain_rotation_of_a_part():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 10))
    y = plain.rotate_half_partial(x, [0, 1, 2, 30, 31], 6, 50.0)
    assert np.array_equal(y[0], x[0]), "position 0 turns nothing"
    assert np.array_equal(y[..., 6:], x[..., 6:]), "the coordinates past the rotated ones pass"
    # pair (1, 4) of head 1 at position 30 by hand
    ang = 30 * 50.0 ** (-2.0 * 1 / 6)
    a, b = x[3, 1, 1], x[3, 1, 4]
    assert np.allclose([y[3, 1, 1], y[3, 1, 4]], [a * np.cos(ang) - b * np.sin(ang), b * np.cos(ang) + a * np.sin(ang)])
    # a rotation keeps every pair's length, and scores depend on the distance alone
    assert np.allclose((y[..., :6] ** 2).sum(-1), (x[..., :6] ** 2).sum(-1))
    q, k = rng.normal(size=(1, 1, 6)), rng.normal(size=(1, 1, 6))
    s = [float((plain.rotate_half_partial(q, [p + 4], 6, 50.0) * plain.rotate_half_partial(k, [p], 6, 50.0)).sum()) for p in (0, 9, 200)]
    assert np.allclose(s, s[0])
    assert plain.rotate_half_partial(x, [3] * 5, 0, 1.0) is x


def test_plain_window_and_the_sink():
    vis = plain.window_mask(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True, False, False, False, False]
    assert plain.window_mask(4, 1).tolist() == np.eye(4, dtype=bool).tolist(), "a window of one token: the query's own key"
    assert plain.window_mask(4, None)[3].all()
    s = np.array([[0.0, 1.0, -2.0, 5.0]])
    p = plain.softmax_plus_one(s, np.array([[True, True, True, False]]))
    e = np.exp([0.0, 1.0, -2.0])
    assert np.allclose(p[0, :3], e / (1.0 + e.sum())) and p[0, 3] == 0.0
    assert p.sum() < 1.0, "the sink takes its share and has no value"
    big = plain.softmax_plus_one(np.array([[800.0, 799.0]]), np.ones((1, 2), dtype=bool))
    assert np.isfinite(big).all() and np.isclose(big.sum(), 1.0)
    small = plain.softmax_plus_one(np.array([[-800.0, -900.0]]), np.ones((1, 2), dtype=bool))
    assert np.isfinite(small).all() and small.sum() < 1e-300


def test_plain_convolution_carries_its_inputs():
    rng = np.random.default_rng(1)
    x, w = rng.normal(size=(11, 5)), rng.normal(size=(5, 4))
    whole = plain.short_conv(x, w)
    assert np.allclose(whole[0], x[0] * w[:, 3]), "the last column is the current token's, zeros come before the start"
    assert np.allclose(whole[2], x[0] * w[:, 1] + x[1] * w[:, 2] + x[2] * w[:, 3])
    a = plain.short_conv(x[:6], w)
    b = plain.short_conv(x[6:], w, before=x[3:6])
    assert np.allclose(np.concatenate([a, b]), whole)
    assert np.allclose(plain.short_conv(x, w[:, 3:]), x * w[:, 3:].T), "one tap: a scale per channel, nothing to keep"


def test_plain_delta_rule_carries_its_state():
    rng = np.random.default_rng(2)
    n, dk, dv = 9, 4, 3
    q, v = rng.normal(size=(n, dk)), rng.normal(size=(n, dv))
    k = plain.unit_vector(rng.normal(size=(n, dk)))
    beta, g = rng.uniform(0.1, 1.0, size=n), rng.uniform(0.5, 1.0, size=n)
    whole, s_whole = plain.delta_rule(q, k, v, beta, g)
    a, s = plain.delta_rule(q[:4], k[:4], v[:4], beta[:4], g[:4])
    b, s = plain.delta_rule(q[4:], k[4:], v[4:], beta[4:], g[4:], s)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(s, s_whole)
    # beta 1 and a unit key: right after the write the state answers the key with the value
    o, s = plain.delta_rule(k, k, v, np.ones(n), g)
    assert np.allclose(o, v, atol=1e-5)
    # no decay, beta 1, keys at right angles: every value is still there at the end
    eye = np.eye(4)
    o, s = plain.delta_rule(eye, eye, v[:4], np.ones(4), np.ones(4))
    assert np.allclose(s, v[:4]) and np.allclose(s.T @ eye[1], v[1])
    # the read-out sees the write of its own token: with a zero state o_0 = (q_0 . k_0) beta_0 v_0
    assert np.allclose(whole[0], (q[0] @ k[0]) * beta[0] * v[0])


def test_plain_router_groups_and_correction():
    router = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}, "scale": 2.0}
    z = np.log(np.array([[0.6, 0.1, 0.3, 0.35, 0.2, 0.7]]) / (1 - np.array([[0.6, 0.1, 0.3, 0.35, 0.2, 0.7]])))
    w = {"router": np.eye(6), "correction": np.zeros(6)}
    ids, weights = plain.route(z, w, "", router)
    assert ids.tolist() == [[5, 4]], "group 2 (0.9 by its two largest) beats group 0 (0.7): 0.6 of group 0 cannot be chosen"
    assert np.allclose(weights[0], np.array([0.7, 0.2]) / 0.9 * 2.0)
    # the correction moves the choice, not the weights; a choice score below zero still beats an expert that is out
    w["correction"] = np.array([-9.0, -9.0, -1.0, -1.2, -9.0, -9.0])
    ids, weights = plain.route(z, w, "", router)
    assert ids.tolist() == [[2, 3]], "every choice score is negative; the experts of the groups that are out count as minus infinity, not 0"
    assert np.allclose(weights[0], np.array([0.3, 0.35]) / 0.65 * 2.0)
    # groups of one expert: the group's score is that expert's
    one = {"experts": 4, "top": 1, "groups": {"count": 4, "keep": 2}}
    ids, weights = plain.route(z[:, :4], {"router": np.eye(4), "correction": np.zeros(4)}, "", one)
    assert ids.tolist() == [[0]] and np.allclose(weights, 1.0)
    margins = []
    plain.route(z, {"router": np.eye(6), "correction": np.zeros(6)}, "", router, margins)
    assert np.allclose(margins[0], [0.2]), "by how much the last choice was ahead: 0.9 against 0.7 between the groups"


def test_plain_cap_and_activation():
    assert np.allclose(plain.soft_cap(np.array([0.01, 100.0, -100.0]), 5.0), [0.01, 5.0, -5.0], atol=1e-6)
    assert np.allclose(plain.gelu_erf(np.array([0.0, 1.0, -1.0, 6.0])), [0.0, 0.8413447, -0.1586553, 6.0], atol=1e-6)
    assert np.allclose(plain.softplus(np.array([-800.0, 0.0, 800.0])), [0.0, np.log(2.0), 800.0])
