"""Varolix on the host: configuration, the model as data, the loop's run order, what the cache manager makes of its
mixers, and the plain implementation's own mechanisms."""
import copy
import math

import numpy as np
import pytest

from machserve_b200.cache import CacheManager
from machserve_b200.config import ConfigError, config_from_json
from machserve_b200.parts import CacheSet, DecoderModel, FixedState, PagedCache
from tests.plain import varolix as plain
from tests.varolix_cases import CASES


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
        m, p = layer["mixer"], f"l{i}.mix."
        assert decl[f"l{i}.norm1"] == (w,)
        if layer["type"] == "attention":
            assert decl[p + "q"] == (m["heads"] * m["dim"], w) and decl[p + "q.b"] == (m["heads"] * m["dim"],)
            assert decl[p + "k"] == (m["kv_heads"] * m["dim"], w) and decl[p + "k.b"] == (m["kv_heads"] * m["dim"],)
            assert decl[p + "v"] == (m["kv_heads"] * m["vdim"], w) and decl[p + "v.b"] == (m["kv_heads"] * m["vdim"],)
            assert decl[p + "o"] == (w, m["heads"] * m["vdim"]) and p + "o.b" not in decl and p + "g" not in decl
        elif layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            assert decl[p + "left.q"] == (a["heads"] * a["dim"], w) and decl[p + "left.k.b"] == (a["kv_heads"] * a["dim"],)
            assert decl[p + "left.v.b"] == (a["kv_heads"] * a["vdim"],) and decl[p + "left.o.b"] == (w,)
            assert decl[p + "left.q.norm"] == (a["dim"],) and decl[p + "left.k.norm"] == (a["dim"],)
            assert decl[p + "left.o"] == (w, a["heads"] * a["vdim"])
            assert decl[p + "right.q"] == (b["heads"] * b["dim"], w) and decl[p + "right.k"] == (b["heads"] * b["dim"], w)
            assert decl[p + "right.v"] == (b["heads"] * b["vdim"], w) and decl[p + "right.g"] == (b["heads"] * b["vdim"], w)
            assert decl[p + "right.i"] == (b["heads"], w) and decl[p + "right.f.b"] == (b["heads"],)
            assert decl[p + "right.norm"] == (b["heads"] * b["vdim"],) and decl[p + "right.o"] == (w, b["heads"] * b["vdim"])
            assert p + "left.out" not in decl and p + "right.out" not in decl
        else:
            hd = m["dim"] + m["rot_dim"]
            assert decl[p + "dq"] == (m["q_rank"], w) and decl[p + "dq.norm"] == (m["q_rank"],) and decl[p + "uq"] == (m["heads"] * hd, m["q_rank"])
            assert decl[p + "dkv"] == (m["kv_rank"] + m["rot_dim"], w) and decl[p + "dkv.norm"] == (m["kv_rank"],)
            assert decl[p + "uk"] == (m["heads"] * m["dim"], m["kv_rank"]) and decl[p + "uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert decl[p + "sink"] == (m["heads"],) and decl[p + "g"] == (m["heads"], w) and decl[p + "o"] == (w, m["heads"] * m["vdim"])
            assert p + "q" not in decl
        if layer["mlp"] is None:
            assert f"l{i}.norm2" not in decl and not any(k.startswith(f"l{i}.mlp.") for k in decl)
        else:
            assert decl[f"l{i}.norm2"] == (w,) and decl[f"l{i}.mlp.gate"] == (layer["mlp"]["ff"], w)
            assert decl[f"l{i}.mlp.up"] == (layer["mlp"]["ff"], w) and decl[f"l{i}.mlp.down"] == (w, layer["mlp"]["ff"])
    assert model.kernel_files() is not None and "matrix_memory" in model.kernel_files() or name == "E"


def test_optional_keys():
    raw = copy.deepcopy(CASES["A"]["config"])
    raw.pop("loop")
    att, pair = raw["layers"][0]["mixer"], raw["layers"][1]["mixer"]
    att["rot"].pop("scaling")
    att.pop("kv_heads")
    att.pop("vdim")
    pair["left"].pop("q_temp")
    pair["right"].pop("vdim")
    cfg = config_from_json(raw)
    a, p = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (a.kv_heads, a.vdim, a.scaling) == (a.heads, a.dim, None) and p.left.temp_coef == 0.0 and p.right.vdim == p.right.dim
    assert cfg.loop is None and [r.layer for r in cfg.run_order()] == [0, 1, 2, 3]
    assert type(cfg).from_json(cfg.to_json()) == cfg
    raw["layers"][3]["mixer"].pop("rot")
    spec = config_from_json(raw).model_spec()
    assert spec.layers[3].mixer["position"] is None and spec.layers[0].mixer["position"]["scaling"] is None


def test_the_loop_runs_a_range_of_layers_several_times():
    for name, want in (("A", [0, 1, 2, 1, 2, 1, 2, 3]), ("B", [0, 1, 2, 3]), ("C", [0, 1, 0, 1, 2, 3, 4]), ("D", [0, 1, 2]),
                       ("E", [0, 1, 2, 1, 2]), ("F", [0, 1, 0, 1])):
        cfg = config_from_json(CASES[name]["config"])
        runs = cfg.model_spec().run_order
        assert [r.layer for r in runs] == want == plain.run_order(CASES[name]["config"])
        assert all(r.cache_of is None and r.entry is None for r in runs), "every pass owns its cache or state; nothing between passes"


def test_cache_needs_pages_states_and_groups():
    cfg = config_from_json(CASES["A"]["config"])
    needs = DecoderModel(cfg.model_spec()).cache_needs()
    kinds = [type(n) for n in needs]
    assert kinds == [PagedCache, CacheSet, PagedCache, CacheSet, PagedCache, CacheSet, PagedCache, PagedCache]
    pair = CASES["A"]["config"]["layers"][1]["mixer"]
    left, right = needs[1].needs
    assert isinstance(left, PagedCache) and left.window is None and [(p.heads, p.width) for p in left.planes] == [(2, 16), (2, 8)]
    b = pair["right"]
    assert isinstance(right, FixedState) and right.shape == (b["heads"] * b["dim"] * (b["vdim"] + 1) + b["heads"],), \
        "a slot holds the matrices with the normalizer as one more column, and a stabilizer a head"
    latent = needs[2]
    assert [(p.heads, p.width) for p in latent.planes] == [(1, 16 + 4)], "one plane of latent and rotated key part"
    cache = CacheManager(needs, page_size=8, num_pages=16, num_state_slots=2)
    assert sorted(cache.state_runs) == [(1, 1), (3, 1), (5, 1)], "each pass over the looped pair has a state of its own"
    by_runs = [list(g.runs) for g in cache.groups]
    assert [(1, 0), (3, 0), (5, 0)] in by_runs and [2, 4, 6] in by_runs, "the passes' pages lie in one group a layer"
    cache.begin("a")
    cache.reserve("a", 20)
    cache.commit("a", 20)
    cache.check()
    assert all(g.pool.num_held == 3 for g in cache.groups), "20 tokens are three pages of eight in every group"
    cache.release("a")
    assert all(g.pool.num_held == 0 for g in cache.groups)
    # a model without a matrix memory keeps no state
    none = CacheManager(DecoderModel(config_from_json(CASES["E"]["config"]).model_spec()).cache_needs(), 16, 8, 1)
    assert not none.state_runs


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "serial"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "at most"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 6), "at most"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "not supported"),
    (lambda c: c["loop"].__setitem__("stop", 9), "not a range"),
    (lambda c: c.pop("width"), "'width' is required"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "'scale' is required"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("gate_cap"), "'gate_cap' is required"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "'left_scale' is required"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "'q_rank' is required"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
    (lambda c: c.__setitem__("layers", []), "at least one layer"),
])
def test_config_errors_name_the_key(change, message):
    raw = copy.deepcopy(CASES["A"]["config"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_json(raw)


def test_the_rotary_part_builds_the_stretched_table_of_the_plain_formula():
    """The engine's table (float64 on the host, no device needed) against the plain frequencies, with and without stretching."""
    from machserve_b200.config import part
    from machserve_b200.parts.base import POSITION_ENCODINGS

    for dims, base, scaling in ((8, 100.0, (4.0, 32, 8.0, 1.0)), (32, 10000.0, (4.0, 64, 16.0, 2.0)), (16, 20000.0, (16.0, 16, 4.0, 0.5)),
                                (12, 200.0, None), (2, 7.0, (8.0, 1024, 32.0, 1.0))):
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        enc = POSITION_ENCODINGS.build(part("rope", head_dim=dims, rotary_dim=dims, theta=base, pairing="half", scaling=sc))
        f, m = enc.frequencies()
        pf, pm = plain.rotary_frequencies(dims, base, sc)
        assert np.allclose(f, pf, rtol=1e-15, atol=0) and m == pm
        if scaling:
            plain_f = base ** (-2.0 * np.arange(dims // 2) / dims)
            assert np.all(f <= plain_f * (1 + 1e-12)) and np.all(f >= plain_f / scaling[0] * (1 - 1e-12))
            assert m == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)


# ------------------------------------------------------------------ the mechanisms on the host


def test_plain_rotation_in_halves_of_a_part_with_stretched_waves():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(6, 2, 10))
    rot = {"dims": 6, "base": 50.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    y = plain.rotate_half(x, [0, 1, 2, 9, 30, 31], rot)
    f, m = plain.rotary_frequencies(6, 50.0, rot["scaling"])
    assert np.array_equal(y[..., 6:], x[..., 6:]) and np.allclose(y[0], x[0] * np.r_[np.full(6, m), np.ones(4)])
    for i in range(3):  # pair (i, i + 3): a turn by p * f_i, lengths times m
        a = 30 * f[i]
        assert y[4, 1, i] == pytest.approx(m * (x[4, 1, i] * math.cos(a) - x[4, 1, i + 3] * math.sin(a)))
        assert y[4, 1, i + 3] == pytest.approx(m * (x[4, 1, i + 3] * math.cos(a) + x[4, 1, i] * math.sin(a)))
    plain_f = 50.0 ** (-2.0 * np.arange(3) / 6)
    assert f[0] == plain_f[0] or f[0] < plain_f[0]
    assert f[-1] == pytest.approx(plain_f[-1] / 4.0), "the slowest wave is stretched by the whole factor"


def test_plain_softmax_with_a_sink_and_the_temperature():
    s = np.array([[1.0, 9.0, 9.0], [0.5, -0.25, 9.0], [2.0, 0.0, 1.0]])
    p = plain.causal_softmax(s)
    assert p[0, 0] == 1.0 and p[1, 2] == 0.0 and np.allclose(p.sum(-1), 1.0)
    q = plain.causal_softmax(s, 1.5)
    assert q[0, 0] == pytest.approx(math.e / (math.e + math.exp(1.5))), "the sink counts once, unscaled, without a value"
    assert np.all(q.sum(-1) < 1.0)
    t = plain.query_temperature([0, 3, 4, 9, 10], {"coef": 0.5, "every": 5})
    assert np.allclose(t, [1.0, 1.0, 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(3), 1.0 + 0.5 * math.log(3)])


def test_plain_matrix_memory_carries_its_state_and_stays_in_range():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(40, 6)), rng.normal(size=(40, 6)), rng.normal(size=(40, 5))
    i_log, f_log = rng.normal(size=40) * 3, -np.abs(rng.normal(size=40))
    whole, (S, n, m) = plain.matrix_memory(q, k, v, i_log, f_log)
    first, state = plain.matrix_memory(q[:17], k[:17], v[:17], i_log[:17], f_log[:17])
    second, (S2, n2, m2) = plain.matrix_memory(q[17:], k[17:], v[17:], i_log[17:], f_log[17:], state)
    assert np.allclose(np.concatenate([first, second]), whole, atol=1e-12) and np.allclose(S, S2) and np.allclose(n, n2) and m == m2
    # against the unstabilized sums: S_t = sum_j exp(i_j + sum_(l > j) f_l) k_j v_j^T, with the same denominator rule
    t = 12
    w = np.array([math.exp(i_log[j] + f_log[j + 1 : t + 1].sum()) for j in range(t + 1)])
    St = (w[:, None, None] * k[: t + 1, :, None] * v[: t + 1, None, :]).sum(0)
    nt = (w[:, None] * k[: t + 1]).sum(0)
    ms = plain.matrix_memory(q[: t + 1], k[: t + 1], v[: t + 1], i_log[: t + 1], f_log[: t + 1])[1][2]
    want = St.T @ q[t] / (max(abs(nt @ q[t]), 1.0) + 1e-6 * math.exp(ms))
    assert np.allclose(whole[t], want, rtol=1e-9)
    # the stabilizer starts at zero, not at minus infinity: a first input gate below zero leaves m at f
    _, (_, _, m1) = plain.matrix_memory(q[:1], k[:1], v[:1], np.array([-4.0]), np.array([-0.5]))
    assert m1 == -0.5
    # gates far out of range do not overflow
    big, _ = plain.matrix_memory(q, k, v, np.full(40, 80.0), np.full(40, -1e-3))
    assert np.isfinite(big).all()


def test_plain_gates_are_capped_before_the_logsigmoid():
    h = np.array([[100.0], [-100.0], [0.3]])
    w = {"i": np.ones((1, 1)), "i.b": np.zeros(1), "f": np.ones((1, 1)), "f.b": np.array([0.2])}
    i_log, f_log = plain.memory_gates(h, w, "", 5.0)
    assert i_log[0, 0] == pytest.approx(5.0) and i_log[1, 0] == pytest.approx(-5.0)
    assert f_log[0, 0] == pytest.approx(-math.log1p(math.exp(-5.0))) and f_log[1, 0] == pytest.approx(-5.0 - math.log1p(math.exp(-5.0)))
    assert f_log[2, 0] == pytest.approx(-math.log1p(math.exp(-5.0 * math.tanh(0.1))))
    assert plain.gelu_tanh(np.array([0.0]))[0] == 0.0 and plain.gelu_tanh(np.array([3.0]))[0] == pytest.approx(2.99636, abs=1e-4)
