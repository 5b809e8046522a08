"""Tiny Varolix configurations for the tests, and how their model folders are made.

They differ from one another in every size and constant: one to five query heads per key head, key and value widths that are
equal and unequal, rotations of a part and of all of a head with and without stretched waves, temperatures that step every
position and every few and none at all, matrix memories of one to three heads with tight and loose gate caps and with forget
gates that forget at once and that last, multipliers of the two halves that are one and that are not, latents narrower and
wider than a head, layers without a feed-forward, loops over the first, the middle and the last layers, a loop of one pass
and no loop.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np


def _attention(heads, kv_heads, dim, vdim, scale, rot=None, scaling=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        out["rot"] = {"dims": rot[0], "base": rot[1]}
        if scaling:
            out["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention", "mixer": out}


def _pair(left, right, left_scale, right_scale):
    heads, kv_heads, dim, vdim, scale, temp = left
    l = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if temp:
        l["q_temp"] = {"coef": temp[0], "every": temp[1]}
    r = dict(zip(("heads", "dim", "vdim", "gate_cap"), right))
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, rot_dims=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "q_rank": q_rank, "scale": scale, "rot": {"base": base, "dims": rot_dims or rot_dim}}}


def _with(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff} if ff else None)


def _config(vocab, width, eps, layers, loop=None):
    out = {"architecture": "Varolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


CASES = {
    # the three mixers, the middle two run three times; a layer without a feed-forward; stretched waves whose ramp lies inside
    # the rotated pairs; a temperature that steps every five positions
    "A": dict(config=_config(150, 64, 1e-5, [
        _with(_attention(4, 2, 16, 24, 0.3, (8, 100.0), (4.0, 32, 8.0, 1.0)), 48),
        _with(_pair((4, 2, 16, 8, 0.35, (0.3, 5)), (2, 8, 12, 4.0), 0.7, 1.3), None),
        _with(_latent(3, 8, 4, 12, 16, 10, 0.28, 300.0), 40),
        _with(_attention(2, 2, 8, 8, 0.4, (8, 30.0)), 24),
    ], loop=(1, 3, 3)), seed=41, page=8),
    # odd sizes everywhere; no loop, no temperature, no stretching; one head for all keys; a latent wider than a head; a rotation
    # of a part of the rotated coordinates
    "B": dict(config=_config(131, 50, 1e-6, [
        _with(_pair((3, 3, 10, 7, 0.31, None), (3, 7, 9, 11.0), 1.0, 1.0), 21),
        _with(_attention(5, 1, 6, 5, 0.45, (2, 7.0)), 37),
        _with(_latent(1, 5, 6, 3, 9, 7, 0.5, 13.0, 4), None),
        _with(_pair((2, 1, 6, 11, 0.4, (0.9, 1)), (1, 5, 3, 2.5), -0.8, 0.6), 33),
    ]), seed=42, page=16),
    # widths that the bfloat16 engine's tensor-core attention covers (64 and 128 for prompts on tcgen05, steps of 16 for the
    # cluster kernel); the first two layers run twice
    "C": dict(config=_config(128, 96, 1e-6, [
        _with(_attention(4, 1, 64, 64, 0.12, (32, 10000.0), (4.0, 64, 16.0, 2.0)), 64),
        _with(_pair((2, 2, 64, 64, 0.11, (0.6, 16)), (2, 32, 64, 12.0), 1.25, 0.75), 128),
        _with(_latent(4, 32, 16, 32, 48, 24, 0.14, 5000.0), 64),
        _with(_attention(2, 2, 128, 128, 0.09, (128, 500.0)), 96),
        _with(_pair((4, 1, 32, 32, 0.17, (0.2, 40)), (1, 64, 32, 8.0), 0.5, 1.5), 64),
    ], loop=(0, 2, 2)), seed=43, page=16),
    # memories that last (forget gates near one) behind a loose cap; a loop of one pass; the last layers looped
    "D": dict(config=_config(144, 64, 1e-5, [
        _with(_pair((2, 2, 16, 48, 0.25, (0.4, 3)), (3, 12, 8, 20.0), 1.1, 0.8), 40),
        _with(_pair((8, 2, 48, 16, 0.14, (1.5, 64)), (2, 20, 20, 30.0), 0.9, 1.4), None),
        _with(_attention(2, 1, 16, 16, 0.35, (16, 20000.0), (16.0, 16, 4.0, 0.5)), 24),
    ], loop=(0, 1, 1)), seed=44, page=8, forget_shift=5.0),
    # attention of both kinds only: no state at all; the last two layers run twice
    "E": dict(config=_config(90, 48, 1e-6, [
        _with(_attention(3, 1, 16, 8, 0.25, (12, 200.0), (2.0, 24, 6.0, 1.5)), 32),
        _with(_latent(2, 16, 8, 24, 20, 32, 0.2, 1000.0), 96),
        _with(_latent(5, 4, 2, 6, 8, 6, 0.6, 50.0), 16),
    ], loop=(1, 3, 2)), seed=45, page=16),
    # matrix memories beside attention only: one mixer kind, a tight cap, a forget gate that forgets at once
    "F": dict(config=_config(101, 40, 1e-5, [
        _with(_pair((2, 1, 8, 8, 0.5, None), (2, 16, 8, 1.5), 1.0, 2.0), 24),
        _with(_pair((1, 1, 24, 16, 0.2, (0.7, 2)), (4, 4, 12, 6.0), 2.0, 1.0), 56),
    ], loop=(0, 2, 2)), seed=46, page=8, forget_shift=-3.0),
}


def random_case(seed: int) -> dict:
    """A configuration drawn from many sizes: widths, head counts and groups, key and value widths that the tensor-core kernels
    cover and that they do not, rotations of all, a part and none of a head with and without stretching, latents of many ranks,
    two to six layers of the three kinds in any order, with and without a loop."""
    import random

    rng = random.Random(seed)

    def att():
        dim = rng.choice([16, 32, 48, 64, 80, 96, 128, 192, 256])
        kv, g = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4, 8])
        dims = rng.choice([dim, dim // 2, dim // 4 * 2, 8, 0]) // 2 * 2
        scaling = None
        if dims and rng.random() < 0.7:
            scaling = (rng.choice([2.0, 8.0, 32.0]), rng.choice([16, 64, 1024, 4096]), rng.choice([32.0, 8.0, 4.0]), rng.choice([1.0, 0.5, 2.0]))
        return _attention(kv * g, kv, dim, rng.choice([dim, dim, 32, 64, 128, 40]), dim ** -0.5 * rng.choice([1.0, 0.7, 1.3]),
                          (dims, rng.choice([100.0, 10000.0, 40000.0, 1e6])) if dims else None, scaling)

    def pair():
        dim = rng.choice([16, 32, 48, 64, 96, 128])
        kv, g = rng.choice([1, 2, 3]), rng.choice([1, 2, 4, 6])
        left = (kv * g, kv, dim, rng.choice([dim, 32, 64, 128, 24]), rng.choice([0.11, dim ** -0.5, 0.3]),
                (rng.choice([0.6, 0.1, 1.0]), rng.choice([1, 7, 32, 100])))
        right = (rng.choice([1, 2, 3, 4]), rng.choice([8, 16, 24, 48, 64, 100, 128]), rng.choice([8, 16, 33, 64, 96, 128]), rng.choice([12.0, 5.0, 30.0]))
        return _pair(left, right, rng.choice([1.25, 1.0, 0.5]), rng.choice([0.75, 1.0, 1.5]))

    def lat():
        dim, rd = rng.choice([16, 32, 64, 96, 128]), rng.choice([8, 16, 32, 64, 24])
        return _latent(rng.choice([1, 2, 4, 8, 12, 16, 20]), dim, rd, rng.choice([dim, 32, 64, 48]), rng.choice([32, 64, 128, 192, 256, 72]),
                       rng.choice([24, 72, 96, 200]), (dim + rd) ** -0.5, rng.choice([40000.0, 10000.0]))

    width = rng.choice([64, 96, 160, 192, 288, 384])
    n = rng.choice([2, 3, 4, 6])
    layers = [_with(rng.choice([att, pair, lat])(), rng.choice([64, 256, 200]) if rng.random() < 0.85 else None) for _ in range(n)]
    loop = None
    if rng.random() < 0.7:
        a = rng.randrange(0, n)
        loop = (a, rng.randrange(a + 1, n + 1), rng.choice([1, 2, 3]))
    return _config(rng.choice([100, 512, 1000, 257]), width, rng.choice([1e-6, 1e-5]), layers, loop)


def make_model_dir(root, name: str) -> Path:
    """Writes the tiny model `name` (config.json, model.safetensors in bfloat16-exact float32) under root."""
    import torch

    from machserve_b200.config import config_from_json
    from machserve_b200.weights import write_random_model
    from machserve_b200.weights.safetensors_io import write_safetensors

    case = CASES[name]
    out = Path(root) / f"varolix_{name}"
    if (out / "model.safetensors").exists():
        return out
    raw = Path(root) / f"varolix_{name}_drawn"
    write_random_model(config_from_json(case["config"]), raw, case["seed"], torch.float32, 0.12, 0.3, 0.1)
    _, w = read_weights(raw)
    tensors = {}
    for k, v in w.items():
        a = np.asarray(v)
        t = torch.from_numpy(a.astype(np.float32) if a.dtype.kind == "f" else a)
        if k.endswith(".f.b"):
            t = t + case.get("forget_shift", 0.0)
        tensors[k] = t.to(torch.bfloat16).to(torch.float32) if t.dtype == torch.float32 else t
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text((raw / "config.json").read_text())
    write_safetensors(out / "model.safetensors", tensors)
    return out


def read_weights(model_dir, round_to_bf16: bool = False):
    from tests.plain import read_model_dir

    return read_model_dir(model_dir, round_to_bf16=round_to_bf16)


def plain_logits(model_dir, tokens, bf16_weights: bool = False) -> np.ndarray:
    from tests.plain.varolix import forward

    cfg, w = read_weights(model_dir, bf16_weights)
    return forward(cfg, w, tokens)


def _jitter(rel: float, seed: int):
    """A function that multiplies every element by 1 + rel * u, u uniform in [-1, 1]: rounding noise of a chosen size."""
    rng = np.random.default_rng(seed)
    return lambda a: np.asarray(a) * (1.0 + rel * rng.uniform(-1.0, 1.0, size=np.shape(a)))


def plain_with_reach(model_dir, tokens, dtype: str):
    """(logits [T, vocab], streams after every run, reach [T], reaches of the streams): `reach[t]` is how far row t's logits
    move (largest element) when what an engine of that dtype rounds is disturbed by noise of its rounding's size and all else
    stays as it is; the largest of several draws (near a cancellation one draw may happen to move little).  Most rows move little.  A row moves far where a head of a matrix memory has
    few live terms that cancel: its read-out is divided by its own root mean square, which is then all rounding.  A float32
    engine: noise of a few units in the last place of 24 bits on everything it hands on and on what enters and leaves the
    recurrence.  A bfloat16 engine: the layers' normed inputs, queries, kept keys and values, the softmax's weights and the
    rows that output projections read rounded to bfloat16 (the inputs alone; all of them; all of them with noise of that size
    instead, twice), with the float32 noise on the recurrence."""
    import torch

    from tests.plain.varolix import forward

    cfg, w = read_weights(model_dir, dtype == "bfloat16")
    streams = []
    logits = forward(cfg, w, tokens, streams)
    r16 = lambda h: torch.from_numpy(np.ascontiguousarray(h).astype(np.float32)).to(torch.bfloat16).to(torch.float64).numpy()
    fine = 2.0 ** -22
    if dtype == "float32":
        draws = [(_jitter(fine, 3 * n), _jitter(fine, 3 * n + 1) if n % 2 else None, _jitter(fine, 3 * n + 2)) for n in range(6)]
    else:
        draws = [(r16, None, _jitter(fine, 3)), (r16, r16, _jitter(fine, 5)), (_jitter(2.0 ** -8, 6), _jitter(2.0 ** -8, 7), _jitter(fine, 8)),
                 (_jitter(2.0 ** -8, 9), _jitter(2.0 ** -8, 10), _jitter(fine, 11))]
    reach = np.zeros(len(tokens))
    stream_reach = [np.zeros(len(tokens)) for _ in streams]
    for rh, ri, rr in draws:
        taps = []
        moved = forward(cfg, w, tokens, taps, rh, ri, rr)
        reach = np.maximum(reach, np.abs(moved - logits).max(-1))
        for j, (a, b) in enumerate(zip(taps, streams)):
            stream_reach[j] = np.maximum(stream_reach[j], np.abs(a - b).max(-1))
    return logits, streams, reach, stream_reach


def assert_rows_close(got, want, reach, tol: float, what: str, tight: float = 0.7) -> int:
    """Row t of `got` within max(tol * max(1, largest |want|), 4 * reach[t]) of `want`; at least `tight` of the rows are
    held to the first of the two, and the median row lies within half of it (the test keeps its teeth).  Returns how many rows
    are held to the tolerance itself."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    base = tol * max(1.0, float(np.abs(want).max()))
    allowed = np.maximum(base, 4.0 * np.asarray(reach))
    err = np.abs(got - want).max(-1)
    bad = np.nonzero(err > allowed)[0]
    assert len(bad) == 0, (f"{what}: {len(bad)} rows differ by more than max({base:.3g}, 4 x what rounding moves them); first bad row "
                           f"{bad[0]} (error {err[bad[0]]:.3g}, allowed {allowed[bad[0]]:.3g}), worst {err.max():.3g}")
    held = int((allowed <= base).sum())
    assert held >= tight * len(err), f"{what}: rounding alone moves all but {held} of {len(err)} rows by more than a quarter of the tolerance"
    assert np.median(err) <= 0.5 * base, f"{what}: the median row differs by {np.median(err):.3g}, more than half of {base:.3g}"
    return held
