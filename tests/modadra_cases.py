"""Tiny Modadra configurations for the tests, and how their model folders are made.

They differ from one another in every size and constant: one to five query heads per key head on the attention side and one to
three value heads per key head on the recurrent side, key and value widths that are equal and unequal, rotations of none, a
part and all of a head, windows of one token, of no multiple of a page, of one past a key tile, longer than every prompt and
none at all, convolutions of one to six taps, routers with one group, with as many kept as there are, with groups of one
expert and with all experts chosen, layers without a feed-forward, a multiplier of one, no cap on the logits.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np


def _left(heads, kv_heads, dim, vdim, scale, rot=None, window=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        out["rot"] = {"dims": rot[0], "base": rot[1]}
    if window:
        out["mask"] = {"size": window}
    return out


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(ff, experts, top, groups=None, scale=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _layer(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _config(vocab, width, eps, layers, mult=None, cap=None):
    out = {"architecture": "Modadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if mult is not None:
        out["residual_mult"] = mult
    if cap is not None:
        out["logit_softcap"] = cap
    return out


CASES = {
    # three layers that differ in everything; windows of 12, 7 and 20 (no multiples of the page of 8); a layer without a feed-forward
    "A": dict(config=_config(150, 64, 1e-5, [
        _layer(_left(4, 2, 16, 24, 0.3, (8, 100.0), 12), _right(4, 2, 8, 16, 3), _moe(32, 6, 2, (3, 2), 1.5)),
        _layer(_left(3, 3, 8, 8, 0.5, (8, 10000.0), 7), _right(2, 1, 16, 12, 2), None),
        _layer(_left(2, 1, 32, 16, 0.2, None, 20), _right(3, 3, 12, 20, 5), _moe(48, 8, 3, (2, 1), 1.0)),
    ], mult=0.5, cap=8.0), seed=31, page=8),
    # odd sizes everywhere; no multiplier, no cap, no groups, no weight scale; a window longer than every prompt; a convolution
    # of one tap (no inputs to keep); groups of three of which one is kept, one expert a token
    "B": dict(config=_config(131, 50, 1e-6, [
        _layer(_left(5, 1, 6, 5, 0.45, (2, 7.0), 13), _right(3, 1, 7, 9, 4), _moe(21, 5, 2)),
        _layer(_left(1, 1, 10, 7, 0.31, (10, 3000.0), 500), _right(1, 1, 5, 3, 1), _moe(37, 9, 1, (3, 1), 0.7)),
    ]), seed=32, page=16),
    # widths that the bfloat16 engine's tensor-core attention covers; windows of 64 (a key tile) and 33 (one past half of it);
    # every expert chosen; as many groups kept as there are
    "C": dict(config=_config(128, 96, 1e-6, [
        _layer(_left(4, 1, 32, 32, 0.17, (16, 50000.0), 64), _right(2, 2, 32, 64, 4), _moe(64, 8, 2, (4, 2), 2.0)),
        _layer(_left(2, 2, 64, 64, 0.11, (64, 500.0), 33), _right(4, 1, 16, 32, 3), _moe(128, 4, 4, (2, 2), 1.0)),
    ], mult=0.7, cap=20.0), seed=33, page=16),
    # no window at all in one layer and a window of one token (the query's own key) in another; a fast rotation; groups of one
    # expert; a last layer without a feed-forward; a convolution of six taps
    "D": dict(config=_config(144, 64, 1e-5, [
        _layer(_left(2, 2, 16, 48, 0.25, (4, 10.0), None), _right(6, 2, 12, 8, 2), _moe(40, 4, 1, (4, 2), 2.5)),
        _layer(_left(8, 2, 48, 16, 0.14, (24, 1000.0), 1), _right(2, 2, 20, 20, 6), _moe(24, 12, 4, (4, 2), 0.5)),
        _layer(_left(2, 1, 16, 16, 0.35, (16, 20000.0), 48), _right(1, 1, 64, 32, 4), None),
    ], mult=0.25, cap=30.0), seed=34, page=8),
    # a memory that lasts (decays close to one) and corrections as large as the scores, below zero for most experts
    "E": dict(config=_config(90, 48, 1e-6, [
        _layer(_left(3, 1, 16, 8, 0.25, (12, 200.0), 24), _right(4, 2, 16, 24, 3), _moe(32, 10, 3, (5, 2), 1.2)),
        _layer(_left(2, 2, 8, 32, 0.4, None, 10), _right(2, 1, 24, 16, 4), _moe(96, 6, 2, (2, 1))),
    ], mult=0.4), seed=35, page=16, a_log_shift=-3.5, correction=(-0.8, 6.0)),
}


def _rewrite(src: Path, dst: Path, change) -> None:
    import torch

    from machserve_b200.weights.safetensors_io import write_safetensors

    dst.mkdir(parents=True, exist_ok=True)
    _, w = read_weights(src)
    tensors = {}
    for k, v in w.items():
        a = np.asarray(v)
        t = torch.from_numpy(a.astype(np.float32) if a.dtype.kind == "f" else a)
        tensors[k] = change(k, t)
    (dst / "config.json").write_text((src / "config.json").read_text())
    write_safetensors(dst / "model.safetensors", tensors)


def make_model_dir(root, name: str, steady_routers: bool = False) -> Path:
    """Writes the tiny model `name` (config.json, model.safetensors in bfloat16-exact float32) under root.
    `steady_routers`: a second folder whose routers weigh the token 30 times less and whose corrections are three times as
    large, so that the corrections decide most choices by margins that rounding to bfloat16 cannot turn."""
    import torch

    from machserve_b200.config import config_from_json
    from machserve_b200.weights import write_random_model

    case = CASES[name]
    out = Path(root) / f"modadra_{name}"
    if not (out / "model.safetensors").exists():
        raw = Path(root) / f"modadra_{name}_drawn"
        write_random_model(config_from_json(case["config"]), raw, case["seed"], torch.float32, 0.12, 0.3, 0.1)
        shift, corr = case.get("a_log_shift", 0.0), case.get("correction", (0.0, 1.0))

        def change(k, t):
            if k.endswith(".A_log"):
                t = t + shift
            if k.endswith("mlp.correction"):
                t = t * corr[1] + corr[0]
            return t.to(torch.bfloat16).to(torch.float32) if t.dtype == torch.float32 else t

        _rewrite(raw, out, change)
    if not steady_routers:
        return out
    steady = Path(root) / f"modadra_{name}_steady"
    if not (steady / "model.safetensors").exists():
        import torch

        def steadier(k, t):
            if k.endswith("mlp.router"):
                t = t / 30.0
            if k.endswith("mlp.correction"):
                t = t * 3.0
            return t.to(torch.bfloat16).to(torch.float32) if t.dtype == torch.float32 else t

        _rewrite(out, steady, steadier)
    return steady


def read_weights(model_dir, round_to_bf16: bool = False):
    from tests.plain import read_model_dir

    return read_model_dir(model_dir, round_to_bf16=round_to_bf16)


def plain_logits(model_dir, tokens, bf16_weights: bool = False) -> np.ndarray:
    from tests.plain.modadra import forward

    cfg, w = read_weights(model_dir, bf16_weights)
    return forward(cfg, w, tokens)


CLOSE_CALL = 0.01  # a margin of a router's choice below this can fall either way under bfloat16 rounding


def plain_logits_and_close_calls(model_dir, tokens, bf16_weights: bool = False, tol: float = 0.02):
    """(logits [T, vocab], unsure [T] bool).  `unsure[t]` says that the plain model itself cannot vouch for row t under
    bfloat16 rounding: some router chose an expert or a group by less than CLOSE_CALL at token t, or the row's logits move by
    more than `tol` (times their largest) when what a bfloat16 engine hands on in 16 bits (the layers' normed inputs, kept keys
    and values, the rows that the output projections read) is rounded to bfloat16 and all else stays as it is (or the normed
    inputs alone: two draws of the same noise).  A recurrent
    layer hands a wrong choice on to the rows after it, so every row after a close call of such a model is unsure too for as
    long as the state remembers: the callers compare long sequences of those cases in float32."""
    import torch

    from tests.plain.modadra import forward

    cfg, w = read_weights(model_dir, bf16_weights)
    margins = []
    logits = forward(cfg, w, tokens, None, margins)
    unsure = np.zeros(len(tokens), dtype=bool)
    for m in margins:
        unsure |= m < CLOSE_CALL
    r16 = lambda h: torch.from_numpy(h.astype(np.float32)).to(torch.bfloat16).to(torch.float64).numpy()
    for inner in (None, r16):  # two draws of the rounding: the normed inputs alone, and every place named above
        rounded = forward(cfg, w, tokens, None, None, r16, inner)
        unsure |= np.abs(rounded - logits).max(-1) > tol * max(1.0, float(np.abs(logits).max()))
    return logits, unsure
