"""Plain, slow, whole-sequence numpy implementation of the Modadra decoder, one function per mechanism.

Written from the design's equations; it keeps no cache and no state between calls, computes a whole sequence at once
in float64, and imports nothing from the engine package: it is what the engine is compared with.

Notation: d the model width, T the tokens of the sequence, p the position of a token (from 0), W [out, in] a matrix
applied as x . W^T.
"""
from __future__ import annotations

import math

import numpy as np


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


# ------------------------------------------------------------------------------------------ the attention half


def rotate_half_partial(x, positions, dims, base):
    """x [T, heads, width]: of each head's first `dims` coordinates, i is paired with i + dims/2; the pair (a, b) at
    position p becomes (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims).  The other coordinates stay."""
    if not dims:
        return x
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def window_mask(t, size):
    """visible[i, j]: 0 <= i - j < size (every earlier key when size is None)."""
    dist = np.arange(t)[:, None] - np.arange(t)[None, :]
    return (dist >= 0) if size is None else (dist >= 0) & (dist < size)


def softmax_plus_one(s, visible):
    """exp(s_j) / (1 + sum over the visible j of exp(s_j)): a sink of score 0 that has no value."""
    s = np.where(visible, s, -np.inf)
    m = np.maximum(s.max(-1, keepdims=True), 0.0)
    e = np.exp(s - m)
    return e / (np.exp(-m) + e.sum(-1, keepdims=True))


def windowed_attention(h, w, p, cfg, rnd=None):
    """Grouped heads, key and value widths of their own, rotation of a part of every head, a sliding window, the softmax
    with one added to its denominator, a gate per head from the mixer's input, the output projection."""
    t = h.shape[0]
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    pos = np.arange(t)
    rot = cfg.get("rot") or {}
    q = rotate_half_partial((h @ w[p + "q"].T).reshape(t, H, dk), pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_half_partial((h @ w[p + "k"].T).reshape(t, G, dk), pos, rot.get("dims", 0), rot.get("base", 1.0))
    v = (h @ w[p + "v"].T).reshape(t, G, dv)
    rnd = rnd or (lambda a: a)  # (a rounding of what is kept for later tokens and of what the output projection reads)
    k, v = rnd(k), rnd(v)
    gate = sigmoid(h @ w[p + "g"].T)  # [T, H]
    vis = window_mask(t, (cfg.get("mask") or {}).get("size"))
    out = np.zeros((t, H, dv))
    for head in range(H):
        g = head // (H // G)
        prob = softmax_plus_one(q[:, head] @ k[:, g].T * cfg["scale"], vis)
        out[:, head] = (prob @ v[:, g]) * gate[:, head : head + 1]
    return rnd(out.reshape(t, H * dv)) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ the recurrent half


def short_conv(x, taps_w, before=None):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] * x_(t - (taps-1) + j), zeros (or `before`, the taps - 1 rows
    that came before) ahead of the first row."""
    taps = taps_w.shape[1]
    pad = np.zeros((taps - 1, x.shape[1])) if before is None else before
    xx = np.concatenate([pad, x], axis=0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += xx[j : j + x.shape[0]] * taps_w[:, j][None, :]
    return y


def unit_vector(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def delta_rule(q, k, v, beta, g, state=None):
    """One head.  q, k [T, dk], v [T, dv], beta, g [T].  S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T;
    o_t = S^T q_t (after the write).  Returns (o [T, dv], S)."""
    dk, dv = q.shape[1], v.shape[1]
    s = np.zeros((dk, dv)) if state is None else state.copy()
    o = np.zeros((q.shape[0], dv))
    for t in range(q.shape[0]):
        s = g[t] * s
        u = beta[t] * (v[t] - s.T @ k[t])
        s = s + np.outer(k[t], u)
        o[t] = s.T @ q[t]
    return o, s


def gated_delta(h, w, p, cfg, eps, rnd=None):
    t = h.shape[0]
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(t, G, dk)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(t, G, dk)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(t, H, dv)
    q = unit_vector(q) * dk ** -0.5
    k = unit_vector(k)
    beta = sigmoid(h @ w[p + "b"].T)  # [T, H]
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))  # [T, H]
    o = np.zeros((t, H, dv))
    for head in range(H):
        g = head // (H // G)
        o[:, head], _ = delta_rule(q[:, g], k[:, g], v[:, head], beta[:, head], decay[:, head])
    o = unit_rms(o, eps) * w[p + "norm"]
    y = o.reshape(t, H * dv) * silu(h @ w[p + "g"].T)
    return (y if rnd is None else rnd(y)) @ w[p + "o"].T


def two_mixers(h, w, p, cfg, eps, rnd=None):
    """Both halves read h; each output is normed over the width with a weight of its own; half their sum."""
    left = windowed_attention(h, w, p + "left.", cfg["left"], rnd)
    right = gated_delta(h, w, p + "right.", cfg["right"], eps, rnd)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ------------------------------------------------------------------------------------------ the feed-forward


def route(h, w, p, router, margins=None):
    """(ids [T, top], weights [T, top]).  Scores s = sigmoid(W h); an expert is chosen by s + correction, among the experts
    of the `keep` best groups only (a group's score: the sum of its two largest choice scores); the weights are the chosen
    experts' s over their sum, times `scale`.  `margins`, a list, receives [T]: by how much the last choice (of an expert or of
    a group) was ahead of the best alternative."""
    n, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    s = sigmoid(h @ w[p + "router"].T)
    c = s + w[p + "correction"]
    per = n // count
    grouped = np.sort(c.reshape(-1, count, per), axis=-1)
    gscore = grouped[..., -2:].sum(-1)  # [T, count] (a group of one expert: that expert's score)
    gorder = np.argsort(-gscore, axis=-1, kind="stable")
    allowed = np.zeros((h.shape[0], count), dtype=bool)
    np.put_along_axis(allowed, gorder[:, :keep], True, axis=-1)
    masked = np.where(np.repeat(allowed, per, axis=-1), c, -np.inf)
    order = np.argsort(-masked, axis=-1, kind="stable")
    ids = order[:, :top]
    if margins is not None:
        sm = np.take_along_axis(masked, order, -1)
        m = sm[:, top - 1] - sm[:, top] if top < n else np.full(h.shape[0], np.inf)
        m = np.where(np.isfinite(m), m, np.inf)
        if keep < count:
            gs = np.take_along_axis(gscore, gorder, -1)
            m = np.minimum(m, gs[:, keep - 1] - gs[:, keep])
        margins.append(m)
    chosen = np.take_along_axis(s, ids, -1)
    return ids, chosen / (chosen.sum(-1, keepdims=True) + 1e-20) * router.get("scale", 1.0)


def expert(x, w, q, rnd=None):
    mid = gelu_erf(x @ w[q + "up"].T)
    return (mid if rnd is None else rnd(mid)) @ w[q + "down"].T


def routed_mlp(h, w, p, cfg, margins=None, rnd=None):
    ids, weights = route(h, w, p, cfg["router"], margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], weights[t]):
            out[t] += a * expert(h[t], w, f"{p}e{int(e)}.", rnd)
    return out


# ------------------------------------------------------------------------------------------ the model


def layer(x, w, i, spec, eps, mult, margins=None, round_h=None, round_inner=None):
    """x <- x + m * mixer(norm1(x)); then, if the layer has a feed-forward, x <- x + m * ff(norm2(x)).  `round_h`, a
    function, is applied to the normed rows, and `round_inner` to keys and values and to the rows that output projections
    read: what an engine does that hands them on in fewer bits."""
    p = f"l{i}."
    rnd = round_h or (lambda a: a)
    x = x + mult * two_mixers(rnd(rms_norm(x, w[p + "norm1"], eps)), w, p + "mix.", spec["mixer"], eps, round_inner)
    if spec.get("mlp") is not None:
        x = x + mult * routed_mlp(rnd(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.", spec["mlp"], margins, round_inner)
    return x


def soft_cap(z, cap):
    return cap * np.tanh(z / cap)


def forward(config, w, tokens, taps=None, margins=None, round_h=None, round_inner=None):
    """Logits [T, vocab] of a whole sequence; `taps`, a list, receives the stream after every layer; `margins`, a list,
    receives the router's margins [T] of every routed feed-forward (see `route`)."""
    w = {k: np.asarray(v, dtype=np.float64) if np.asarray(v).dtype.kind == "f" else np.asarray(v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens, dtype=np.int64)]
    for i, spec in enumerate(config["layers"]):
        x = layer(x, w, i, spec, eps, config.get("residual_mult", 1.0), margins, round_h, round_inner)
        if taps is not None:
            taps.append(x.copy())
    z = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    return soft_cap(z, cap) if cap else z
