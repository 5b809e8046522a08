"""Plain, slow, whole-sequence numpy implementation of the Varolix decoder, one function per mechanism.

Written from the design's equations; it keeps no cache and no state between calls, computes a whole sequence at once
in float64, and imports nothing from the engine package: it is what the engine is compared with.

Notation: d the model width, T the tokens of the sequence, p the position of a token (from 0), W [out, in] a matrix
applied as x . W^T.  `rnd`, where a function takes it, rounds what an engine hands on in fewer bits (keys and values that
are kept for later tokens, rows that output projections read); None rounds nothing.  `rec` likewise disturbs what enters and
leaves a recurrence, which an engine computes in 32 bits: a test finds with it the rows whose result hangs on the last bits.
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


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def _same(a):
    return a


# ------------------------------------------------------------------------------------------ rotation


def rotary_frequencies(dims, base, scaling=None):
    """(f [dims/2], m): the angle of pair i at position p is p * f_i, and cos and sin are multiplied by m.
    Without scaling f_i = base^(-2i/dims), m = 1.  With scaling {factor, original, fast, slow}: the pair index at which a
    wave makes t turns over `original` positions is n(t) = dims * ln(original / (2 pi t)) / (2 ln base);
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
    f_i <- f_i / factor * r_i + f_i * (1 - r_i);  m = 0.1 ln(factor) + 1."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0

    def n(turns):
        return dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(n(scaling["fast"])), 0)
    hi = min(math.ceil(n(scaling["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / scaling["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate_half(x, positions, rot):
    """x [T, heads, width]: of each head's first rot.dims coordinates, i is paired with i + dims/2; the pair (u, v) at
    position p becomes (u c - v s, v c + u s) with c = m cos(p f_i), s = m sin(p f_i).  The other coordinates stay."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    half = dims // 2
    f, m = rotary_frequencies(dims, rot["base"], rot.get("scaling"))
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (m * np.cos(ang))[:, None, :], (m * np.sin(ang))[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------ softmax attention


def causal_softmax(s, sink=None):
    """s [T, T] scores; row i sees the columns j <= i.  `sink`, a number: exp(sink) joins the denominator once."""
    t = s.shape[0]
    s = np.where(np.arange(t)[:, None] >= np.arange(t)[None, :], s, -np.inf)
    m = s.max(-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink)
    e = np.exp(s - m)
    den = e.sum(-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - m)
    return e / den


def grouped_attend(q, k, v, scale, rnd=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H*dv]; query head h reads key/value head h // (H/G).  `rnd` rounds the
    queries and the softmax's weights (a tensor core's operands)."""
    rnd = rnd or _same
    t, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((t, H, v.shape[2]))
    q = rnd(q)
    for h in range(H):
        g = h // (H // G)
        out[:, h] = rnd(causal_softmax(q[:, h] @ k[:, g].T * scale)) @ v[:, g]
    return out.reshape(t, -1)


def rotary_attention(h, w, p, cfg, rnd=None):
    """Mixer `attention`: biased q, k, v; rotation of the first rot.dims coordinates of every head; causal softmax."""
    rnd = rnd or _same
    t = h.shape[0]
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    pos = np.arange(t)
    q = rotate_half((h @ w[p + "q"].T + w[p + "q.b"]).reshape(t, H, dk), pos, cfg.get("rot"))
    k = rotate_half((h @ w[p + "k"].T + w[p + "k.b"]).reshape(t, G, dk), pos, cfg.get("rot"))
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(t, G, dv)
    return rnd(grouped_attend(q, rnd(k), rnd(v), cfg["scale"], rnd)) @ w[p + "o"].T


def query_temperature(positions, temp):
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = np.asarray(positions, dtype=np.float64)
    return 1.0 + temp["coef"] * np.log(np.floor((p + 1.0) / temp["every"]) + 1.0)


def normed_attention(h, w, p, cfg, eps, rnd=None):
    """The left half of mixer `parallel`: biased q, k, v and output; every q and k head normed with a weight that the
    heads share; no rotation; the query multiplied by a temperature that grows with the position; causal softmax."""
    rnd = rnd or _same
    t = h.shape[0]
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = rms_norm((h @ w[p + "q"].T + w[p + "q.b"]).reshape(t, H, dk), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T + w[p + "k.b"]).reshape(t, G, dk), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(t, G, dv)
    if cfg.get("q_temp"):
        q = q * query_temperature(np.arange(t), cfg["q_temp"])[:, None, None]
    return rnd(grouped_attend(q, rnd(k), rnd(v), cfg["scale"], rnd)) @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------------------------------ matrix memory


def soft_cap(z, cap):
    return cap * np.tanh(z / cap)


def matrix_memory(q, k, v, i_log, f_log, state=None):
    """One head.  q, k [T, dk], v [T, dv]; i_log, f_log [T] the logarithms of the input and forget gates.
    m_t = max(f_t + m_(t-1), i_t);  S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T;  n_t likewise
    with k_t alone;  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).  S, n and m start at zero (or at `state`).
    Returns (o [T, dv], (S, n, m))."""
    dk, dv = q.shape[1], v.shape[1]
    S, n, m = (np.zeros((dk, dv)), np.zeros(dk), 0.0) if state is None else (state[0].copy(), state[1].copy(), float(state[2]))
    o = np.zeros((q.shape[0], dv))
    for t in range(q.shape[0]):
        m_new = max(f_log[t] + m, i_log[t])
        a, b = math.exp(f_log[t] + m - m_new), math.exp(i_log[t] - m_new)
        S = a * S + b * np.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        o[t] = S.T @ q[t] / (max(abs(float(n @ q[t])), math.exp(-m)) + 1e-6)
    return o, (S, n, m)


def memory_gates(h, w, p, cap):
    """(i_log, f_log) [T, H]: i = cap tanh((W_i h + b_i) / cap); f = logsigmoid(cap tanh((W_f h + b_f) / cap))."""
    return soft_cap(h @ w[p + "i"].T + w[p + "i.b"], cap), log_sigmoid(soft_cap(h @ w[p + "f"].T + w[p + "f.b"], cap))


def matrix_memory_mixer(h, w, p, cfg, eps, rnd=None, rec=None):
    """The right half of mixer `parallel`."""
    rnd, rec = rnd or _same, rec or _same
    t = h.shape[0]
    H, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = rec((h @ w[p + "q"].T).reshape(t, H, dk) * dk ** -0.5)
    k = rec((h @ w[p + "k"].T).reshape(t, H, dk))
    v = rec((h @ w[p + "v"].T).reshape(t, H, dv))
    i_log, f_log = memory_gates(h, w, p, cfg["gate_cap"])
    i_log, f_log = rec(i_log), rec(f_log)
    o = np.zeros((t, H, dv))
    for head in range(H):
        o[:, head], _ = matrix_memory(q[:, head], k[:, head], v[:, head], i_log[:, head], f_log[:, head])
    y = unit_rms(rec(o), eps).reshape(t, H * dv) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return rnd(y) @ w[p + "o"].T


def two_mixers_sum(h, w, p, cfg, eps, rnd=None, rec=None):
    """Mixer `parallel`: both halves read h; left_scale * left + right_scale * right."""
    left = normed_attention(h, w, p + "left.", cfg["left"], eps, rnd)
    right = matrix_memory_mixer(h, w, p + "right.", cfg["right"], eps, rnd, rec)
    return cfg["left_scale"] * left + cfg["right_scale"] * right


# ------------------------------------------------------------------------------------------ latent attention


def latent_attention(h, w, p, cfg, eps, rnd=None):
    """Mixer `latent_attention`: queries through a normed latent; one normed latent and one rotated key part a token, from
    which every head's unrotated keys and values are made; a sink in every head's softmax; a gate per head."""
    rnd = rnd or _same
    t = h.shape[0]
    H, dn, dr, dv, r = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    pos = np.arange(t)
    rot = dict(cfg["rot"])
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (rnd(cq) @ w[p + "uq"].T).reshape(t, H, dn + dr)
    q_plain, q_rot = rnd(q[..., :dn]), rnd(rotate_half(q[..., dn:], pos, rot))
    down = h @ w[p + "dkv"].T
    c = rnd(rms_norm(down[:, :r], w[p + "dkv.norm"], eps))
    k_rot = rnd(rotate_half(down[:, None, r:], pos, rot)[:, 0])  # [T, dr], shared by the heads
    k_plain = (c @ w[p + "uk"].T).reshape(t, H, dn)
    v = (c @ w[p + "uv"].T).reshape(t, H, dv)
    gate = sigmoid(h @ w[p + "g"].T)  # [T, H]
    out = np.zeros((t, H, dv))
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * cfg["scale"]
        out[:, head] = rnd(causal_softmax(s, float(w[p + "sink"][head]))) @ v[:, head] * gate[:, head:head + 1]
    return rnd(out.reshape(t, H * dv)) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ the feed-forward and the model


def dense_mlp(h, w, p, rnd=None):
    rnd = rnd or _same
    return rnd(gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixer(h, w, p, spec, eps, rnd=None, rec=None):
    if spec["type"] == "attention":
        return rotary_attention(h, w, p, spec["mixer"], rnd)
    if spec["type"] == "parallel":
        return two_mixers_sum(h, w, p, spec["mixer"], eps, rnd, rec)
    if spec["type"] == "latent_attention":
        return latent_attention(h, w, p, spec["mixer"], eps, rnd)
    raise ValueError(spec["type"])


def layer(x, w, i, spec, eps, round_h=None, rnd=None, rec=None):
    """x <- x + mixer(norm1(x)); then, if the layer has a feed-forward, x <- x + ff(norm2(x))."""
    p = f"l{i}."
    rh = round_h or _same
    x = x + mixer(rh(rms_norm(x, w[p + "norm1"], eps)), w, p + "mix.", spec, eps, rnd, rec)
    if spec.get("mlp") is not None:
        x = x + dense_mlp(rh(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.", rnd)
    return x


def run_order(config):
    """The layers in the order they run: the looped range `times` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def forward(config, w, tokens, taps=None, round_h=None, round_inner=None, round_rec=None):
    """Logits [T, vocab] of a whole sequence; `taps`, a list, receives the stream after every run of a layer."""
    w = {k: np.asarray(v, dtype=np.float64) if np.asarray(v).dtype.kind == "f" else np.asarray(v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens, dtype=np.int64)]
    for i in run_order(config):
        x = layer(x, w, i, config["layers"][i], eps, round_h, round_inner, round_rec)
        if taps is not None:
            taps.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
