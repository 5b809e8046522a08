"""Modadra on the GPU against the plain implementation: each mechanism's kernel alone, then the model in every way of cutting
the work (whole, token by token, portions down to two tokens, unequal requests side by side on reused pages and state slots),
and greedy generation through the engine."""
import json
import sys

import numpy as np
import pytest

from tests.helpers import (BF16_TOL, F32_TOL, REPO, assert_close, collect_rows, random_tokens, trace_portions, trace_tail_decode,
                           trace_whole)
from tests.modadra_cases import CASES, make_model_dir, plain_logits, plain_logits_and_close_calls, read_weights
from tests.plain import modadra as plain

pytestmark = pytest.mark.gpu

MODEL_CASES = [(n, d) for n in sorted(CASES) for d in ("float32", "bfloat16")]


def _torch():
    import torch

    return torch


def _dev(a, dtype=None):
    torch = _torch()
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _ints(v):
    torch = _torch()
    return torch.tensor(list(v), dtype=torch.int32, device="cuda")


def _held(a, tdt):
    """The values of `a` as an array of dtype tdt holds them, as float64."""
    return _dev(np.asarray(a, dtype=np.float32), tdt).float().cpu().numpy().astype(np.float64)


# ----------------------------------------------------------------------------------- mechanisms, one kernel each


def _paged(rng, tokens_per_seq, heads, width, page, spare=3):
    """Pages in shuffled order for sequences of the given lengths: (pages array, block table)."""
    per = [-(-n // page) for n in tokens_per_seq]
    ids = rng.permutation(sum(per) + spare)
    table = np.full((len(per), max(per) + 1), -1, dtype=np.int32)
    pages = np.zeros((sum(per) + spare, heads, page, width), dtype=np.float32)
    at = 0
    for s, n in enumerate(per):
        table[s, :n] = ids[at : at + n]
        at += n
    return pages, table


def _fill_pages(pages, table, seq, values, page):
    for p in range(values.shape[0]):
        pages[table[seq, p // page], :, p % page, :] = values[p]


@pytest.mark.parametrize("hq,hkv,dk,dv,rot,base,page", [(4, 2, 16, 24, 8, 100.0, 8), (3, 3, 10, 6, 10, 7.0, 16), (2, 1, 12, 20, 0, 1.0, 8),
                                                          (5, 1, 6, 5, 2, 3000.0, 16), (2, 2, 64, 64, 32, 50000.0, 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_of_a_part_of_every_head_and_the_store(hq, hkv, dk, dv, rot, base, page, dtype):
    """The first `rot` coordinates of every query and key head are turned in halves, the rest pass; values pass; keys and
    values land in their pages at the rows' positions; the queries come out in float32 and as a bfloat16 copy."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(hq * 100 + dk)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    positions = [0, 1, 2, 7, 8, 15, 16, 37, 90]
    qw, kw, vw = hq * dk, hkv * dk, hkv * dv
    proj = rng.normal(size=(len(positions), qw + kw + vw + hq + 3)).astype(np.float32)  # a wider product: gates lie behind
    cos_sin = None
    if rot:
        ang = np.arange(96, dtype=np.float64)[:, None] * (base ** (-2.0 * np.arange(rot // 2) / rot))[None, :]
        cos_sin = _dev(np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32))
    kp, table = _paged(rng, [91], hkv, dk, page)
    k_pages = torch.zeros(kp.shape, dtype=tdt, device="cuda")
    v_pages = torch.zeros(kp.shape[:3] + (dv,), dtype=tdt, device="cuda")
    q_out = torch.empty(len(positions), qw, device="cuda")
    q_half = torch.empty(len(positions), qw, dtype=torch.bfloat16, device="cuda")
    ops.rope_store(_dev(proj), cos_sin, rot, False, _ints(positions), _ints([0] * len(positions)), _dev(table), q_out, k_pages, v_pages,
                   hq, hkv, dk, dv, store=True, q_half=q_half)
    p64 = proj.astype(np.float64)
    want_q = plain.rotate_half_partial(p64[:, :qw].reshape(-1, hq, dk), positions, rot, base).reshape(-1, qw)
    want_k = plain.rotate_half_partial(p64[:, qw : qw + kw].reshape(-1, hkv, dk), positions, rot, base)
    assert_close(q_out.cpu().numpy(), want_q, 2e-6, "queries")
    assert_close(q_half.float().cpu().numpy(), want_q, 1e-2, "the bfloat16 copy of the queries")
    if rot < dk:
        assert np.array_equal(q_out.cpu().numpy().reshape(-1, hq, dk)[..., rot:], proj[:, :qw].reshape(-1, hq, dk)[..., rot:])
    tol = 2e-6 if dtype == "float32" else 1e-2
    for i, p in enumerate(positions):
        page_id = table[0, p // page]
        assert_close(k_pages[page_id, :, p % page].float().cpu().numpy(), want_k[i], tol, f"key at {p}")
        assert_close(v_pages[page_id, :, p % page].float().cpu().numpy().reshape(-1), p64[i, qw + kw : qw + kw + vw], tol, f"value at {p}")
    # a run that reads another run's pages stores nothing
    k2, v2 = torch.zeros_like(k_pages), torch.zeros_like(v_pages)
    ops.rope_store(_dev(proj), cos_sin, rot, False, _ints(positions), _ints([0] * len(positions)), _dev(table), q_out, k2, v2, hq, hkv, dk, dv,
                   store=False)
    assert float(k2.abs().max()) == 0.0 and float(v2.abs().max()) == 0.0
    assert_close(q_out.cpu().numpy(), want_q, 2e-6, "queries, nothing stored")


def _plain_attend(q, k, v, positions, window, scale, groups):
    """q [T, H, dk] at `positions` of one sequence whose keys k [N, G, dk] and values v [N, G, dv] are all there; the softmax
    has one added to its denominator."""
    t, h, _ = q.shape
    out = np.zeros((t, h, v.shape[2]))
    for i, p in enumerate(positions):
        lo = 0 if not window else max(0, p - window + 1)
        vis = np.zeros((1, k.shape[0]), dtype=bool)
        vis[0, lo : p + 1] = True
        for head in range(h):
            g = head // groups
            s = (q[i, head][None, :] @ k[:, g].T) * scale
            out[i, head] = (plain.softmax_plus_one(s, vis) @ v[:, g])[0]
    return out


def _attend_every_form(ops, q, kd, vd, table, rows, hq, hkv, dk, dv, window, scale, dtype):
    """The rows (sequence, position) of q through every attention kernel that the design's mixer may use at these widths:
    {name: out [T, hq, dv]}.  Rows that follow one another in a sequence are a portion; the others are decoded rows."""
    torch = _torch()
    t = len(rows)
    sinks = torch.zeros(hq, device="cuda")  # a sink of score zero: one more in the denominator
    pos, slot = _ints(p for _, p in rows), _ints(s for s, _ in rows)
    tab = _dev(table)
    outs = {}
    for share in (True, False):
        out = torch.zeros(t, hq * dv, dtype=kd.dtype, device="cuda")
        ops.attention_wide(_dev(q).view(t, hq * dk), kd, vd, out, sinks, pos, slot, tab, hq, hkv, dk, dv, window, scale, share_rows=share)
        outs["exact, rows share" if share else "exact, heads share"] = out.float().cpu().numpy().reshape(t, hq, dv)
    assert np.array_equal(outs["exact, rows share"], outs["exact, heads share"]), "the two forms of the exact kernel give the same bits"
    if dtype != "bfloat16":
        return outs
    # portions: runs of consecutive rows of one sequence; singles: the rest
    runs, singles, i = [], [], 0
    while i < t:
        j = i
        while j + 1 < t and rows[j + 1] == (rows[j][0], rows[j][1] + 1):
            j += 1
        (runs.append((i, j - i + 1)) if j > i else singles.append(i))
        i = j + 1
    if ops.attention_wide_mma_supports(dk, dv, dv, True):
        tile = ops.attention_wide_mma_tile_rows(dv)
        t0 = [a + b for a, n in runs for b in range(0, n, tile)]
        tn = [min(tile, n - b) for a, n in runs for b in range(0, n, tile)]
        for splits in (1, 3):
            out = torch.zeros(t, hq * dv, dtype=torch.bfloat16, device="cuda")
            if t0:
                ops.attention_wide_mma(_dev(q).view(t, hq * dk), kd, vd, out, sinks, pos, slot, tab, _ints(t0), _ints(tn), len(t0), False,
                                       hq, hkv, dk, dv, window, scale)
            if singles:
                items = len(singles) * hkv * (-(-(hq // hkv) // 16))
                scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(items, dv, splits)), device="cuda")
                ops.attention_wide_mma(_dev(q).view(t, hq * dk), kd, vd, out, sinks, pos, slot, tab, _ints(singles), None, len(singles), True,
                                       hq, hkv, dk, dv, window, scale, splits, scratch)
            outs[f"mma.sync, {splits} runs of keys"] = out.float().cpu().numpy().reshape(t, hq, dv)
    if dk == dv and dk in (64, 128) and ops.attention_prefill_tc_supports(dk, kd.shape[2]):
        from types import SimpleNamespace

        from machserve_b200.parts.attention import decode_launch

        qh = _dev(q).view(t, hq * dk).to(torch.bfloat16)
        out = torch.zeros(t, hq * dv, dtype=torch.bfloat16, device="cuda")
        t0 = [a + b for a, n in runs for b in range(0, n, 128)]
        tn = [min(128, n - b) for a, n in runs for b in range(0, n, 128)]
        if t0:
            ops.attention_prefill_tc(qh, kd, vd, out, _ints(t0), _ints(tn), len(t0), pos, slot, tab, hq, hkv, dk, window, scale, 1, None, None,
                                     sinks=sinks)
        if singles and not (ops.attention_decode_supports(dk, hq // hkv) and ops.attention_prefill_supports(dk)):
            scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(len(singles) * hkv * (-(-(hq // hkv) // 16)), dv, 1)), device="cuda")
            ops.attention_wide_mma(_dev(q).view(t, hq * dk), kd, vd, out, sinks, pos, slot, tab, _ints(singles), None, len(singles), True,
                                   hq, hkv, dk, dv, window, scale, 1, scratch)
        elif singles:
            rt = SimpleNamespace(sm_count=torch.cuda.get_device_properties(0).multi_processor_count)
            longest = max(rows[i][1] for i in singles) + 1
            tiles = -(-longest // 64) if not window else min(-(-longest // 64), (window + 63) // 64 + 1)
            splits, stages, warps, kpw, parts = decode_launch(rt, dk, ops.attention_decode_cluster_max_stages(dk), {}, len(singles) * hkv, tiles)
            scratch = counters = None
            if parts > 1:
                scratch = torch.zeros(ops.attention_decode_cluster_scratch_words(len(singles), hq, hkv, dk, parts), device="cuda")
                counters = torch.zeros(len(singles) * hkv, dtype=torch.int32, device="cuda")
            ops.attention_decode_cluster(qh, kd, vd, out, pos, slot, tab, hq, hkv, dk, window, scale, splits, stages, rows=_ints(singles),
                                         num_rows=len(singles), warps=warps, keys_per_warp=kpw, parts=parts, scratch=scratch, counters=counters,
                                         sinks=sinks)
        assert ops.tc_status_codes() == (0, 0)
        outs["tcgen05 portions, cluster decoding"] = out.float().cpu().numpy().reshape(t, hq, dv)
    return outs


@pytest.mark.parametrize("dk,dv,hq,hkv,window,page", [
    (16, 24, 4, 2, 12, 8), (6, 5, 5, 1, 13, 16), (32, 16, 2, 1, 20, 8), (48, 80, 6, 3, 40, 16), (64, 64, 4, 1, 64, 16), (64, 64, 2, 2, 33, 16),
    (128, 128, 4, 2, 100, 16), (16, 48, 2, 2, None, 8), (48, 16, 8, 2, 1, 8), (32, 32, 4, 1, 500, 16),
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_attention_with_one_more_in_the_denominator(dk, dv, hq, hkv, window, page, dtype):
    """Portions of two sequences side by side and decoded rows, the first tokens of a sequence among them, against the plain
    softmax with its sink of score zero; through the exact kernel and, in bfloat16, every tensor-core kernel that covers the
    widths."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(dk * 1000 + dv)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    lens = [150, 41]
    kp, table = _paged(rng, lens, hkv, dk, page)
    vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
    ks = [rng.normal(size=(n, hkv, dk)).astype(np.float32) for n in lens]
    vs = [rng.normal(size=(n, hkv, dv)).astype(np.float32) for n in lens]
    for s in range(2):
        _fill_pages(kp, table, s, ks[s], page)
        _fill_pages(vp, table, s, vs[s], page)
    kd, vd = _dev(kp, tdt), _dev(vp, tdt)
    ks, vs = [_held(k, tdt) for k in ks], [_held(v, tdt) for v in vs]
    scale = 1.2 / np.sqrt(dk)
    # a portion of sequence 0, its last position decoded, the first three positions of sequence 1, its last position decoded
    rows = [(0, p) for p in range(100, 137)] + [(0, 149)] + [(1, p) for p in range(3)] + [(1, 40)]
    q = rng.normal(size=(len(rows), hq, dk)).astype(np.float32)
    q[5] *= -6.0  # a row whose scores are far below zero: the one in the denominator takes nearly all of its weight
    outs = _attend_every_form(ops, q, kd, vd, table, rows, hq, hkv, dk, dv, window, scale, dtype)
    assert dtype == "float32" or len(outs) > 2 or dk % 16 or dv % 8, "a tensor-core kernel covers these widths"
    for name, got in outs.items():
        q_held = _held(q, torch.bfloat16) if name.startswith(("mma", "tcgen05")) else q.astype(np.float64)
        want = np.zeros((len(rows), hq, dv))
        for s in range(2):
            idx = [i for i, (ss, _) in enumerate(rows) if ss == s]
            want[idx] = _plain_attend(q_held[idx], ks[s], vs[s], [rows[i][1] for i in idx], window, scale, hq // hkv)
        tol = 2e-5 if dtype == "float32" else 1.5e-2
        assert_close(got.reshape(len(rows), -1), want.reshape(len(rows), -1), tol, f"{name} ({dk}, {dv}, window {window})")
    # the first token of a sequence sees its own key alone: weight e^s / (1 + e^s), not 1
    first = [i for i, r in enumerate(rows) if r == (1, 0)][0]
    s0 = (q[first].astype(np.float64).reshape(hq, dk) * ks[1][0].repeat(hq // hkv, axis=0)).sum(-1) * scale
    want0 = (1.0 / (1.0 + np.exp(-s0)))[:, None] * vs[1][0].repeat(hq // hkv, axis=0)
    assert_close(outs["exact, rows share"][first], want0, 2e-5 if dtype == "float32" else 1.5e-2, "the first token of a sequence")


@pytest.mark.parametrize("dk,dv,window,page,n", [(16, 24, 12, 8, 90), (64, 64, 40, 16, 200), (32, 16, 17, 8, 75), (48, 80, 64, 16, 330)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_key_stands_out_at_the_windows_edge(dk, dv, window, page, n, dtype):
    """Among keys of small scores one key answers the query's direction.  When it is the oldest key of the window it carries the
    row; one token later it is outside and must leave no trace.  Queries in a portion and queries decoded alone, with the edge
    at, before and behind a page's border; and a key far behind the window, which nothing may see."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(window * 7 + dk)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    hq, hkv = 2, 1
    scale = 1.0 / np.sqrt(dk)
    direction = np.zeros(dk, dtype=np.float32)
    direction[3] = 1.0
    marks = [m for m in (5, page - 1, page, 2 * page + 1, n - window - 2) if 0 <= m < n - window]
    k = (0.05 * rng.normal(size=(n, hkv, dk))).astype(np.float32)
    v = rng.normal(size=(n, hkv, dv)).astype(np.float32)
    for m in marks:
        k[m, 0] = 16.0 * np.sqrt(dk) * direction  # score 16 * |q_3| against scores near zero
        v[m, 0] = 100.0 + m
    kp, table = _paged(rng, [n], hkv, dk, page)
    vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
    _fill_pages(kp, table, 0, k, page)
    _fill_pages(vp, table, 0, v, page)
    kd, vd = _dev(kp, tdt), _dev(vp, tdt)
    edge = sorted({p for m in marks for p in (m, m + 1, m + window - 1, m + window, m + window + 1) if p < n})
    # one portion that covers every edge; then the positions at the edges decoded alone (three calls, so that no two rows of
    # a call follow one another: rows that do are a portion)
    calls = {"portion": [list(range(min(marks), min(n, max(marks) + window + 2)))],
             "alone": [[p for p in edge if p % 3 == r] for r in range(3)]}
    for how, groups in calls.items():
        got = {}
        for group in groups:
            if not group:
                continue
            q = np.tile(direction, (len(group), hq, 1)).astype(np.float32)
            outs = _attend_every_form(ops, q, kd, vd, table, [(0, p) for p in group], hq, hkv, dk, dv, window, scale, dtype)
            for name, o in outs.items():
                for i, p in enumerate(group):
                    got.setdefault(name, {})[p] = o[i]
        for name, by_pos in got.items():
            for p in edge:
                seen = [m for m in marks if 0 <= p - m < window]
                level = np.abs(by_pos[p]).max()
                if seen:  # the marked keys in the window share the weight; their values are 100 + mark
                    want = np.mean([100.0 + m for m in seen])
                    assert abs(by_pos[p].mean() - want) < 2.0, f"{name}: position {p} ({how}) must see the keys at {seen}, and no other marked key"
                else:
                    assert level < 10.0, f"{name}: position {p} ({how}) is {level:.3g}: it sees a marked key that its window has left"


def _gdr_inputs(rng, total, heads, groups, dk, dv, taps, extra=3):
    kw, vw = groups * dk, heads * dv
    c = 2 * kw + vw
    ld = extra + c + vw + 2 * heads + 2
    proj = rng.normal(size=(total, ld)).astype(np.float32)
    conv = (rng.normal(size=(c, taps)) / np.sqrt(taps)).astype(np.float32)
    a_log = rng.normal(size=heads).astype(np.float32) - 1.0
    dt_bias = rng.normal(size=heads).astype(np.float32)
    return proj, conv, a_log, dt_bias, dict(x=extra, b=extra + c + vw, a=extra + c + vw + heads, c=c, kw=kw, vw=vw)


def _plain_gdr(rows, conv, a_log, dt_bias, off, heads, groups, dk, dv):
    """One sequence whole: (q, k, v after convolution, SiLU and unit vectors; beta; decay; o)."""
    n = rows.shape[0]
    kw, c = off["kw"], off["c"]
    y = plain.silu(plain.short_conv(rows[:, off["x"] : off["x"] + c], conv.astype(np.float64)))
    q = plain.unit_vector(y[:, :kw].reshape(n, groups, dk)) * dk ** -0.5
    k = plain.unit_vector(y[:, kw : 2 * kw].reshape(n, groups, dk))
    v = y[:, 2 * kw :].reshape(n, heads, dv)
    beta = plain.sigmoid(rows[:, off["b"] : off["b"] + heads])
    g = np.exp(-np.exp(a_log.astype(np.float64)) * plain.softplus(rows[:, off["a"] : off["a"] + heads] + dt_bias))
    o = np.zeros((n, heads, dv))
    for h in range(heads):
        o[:, h], _ = plain.delta_rule(q[:, h // (heads // groups)], k[:, h // (heads // groups)], v[:, h], beta[:, h], g[:, h])
    return np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], -1), beta, g, o.reshape(n, -1)


def _run_gdr(ops, proj, conv, a_log, dt_bias, off, state, conv_off, parts, heads, groups, dk, dv, narrow=None):
    """One step of the engine's three kernels over `parts` [(slot, rows of proj)]: (qkv, bg, o) of the step's rows."""
    torch = _torch()
    rows = np.concatenate([r for _, r in parts])
    cu = np.concatenate([[0], np.cumsum([len(r) for _, r in parts])]).astype(np.int32)
    seq_of = np.concatenate([np.full(len(r), i) for i, (_, r) in enumerate(parts)]).astype(np.int32)
    slot_of = np.concatenate([np.full(len(r), s) for s, r in parts]).astype(np.int32)
    t, taps = len(rows), conv.shape[1]
    dproj = _dev(proj[rows])
    qkv = torch.empty((t, off["c"]), device="cuda")
    bg = torch.empty((t, 2 * heads), device="cuda")
    slots = _dev(np.array([s for s, _ in parts], dtype=np.int32))
    ops.gdr_prepare(dproj, off["x"], off["b"], off["a"], _dev(conv), _dev(a_log), _dev(dt_bias), state, conv_off, _dev(cu), _dev(seq_of),
                    _dev(slot_of), qkv, bg, heads, groups, dk, dv, dk ** -0.5)
    ops.gdr_conv_update(dproj, off["x"], taps, off["c"], state, conv_off, _dev(cu), slots, _dev(slot_of), len(parts))
    o = torch.empty((t, heads * dv), device="cuda")
    longest = max(len(r) for _, r in parts)
    ops.gdr_scan(qkv, bg, state, _dev(cu), slots, _dev(slot_of), o, len(parts), heads, groups, dk, dv,
                 narrow=(longest > 16) if narrow is None else narrow)
    return qkv.cpu().numpy(), bg.cpu().numpy(), o.cpu().numpy(), cu


@pytest.mark.parametrize("heads,groups,dk,dv,taps", [(4, 2, 8, 16, 3), (3, 1, 7, 9, 4), (1, 1, 5, 3, 1), (6, 2, 12, 8, 2), (2, 2, 20, 20, 6),
                                                      (1, 1, 64, 32, 4), (4, 2, 128, 40, 4), (2, 1, 100, 33, 5)])
def test_convolution_unit_vectors_gates_and_the_delta_rule(heads, groups, dk, dv, taps):
    """Sequences of unequal lengths side by side, cut into three steps (one of them of single tokens) with the matrices and the
    convolution's last inputs carried in their slots; a sequence shorter than the convolution; slots of other requests stay
    as they are."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(heads * 100 + dk)
    lens, cuts, slots = [37, 1, 12, 70, 2], [(20, 21), (0, 1), (2, 3), (52, 69), (1, 2)], [3, 0, 2, 5, 6]
    total = sum(lens)
    proj, conv, a_log, dt_bias, off = _gdr_inputs(rng, total, heads, groups, dk, dv, taps)
    starts = np.concatenate([[0], np.cumsum(lens)])
    p64 = proj.astype(np.float64)
    want = [_plain_gdr(p64[starts[s] : starts[s + 1]], conv, a_log, dt_bias, off, heads, groups, dk, dv) for s in range(len(lens))]
    conv_off = heads * dk * dv
    stride = conv_off + (taps - 1) * off["c"] + 5
    state = torch.full((8, stride), 7.0, device="cuda")
    state[slots] = 0.0  # (the engine clears a slot when it hands it out)
    got = [[np.zeros_like(w) for w in ww] for ww in want]
    for step in range(3):
        parts = []
        for s, n in enumerate(lens):
            a, b = (0, cuts[s][0]) if step == 0 else (cuts[s][0], cuts[s][1]) if step == 1 else (cuts[s][1], n)
            if b > a:
                parts.append((slots[s], np.arange(starts[s] + a, starts[s] + b)))
        qkv, bg, o, cu = _run_gdr(ops, proj, conv, a_log, dt_bias, off, state, conv_off, parts, heads, groups, dk, dv)
        for i, (slot, r) in enumerate(parts):
            s = slots.index(slot)
            at = r - starts[s]
            got[s][0][at], got[s][3][at] = qkv[cu[i] : cu[i + 1]], o[cu[i] : cu[i + 1]]
            got[s][1][at], got[s][2][at] = bg[cu[i] : cu[i + 1], :heads], bg[cu[i] : cu[i + 1], heads:]
    for s in range(len(lens)):
        for j, what in enumerate(("convolved inputs", "beta", "decay", "read-out")):
            assert_close(got[s][j], want[s][j], 3e-5, f"{what} of sequence {s} ({heads} heads, {groups} key heads, {dk}x{dv}, {taps} taps)")
    for free in (1, 4, 7):
        assert float(state[free].min()) == 7.0 and float(state[free].max()) == 7.0, "slots of other requests are not touched"
    for s, slot in enumerate(slots):  # what a slot holds behind the matrices: the sequence's last taps - 1 inputs, oldest first
        rows = p64[starts[s] : starts[s + 1], off["x"] : off["x"] + off["c"]]
        held = np.concatenate([np.zeros((taps - 1, off["c"])), rows])[len(rows) :]
        assert np.array_equal(state[slot, conv_off : conv_off + (taps - 1) * off["c"]].cpu().numpy().reshape(taps - 1, off["c"]), held.astype(np.float32))
        assert float(state[slot, conv_off + (taps - 1) * off["c"] :].min()) == 0.0


def test_a_far_write_lives_on_in_the_state():
    """A key that only the first token writes, read 600 tokens later through decays close to one, in portions and single
    tokens; blocks of 32 and of 8 value columns, whole or cut: the same bits."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(6)
    heads, groups, dk, dv, n = 2, 1, 16, 32, 640
    kw, vw = groups * dk, heads * dv
    c = 2 * kw + vw
    qkv = np.zeros((n, c), dtype=np.float32)
    far = plain.unit_vector(rng.normal(size=dk))
    others = rng.normal(size=(n, dk))
    others -= np.outer(others @ far, far)  # every other key is at a right angle to the far one: nothing overwrites it
    qkv[:, kw : 2 * kw] = plain.unit_vector(others)
    qkv[:, :kw] = 0.25 * plain.unit_vector(others[::-1])
    qkv[:, 2 * kw :] = 0.05 * rng.normal(size=(n, vw))
    qkv[0, kw : 2 * kw], qkv[0, 2 * kw :] = far, np.arange(vw) + 1.0
    qkv[600, :kw] = far
    bg = np.concatenate([np.full((n, heads), 0.9), np.full((n, heads), np.exp(-1e-4))], -1).astype(np.float32)
    want = np.zeros((n, heads, dv))
    q64 = qkv.astype(np.float64)
    for h in range(heads):
        want[:, h], _ = plain.delta_rule(q64[:, :kw], q64[:, kw : 2 * kw], q64[:, 2 * kw + h * dv : 2 * kw + (h + 1) * dv], bg[:, h].astype(np.float64),
                                         bg[:, heads + h].astype(np.float64))
    assert np.abs(want[600]).max() > 20 * np.abs(want[599]).max(), "the test's far key carries row 600"
    state = torch.zeros((1, heads * dk * dv), device="cuda")
    one = _dev(np.zeros(1, dtype=np.int32))
    got, at = np.zeros((n, vw), dtype=np.float32), 0
    sizes = [1, 2, 130, 1, 1, 300, 7] + [1] * 40
    while at < n:
        m = min(sizes.pop(0) if sizes else 64, n - at)
        o = torch.empty((m, vw), device="cuda")
        ops.gdr_scan(_dev(qkv[at : at + m]), _dev(bg[at : at + m]), state, _dev(np.array([0, m], dtype=np.int32)), one, _dev(np.zeros(m, dtype=np.int32)),
                     o, 1, heads, groups, dk, dv, narrow=m > 16)
        got[at : at + m] = o.cpu().numpy()
        at += m
    assert_close(got, want.reshape(n, -1), 1e-4, "rows in portions and alone against the whole sequence")
    for narrow in (False, True):
        state.zero_()
        o = torch.empty((n, vw), device="cuda")
        ops.gdr_scan(_dev(qkv), _dev(bg), state, _dev(np.array([0, n], dtype=np.int32)), one, _dev(np.zeros(n, dtype=np.int32)), o, 1, heads, groups,
                     dk, dv, narrow=narrow)
        assert np.array_equal(o.cpu().numpy(), got), "the scan's result must not depend on how the rows were cut"


@pytest.mark.parametrize("experts,top,groups,keep,scale", [(6, 2, 3, 2, 1.5), (8, 3, 2, 1, 1.0), (5, 2, 1, 1, 1.0), (9, 1, 3, 1, 0.7), (8, 2, 4, 2, 2.0),
                                                           (4, 4, 2, 2, 1.0), (4, 1, 4, 2, 2.5), (12, 4, 4, 2, 0.5), (64, 6, 8, 3, 2.5)])
def test_choice_by_scores_with_a_correction_and_groups(experts, top, groups, keep, scale):
    """Corrections as large as the scores and below zero: an expert outside the kept groups is not chosen although its choice
    score beats a negative one inside; the weights are the scores without the correction."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(experts * 10 + top)
    t = 200
    logits = (2.0 * rng.normal(size=(t, experts))).astype(np.float32)
    for corr in (None, rng.normal(size=experts).astype(np.float32), (rng.normal(size=experts) - 2.0).astype(np.float32)):
        ids = torch.empty((t, top), dtype=torch.int32, device="cuda")
        weights = torch.empty((t, top), device="cuda")
        ops.moe_route_scored(_dev(logits), top, ids, weights, None if corr is None else _dev(corr), groups, keep, scale)
        w = {"router": np.eye(experts), "correction": np.zeros(experts) if corr is None else corr.astype(np.float64)}
        margins = []
        want_ids, want_w = plain.route(logits.astype(np.float64), w, "", {"experts": experts, "top": top, "scale": scale,
                                                                         "groups": {"count": groups, "keep": keep}}, margins)
        sure = margins[0] > 1e-5
        assert sure.sum() > 0.9 * t
        assert np.array_equal(ids.cpu().numpy()[sure], want_ids[sure]), f"{top} of {experts} in {keep} of {groups} groups"
        assert_close(weights.cpu().numpy()[sure], want_w[sure], 3e-6, "weights from the scores without the correction")
        if corr is not None and (corr < -1.0).all() and keep < groups:
            per = experts // groups
            got = ids.cpu().numpy()
            assert (np.ptp(got // per, axis=1) < groups).all() and all(len(set(r // per)) <= keep for r in got)


@pytest.mark.parametrize("experts,top,d,ff", [(5, 2, 64, 32), (3, 3, 50, 21), (12, 4, 96, 24)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_without_a_gate(experts, top, d, ff, dtype):
    """down(gelu(up x)) with the exact gelu, pair by pair and (bfloat16, sizes it covers) in sorted tiles."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(experts + d)
    t = 70
    rt = torch.float32 if dtype == "float32" else torch.bfloat16
    h = _held(rng.normal(size=(t, d)), rt)
    up = _held(0.3 * rng.normal(size=(experts, ff, d)), rt)
    down = _held(0.3 * rng.normal(size=(experts, d, ff)), rt)
    ids = torch.empty((t, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((t, top), device="cuda")
    ops.moe_route_scored(_dev(rng.normal(size=(t, experts)).astype(np.float32)), top, ids, weights, None, 1, 1, 1.3)
    slots = np.zeros(t, dtype=np.int32)
    slots[4] = -1  # a row of no request gets zeros
    want = np.zeros((t, d))
    for r in range(t):
        if slots[r] >= 0:
            for e, a in zip(ids.cpu().numpy()[r], weights.cpu().numpy()[r].astype(np.float64)):
                hidden = plain.gelu_erf(up[e] @ h[r])
                want[r] += a * ((hidden if dtype == "float32" else _held(hidden, rt)) @ down[e].T)
    hid = torch.empty((t * top, ff), dtype=rt, device="cuda")
    ops.moe_gate_up_pairs(_dev(h.astype(np.float32), rt), _dev(up.astype(np.float32), rt), None, ids, _dev(slots), hid, "gelu")
    y = torch.empty((t, d), device="cuda")
    ops.moe_down_pairs(hid, _dev(down.astype(np.float32), rt), ids, weights, _dev(slots), y)
    assert_close(y.cpu().numpy(), want, 2e-5 if dtype == "float32" else 3e-3, f"{top} of {experts} experts, pair by pair")
    if dtype == "bfloat16" and ops.moe_grouped_supports(d, ff, experts):
        scratch = torch.empty(ops.moe_grouped_scratch_ints(t * top, experts), dtype=torch.int32, device="cuda")
        z = torch.empty((t * top, d), device="cuda")
        y2 = torch.empty((t, d), device="cuda")
        ops.moe_grouped(_dev(h.astype(np.float32), rt), _dev(up.astype(np.float32), rt), None, _dev(down.astype(np.float32), rt), ids, weights,
                        _dev(slots), scratch, hid, z, y2, "gelu")
        assert_close(y2.cpu().numpy(), want, 3e-3, f"{top} of {experts} experts, in sorted tiles")


@pytest.mark.parametrize("d", [24, 50, 64, 256, 1000, 4096])
def test_mean_of_two_normed_rows_head_gates_and_the_cap(d):
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(d)
    t = 19
    a, b = (3.0 * rng.normal(size=(t, d))).astype(np.float32), (0.01 * rng.normal(size=(t, d))).astype(np.float32)
    wa, wb = rng.normal(size=d).astype(np.float32), rng.normal(size=d).astype(np.float32)
    for eps, scale in ((1e-6, 0.5), (1e-3, 1.0)):
        out = torch.empty((t, d), device="cuda")
        ops.norm_pair_mean(_dev(a), _dev(b), _dev(wa), _dev(wb), out, eps, scale)
        a64, b64 = a.astype(np.float64), b.astype(np.float64)
        want = scale * (plain.rms_norm(a64, wa.astype(np.float64), eps) + plain.rms_norm(b64, wb.astype(np.float64), eps))
        assert_close(out.cpu().numpy(), want, 3e-6, f"mean of two normed rows of {d}")
    heads = 5 if d % 5 == 0 else 4 if d % 4 == 0 else 1
    dv = d // heads
    gate = rng.normal(size=(t, heads + 3)).astype(np.float32)
    for tdt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        x = _dev(a, tdt)
        got = ops.head_gate_mul(x, _dev(gate)[:, 2 : 2 + heads], torch.empty_like(x), heads, dv)
        want = (x.float().cpu().numpy().astype(np.float64).reshape(t, heads, dv) * plain.sigmoid(gate[:, 2 : 2 + heads].astype(np.float64))[..., None])
        assert_close(got.float().cpu().numpy(), want.reshape(t, d), tol, f"{heads} head gates over rows of {d}")
    for cap in (8.0, 30.0, 0.5):
        z = _dev((10.0 * a).astype(np.float32))
        ops.softcap(z, cap)
        assert_close(z.cpu().numpy(), plain.soft_cap(10.0 * a.astype(np.float64), cap), 2e-6, f"cap of {cap}")


# ----------------------------------------------------------------------------------- the model, cut every way


def _replay(model_dir, dtype, steps, max_tokens, page, max_requests=4):
    from machserve_b200.engine.replay import make_replay_runner, replay

    runner = make_replay_runner(model_dir, dtype, max_tokens, page, max_requests)
    out = replay(runner, steps)
    runner.cache.check()
    assert not runner.cache.requests, "requests still hold cache after the trace ended"
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    return out


def _compare_rows(got, model_dir, dtype, tokens, what, rows=None):
    """The engine's logits for `tokens` (or for the rows `rows` of them) against the plain model.  In float32 every row must
    agree.  In bfloat16 a row is left out where the plain model itself cannot vouch for it (a router's close call at or
    before that token, or logits that rounding of the layers' inputs alone moves): every other row must agree, and most rows
    must be of that other kind."""
    if dtype == "float32":
        want = plain_logits(model_dir, tokens)
        return assert_close(got, want if rows is None else want[rows], F32_TOL, what)
    want, close = plain_logits_and_close_calls(model_dir, tokens, bf16_weights=True)
    close = np.maximum.accumulate(close)  # the recurrent half hands a wrong choice on to the rows after it
    if rows is not None:
        want, close = want[rows], close[rows]
    sure = ~close
    assert np.isfinite(np.asarray(got)).all()
    if sure.any():
        assert_close(np.asarray(got)[sure], want[sure], BF16_TOL, what + " (rows before a close call of a router)")
    return int(sure.sum())


def _dir(model_root, name, dtype):
    return make_model_dir(model_root, name, dtype == "bfloat16")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_whole_prompts(model_root, name, dtype):
    """Each request alone and whole, every position wanted: the first tokens of a sequence are among them."""
    d = _dir(model_root, name, dtype)
    requests = {f"r{n}": random_tokens(CASES[name]["config"]["vocab"], n, 300 + n) for n in (1, 2, 9, 33, 70)}
    steps = trace_whole(requests)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))
    sure = sum(_compare_rows(got[rid], d, dtype, toks, f"{name} {dtype} whole {rid}") or 0 for rid, toks in requests.items())
    assert dtype == "float32" or sure >= 40, f"{name}: the test's tokens leave {sure} rows of 115 without a close call"


@pytest.mark.parametrize("name", sorted(CASES))
def test_layers_follow_the_plain_layers(model_root, name):
    """The stream after every layer against the plain layers, in float32."""
    from machserve_b200.engine.replay import make_replay_runner
    from machserve_b200.engine.runner import StepEntry

    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 37, 1)
    runner = make_replay_runner(d, "float32", 64, CASES[name]["page"])
    taps = []
    runner.step([StepEntry("a", toks, [0])], tap=lambda i, h: taps.append(h.cpu().numpy()) if i >= 0 else None)
    cfg, w = read_weights(d)
    want = []
    plain.forward(cfg, w, toks, want)
    assert len(taps) == len(want) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(taps, want)):
        assert_close(a, b, F32_TOL, f"{name}: stream after layer {i}")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_decoded_tail_passes_every_window(model_root, name, dtype):
    """Most of it in one step, the last 60 tokens one by one: more than the windows of the tiny models, so that keys a prompt's
    step stored leave the windows of decoded tokens, and the state and the convolution's inputs go from a prompt's step into
    single tokens."""
    d = _dir(model_root, name, dtype)
    toks = random_tokens(CASES[name]["config"]["vocab"], 100, 7)
    steps = trace_tail_decode("a", toks, 60)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))
    _compare_rows(got["a"], d, dtype, toks, f"{name} {dtype} tail")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_portions_down_to_two_tokens(model_root, name, dtype):
    """Portions shorter than the convolution, portions that end in the middle of a page and of a window."""
    d = _dir(model_root, name, dtype)
    toks = random_tokens(CASES[name]["config"]["vocab"], 100, 11)
    steps = trace_portions("a", toks, [7, 2, 13, 3, 2, 16, 5, 9, 31])
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))["a"]
    _compare_rows(got, d, dtype, toks, f"{name} {dtype} portions")
    if dtype == "float32":  # the arithmetic of a row depends on its position and on the tokens before it alone
        whole = trace_whole({"a": toks})
        alone = collect_rows(whole, _replay(d, dtype, whole, 128, CASES[name]["page"]))["a"]
        assert_close(got, alone, 2e-6, "float32 logits must not depend on how the prompt was cut")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_unequal_requests_side_by_side_on_reused_pages_and_slots(model_root, name, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool so small that later requests run
    on pages and state slots that earlier ones gave back; each against itself alone."""
    from tests.test_replay_gpu import mixed_trace

    d = _dir(model_root, name, dtype)
    requests, steps = mixed_trace(CASES[name]["config"]["vocab"], seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    got = collect_rows(steps, _replay(d, dtype, steps, 256, CASES[name]["page"], max_requests=4))
    for rid, toks in requests.items():
        _compare_rows(got[rid], d, dtype, toks, f"{name} {dtype} mixed {rid}")
    whole = trace_whole(requests)
    alone = collect_rows(whole, _replay(d, dtype, whole, 256, CASES[name]["page"]))
    for rid in requests:
        if dtype == "float32":
            assert_close(got[rid], alone[rid], 2e-6, f"float32 logits of {rid} must not depend on the batch, the pages or the slot")


def test_long_decoding_from_a_short_prompt(model_root):
    """Four tokens of prompt and then 180 tokens one by one, in float32: the state, the convolution's inputs and the window
    pass many pages of decoded tokens; a drift or a slip by one shows in the last rows."""
    d = make_model_dir(model_root, "E")
    toks = random_tokens(CASES["E"]["config"]["vocab"], 184, 21)
    steps = trace_tail_decode("a", toks, 180)
    got = collect_rows(steps, _replay(d, "float32", steps, 192, CASES["E"]["page"]))
    _compare_rows(got["a"], d, "float32", toks, "E float32 long decoding")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "float32"), ("E", "float32"), ("C", "bfloat16")])
def test_greedy_generation_through_the_engine(model_root, name, dtype):
    """`Engine.generate`: scheduler, portions under a token budget, decoding, sampler.  In float32 the tokens are the
    plain model's greedy tokens; in bfloat16 every generated token is the plain model's choice or within its rounding."""
    from machserve_b200 import Engine

    d = make_model_dir(model_root, name, dtype == "bfloat16")
    vocab = CASES[name]["config"]["vocab"]
    prompts = [random_tokens(vocab, n, 40 + n) for n in (3, 29, 14, 1, 50)]
    eng = Engine(str(d), dtype, capacity=4, prefill_rows=16, tpp=CASES[name]["page"], max_seq=128)
    outs = eng.generate(prompts, max_new_tokens=12)
    eng.runner.cache.check()
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        seq = list(prompt)
        for tok in out:
            logits = plain_logits(d, seq, bf16_weights=(dtype == "bfloat16"))[-1]
            best = int(np.argmax(logits))
            if dtype == "float32":
                assert tok == best, f"{name}: token {len(seq) - len(prompt)} of a prompt of {len(prompt)} is {tok}, the plain model's is {best}"
            else:
                assert logits[best] - logits[tok] <= 2 * BF16_TOL * max(1.0, np.abs(logits).max())
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_root, tmp_path, dtype):
    """bin/trace_run itself on a model folder of this design, as a user drives it: steps on standard input, a line per step
    on standard output, the wanted rows in files."""
    import subprocess

    d = make_model_dir(model_root, "A", dtype == "bfloat16")
    toks = random_tokens(CASES["A"]["config"]["vocab"], 60, 9)
    steps = trace_portions("a", toks, [20, 2, 17, 1, 1, 1, 18])
    out = tmp_path / "out"
    cmd = [sys.executable, str(REPO / "bin" / "trace_run"), "--model", str(d), "--dtype", dtype, "--out", str(out),
           "--max-tokens", "64", "--page-size", "8"]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {st['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    rows = [np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, CASES["A"]["config"]["vocab"]) for st in steps]
    _compare_rows(np.concatenate(rows, 0), d, dtype, toks, f"A {dtype} trace_run")
