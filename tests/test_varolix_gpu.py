"""Varolix on the GPU against the plain implementation: each mechanism's kernel alone, then the model in every way of cutting
the work (whole, token by token, portions down to two tokens, unequal requests side by side on reused pages and state slots),
and greedy generation through the engine."""
import json
import sys

import numpy as np
import pytest

from tests.helpers import (BF16_TOL, F32_TOL, REPO, assert_close, collect_rows, random_tokens, trace_portions, trace_tail_decode,
                           trace_whole)
from tests.plain import varolix as plain
from tests.varolix_cases import CASES, assert_rows_close, make_model_dir, plain_logits, plain_with_reach, read_weights

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


def _table(dims, base, scaling, positions=128):
    f, m = plain.rotary_frequencies(dims, base, scaling)
    ang = np.arange(positions, dtype=np.float64)[:, None] * f[None, :]
    return _dev((np.stack([np.cos(ang), np.sin(ang)], -1) * m).astype(np.float32))


# ----------------------------------------------------------------------------------- mechanisms, one kernel each


@pytest.mark.parametrize("hq,hkv,dk,dv,rot,base,scaling,page", [
    (4, 2, 16, 24, 8, 100.0, (4.0, 32, 8.0, 1.0), 8), (5, 1, 6, 5, 2, 7.0, None, 16), (2, 2, 64, 64, 32, 10000.0, (4.0, 64, 16.0, 2.0), 16),
    (2, 1, 16, 16, 16, 20000.0, (16.0, 16, 4.0, 0.5), 8), (3, 3, 10, 7, 0, 1.0, None, 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_biases_rotation_with_stretched_waves_and_the_store(hq, hkv, dk, dv, rot, base, scaling, page, dtype):
    """q, k and v get their biases as the product is read; the first `rot` coordinates of every query and key head are turned
    in halves by the stretched angles and lengthened; values pass; keys and values land in their pages."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(hq * 100 + dk)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    positions = [0, 1, 2, 7, 8, 15, 16, 37, 90]
    qw, kw, vw = hq * dk, hkv * dk, hkv * dv
    proj = rng.normal(size=(len(positions), qw + kw + vw + 5)).astype(np.float32)
    bias = rng.normal(size=qw + kw + vw).astype(np.float32)
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    cos_sin = _table(rot, base, sc) if rot else None
    kp, table = _paged(rng, [91], hkv, dk, page)
    k_pages = torch.zeros(kp.shape, dtype=tdt, device="cuda")
    v_pages = torch.zeros(kp.shape[:3] + (dv,), dtype=tdt, device="cuda")
    q_out = torch.empty(len(positions), qw, device="cuda")
    q_half = torch.empty(len(positions), qw, dtype=torch.bfloat16, device="cuda")
    ops.rope_store(_dev(proj), cos_sin, rot, False, _ints(positions), _ints([0] * len(positions)), _dev(table), q_out, k_pages, v_pages,
                   hq, hkv, dk, dv, store=True, q_half=q_half, bias=_dev(bias))
    p64 = proj[:, : qw + kw + vw].astype(np.float64) + bias.astype(np.float64)
    r = {"dims": rot, "base": base, "scaling": sc}
    want_q = plain.rotate_half(p64[:, :qw].reshape(-1, hq, dk), positions, r).reshape(-1, qw)
    want_k = plain.rotate_half(p64[:, qw : qw + kw].reshape(-1, hkv, dk), positions, r)
    assert_close(q_out.cpu().numpy(), want_q, 2e-6, "queries")
    assert_close(q_half.float().cpu().numpy(), want_q, 1e-2, "the bfloat16 copy of the queries")
    tol = 2e-6 if dtype == "float32" else 1e-2
    for i, p in enumerate(positions):
        page_id = table[0, p // page]
        assert_close(k_pages[page_id, :, p % page].float().cpu().numpy(), want_k[i], tol, f"key at {p}")
        assert_close(v_pages[page_id, :, p % page].float().cpu().numpy().reshape(-1), p64[i, qw + kw :], tol, f"value at {p}")


@pytest.mark.parametrize("hq,hkv,dk,dv,coef,every,page", [(4, 2, 16, 8, 0.3, 5, 8), (3, 3, 10, 7, 0.0, 1, 16), (2, 1, 6, 11, 0.9, 1, 16),
                                                          (2, 2, 64, 64, 0.5, 16, 16), (8, 2, 48, 16, 1.5, 64, 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_norms_with_a_shared_weight_biases_and_the_temperature(hq, hkv, dk, dv, coef, every, page, dtype):
    """Every q and k head over its own root mean square times a weight the heads share; the biases of q, k and v added
    first; the query times 1 + coef ln(floor((p + 1) / every) + 1); the values as they are."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(hq * 10 + dk)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    positions = [0, 1, every - 1, every, 2 * every - 1, 2 * every, 37, 90, 5 * every + 3]
    positions = sorted({p for p in positions if 0 <= p <= 400})
    n = len(positions)
    qw, kw, vw = hq * dk, hkv * dk, hkv * dv
    proj = rng.normal(size=(n, qw + kw + vw + 3)).astype(np.float32)
    bias = rng.normal(size=qw + kw + vw).astype(np.float32)
    wq, wk = (1 + 0.3 * rng.normal(size=dk)).astype(np.float32), (1 + 0.3 * rng.normal(size=dk)).astype(np.float32)
    kp, table = _paged(rng, [max(positions) + 1], hkv, dk, page)
    k_pages = torch.zeros(kp.shape, dtype=tdt, device="cuda")
    v_pages = torch.zeros(kp.shape[:3] + (dv,), dtype=tdt, device="cuda")
    q_out = torch.empty(n, qw, device="cuda")
    q_half = torch.empty(n, qw, dtype=torch.bfloat16, device="cuda")
    ops.head_norm_store(_dev(proj), 1e-5, _ints(positions), _ints([0] * n), _dev(table), q_out, k_pages, v_pages, hq, hkv, dk, dv, qw + kw,
                        norm=True, wq=_dev(wq), wk=_dev(wk), store=True, q_half=q_half, bias=_dev(bias), temp_coef=coef, temp_every=every)
    p64 = proj[:, : qw + kw + vw].astype(np.float64) + bias
    temp = plain.query_temperature(positions, {"coef": coef, "every": every}) if coef else np.ones(n)
    want_q = (plain.rms_norm(p64[:, :qw].reshape(n, hq, dk), wq.astype(np.float64), 1e-5) * temp[:, None, None]).reshape(n, qw)
    want_k = plain.rms_norm(p64[:, qw : qw + kw].reshape(n, hkv, dk), wk.astype(np.float64), 1e-5)
    assert_close(q_out.cpu().numpy(), want_q, 3e-6, "queries")
    assert_close(q_half.float().cpu().numpy(), want_q, 1e-2, "the bfloat16 copy of the queries")
    if coef:
        assert temp[0] == 1.0 or every == 1, "the first positions have a temperature of one"
        assert len(set(np.round(temp, 9))) > 2, "the test's positions lie on several steps of the temperature"
    tol = 3e-6 if dtype == "float32" else 1e-2
    for i, p in enumerate(positions):
        page_id = table[0, p // page]
        assert_close(k_pages[page_id, :, p % page].float().cpu().numpy(), want_k[i], tol, f"key at {p}")
        assert_close(v_pages[page_id, :, p % page].float().cpu().numpy().reshape(-1), p64[i, qw + kw :], tol, f"value at {p}")


@pytest.mark.parametrize("heads,dn,dr,r,rot,interleaved,page", [(3, 8, 4, 16, 4, False, 8), (1, 5, 6, 9, 4, False, 16), (4, 32, 16, 48, 16, False, 16),
                                                                (2, 16, 8, 20, 8, True, 8), (5, 4, 2, 8, 2, False, 16), (2, 64, 32, 256, 32, False, 16),
                                                                (3, 16, 16, 32, 8, False, 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_norm_rotation_in_halves_and_queries_from_a_product_of_their_own(heads, dn, dr, r, rot, interleaved, page, dtype):
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(heads * 31 + r)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    positions = [0, 1, 7, 8, 16, 37, 90]
    n, hd, wide = len(positions), dn + dr, r + dr
    # the columns ahead of the down-projection in the input product (the queries' own latent) and the rows' lengths: on
    # 16-byte boundaries where the sizes allow the kernel's 16-byte form, off them otherwise
    by4 = dn % 4 == 0 and dr % 4 == 0 and r % 4 == 0 and rot % 8 == 0 and not interleaved
    lead = 8 if by4 else 6
    proj = rng.normal(size=(n, -(-(lead + wide + heads) // 4) * 4 if by4 else lead + wide + heads)).astype(np.float32)
    queries = rng.normal(size=(n, heads * hd + (4 if by4 else 2))).astype(np.float32)
    w = (1 + 0.2 * rng.normal(size=r)).astype(np.float32)
    cos_sin = _table(rot, 50.0, None)
    pp, table = _paged(rng, [91], 1, wide, page)
    pages = torch.zeros(pp.shape, dtype=tdt, device="cuda")
    q_wide = torch.zeros(n, heads, wide, device="cuda")
    q_plain = torch.zeros(n, heads, dn, dtype=tdt, device="cuda")
    ops.latent_encode(_dev(proj), lead, _dev(w), 1e-6, cos_sin, rot, _ints(positions), _ints([0] * n), _dev(table), q_wide, q_plain, pages,
                      heads, dn, dr, r, store=True, queries=_dev(queries), interleaved=interleaved)
    q64 = queries[:, : heads * hd].astype(np.float64).reshape(n, heads, hd)
    kv = proj[:, lead : lead + wide].astype(np.float64)

    def turn(x):
        if not interleaved:
            return plain.rotate_half(x, positions, {"dims": rot, "base": 50.0})
        y = x.copy()  # pairs (2i, 2i + 1): the halves' rotation of the coordinates taken evens first
        order = list(range(0, rot, 2)) + list(range(1, rot, 2))
        y[..., order] = plain.rotate_half(x[..., order], positions, {"dims": rot, "base": 50.0})
        return y

    assert_close(q_wide[:, :, r:].cpu().numpy().reshape(n, -1), turn(q64[..., dn:]).reshape(n, -1), 2e-6, "the queries' rotated parts")
    assert_close(q_plain.float().cpu().numpy().reshape(n, -1), q64[..., :dn].reshape(n, -1), 2e-6 if dtype == "float32" else 1e-2, "unrotated parts")
    tol = 3e-6 if dtype == "float32" else 1e-2
    want_c = plain.rms_norm(kv[:, :r], w.astype(np.float64), 1e-6)
    want_kr = turn(kv[:, None, r:])[:, 0]
    for i, p in enumerate(positions):
        row = pages[table[0, p // page], 0, p % page].float().cpu().numpy()
        assert_close(row[:r], want_c[i], tol, f"latent at {p}")
        assert_close(row[r:], want_kr[i], tol, f"rotated key part at {p}")


@pytest.mark.parametrize("rows,d", [(1, 24), (5, 50), (33, 64), (7, 1000), (3, 4096)])
def test_weighted_sum_of_two_halves_and_the_norm_of_a_column_range(rows, d):
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(d)
    a, b = rng.normal(size=(rows, d)).astype(np.float32), rng.normal(size=(rows, d)).astype(np.float32)
    ba = rng.normal(size=d).astype(np.float32)
    out = torch.empty(rows, d, device="cuda")
    ops.pair_weighted_sum(_dev(a), _dev(b), out, 1.2, -0.9, bias_a=_dev(ba))
    assert_close(out.cpu().numpy(), 1.2 * (a.astype(np.float64) + ba) - 0.9 * b, 1e-6, "weighted sum with the left bias")
    ops.pair_weighted_sum(_dev(a), _dev(b), out, 1.0, 1.0)
    assert_close(out.cpu().numpy(), a.astype(np.float64) + b, 1e-6, "plain sum")
    # the norm of the rows of a column range of a wider product (one "head" that is the whole range, no gate)
    wide = rng.normal(size=(rows, d + 13)).astype(np.float32)
    w = (1 + 0.2 * rng.normal(size=d)).astype(np.float32)
    for tdt, tol in ((torch.float32, 3e-6), (torch.bfloat16, 1e-2)):
        normed = torch.empty(rows, d, dtype=tdt, device="cuda")
        ops.gla_output(_dev(wide)[:, 5 : 5 + d], None, _dev(w), 1e-5, normed, 1, d)
        assert_close(normed.float().cpu().numpy(), plain.rms_norm(wide[:, 5 : 5 + d].astype(np.float64), w.astype(np.float64), 1e-5), tol, "norm")


# ----------------------------------------------------------------------------------- softmax attention in every kernel


def _plain_attend(q, k, v, positions, scale, groups, sinks=None):
    """q [T, H, dk] at `positions` of one sequence whose keys k [N, G, dk] and values v [N, G, dv] are all there."""
    t, h, _ = q.shape
    out = np.zeros((t, h, v.shape[2]))
    for i, p in enumerate(positions):
        for head in range(h):
            g = head // groups
            s = (k[: p + 1, g] @ q[i, head]) * scale
            m = s.max() if sinks is None else max(s.max(), sinks[head])
            e = np.exp(s - m)
            out[i, head] = (e @ v[: p + 1, g]) / (e.sum() + (0.0 if sinks is None else np.exp(sinks[head] - m)))
    return out


def _attend_every_form(ops, q, kd, vd, table, rows, hq, hkv, dk, dv, scale, dtype, sinks=None, one_plane=False):
    """The rows (sequence, position) of q through every attention kernel that the design's mixers may use at these widths:
    {name: out [T, hq, dv]}.  Rows that follow one another in a sequence are a portion; the others are decoded rows.
    `one_plane`: the values are the first dv coordinates of the keys' plane (a latent cache)."""
    torch = _torch()
    t = len(rows)
    sk = _dev(np.asarray(sinks, dtype=np.float32)) if sinks is not None else None
    pos, slot = _ints(p for _, p in rows), _ints(s for s, _ in rows)
    tab = _dev(table)
    outs = {}
    for share in (True, False):
        out = torch.zeros(t, hq * dv, dtype=kd.dtype, device="cuda")
        ops.attention_wide(_dev(q).view(t, hq * dk), kd, vd, out, sk, pos, slot, tab, hq, hkv, dk, dv, None, scale, share_rows=share)
        outs["exact, rows share" if share else "exact, heads share"] = out.float().cpu().numpy().reshape(t, hq, dv)
    assert np.array_equal(outs["exact, rows share"], outs["exact, heads share"]), "the two forms of the exact kernel give the same bits"
    if dtype != "bfloat16":
        return outs
    runs, singles, i = [], [], 0
    while i < t:
        j = i
        while j + 1 < t and rows[j + 1] == (rows[j][0], rows[j][1] + 1):
            j += 1
        (runs.append((i, j - i + 1)) if j > i else singles.append(i))
        i = j + 1
    if ops.attention_wide_mma_supports(dk, dv, dk if one_plane else dv, not one_plane):
        tile = ops.attention_wide_mma_tile_rows(dv)
        t0 = [a + b for a, n in runs for b in range(0, n, tile)]
        tn = [min(tile, n - b) for a, n in runs for b in range(0, n, tile)]
        for splits in (1, 3):
            out = torch.zeros(t, hq * dv, dtype=torch.bfloat16, device="cuda")
            if t0:
                ops.attention_wide_mma(_dev(q).view(t, hq * dk), kd, vd, out, sk, pos, slot, tab, _ints(t0), _ints(tn), len(t0), False,
                                       hq, hkv, dk, dv, None, scale)
            if singles:
                items = len(singles) * hkv * (-(-(hq // hkv) // 16))
                scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(items, dv, splits)), device="cuda")
                ops.attention_wide_mma(_dev(q).view(t, hq * dk), kd, vd, out, sk, pos, slot, tab, _ints(singles), None, len(singles), True,
                                       hq, hkv, dk, dv, None, scale, splits, scratch)
            outs[f"mma.sync, {splits} runs of keys"] = out.float().cpu().numpy().reshape(t, hq, dv)
    if not one_plane and dk == dv and dk in (64, 128) and ops.attention_prefill_tc_supports(dk, kd.shape[2]) \
            and ops.attention_decode_supports(dk, hq // hkv) and ops.attention_prefill_supports(dk):
        from types import SimpleNamespace

        from machserve_b200.parts.attention import decode_launch

        qh = _dev(q).view(t, hq * dk).to(torch.bfloat16)
        out = torch.zeros(t, hq * dv, dtype=torch.bfloat16, device="cuda")
        t0 = [a + b for a, n in runs for b in range(0, n, 128)]
        tn = [min(128, n - b) for a, n in runs for b in range(0, n, 128)]
        if t0:
            ops.attention_prefill_tc(qh, kd, vd, out, _ints(t0), _ints(tn), len(t0), pos, slot, tab, hq, hkv, dk, None, scale, 1, None, None,
                                     sinks=sk)
        if singles:
            rt = SimpleNamespace(sm_count=torch.cuda.get_device_properties(0).multi_processor_count)
            tiles = -(-(max(rows[i][1] for i in singles) + 1) // 64)
            splits, stages, warps, kpw, parts = decode_launch(rt, dk, ops.attention_decode_cluster_max_stages(dk), {}, len(singles) * hkv, tiles)
            scratch = counters = None
            if parts > 1:
                scratch = torch.zeros(ops.attention_decode_cluster_scratch_words(len(singles), hq, hkv, dk, parts), device="cuda")
                counters = torch.zeros(len(singles) * hkv, dtype=torch.int32, device="cuda")
            ops.attention_decode_cluster(qh, kd, vd, out, pos, slot, tab, hq, hkv, dk, None, scale, splits, stages, rows=_ints(singles),
                                         num_rows=len(singles), warps=warps, keys_per_warp=kpw, parts=parts, scratch=scratch, counters=counters,
                                         sinks=sk)
        assert ops.tc_status_codes() == (0, 0)
        outs["tcgen05 portions, cluster decoding"] = out.float().cpu().numpy().reshape(t, hq, dv)
    return outs


@pytest.mark.parametrize("dk,dv,hq,hkv,page,sink,one_plane", [
    (16, 24, 4, 2, 8, False, False), (6, 5, 5, 1, 16, False, False), (64, 64, 4, 1, 16, False, False), (128, 128, 2, 2, 16, False, False),
    (48, 16, 8, 2, 8, False, False), (20, 16, 3, 1, 8, True, True), (64, 48, 4, 1, 16, True, True), (15, 9, 1, 1, 16, True, True)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_causal_softmax_with_and_without_a_learned_sink(dk, dv, hq, hkv, page, sink, one_plane, dtype):
    """Portions of two sequences side by side and decoded rows, the first tokens of a sequence among them; with a learned sink
    per head over a cache of one plane (latent attention's form) and without one over keys and values."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(dk * 1000 + dv)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    lens = [150, 41]
    kp, table = _paged(rng, lens, hkv, dk, page)
    ks = [rng.normal(size=(n, hkv, dk)).astype(np.float32) for n in lens]
    vs = [k[..., :dv] if one_plane else rng.normal(size=(k.shape[0], hkv, dv)).astype(np.float32) for k in ks]
    vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
    for s in range(2):
        _fill_pages(kp, table, s, ks[s], page)
        _fill_pages(vp, table, s, vs[s], page)
    kd = _dev(kp, tdt)
    vd = kd if one_plane else _dev(vp, tdt)
    ks, vs = [_held(k, tdt) for k in ks], [_held(v, tdt) for v in vs]
    scale = 1.2 / np.sqrt(dk)
    sinks = rng.normal(size=hq) * 2.0 + 1.0 if sink else None
    rows = [(0, p) for p in range(100, 137)] + [(0, 149)] + [(1, p) for p in range(3)] + [(1, 40)]
    q = rng.normal(size=(len(rows), hq, dk)).astype(np.float32)
    q[5] *= -6.0  # a row whose scores are far below zero: a sink takes nearly all of its weight
    outs = _attend_every_form(ops, q, kd, vd, table, rows, hq, hkv, dk, dv, scale, dtype, sinks, one_plane)
    assert dtype == "float32" or len(outs) > 2 or dk % 16 or dv % 8, "a tensor-core kernel covers these widths"
    for name, got in outs.items():
        q_held = _held(q, torch.bfloat16) if name.startswith(("mma", "tcgen05")) else q.astype(np.float64)
        want = np.zeros((len(rows), hq, dv))
        for s in range(2):
            idx = [i for i, (ss, _) in enumerate(rows) if ss == s]
            want[idx] = _plain_attend(q_held[idx], ks[s], vs[s], [rows[i][1] for i in idx], scale, hq // hkv, sinks)
        assert_close(got.reshape(len(rows), -1), want.reshape(len(rows), -1), 2e-5 if dtype == "float32" else 1.5e-2, f"{name} ({dk}, {dv})")


@pytest.mark.parametrize("dk,dv,page,n,sink", [(16, 24, 8, 700, None), (64, 64, 16, 900, None), (128, 128, 16, 520, None), (64, 32, 16, 650, 3.0)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_key_among_hundreds_carries_the_row(dk, dv, page, n, sink, dtype):
    """Among keys of small scores one key answers the query's direction: the first key of the sequence, keys at, before and
    behind a page's border, a key hundreds of tokens back.  A query sees it from its own position on and never before; queries
    in a portion and queries decoded alone; a sink level with the marked score takes half of the weight."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(n + dk)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    hq, hkv = 2, 1
    scale = 1.0 / np.sqrt(dk)
    marks = [0, page - 1, page, 5 * page + 1, n - 40]
    k = (0.05 * rng.normal(size=(n, hkv, dk))).astype(np.float32)
    v = rng.normal(size=(n, hkv, dv)).astype(np.float32)
    for j, m in enumerate(marks):  # each mark has a direction of its own: 32 - 16 for a query that asks for it, -16 for every other
        k[m, 0] = 0.0
        k[m, 0, j] = 32.0 * np.sqrt(dk)
        k[m, 0, dk - 1] = -16.0 * np.sqrt(dk)
        v[m, 0] = 100.0 + m
    kp, table = _paged(rng, [n], hkv, dk, page)
    vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
    _fill_pages(kp, table, 0, k, page)
    _fill_pages(vp, table, 0, v, page)
    kd, vd = _dev(kp, tdt), _dev(vp, tdt)
    sinks = [16.0, -30.0] if sink else None  # head 0: level with the marked score; head 1: out of sight
    for j, m in enumerate(marks):
        q1 = np.zeros((hq, dk), dtype=np.float32)
        q1[:, j] = 1.0
        q1[:, dk - 1] = 1.0
        portion = list(range(max(0, m - 3), min(n, m + 4)))
        alone = [p for p in (m - 1, m + 1, min(n - 1, m + 300), n - 1) if 0 <= p < n and p not in (m,)] + [m]
        for how, group in (("portion", portion), ("alone", sorted(set(alone))[::2]), ("alone", sorted(set(alone))[1::2])):
            if not group:
                continue
            q = np.tile(q1, (len(group), 1, 1))
            outs = _attend_every_form(ops, q, kd, vd, table, [(0, p) for p in group], hq, hkv, dk, dv, scale, dtype, sinks)
            for name, o in outs.items():
                for i, p in enumerate(group):
                    for head in range(hq):
                        got = o[i, head].mean()
                        if p < m:
                            assert abs(got) < 10.0, f"{name}: position {p} ({how}) sees the key at {m}, which lies ahead of it"
                        else:
                            want = (100.0 + m) * (0.5 if sink and head == 0 else 1.0)
                            assert abs(got - want) < 2.0 + 0.005 * want, f"{name}: position {p} ({how}), head {head}, must see the key at {m}: {got:.4g} for {want}"


# ----------------------------------------------------------------------------------- the matrix memory


def _mm_offsets(heads, dk, dv):
    """Columns of a product that holds q | k | v | g | i | f among others: on 16-byte boundaries where the sizes allow the
    kernel's 16-byte copies, off them otherwise."""
    kw, vw = heads * dk, heads * dv
    extra = 4 if dk % 4 == 0 and dv % 4 == 0 else 3
    off = dict(q=extra, k=extra + kw, v=extra + 2 * kw, g=extra + 2 * kw + vw + 1)
    off["i"] = off["g"] + vw
    off["f"] = off["i"] + heads
    off["ld"] = -(-(off["f"] + heads + 2) // 4) * 4 if extra == 4 else off["f"] + heads + 2
    return off


def _plain_mm(rows, off, bi, bf, cap, norm, eps, heads, dk, dv, state=None, rec=None):
    """One sequence whole through the plain functions: (y [T, heads*dv], states per head).  `rec` disturbs what enters and
    leaves the recurrence (rounding noise of a chosen size)."""
    n = rows.shape[0]
    r = rows.astype(np.float64)
    rec = rec or (lambda a: a)
    q = rec(r[:, off["q"] : off["q"] + heads * dk].reshape(n, heads, dk) * dk ** -0.5)
    k = rec(r[:, off["k"] : off["k"] + heads * dk].reshape(n, heads, dk))
    v = rec(r[:, off["v"] : off["v"] + heads * dv].reshape(n, heads, dv))
    i_log = rec(plain.soft_cap(r[:, off["i"] : off["i"] + heads] + bi, cap))
    f_log = rec(plain.log_sigmoid(plain.soft_cap(r[:, off["f"] : off["f"] + heads] + bf, cap)))
    o, states = np.zeros((n, heads, dv)), []
    for h in range(heads):
        o[:, h], st = plain.matrix_memory(q[:, h], k[:, h], v[:, h], i_log[:, h], f_log[:, h], None if state is None else state[h])
        states.append(st)
    y = plain.unit_rms(rec(o), eps).reshape(n, heads * dv) * norm * plain.sigmoid(r[:, off["g"] : off["g"] + heads * dv])
    return y, states


def _mm_reach(y, *args):
    """How far rounding noise of float32's size on the recurrence's inputs and read-out moves each row of y (two draws)."""
    from tests.varolix_cases import _jitter

    return np.max([np.abs(_plain_mm(*args, rec=_jitter(2.0 ** -22, seed))[0] - y).max(-1) for seed in (11, 12)], axis=0)


def _run_mm(ops, proj, off, bi, bf, cap, norm, eps, state, parts, heads, dk, dv, narrow=None, out_dtype=None):
    """One step of the engine's three kernels over `parts` [(slot, rows of proj)]: y of the step's rows."""
    torch = _torch()
    rows = np.concatenate([r for _, r in parts])
    cu = np.concatenate([[0], np.cumsum([len(r) for _, r in parts])]).astype(np.int32)
    slot_of = np.concatenate([np.full(len(r), s) for s, r in parts]).astype(np.int32)
    t = len(rows)
    dproj = _dev(proj[rows])
    slots = _dev(np.array([s for s, _ in parts], dtype=np.int32))
    gates = torch.empty((t, heads, 4), device="cuda")
    ops.mm_gates(dproj, off["i"], off["f"], _dev(bi), _dev(bf), cap, state, _dev(cu), slots, _dev(slot_of), gates, len(parts), heads, dk, dv)
    o = torch.empty((t, heads, dv + 1), device="cuda")
    longest = max(len(r) for _, r in parts)
    ops.mm_scan(dproj, off["q"], off["k"], off["v"], gates, dk ** -0.5, state, _dev(cu), slots, _dev(slot_of), o, len(parts), heads, dk, dv,
                narrow=(longest > 16) if narrow is None else narrow)
    y = torch.empty((t, heads * dv), dtype=out_dtype or torch.float32, device="cuda")
    ops.mm_output(o, gates, dproj[:, off["g"] : off["g"] + heads * dv], _dev(norm), eps, y, heads, dv)
    return y.float().cpu().numpy(), cu


@pytest.mark.parametrize("heads,dk,dv,cap,forget", [(2, 8, 12, 4.0, 0.0), (3, 7, 9, 11.0, 0.0), (1, 5, 3, 2.5, 2.0), (2, 32, 64, 12.0, 4.0),
                                                     (1, 64, 32, 8.0, -2.0), (4, 4, 12, 6.0, 1.0), (2, 100, 33, 30.0, 6.0), (2, 128, 128, 20.0, 3.0)])
def test_gates_memory_and_read_out_over_unequal_sequences_cut_into_steps(heads, dk, dv, cap, forget):
    """Three sequences of unequal lengths side by side, cut into three steps at places of their own (one of them a single
    token at a time), on slots of which one holds an earlier request's leftovers until it is handed out: every row against
    the plain memory run whole, and the slots' matrices, normalizers and stabilizers at the end against its state."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(heads * 1000 + dk * 10 + dv)
    off = _mm_offsets(heads, dk, dv)
    lens = [37, 3, 20]
    total = sum(lens)
    proj = rng.normal(size=(total, off["ld"])).astype(np.float32)
    proj[:, off["i"] : off["i"] + heads] *= 3.0  # input gates that reach the cap and lie far below it
    proj[:, off["f"] : off["f"] + heads] = 2.0 * proj[:, off["f"] : off["f"] + heads] + forget
    bi, bf = rng.normal(size=heads).astype(np.float32), rng.normal(size=heads).astype(np.float32)
    norm = (1 + 0.2 * rng.normal(size=heads * dv)).astype(np.float32)
    eps = 1e-5
    words = ops.mm_state_floats(heads, dk, dv)
    state = torch.full((5, words), 7.5, device="cuda")  # leftovers everywhere
    starts = np.concatenate([[0], np.cumsum(lens)])
    seq_rows = [np.arange(starts[s], starts[s + 1]) for s in range(3)]
    slot = {0: 3, 1: 0, 2: 4}
    cuts = {0: [0, 20, 21, 37], 1: [0, 1, 2, 3], 2: [0, 2, 19, 20]}
    got = np.zeros((total, heads * dv))
    for step in range(3):
        parts = []
        for s in (2, 0, 1):  # the step's order of sequences is not the slots' order
            if step == 0:
                state[slot[s]].zero_()  # a slot is cleared when it is handed out
            lo, hi = cuts[s][step], cuts[s][step + 1]
            if hi > lo:
                parts.append((slot[s], seq_rows[s][lo:hi]))
        y, cu = _run_mm(ops, proj, off, bi, bf, cap, norm, eps, state, parts, heads, dk, dv)
        for i, (_, r) in enumerate(parts):
            got[r] = y[cu[i] : cu[i + 1]]
    final = state.cpu().numpy()
    assert np.all(final[1] == 7.5) and np.all(final[2] == 7.5), "slots of no request of the step are not touched"
    for s in range(3):
        args = (proj[seq_rows[s]], off, bi.astype(np.float64), bf.astype(np.float64), cap, norm.astype(np.float64), eps, heads, dk, dv)
        want, states = _plain_mm(*args)
        # (a read-out whose few live terms cancel is divided by a root mean square that is all rounding: such rows get what
        # rounding alone moves them by)
        assert_rows_close(got[seq_rows[s]], want, _mm_reach(want, *args), 3e-5, f"sequence {s} ({heads} heads of {dk} x {dv})", tight=0.6)
        mats = final[slot[s], : heads * dk * (dv + 1)].reshape(heads, dk, dv + 1)
        for h, (S, n, m) in enumerate(states):
            assert_close(mats[h, :, :dv], S, 3e-5, f"matrix of sequence {s}, head {h}")
            assert_close(mats[h, :, dv], n, 3e-5, f"normalizer of sequence {s}, head {h}")
            assert abs(final[slot[s], heads * dk * (dv + 1) + h] - m) < 1e-4 * max(1.0, abs(m)), f"stabilizer of sequence {s}, head {h}"
    # blocks of 8 columns and of 32 give the same bits; a bfloat16 result is the float32 one rounded
    state_a, state_b = torch.zeros(1, words, device="cuda"), torch.zeros(1, words, device="cuda")
    ya, _ = _run_mm(ops, proj, off, bi, bf, cap, norm, eps, state_a, [(0, seq_rows[0])], heads, dk, dv, narrow=True)
    yb, _ = _run_mm(ops, proj, off, bi, bf, cap, norm, eps, state_b, [(0, seq_rows[0])], heads, dk, dv, narrow=False)
    assert np.array_equal(ya, yb) and torch.equal(state_a, state_b)
    yh, _ = _run_mm(ops, proj, off, bi, bf, cap, norm, eps, torch.zeros(1, words, device="cuda"), [(0, seq_rows[0])], heads, dk, dv,
                    out_dtype=torch.bfloat16)
    assert np.array_equal(yh, torch.from_numpy(ya.astype(np.float32)).to(torch.bfloat16).float().numpy())


def test_a_far_write_lives_on_in_the_memory():
    """One token writes with an open input gate into a memory whose forget gate stays shut for 600 tokens, through portions
    and single tokens; every other token's input gate is closed.  A query in the written key's direction reads the written
    value back, 600 tokens later as well as at once; a query across it reads nothing of it; before the write there is nothing."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(5)
    heads, dk, dv, cap, eps = 2, 16, 8, 16.0, 1e-6
    off = _mm_offsets(heads, dk, dv)
    n, mark = 640, 23
    proj = (0.1 * rng.normal(size=(n, off["ld"]))).astype(np.float32)
    proj[:, off["i"] : off["i"] + heads] = -100.0  # closed: i = -cap
    proj[:, off["f"] : off["f"] + heads] = 100.0   # kept: f = logsigmoid(cap), a few 1e-7 below zero
    proj[mark, off["i"] : off["i"] + heads] = 100.0
    direction = np.zeros(dk, dtype=np.float32)
    direction[2] = 1.0
    value = np.arange(1, dv + 1, dtype=np.float32)
    for h in range(heads):
        proj[mark, off["k"] + h * dk : off["k"] + (h + 1) * dk] = 3.0 * direction
        proj[mark, off["v"] + h * dv : off["v"] + (h + 1) * dv] = value * (h + 1)
    readers = [mark, mark + 1, 100, 333, 639]
    for p in readers:
        proj[p, off["q"] : off["q"] + heads * dk] = np.tile(5.0 * direction, heads)
    across = [50, 400]
    for p in across:
        proj[p, off["q"] : off["q"] + heads * dk] = 0.0
        proj[p, off["q"] + 5] = 4.0
    proj[:, off["g"] : off["g"] + heads * dv] = 50.0  # an open output gate
    zeros, ones = np.zeros(heads, dtype=np.float32), np.ones(heads * dv, dtype=np.float32)
    state = torch.zeros(1, ops.mm_state_floats(heads, dk, dv), device="cuda")
    got = np.zeros((n, heads * dv))
    at, sizes, i = 0, [17, 1, 1, 30, 2, 64, 1, 5, 128], 0
    while at < n:
        m = min(sizes[i % len(sizes)], n - at)
        y, _ = _run_mm(ops, proj, off, zeros, zeros, cap, ones, eps, state, [(0, np.arange(at, at + m))], heads, dk, dv)
        got[at : at + m] = y
        at, i = at + m, i + 1
    want, _ = _plain_mm(proj, off, zeros.astype(np.float64), zeros.astype(np.float64), cap, ones.astype(np.float64), eps, heads, dk, dv)
    live = np.r_[mark:n]  # (before the write the read-out is noise of closed gates, far below the norm's eps)
    assert_close(got[live], want[live], 1e-3, "the memory over 640 tokens in portions and single steps")
    unit = value / np.sqrt((value * value).mean())  # the read-out is divided by its root mean square
    for p in readers:
        for h in range(heads):
            assert_close(got[p, h * dv : (h + 1) * dv], unit, 1e-3, f"position {p}, head {h}: the value written at {mark}")
    assert np.abs(got[:mark]).max() < 0.9, "before the write the memory holds noise of closed gates alone"
    for p in across:
        assert np.abs(got[p] - np.tile(unit, heads)).max() > 0.3, f"position {p} asks across the written key"


# ----------------------------------------------------------------------------------- the model, cut every way


def _replay(model_dir, dtype, steps, max_tokens, page, max_requests=4):
    from machserve_b200.engine.replay import make_replay_runner, replay

    runner = make_replay_runner(model_dir, dtype, max_tokens, page, max_requests)
    out = replay(runner, steps)
    runner.cache.check()
    assert not runner.cache.requests, "requests still hold cache after the trace ended"
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    return out


def _compare_rows(got, model_dir, dtype, tokens, what, rows=None, tight=0.7):
    """The engine's logits for `tokens` (or for the rows `rows` of them) against the plain model: every row within the
    tolerance, or, where rounding alone moves the plain model's row by more than a third of it (`plain_with_reach`), within
    three times that.  Returns how many rows were held to the tolerance itself."""
    want, _, reach, _ = plain_with_reach(model_dir, tokens, dtype)
    if rows is not None:
        want, reach = want[rows], reach[rows]
    if dtype == "float32":
        return assert_rows_close(got, want, reach, F32_TOL, what, tight)
    return assert_rows_close(got, want, reach, BF16_TOL, what, 0.0)  # (float32 is the sharp comparison)


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_whole_prompts(model_root, name, dtype):
    """Each request alone and whole, every position wanted: the first tokens of a sequence are among them."""
    d = make_model_dir(model_root, name)
    requests = {f"r{n}": random_tokens(CASES[name]["config"]["vocab"], n, 300 + n) for n in (1, 2, 9, 33, 70)}
    steps = trace_whole(requests)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))
    held = sum(_compare_rows(got[rid], d, dtype, toks, f"{name} {dtype} whole {rid}", tight=0.0) for rid, toks in requests.items())
    assert held >= (90 if dtype == "float32" else 40), f"{name}: rounding alone moves all but {held} rows of 115 by more than a quarter of the tolerance"


@pytest.mark.parametrize("name", sorted(CASES))
def test_layers_follow_the_plain_layers(model_root, name):
    """The stream after every run of a layer (a looped layer counts each time) against the plain layers, in float32."""
    from machserve_b200.engine.replay import make_replay_runner
    from machserve_b200.engine.runner import StepEntry

    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 37, 1)
    runner = make_replay_runner(d, "float32", 64, CASES[name]["page"])
    taps = []
    runner.step([StepEntry("a", toks, [0])], tap=lambda i, h: taps.append(h.cpu().numpy()) if i >= 0 else None)
    cfg, _ = read_weights(d)
    _, want, _, reach = plain_with_reach(d, toks, "float32")
    assert len(taps) == len(want) == len(plain.run_order(cfg))
    for i, (a, b) in enumerate(zip(taps, want)):
        assert_rows_close(a, b, reach[i], F32_TOL, f"{name}: stream after run {i}", tight=0.8)


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_prefill_against_token_by_token_decoding(model_root, name, dtype):
    """Most of it in one step, the last 60 tokens one by one: the keys, the latents and the memories' states go from a
    prompt's step into single tokens."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 100, 7)
    steps = trace_tail_decode("a", toks, 60)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))
    _compare_rows(got["a"], d, dtype, toks, f"{name} {dtype} tail")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_portions_down_to_two_tokens(model_root, name, dtype):
    """Portions of many sizes that end in the middle of a page and of a temperature's step."""
    d = make_model_dir(model_root, name)
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

    d = make_model_dir(model_root, name)
    requests, steps = mixed_trace(CASES[name]["config"]["vocab"], seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    got = collect_rows(steps, _replay(d, dtype, steps, 256, CASES[name]["page"], max_requests=4))
    for rid, toks in requests.items():
        _compare_rows(got[rid], d, dtype, toks, f"{name} {dtype} mixed {rid}")
    if dtype == "float32":
        whole = trace_whole(requests)
        alone = collect_rows(whole, _replay(d, dtype, whole, 256, CASES[name]["page"]))
        for rid in requests:
            assert_close(got[rid], alone[rid], 2e-6, f"float32 logits of {rid} must not depend on the batch, the pages or the slot")


@pytest.mark.parametrize("seed", range(16))
def test_configurations_drawn_from_many_sizes(model_root, seed):
    """Sixteen configurations drawn from many sizes (head counts, groups, widths inside and outside what the tensor-core
    kernels cover, ranks, rotations, layer orders, loops): a prompt of 130 rows and 20 rows decoded one by one, in both dtypes,
    against the plain model.  The typical row within float32's and bfloat16's rounding; no row far off (a row of a matrix
    memory whose live terms cancel may be off by more than the typical one: see `plain_with_reach`)."""
    import torch

    from machserve_b200.config import config_from_json
    from machserve_b200.weights import write_random_model
    from tests.varolix_cases import random_case

    raw = random_case(seed)
    d = model_root / f"varolix_drawn_{seed}"
    if not (d / "model.safetensors").exists():
        write_random_model(config_from_json(raw), d, seed, torch.bfloat16, 0.06, 0.2, 0.1)
    toks = random_tokens(raw["vocab"], 150, seed)
    want = plain_logits(d, toks)
    spread = np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())
    steps = trace_tail_decode("a", toks, 20)
    for dtype, typical, far in (("float32", 2e-5, 2e-3), ("bfloat16", 6e-2, 1.0)):
        got = collect_rows(steps, _replay(d, dtype, steps, 192, 16))["a"]
        assert np.isfinite(got).all()
        diff = got - want
        err = np.sqrt(((diff - diff.mean(-1, keepdims=True)) ** 2).mean(-1)) / spread
        assert np.median(err) < typical and err.max() < far, f"seed {seed} {dtype}: median {np.median(err):.3g}, largest {err.max():.3g} at row {int(err.argmax())}"


@pytest.mark.parametrize("name", ["D", "A"])
def test_long_decoding_from_a_short_prompt(model_root, name):
    """Four tokens of prompt and then 180 tokens one by one, in float32: the memories (lasting ones in D) and the caches pass
    many pages of decoded tokens, the decoding steps run from recorded graphs; a drift or a slip by one shows in the last rows."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 184, 21)
    steps = trace_tail_decode("a", toks, 180)
    got = collect_rows(steps, _replay(d, "float32", steps, 192, CASES[name]["page"]))
    _compare_rows(got["a"], d, "float32", toks, f"{name} float32 long decoding")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("D", "float32"), ("C", "bfloat16")])
def test_greedy_generation_through_the_engine(model_root, name, dtype):
    """`Engine.generate`: scheduler, portions under a token budget, decoding, sampler.  In float32 the tokens are the
    plain model's greedy tokens; in bfloat16 every generated token is the plain model's choice or within its rounding."""
    from machserve_b200 import Engine

    d = make_model_dir(model_root, name)
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

    d = make_model_dir(model_root, "A")
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
