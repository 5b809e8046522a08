"""Grouped-query attention whose positions enter through the scores alone: every head normed on its own, a soft cap, a
learned bias by distance, and a mask by chunks."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from . import wide_attend
from ..weights.loader import TensorDecl
from .base import CachePlane, Mixer, PagedCache, matrix, register_mixer, vector_f32


def distance_bucket(n: int, rows: int, reach: float) -> int:
    """The row of a bias table of `rows` rows that distance n >= 0 reads: the first half of the rows one distance each, the
    other half spaced evenly in the logarithm of the distance up to `reach`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def bias_by_distance(table: torch.Tensor, reach: float, longest: int) -> torch.Tensor:
    """table [rows, heads] -> float32 [heads, longest]: entry [h, n] is the bias of head h at distance n (the kernels clamp
    larger distances to the last entry, which by then is the table's last row or `longest` covers every distance)."""
    rows = table.shape[0]
    idx = torch.tensor([distance_bucket(n, rows, reach) for n in range(longest)], dtype=torch.long)
    return table.to(torch.float32)[idx].t().contiguous()


@register_mixer("chunked_attention")
class ChunkedAttention(wide_attend.WideAttendPlan, Mixer):
    """q = Wq x (+ bq), k = Wk x (+ bk), one product; v = Wv x (+ bv with `value_bias`), or, `values_are_keys`, the keys as
    projected (no Wv).  With `head_norm`, every query head and every key head is divided by its own root mean square over the
    head's coordinates (eps inside the root; with `norm_weight` times a weight [key_dim] that the heads share, one for the
    queries and one for the keys); the values are not.  With `temp_coef` c the normed query at position p is multiplied by
    1 + c * ln(floor((p + 1) / temp_every) + 1).  Query head h reads key/value head
    h // (heads / kv_heads).  score = scale * q . k; then, with `softcap` c, score <- c * tanh(score / c); then, with a
    bias table [rows, heads], score += table[bucket(i - j), h] (`distance_bucket`; not scaled); position i sees the keys
    j <= i of its own chunk floor(i / chunk) (every earlier key without `chunk`); an ordinary softmax; the heads' outputs
    side by side go through Wo (+ bo with `out_bias`).  Norms, temperature, scores, the cap, the bias and the softmax are
    float32.  Without cap, bias table and chunks the scores are plain, and in bfloat16 the rows go to the framework's kernels
    for keys and values of one width where those cover the sizes (portions of prompts to the tcgen05 kernel, decoding rows to
    the cluster kernel).

    params: prefix, hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, eps, bias (bool: q and k biases),
    values_are_keys, head_norm, norm_weight, value_bias, out_bias, temp_coef (0: none), temp_every, softcap (or None),
    bias_rows (or None: no distance bias), bias_reach, chunk (or None), max_positions.  Tensors under the prefix: q, k, (v),
    o, (q.b, k.b), (v.b), (o.b), (q.norm, k.norm [key_dim]), (rel [bias_rows, heads]).
    """

    graph_safe = True
    kernel_files = ('head_norm_store', 'attention_wide', 'attention_wide_mma')

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden = int(spec["hidden_size"])
        self.hq, self.hkv = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.dk, self.dv = int(spec["key_dim"]), int(spec["value_dim"])
        if self.hq % self.hkv:
            raise ValueError(f"chunked_attention: {self.hq} heads are not a multiple of {self.hkv} kv heads")
        self.values_are_keys = bool(spec.get("values_are_keys", False))
        if self.values_are_keys and self.dv != self.dk:
            raise ValueError(f"chunked_attention: values that are the keys have the keys' size ({self.dk}), not {self.dv}")
        if self.dv > 512:
            raise ValueError(f"chunked_attention: values of {self.dv} coordinates per head are more than the kernel covers (512)")
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.has_bias = bool(spec.get("bias", False))
        self.head_norm = bool(spec.get("head_norm", True))
        self.norm_weight = bool(spec.get("norm_weight", False))
        self.value_bias, self.out_bias = bool(spec.get("value_bias", False)), bool(spec.get("out_bias", False))
        self.coef, self.every = float(spec.get("temp_coef", 0.0)), int(spec.get("temp_every", 1))
        if self.norm_weight and not self.head_norm:
            raise ValueError("chunked_attention: a norm weight without the norm")
        if self.value_bias and self.values_are_keys:
            raise ValueError("chunked_attention: values that are the keys have no bias of their own")
        if self.coef and self.every < 1:
            raise ValueError(f"chunked_attention: a temperature that steps every {self.every} positions")
        self.softcap: Optional[float] = spec.get("softcap")
        self.bias_rows: Optional[int] = spec.get("bias_rows")
        self.bias_reach = spec.get("bias_reach")
        self.chunk: Optional[int] = spec.get("chunk")
        self.max_positions = int(spec["max_positions"])
        if self.bias_rows is not None and (self.bias_rows < 2 or self.bias_reach is None or self.bias_reach <= self.bias_rows // 2):
            raise ValueError(f"chunked_attention: a bias table of {self.bias_rows} rows that reaches {self.bias_reach}")
        self.qw, self.kw = self.hq * self.dk, self.hkv * self.dk
        self.vw = 0 if self.values_are_keys else self.hkv * self.dv
        self.plain_scores = not self.softcap and self.bias_rows is None and not self.chunk
        if self.plain_scores and self.dk == self.dv:  # widths the framework's kernels for equal keys and values may cover
            self.kernel_files = (*type(self).kernel_files, "attention_decode", "attention_prefill", "attention_decode_cluster",
                                 "attention_prefill_tc")
        self._bias_deferred = False

    def cache_need(self):
        return PagedCache((CachePlane("k", self.hkv, self.dk), CachePlane("v", self.hkv, self.dv)), None, self.chunk)

    def tensors(self):
        p = self.prefix
        out = [TensorDecl(p + "q", (self.qw, self.hidden)), TensorDecl(p + "k", (self.kw, self.hidden))]
        if not self.values_are_keys:
            out.append(TensorDecl(p + "v", (self.vw, self.hidden)))
        if self.has_bias:
            out += [TensorDecl(p + "q.b", (self.qw,), init="bias"), TensorDecl(p + "k.b", (self.kw,), init="bias")]
        if self.value_bias:
            out.append(TensorDecl(p + "v.b", (self.vw,), init="bias"))
        if self.norm_weight:
            out += [TensorDecl(p + "q.norm", (self.dk,), init="scale"), TensorDecl(p + "k.norm", (self.dk,), init="scale")]
        if self.out_bias:
            out.append(TensorDecl(p + "o.b", (self.hidden,), init="bias"))
        if self.bias_rows is not None:
            out.append(TensorDecl(p + "rel", (self.bias_rows, self.hq), init="bias"))
        out.append(TensorDecl(p + "o", (self.hidden, self.hq * self.dv)))
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        mats = [tensors[p + "q"], tensors[p + "k"]] + ([] if self.values_are_keys else [tensors[p + "v"]])
        self.w_in = matrix(torch.cat(mats, dim=0), rt)
        self.b_in = None
        if self.has_bias or self.value_bias:
            like = tensors[p + "q"]
            zeros = lambda n: torch.zeros(n, dtype=torch.float32, device=like.device)
            parts = [tensors[p + "q.b"].float(), tensors[p + "k.b"].float()] if self.has_bias else [zeros(self.qw), zeros(self.kw)]
            if not self.values_are_keys:
                parts.append(tensors[p + "v.b"].float() if self.value_bias else zeros(self.vw))
            self.b_in = vector_f32(torch.cat(parts))
        self.w_o = matrix(tensors[p + "o"], rt)
        self.b_o = vector_f32(tensors[p + "o.b"]) if self.out_bias else None
        self.q_norm = vector_f32(tensors[p + "q.norm"]) if self.norm_weight else None
        self.k_norm = vector_f32(tensors[p + "k.norm"]) if self.norm_weight else None
        dist = None
        if self.bias_rows is not None:
            # one entry per distance a query can see: within a chunk, or up to the longest sequence
            longest = min(self.chunk or self.max_positions, self.max_positions, rt.max_positions)
            dist = bias_by_distance(tensors[p + "rel"].detach().to("cpu"), float(self.bias_reach), max(1, longest)).to(rt.device)
        self.dist_bias = dist
        self.score = None
        if self.softcap or dist is not None or self.chunk:
            self.score = ops.ScoreExtras(self.softcap, dist, self.chunk)
        self.fast = wide_attend.supports(rt, self.dk, self.dv, self.dv, True)  # bfloat16: the tensor-core kernel
        # plain scores over keys and values of one width that the framework's decode kernel is built for: decoding rows go there
        self.cluster = {} if (self.fast and self.plain_scores
                              and wide_attend.cluster_covers(rt, self.dk, self.dv, self.hq // self.hkv)) else None

    def defer_output_bias(self):
        """For a part that adds this mixer's delta into a sum of its own: the output projection's bias (float32 [hidden], or
        None), which that part adds from now on instead of this mixer."""
        self._bias_deferred = True
        return self.b_o

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        width = self.qw + (self.kw + self.vw if owns_cache else 0)
        proj = ws.get("chunked_attn.qkv", (t, width), torch.float32)
        ops.linear(x, self.w_in[:width], None, proj)  # (the biases are added where the product is read)
        q = ws.get("chunked_attn.q", (t, self.qw), torch.float32)
        k_pages, v_pages = cache.planes["k"], cache.planes["v"]
        table = cache.block_table(ctx)
        tcgen05 = (self.fast and self.plain_scores and ctx.max_query_len > 1
                   and wide_attend.tcgen05_covers(rt, self.dk, self.dv, k_pages.shape[2]))
        q_half = ws.get("chunked_attn.q_half", (t, self.qw), rt.dtype) if tcgen05 or self.cluster is not None else None
        ops.head_norm_store(proj, self.eps, ctx.positions, ctx.slot_of_token, table, q, k_pages, v_pages, self.hq, self.hkv, self.dk,
                            self.dv, None if self.values_are_keys else self.qw + self.kw, norm=self.head_norm, wq=self.q_norm,
                            wk=self.k_norm, store=owns_cache, q_half=q_half, bias=self.b_in, temp_coef=self.coef, temp_every=self.every)
        out = ws.get("chunked_attn.out", (t, self.hq * self.dv), rt.dtype)
        wide_attend.attend(ctx, rt, self.fast, table, q, k_pages, v_pages, out, None, self.hq, self.hkv, self.dk, self.dv, None,
                           self.scale, q_half=q_half, tcgen05=tcgen05, cluster=self.cluster, score=self.score)
        delta = ws.get("chunked_attn.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(out, self.w_o, None if self._bias_deferred else self.b_o, delta)
