"""Grouped-query attention with keys and values of widths of their own, a rotation of a part of every head, a sliding
window, a sink of score zero in the softmax and a gate per head on the output."""
from __future__ import annotations

import torch

from .. import ops
from . import wide_attend
from ..weights.loader import TensorDecl
from .base import POSITION_ENCODINGS, CachePlane, Mixer, PagedCache, matrix, register_mixer, vector_f32


@register_mixer("rotary_gated_attention")
class RotaryGatedAttention(wide_attend.WideAttendPlan, Mixer):
    """q = Wq x (heads x key_dim), k = Wk x (kv_heads x key_dim), v = Wv x (kv_heads x value_dim), with `bias` each plus a
    bias of its own (added in float32 where the product is read); the position
    encoding (a rotary one over the first rotary_dim coordinates of every query and key head, or none) turns q and k; query
    head h reads key/value head h // (heads / kv_heads); score = scale * q . k over the keys 0..p (or the last `window`,
    the query's own among them).  With `sink` the softmax's denominator has one more term of score zero that has no value:
    p_j = exp(s_j) / (1 + sum exp(s_j)).  With `head_gate` head h's output is multiplied by sigmoid(Wg x)_h, one number a
    head and token.  The heads' values side by side go through the output projection.

    The four input projections are one product with a float32 result.  Angles (the encoding's table), scores, softmax and
    gate are float32; the query stays float32 up to the scores (the exact kernel) or is rounded to bfloat16 as it enters
    the tensor core (bfloat16 runtime, widths the tensor-core kernels cover); the delta is float32.

    params: prefix, hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, window (or None), sink (bool),
    head_gate (bool), bias (bool: q.b, k.b, v.b), position (a PartSpec of a rotary encoding, or None).  Tensors under the
    prefix: q, k, v, o, g [heads, hidden], (q.b, k.b, v.b).
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden = int(spec["hidden_size"])
        self.hq, self.hkv = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.dk, self.dv = int(spec["key_dim"]), int(spec["value_dim"])
        if self.hq % self.hkv:
            raise ValueError(f"rotary_gated_attention: {self.hq} heads are not a multiple of {self.hkv} kv heads")
        if self.dv > 512 or self.dk > 512:
            raise ValueError(f"rotary_gated_attention: heads of {self.dk} key and {self.dv} value coordinates are more than the kernel covers (512)")
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.has_sink, self.has_gate = bool(spec.get("sink", True)), bool(spec.get("head_gate", True))
        self.has_bias = bool(spec.get("bias", False))
        self.position = POSITION_ENCODINGS.build(spec["position"]) if spec.get("position") is not None else None
        self.qw, self.kw, self.vw = self.hq * self.dk, self.hkv * self.dk, self.hkv * self.dv
        files = ["rope_store", "gated", "attention_wide", "attention_wide_mma"]
        if self.dk == self.dv:  # widths the framework's kernels for equal keys and values may cover
            files += ["attention_decode", "attention_prefill", "attention_decode_cluster", "attention_prefill_tc"]
        self.kernel_files = tuple(files)

    def cache_need(self):
        return PagedCache((CachePlane("k", self.hkv, self.dk), CachePlane("v", self.hkv, self.dv)), self.window)

    def tensors(self):
        p = self.prefix
        out = [
            TensorDecl(p + "q", (self.qw, self.hidden)), TensorDecl(p + "k", (self.kw, self.hidden)),
            TensorDecl(p + "v", (self.vw, self.hidden)), TensorDecl(p + "o", (self.hidden, self.hq * self.dv)),
        ]
        if self.has_gate:
            out.append(TensorDecl(p + "g", (self.hq, self.hidden)))
        if self.has_bias:
            out += [TensorDecl(p + "q.b", (self.qw,), init="bias"), TensorDecl(p + "k.b", (self.kw,), init="bias"),
                    TensorDecl(p + "v.b", (self.vw,), init="bias")]
        if self.position is not None:
            out += self.position.tensors()
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        inputs = [tensors[p + "q"], tensors[p + "k"], tensors[p + "v"]] + ([tensors[p + "g"]] if self.has_gate else [])
        self.w_in = matrix(torch.cat(inputs, dim=0), rt)
        self.w_o = matrix(tensors[p + "o"], rt)
        self.b_in = vector_f32(torch.cat([tensors[p + n].float() for n in ("q.b", "k.b", "v.b")])) if self.has_bias else None
        self.sinks = torch.zeros(self.hq, dtype=torch.float32, device=rt.device) if self.has_sink else None
        self.table, self.rot, self.interleaved = None, 0, False
        if self.position is not None:
            self.position.bind(tensors, rt)
            self.table = self.position.rotary_table(rt)
            if self.table is None:
                raise ValueError("rotary_gated_attention: the position encoding must be a rotary one")
            self.rot, self.interleaved = self.position.rotary_dim, self.position.interleaved
            if self.rot > self.dk:
                raise ValueError(f"rotary_gated_attention: {self.rot} rotated coordinates in heads of {self.dk}")
            self.graph_safe = bool(self.position.graph_safe)
        self.fast = wide_attend.supports(rt, self.dk, self.dv, self.dv, True)  # bfloat16: the tensor-core kernel
        # keys and values of one width that the framework's decode kernel is built for: decoding rows go there
        self.cluster = {} if self.fast and wide_attend.cluster_covers(rt, self.dk, self.dv, self.hq // self.hkv) else None

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        gate_at = self.qw + self.kw + self.vw
        proj = ws.get("rg_attn.in", (t, self.w_in.shape[0]), torch.float32)
        ops.linear(x, self.w_in, None, proj)
        q = ws.get("rg_attn.q", (t, self.qw), torch.float32)
        k_pages, v_pages = cache.planes["k"], cache.planes["v"]
        table = cache.block_table(ctx)
        tcgen05 = self.fast and ctx.max_query_len > 1 and wide_attend.tcgen05_covers(rt, self.dk, self.dv, k_pages.shape[2])
        q_half = ws.get("rg_attn.q_half", (t, self.qw), rt.dtype) if tcgen05 or self.cluster is not None else None
        ops.rope_store(proj, self.table, self.rot, self.interleaved, ctx.positions, ctx.slot_of_token, table, q, k_pages, v_pages,
                       self.hq, self.hkv, self.dk, self.dv, store=owns_cache, q_half=q_half, bias=self.b_in)
        out = ws.get("rg_attn.out", (t, self.hq * self.dv), rt.dtype)
        wide_attend.attend(ctx, rt, self.fast, table, q, k_pages, v_pages, out, self.sinks, self.hq, self.hkv, self.dk, self.dv,
                           self.window, self.scale, q_half=q_half, tcgen05=tcgen05, cluster=self.cluster)
        if self.has_gate:
            ops.head_gate_mul(out, proj[:, gate_at:gate_at + self.hq], out, self.hq, self.dv)
        delta = ws.get("mixer.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(out, self.w_o, None, delta)
