"""Attention whose keys and values are made from one latent vector per token: only the latent and one rotated key
part, shared by all heads, are kept in the cache."""
from __future__ import annotations

import torch

from .. import ops
from . import wide_attend
from ..weights.loader import TensorDecl
from .base import POSITION_ENCODINGS, CachePlane, Mixer, PagedCache, matrix, register_mixer, vector_f32


@register_mixer("latent_attention")
class LatentAttention(wide_attend.WideAttendPlan, Mixer):
    """x -> q = Wq x, or, with `query_latent` rq, q = Wuq (Wdq x / rms(Wdq x) * wq) through a normed latent of rq numbers;
    q lies head by head as [dn unrotated | dr rotated];  Wdkv x = [latent (r) | key part (dr)].
    c = latent / rms(latent) * w (eps inside the root); kr = the key part, rotated, shared by all heads.
    Per head h: k_h = Wuk_h c (dn), v_h = Wuv_h c (dv); score = scale * (q_plain . k_h + q_rot . kr) over the keys the
    window lets the row see; a plain softmax, or, with `sink`, one whose denominator also holds exp(sink_h), a learned
    number per head without a key or a value; the heads' values side by side are multiplied by sigmoid(Wg x), one gate per
    element (`gate` True or "element") or one per head ("head"), and go through the output projection.

    The cache holds one plane of r + dr numbers per token, [c | kr].  Keys and values are never made: since
    q_plain . (Wuk_h c) = (Wuk_h^T q_plain) . c, the query is carried into the latent's coordinates, the attention
    runs with ONE key/value head of r + dr key and r value coordinates (both read from the same plane) for all
    query heads, and Wuv_h is applied to the attended latent.  Norm, rotation (the position encoding's table), scores
    and softmax are float32, and so are the carried query and the gate; the delta is float32.

    params: prefix, hidden_size, num_heads, plain_dim (dn), rotated_dim (dr), value_dim (dv), latent_dim (r), scale, eps,
    window (or None), gate (False: no output gate; True or "element"; "head"), sink (bool), query_latent (rq, or None),
    position (a PartSpec of a rotary encoding over the dr coordinates, pairs interleaved or in halves, or None).  Tensors
    under the prefix: q (or dq [rq, hidden], dq.norm [rq], uq [heads*(dn+dr), rq]), dkv, dkv.norm, uk [heads*dn, r],
    uv [heads*dv, r], g ([heads*dv, hidden] or [heads, hidden]), sink [heads], o.
    """

    graph_safe = True
    kernel_files = ('latent_encode', 'gla', 'gated', 'attention_wide', 'attention_wide_mma')

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden, self.heads = int(spec["hidden_size"]), int(spec["num_heads"])
        self.dn, self.dr, self.dv, self.r = int(spec["plain_dim"]), int(spec["rotated_dim"]), int(spec["value_dim"]), int(spec["latent_dim"])
        if self.r > 512:
            raise ValueError(f"latent_attention: a latent of {self.r} coordinates is more than the kernel covers (512)")
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = spec.get("window")
        gate = spec.get("gate", True)
        if gate not in (True, False, None, "element", "head"):
            raise ValueError(f"latent_attention: gate '{gate}' is neither 'element' nor 'head'")
        self.has_gate, self.head_gate = bool(gate), gate == "head"
        self.has_sink = bool(spec.get("sink", False))
        self.rq = int(spec["query_latent"]) if spec.get("query_latent") is not None else None
        self.position = POSITION_ENCODINGS.build(spec["position"]) if spec.get("position") is not None else None
        self.qw, self.kvw, self.ow = self.heads * (self.dn + self.dr), self.r + self.dr, self.heads * self.dv
        self.gw = self.heads if self.head_gate else self.ow
        self.q_cols = self.rq if self.rq is not None else self.qw  # the queries' share of the input product

    def cache_need(self):
        return PagedCache((CachePlane("latent", 1, self.kvw),), self.window)

    def tensors(self):
        p = self.prefix
        if self.rq is not None:
            queries = [TensorDecl(p + "dq", (self.rq, self.hidden)), TensorDecl(p + "dq.norm", (self.rq,), init="scale"),
                       TensorDecl(p + "uq", (self.qw, self.rq))]
        else:
            queries = [TensorDecl(p + "q", (self.qw, self.hidden))]
        out = [
            *queries, TensorDecl(p + "dkv", (self.kvw, self.hidden)),
            TensorDecl(p + "dkv.norm", (self.r,), init="scale"), TensorDecl(p + "uk", (self.heads * self.dn, self.r)),
            TensorDecl(p + "uv", (self.ow, self.r)), TensorDecl(p + "o", (self.hidden, self.ow)),
        ]
        if self.has_gate:
            out.append(TensorDecl(p + "g", (self.gw, self.hidden)))
        if self.has_sink:
            out.append(TensorDecl(p + "sink", (self.heads,), init="bias"))
        if self.position is not None:
            out += self.position.tensors()
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        inputs = [tensors[p + ("dq" if self.rq is not None else "q")], tensors[p + "dkv"]] + ([tensors[p + "g"]] if self.has_gate else [])
        self.w_in = matrix(torch.cat(inputs, dim=0), rt)
        self.w_uq = matrix(tensors[p + "uq"], rt) if self.rq is not None else None
        self.q_norm = vector_f32(tensors[p + "dq.norm"]) if self.rq is not None else None
        self.sinks = vector_f32(tensors[p + "sink"]) if self.has_sink else None
        # per head: the keys' up-projection transposed ([r, dn]: carries a query into the latent's coordinates) and the
        # values' up-projection as it is ([dv, r])
        self.w_uk_t = matrix(tensors[p + "uk"].reshape(self.heads, self.dn, self.r).transpose(1, 2), rt)
        self.w_uv = matrix(tensors[p + "uv"].reshape(self.heads, self.dv, self.r), rt)
        self.w_o = matrix(tensors[p + "o"], rt)
        self.latent_norm = vector_f32(tensors[p + "dkv.norm"])
        self.fast = wide_attend.supports(rt, self.kvw, self.r, self.kvw, False)  # bfloat16: the tensor-core kernel
        self.table, self.rot, self.interleaved = None, 0, True
        if self.position is not None:
            self.position.bind(tensors, rt)
            self.table = self.position.rotary_table(rt)
            if self.table is None:
                raise ValueError("latent_attention: the position encoding must be a rotary one")
            self.rot, self.interleaved = self.position.rotary_dim, bool(self.position.interleaved)
            self.graph_safe = bool(self.position.graph_safe)

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        h, r, wide = self.heads, self.r, self.kvw
        proj = ws.get("latent_attn.in", (t, self.w_in.shape[0]), torch.float32)
        ops.linear(x, self.w_in, None, proj)
        queries = None
        if self.rq is not None:  # the queries' own latent: its norm in float32, then up to the heads
            cq = ws.get("latent_attn.cq", (t, self.rq), rt.dtype)
            ops.gla_output(proj[:, :self.rq], None, self.q_norm, self.eps, cq, 1, self.rq)
            queries = ws.get("latent_attn.queries", (t, self.qw), torch.float32)
            ops.linear(cq, self.w_uq, None, queries)
        q_wide = ws.get("latent_attn.q_wide", (t, h, wide), torch.float32)
        q_plain = ws.get("latent_attn.q_plain", (t, h, self.dn), rt.dtype)
        pages, table = cache.planes["latent"], cache.block_table(ctx)
        ops.latent_encode(proj, self.q_cols, self.latent_norm, self.eps, self.table, self.rot, ctx.positions, ctx.slot_of_token, table,
                          q_wide, q_plain, pages, h, self.dn, self.dr, r, store=owns_cache, queries=queries, interleaved=self.interleaved)
        ops.linear_heads(q_plain, self.w_uk_t, q_wide[:, :, :r])
        attended = ws.get("latent_attn.attended", (t, h, r), rt.dtype)
        wide_attend.attend(ctx, rt, self.fast, table, q_wide.view(t, h * wide), pages, pages, attended.view(t, h * r), self.sinks, h, 1,
                           wide, r, self.window, self.scale)
        values = ws.get("latent_attn.values", (t, h, self.dv), torch.float32)
        ops.linear_heads(attended, self.w_uv, values)
        gate_at = self.q_cols + self.kvw
        if self.head_gate:
            ops.head_gate_mul(values.view(t, self.ow), proj[:, gate_at:gate_at + h], values.view(t, self.ow), h, self.dv)
            gated = values.view(t, self.ow) if rt.dtype == torch.float32 else ws.get("latent_attn.gated", (t, self.ow), rt.dtype).copy_(values.view(t, self.ow))
        elif self.has_gate:
            gated = ws.get("latent_attn.gated", (t, self.ow), rt.dtype)
            ops.sigmoid_gate_mul(values.view(t, self.ow), proj[:, gate_at:], gated)
        elif rt.dtype == torch.float32:
            gated = values.view(t, self.ow)
        else:
            gated = ws.get("latent_attn.gated", (t, self.ow), rt.dtype).copy_(values.view(t, self.ow))
        delta = ws.get("mixer.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(gated, self.w_o, None, delta)
