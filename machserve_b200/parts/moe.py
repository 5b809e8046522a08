"""A routed feed-forward: a mixture of small gated feed-forwards of which every token uses a few."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, matrix, register_feed_forward, vector_f32


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """Router logits z = Wr x (+ br) in float32; of the `experts` experts the `top` with the largest logits are chosen, their
    weights are the softmax over the chosen logits only; delta = sum of weight_e * down_e(act(gate_e(x)) * up_e(x)) over
    the chosen experts; experts have no biases; act "silu" or "gelu_tanh".  The experts' matrices are stacked on the device
    ([experts, ff, hidden] twice, [experts, hidden, ff]); a token's (token, expert) pairs read the chosen experts' rows only.

    Other routers and experts, by parameter.  `scoring` "sigmoid": the scores are s = sigmoid(z); an expert is chosen by
    s + correction (a learned number per expert, tensor `correction`, that enters the choice only), among the experts of the
    `keep` best of `groups` equal groups of neighbours (a group's score is the sum of its two largest choice scores; the
    others' choice scores count as minus infinity); the weights are the chosen experts' s over their sum (+ 1e-20), times
    `weight_scale`.  `gated` False: an expert is down_e(act(up_e(x))), without a gate matrix.  act may also be "gelu" (exact).

    params: prefix, hidden_size, intermediate_size (of one expert), experts, top, activation, router_bias (bool), gated
    (bool), scoring ("softmax_chosen" or "sigmoid"), correction (bool), groups, keep, weight_scale.  Tensors under the
    prefix: router [experts, hidden], router.b, correction [experts], e<i>.gate, e<i>.up, e<i>.down.
    """

    graph_safe = True
    kernel_files = ('moe', 'moe_grouped')
    GROUPED_FROM_ROWS = 17  # fewer rows stream the chosen experts' rows pair by pair (decoding) ...
    GROUPED_FROM_BYTES = 1 << 30  # ... unless the pairs would read this much: sorted, an expert's matrices are read once

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.experts, self.top = int(spec["experts"]), int(spec["top"])
        self.activation = spec.get("activation", "silu")
        self.router_bias = bool(spec.get("router_bias", True))
        self.gated = bool(spec.get("gated", True))
        self.scoring = spec.get("scoring", "softmax_chosen")
        self.has_correction = bool(spec.get("correction", False))
        self.groups, self.keep = int(spec.get("groups", 1)), int(spec.get("keep", 1))
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        if self.scoring not in ("softmax_chosen", "sigmoid"):
            raise ValueError(f"routed_experts: scoring '{self.scoring}' is not known (softmax_chosen, sigmoid)")
        if self.scoring == "softmax_chosen" and (self.has_correction or self.groups != 1 or self.weight_scale != 1.0):
            raise ValueError("routed_experts: a correction, groups and a weight scale belong to the scoring 'sigmoid'")
        if self.scoring == "sigmoid":
            if self.router_bias:
                raise ValueError("routed_experts: the scoring 'sigmoid' has no router bias (its correction enters the choice only)")
            if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups:
                raise ValueError(f"routed_experts: {self.experts} experts in {self.groups} groups of which {self.keep} are kept")
            if self.top > self.experts // self.groups * self.keep:
                raise ValueError(f"routed_experts: {self.top} experts a token, but the {self.keep} kept groups hold "
                                 f"{self.experts // self.groups * self.keep}")
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"routed_experts: {self.top} of {self.experts} experts a token")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"routed_experts: activation '{self.activation}' is not known ({', '.join(ops.ACTIVATIONS)})")

    def tensors(self):
        p = self.prefix
        out = [TensorDecl(p + "router", (self.experts, self.hidden))]
        if self.router_bias:
            out.append(TensorDecl(p + "router.b", (self.experts,), init="bias"))
        if self.has_correction:
            out.append(TensorDecl(p + "correction", (self.experts,), init="bias"))
        for e in range(self.experts):
            if self.gated:
                out.append(TensorDecl(f"{p}e{e}.gate", (self.inter, self.hidden)))
            out += [TensorDecl(f"{p}e{e}.up", (self.inter, self.hidden)), TensorDecl(f"{p}e{e}.down", (self.hidden, self.inter))]
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        self.w_router = matrix(tensors[p + "router"], rt)
        self.b_router = vector_f32(tensors[p + "router.b"]) if self.router_bias else None
        self.correction = vector_f32(tensors[p + "correction"]) if self.has_correction else None
        stack = lambda name: matrix(torch.stack([tensors[f"{p}e{e}.{name}"] for e in range(self.experts)], dim=0), rt)
        # (experts without a gate: their one input matrix stands where the gate's stands, and there is no second one)
        self.w_gate, self.w_up, self.w_down = (stack("gate"), stack("up"), stack("down")) if self.gated else (stack("up"), None, stack("down"))
        self.expert_bytes = (3 if self.gated else 2) * self.inter * self.hidden * self.w_gate.element_size()
        self.grouped = rt.dtype == torch.bfloat16 and ops.moe_grouped_supports(self.hidden, self.inter, self.experts)

    def forward(self, ctx, x):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        logits = ws.get("moe.logits", (t, self.experts), torch.float32)
        ops.linear(x, self.w_router, None, logits)  # (the router's bias is added where the logits are read)
        ids = ws.get("moe.ids", (t, self.top), torch.int32)
        weights = ws.get("moe.weights", (t, self.top), torch.float32)
        if self.scoring == "sigmoid":
            ops.moe_route_scored(logits, self.top, ids, weights, self.correction, self.groups, self.keep, self.weight_scale)
        else:
            ops.moe_route(logits, self.top, ids, weights, self.b_router)
        h = ws.get("moe.h", (t * self.top, self.inter), rt.dtype)
        delta = ws.get("ffn.delta_f32", (t, self.hidden), torch.float32)
        many = t >= self.GROUPED_FROM_ROWS or t * self.top * self.expert_bytes >= self.GROUPED_FROM_BYTES
        if self.grouped and many and t * self.top // 128 + self.experts <= 65535:
            # many rows: sorted by expert on the device, every expert's rows in tiles on the tensor cores
            scratch = ws.get("moe.sorted", (ops.moe_grouped_scratch_ints(t * self.top, self.experts),), torch.int32)
            z = ws.get("moe.z", (t * self.top, self.hidden), torch.float32)
            return ops.moe_grouped(x, self.w_gate, self.w_up, self.w_down, ids, weights, ctx.slot_of_token, scratch, h, z, delta,
                                   self.activation)
        ops.moe_gate_up_pairs(x, self.w_gate, self.w_up, ids, ctx.slot_of_token, h, self.activation)
        return ops.moe_down_pairs(h, self.w_down, ids, weights, ctx.slot_of_token, delta)
