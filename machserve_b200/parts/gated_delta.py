"""The gated delta rule: a recurrent mixer whose matrix state per head is decayed, corrected towards the new value and read,
behind a short causal convolution of its inputs."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, matrix, register_mixer, vector_f32


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """q = Wq x and k = Wk x (kv_heads x key_dim), v = Wv x (heads x value_dim), no biases; value head h reads q/k head
    h // (heads / kv_heads).  Each channel of q, k and v passes a causal convolution over time of `conv` taps (weights
    [channels, conv], the last column the current token's; zeros before the sequence) and SiLU.  Every q and k head is then
    made a unit vector (x / sqrt(sum x^2 + 1e-6)), q also times key_dim^(-1/2).  beta = sigmoid(Wb x) and the decay
    g = exp(-exp(A_log) * softplus(Wa x + dt_bias)) are one number a head and token.  Per head and sequence, with
    S [key_dim, value_dim] zero at the start:

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.

    Each head's o is divided by its root mean square over value_dim (eps inside the root), multiplied by a weight
    [value_dim] that the heads share and by silu(Wg x), and the heads side by side go through Wo.  The six input
    projections are one product with a float32 result; the convolution, the unit vectors, beta, the decay, the state,
    the norm and the gate are float32.  A request's state slot holds the matrices and the convolution's last conv - 1
    inputs.

    params: prefix, hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv, eps.  Tensors under the prefix: q, k, v
    (matrices), q.conv, k.conv, v.conv, b [heads, hidden], a [heads, hidden], A_log [heads], dt_bias [heads], norm [value_dim],
    g [heads*value_dim, hidden], o.
    """

    graph_safe = True
    kernel_files = ('gated_delta', 'gla')

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden = int(spec["hidden_size"])
        self.heads, self.groups = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.dk, self.dv, self.taps = int(spec["key_dim"]), int(spec["value_dim"]), int(spec["conv"])
        self.eps = float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError(f"gated_delta_rule: {self.heads} heads are not a multiple of {self.groups} kv heads")
        if self.dk > 256:
            raise ValueError(f"gated_delta_rule: {self.dk} key channels a head are more than the kernel covers (256)")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"gated_delta_rule: a convolution of {self.taps} taps is not covered (1 to 16)")
        self.kw, self.vw = self.groups * self.dk, self.heads * self.dv
        self.channels = 2 * self.kw + self.vw
        if self.channels * 4 > 48 * 1024:
            raise ValueError(f"gated_delta_rule: {self.channels} convolved channels are more than the kernel covers")
        # columns of the one input product: q | k | v (the convolved channels) | g | b | a
        self.g_off = self.channels
        self.b_off = self.g_off + self.vw
        self.a_off = self.b_off + self.heads
        self.width = self.a_off + self.heads
        self.conv_off = self.heads * self.dk * self.dv  # where a slot's convolution inputs begin, behind its matrices

    def cache_need(self):
        return FixedState((self.conv_off + (self.taps - 1) * self.channels,))

    def tensors(self):
        p, h = self.prefix, self.hidden
        return [
            TensorDecl(p + "q", (self.kw, h)), TensorDecl(p + "k", (self.kw, h)), TensorDecl(p + "v", (self.vw, h)),
            TensorDecl(p + "q.conv", (self.kw, self.taps)), TensorDecl(p + "k.conv", (self.kw, self.taps)),
            TensorDecl(p + "v.conv", (self.vw, self.taps)), TensorDecl(p + "b", (self.heads, h)), TensorDecl(p + "a", (self.heads, h)),
            TensorDecl(p + "A_log", (self.heads,), init="bias"), TensorDecl(p + "dt_bias", (self.heads,), init="bias"),
            TensorDecl(p + "norm", (self.dv,), init="scale"), TensorDecl(p + "g", (self.vw, h)), TensorDecl(p + "o", (h, self.vw)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        self.w_in = matrix(torch.cat([tensors[p + n] for n in ("q", "k", "v", "g", "b", "a")], dim=0), rt)
        self.conv_w = torch.cat([tensors[p + n].to(torch.float32) for n in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = vector_f32(tensors[p + "A_log"]), vector_f32(tensors[p + "dt_bias"])
        self.norm = vector_f32(tensors[p + "norm"])
        self.w_o = matrix(tensors[p + "o"], rt)

    def forward(self, ctx, x, cache, owns_cache=True):
        if not owns_cache:
            raise ValueError("gated_delta_rule: a run cannot read another run's state")
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        state = cache.state
        proj = ws.get("gdr.proj", (t, self.width), torch.float32)
        ops.linear(x, self.w_in, None, proj)
        qkv = ws.get("gdr.qkv", (t, self.channels), torch.float32)
        bg = ws.get("gdr.bg", (t, 2 * self.heads), torch.float32)
        ops.gdr_prepare(proj, 0, self.b_off, self.a_off, self.conv_w, self.a_log, self.dt_bias, state, self.conv_off, ctx.cu_tokens,
                        ctx.seq_of_token, ctx.slot_of_token, qkv, bg, self.heads, self.groups, self.dk, self.dv, self.dk ** -0.5)
        ops.gdr_conv_update(proj, 0, self.taps, self.channels, state, self.conv_off, ctx.cu_tokens, ctx.state_slots, ctx.slot_of_token,
                            ctx.num_seqs)
        o = ws.get("gdr.o", (t, self.vw), torch.float32)
        ops.gdr_scan(qkv, bg, state, ctx.cu_tokens, ctx.state_slots, ctx.slot_of_token, o, ctx.num_seqs, self.heads, self.groups, self.dk,
                     self.dv, narrow=ctx.max_query_len > 16)
        y = ws.get("gdr.y", (t, self.vw), rt.dtype)
        ops.gla_output(o, proj[:, self.g_off:self.g_off + self.vw], self.norm, self.eps, y, self.heads, self.dv)
        delta = ws.get("gdr.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(y, self.w_o, None, delta)
