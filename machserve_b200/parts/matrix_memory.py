"""A matrix memory with exponential gates (the mLSTM cell): a recurrent mixer with a matrix state, a normalizer and a
stabilizer per head."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, matrix, register_mixer, vector_f32


@register_mixer("matrix_memory")
class MatrixMemory(Mixer):
    """q = Wq x * key_dim^(-1/2), k = Wk x (heads x key_dim), v = Wv x (heads x value_dim).  Per head the logarithms of an
    input and a forget gate, one number a token: i = cap tanh((Wi x + bi) / cap), f = logsigmoid(cap tanh((Wf x + bf) / cap)).
    Per head and sequence, with S [key_dim, value_dim], n [key_dim] and m all zero at the start,

        m_t = max(f_t + m_(t-1), i_t),    a_t = exp(f_t + m_(t-1) - m_t),    b_t = exp(i_t - m_t),
        S_t = a_t S_(t-1) + b_t k_t v_t^T,    n_t = a_t n_(t-1) + b_t k_t,
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).

    Each head's o_t is divided by its root mean square over value_dim (eps inside the root); the heads side by side are
    multiplied by a weight [heads*value_dim] and by sigmoid(Wg x) and go through Wo.  The six input projections are one
    product with a float32 result; the gates, their exponentials, m, the state, the division, the norm and the output gate
    are float32.  A request's state slot holds the matrices, with the normalizer as one more column, and the heads' m.

    params: prefix, hidden_size, num_heads, key_dim, value_dim, gate_cap, eps.  Tensors under the prefix: q, k, v, g
    (matrices), i, f [heads, hidden], i.b, f.b [heads], norm [heads*value_dim], o.
    """

    graph_safe = True
    kernel_files = ('matrix_memory',)

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden, self.heads = int(spec["hidden_size"]), int(spec["num_heads"])
        self.dk, self.dv = int(spec["key_dim"]), int(spec["value_dim"])
        self.cap, self.eps = float(spec["gate_cap"]), float(spec["eps"])
        if self.dk > 256:
            raise ValueError(f"matrix_memory: {self.dk} key channels a head are more than the kernel covers (256)")
        if self.cap <= 0:
            raise ValueError(f"matrix_memory: a gate cap of {self.cap}")
        self.kw, self.vw = self.heads * self.dk, self.heads * self.dv
        # columns of the one input product: q | k | v | g | i | f
        self.q_off, self.k_off, self.v_off, self.g_off = 0, self.kw, 2 * self.kw, 2 * self.kw + self.vw
        self.i_off = self.g_off + self.vw
        self.f_off = self.i_off + self.heads
        self.width = self.f_off + self.heads

    def cache_need(self):
        return FixedState((ops.mm_state_floats(self.heads, self.dk, self.dv),))

    def tensors(self):
        p, h = self.prefix, self.hidden
        return [
            TensorDecl(p + "q", (self.kw, h)), TensorDecl(p + "k", (self.kw, h)), TensorDecl(p + "v", (self.vw, h)),
            TensorDecl(p + "g", (self.vw, h)), TensorDecl(p + "i", (self.heads, h)), TensorDecl(p + "i.b", (self.heads,), init="bias"),
            TensorDecl(p + "f", (self.heads, h)), TensorDecl(p + "f.b", (self.heads,), init="bias"),
            TensorDecl(p + "norm", (self.vw,), init="scale"), TensorDecl(p + "o", (h, self.vw)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        self.w_in = matrix(torch.cat([tensors[p + n] for n in ("q", "k", "v", "g", "i", "f")], dim=0), rt)
        self.b_i, self.b_f = vector_f32(tensors[p + "i.b"]), vector_f32(tensors[p + "f.b"])
        self.norm = vector_f32(tensors[p + "norm"])
        self.w_o = matrix(tensors[p + "o"], rt)

    def forward(self, ctx, x, cache, owns_cache=True):
        if not owns_cache:
            raise ValueError("matrix_memory: a run cannot read another run's state")
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        state = cache.state
        proj = ws.get("mm.proj", (t, self.width), torch.float32)
        ops.linear(x, self.w_in, None, proj)
        gates = ws.get("mm.gates", (t, self.heads, 4), torch.float32)
        ops.mm_gates(proj, self.i_off, self.f_off, self.b_i, self.b_f, self.cap, state, ctx.cu_tokens, ctx.state_slots, ctx.slot_of_token,
                     gates, ctx.num_seqs, self.heads, self.dk, self.dv)
        o = ws.get("mm.o", (t, self.heads, self.dv + 1), torch.float32)
        ops.mm_scan(proj, self.q_off, self.k_off, self.v_off, gates, self.dk ** -0.5, state, ctx.cu_tokens, ctx.state_slots,
                    ctx.slot_of_token, o, ctx.num_seqs, self.heads, self.dk, self.dv, narrow=ctx.max_query_len > 16)
        y = ws.get("mm.y", (t, self.vw), rt.dtype)
        ops.mm_output(o, gates, proj[:, self.g_off:self.g_off + self.vw], self.norm, self.eps, y, self.heads, self.dv)
        delta = ws.get("mm.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(y, self.w_o, None, delta)
