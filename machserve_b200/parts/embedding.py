"""The two ends of the model: token embedding, and the head that turns the final hidden rows into logits."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import Head, TokenEmbedding, matrix, register_embedding, register_head


@register_embedding("embedding")
class Embedding(TokenEmbedding):
    """x[r, :] = E[token[r], :] into the float32 residual stream, no scaling
    (crates/mach-model/src/kernels.rs:578-585 of gqf2008/machserve).

    params: tensor, vocab_size, hidden_size.
    """

    graph_safe = True
    kernel_files = ()

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.vocab, self.hidden = spec["tensor"], int(spec["vocab_size"]), int(spec["hidden_size"])

    def tensors(self):
        return [TensorDecl(self.name, (self.vocab, self.hidden))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.table = matrix(tensors[self.name], rt)

    def forward(self, ctx, out):
        return ops.embed_gather(self.table, ctx.token_ids, out)


@register_embedding("scaled_position_embedding")
class ScaledPositionEmbedding(TokenEmbedding):
    """x[r, :] = E[token[r], :] * scale + P[position[r], :] into the float32 residual stream: the table's rows are scaled,
    the learned position vectors (a table [max_positions, hidden], or none) are not.  A head tied to `tensor` reads the
    table itself, without the scale.

    params: tensor, vocab_size, hidden_size, scale, positions (tensor name or None), max_positions.
    """

    graph_safe = True
    kernel_files = ('stream',)

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.vocab, self.hidden = spec["tensor"], int(spec["vocab_size"]), int(spec["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))
        self.positions_name, self.max_positions = spec.get("positions"), int(spec.get("max_positions", 0))
        if self.positions_name is not None and self.max_positions < 1:
            raise ValueError("scaled_position_embedding: a table of positions needs max_positions")

    def tensors(self):
        out = [TensorDecl(self.name, (self.vocab, self.hidden))]
        if self.positions_name is not None:
            out.append(TensorDecl(self.positions_name, (self.max_positions, self.hidden), init="bias"))
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.table = matrix(tensors[self.name], rt)
        self.pos_table = None
        if self.positions_name is not None:
            self.pos_table = tensors[self.positions_name].to(torch.float32).contiguous()

    def forward(self, ctx, out):
        return ops.embed_scaled_pos(self.table, ctx.token_ids, ctx.positions, self.pos_table, out, self.scale)


@register_head("lm_head")
class LMHead(Head):
    """logits = x . W^T in float32, for the rows that are asked for only (the reference computes
    every row, crates/mach-model/src/batched.rs:4594-4626).  With `tied_to` set, the head's own
    tensor may be absent and the embedding table stands in
    (crates/mach-model/src/loader.rs:1025-1033); if it is present it is used.

    With `softcap` c the logits become c * tanh(logits / c), in float32.

    params: tensor, tied_to (name of the embedding tensor, or None), vocab_size, hidden_size, softcap (or None).
    """

    graph_safe = True
    kernel_files = ()

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.tied_to = spec["tensor"], spec.get("tied_to")
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.softcap = float(spec["softcap"]) if spec.get("softcap") else None

    def tensors(self):
        out = [TensorDecl(self.name, (self.vocab, self.hidden), required=self.tied_to is None, random=self.tied_to is None)]
        if self.tied_to is not None:
            out.append(TensorDecl(self.tied_to, (self.vocab, self.hidden)))
        return out

    def bind(self, tensors, rt, embedding=None):
        super().bind(tensors, rt, embedding)
        if self.name in tensors:
            self.weight = matrix(tensors[self.name], rt)
        elif embedding is not None and getattr(embedding, "name", None) == self.tied_to and hasattr(embedding, "table"):
            self.weight = embedding.table  # the embedding's own device tensor: one copy in memory
        else:
            self.weight = matrix(tensors[self.tied_to], rt)

    def forward(self, ctx, x, out):
        ops.linear(x, self.weight, None, out)
        return ops.softcap(out, self.softcap) if self.softcap else out
