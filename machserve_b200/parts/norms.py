"""The norms: RMSNorm and layer norm, each with the residual add fused in front of it."""
from __future__ import annotations

from .. import ops
from ..weights.loader import TensorDecl
from .base import DeltaPair, Norm, ScaledDelta, as_delta, register_norm, vector_f32


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w: eps inside the root, plain x*w, mean over the whole width,
    all in float32 (crates/mach-model/src/kernels.rs:63-80 of gqf2008/machserve).

    params: tensor (name of the weight), size, eps.
    """

    graph_safe = True
    kernel_files = ('stream',)
    accepts_pairs = True  # a `DeltaPair` is summed and added by a kernel of its own (x + (a + b), float32)
    accepts_scaled = True  # a `ScaledDelta` is multiplied by the same kernel as it is added (x + m * a, float32)

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.size, self.eps = spec["tensor"], int(spec["size"]), float(spec["eps"])

    def tensors(self):
        return [TensorDecl(self.name, (self.size,), init="scale")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = vector_f32(tensors[self.name])

    def forward(self, residual, delta, out, rows=None):
        if isinstance(delta, DeltaPair):
            return ops.add_streams_rmsnorm(residual, delta.a, delta.b, None, None, self.weight, out, self.eps, rows)
        if isinstance(delta, ScaledDelta):
            return ops.add_streams_rmsnorm(residual, delta.delta, None, None, None, self.weight, out, self.eps, rows, delta.scale)
        return ops.add_rmsnorm(residual, as_delta(delta), self.weight, out, self.eps, rows)

    def fold_into(self, matrix):
        """W[n][k] *= g[k], in float32 and rounded once; g becomes 1 ((x / rms * g) . W^T = (x . (W g)^T) / rms)."""
        matrix.copy_((matrix.float() * self.weight[None, :]).to(matrix.dtype))
        self.weight.fill_(1.0)
        return True


@register_norm("layernorm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w + b, var the mean of the squared deviations, all in float32.

    Takes a `DeltaPair` as well as one delta: the stream becomes x + (a + b).  `forward_both` writes this norm and a
    second one of the same rows (the two norms of a parallel layer share mean and variance) with one kernel.

    params: tensor (name of the weight), bias (name of the bias), size, eps.
    """

    graph_safe = True
    accepts_pairs = True

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.bias_name, self.size, self.eps = spec["tensor"], spec["bias"], int(spec["size"]), float(spec["eps"])

    def tensors(self):
        return [TensorDecl(self.name, (self.size,), init="scale"), TensorDecl(self.bias_name, (self.size,), init="bias")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = vector_f32(tensors[self.name])
        self.bias = vector_f32(tensors[self.bias_name])

    @staticmethod
    def _deltas(delta):
        if isinstance(delta, DeltaPair):
            return delta.a, delta.b
        return as_delta(delta), None

    def forward(self, residual, delta, out, rows=None):
        a, b = self._deltas(delta)
        return ops.add_layernorm(residual, a, b, self.weight, self.bias, out, self.eps, rows)

    def shares_statistics_with(self, other) -> bool:
        return isinstance(other, LayerNorm) and other.size == self.size and other.eps == self.eps

    def forward_both(self, other: "LayerNorm", residual, delta, out, out_other):
        """out = this norm, out_other = `other`'s norm of the same rows, after the add."""
        a, b = self._deltas(delta)
        ops.add_layernorm(residual, a, b, self.weight, self.bias, out, self.eps, None, other.weight, other.bias, out_other)
        return out, out_other
