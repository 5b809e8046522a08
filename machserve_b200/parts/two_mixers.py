"""A mixer made of two mixers that read the same rows: each output normed over the width with a weight of its own, then
their mean; or the two outputs as they are, each times a number of its own, then their sum."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import MIXERS, CacheSet, Mixer, register_mixer, vector_f32


@register_mixer("two_mixers")
class TwoMixers(Mixer):
    """delta = scale * (left(x) / rms(left(x)) * w_left + right(x) / rms(right(x)) * w_right): `left` and `right` are
    mixers of any registered kind, built from their own specs; each root mean square runs over the model width (eps inside
    the root); `scale` is 1/2 unless said.  Each member keeps what it keeps (`CacheSet`: pages for one, a state for the
    other, or anything else); the members' work lists are the members' own.  In a captured step the two members run as two
    branches of the graph.  With `combine` "weighted_sum" there are no norms: delta = left_scale * left(x) + right_scale *
    right(x), in float32 (a member that offers `defer_output_bias` has its output projection's bias added here).

    params: left, right (PartSpecs of mixers), hidden_size, combine ("normed_mean" if absent, or "weighted_sum"); for the
    mean: left_norm, right_norm (tensor names of the weights), eps, scale; for the sum: left_scale, right_scale.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.left, self.right = MIXERS.build(spec["left"]), MIXERS.build(spec["right"])
        self.combine = spec.get("combine", "normed_mean")
        if self.combine not in ("normed_mean", "weighted_sum"):
            raise ValueError(f"two_mixers: combine '{self.combine}' is neither 'normed_mean' nor 'weighted_sum'")
        self.hidden = int(spec["hidden_size"])
        if self.combine == "normed_mean":
            self.left_name, self.right_name = spec["left_norm"], spec["right_norm"]
            self.eps, self.scale = float(spec["eps"]), float(spec.get("scale", 0.5))
        else:
            self.left_scale, self.right_scale = float(spec["left_scale"]), float(spec["right_scale"])
        self.graph_safe = bool(self.left.graph_safe and self.right.graph_safe)
        files = [m.kernel_files for m in (self.left, self.right)]
        self.kernel_files = None if any(f is None for f in files) else tuple(sorted({"stream", *files[0], *files[1]}))
        if self.left.plan_key() is not None and self.right.plan_key() is not None and self.left.plan_key() != self.right.plan_key():
            raise ValueError("two_mixers: the two members ask for work lists under different keys")
        self._planner = self.left if self.left.plan_key() is not None else self.right

    def cache_need(self):
        return CacheSet((self.left.cache_need(), self.right.cache_need()))

    def tensors(self):
        if self.combine == "weighted_sum":
            return [*self.left.tensors(), *self.right.tensors()]
        return [*self.left.tensors(), *self.right.tensors(), TensorDecl(self.left_name, (self.hidden,), init="scale"),
                TensorDecl(self.right_name, (self.hidden,), init="scale")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.left.bind(tensors, rt)
        self.right.bind(tensors, rt)
        self.graph_safe = bool(self.left.graph_safe and self.right.graph_safe)
        if self.combine == "normed_mean":
            self.w_left, self.w_right = vector_f32(tensors[self.left_name]), vector_f32(tensors[self.right_name])
        else:  # a member's output bias rides in the sum's kernel
            self.bias_left, self.bias_right = (getattr(m, "defer_output_bias", lambda: None)() for m in (self.left, self.right))

    # the members' work lists (at most one key between them)
    def plan_key(self):
        return self._planner.plan_key()

    def plan(self, step):
        return self._planner.plan(step)

    def plan_words(self, max_rows, max_seqs):
        return self._planner.plan_words(max_rows, max_seqs)

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        left_cache, right_cache = cache
        main, side = torch.cuda.current_stream(), rt.side_stream()
        if torch.cuda.is_current_stream_capturing() and main != side:  # the members share no scratch memory: two branches of the graph
            side.wait_stream(main)
            with torch.cuda.stream(side):
                b = self.right.forward(ctx, x, right_cache, owns_cache)
            a = self.left.forward(ctx, x, left_cache, owns_cache)
            main.wait_stream(side)
        else:
            a = self.left.forward(ctx, x, left_cache, owns_cache)
            b = self.right.forward(ctx, x, right_cache, owns_cache)
        delta = rt.workspace.get("two_mixers.delta", (t, self.hidden), torch.float32)
        if self.combine == "weighted_sum":
            return ops.pair_weighted_sum(a, b, delta, self.left_scale, self.right_scale, self.bias_left, self.bias_right)
        return ops.norm_pair_mean(a, b, self.w_left, self.w_right, delta, self.eps, self.scale)
