"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import Block, DeltaPair, ScaledDelta, as_delta, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x))
    (crates/mach-model/src/batched.rs:3200, :4031, :4050, :4453 of gqf2008/machserve).

    The adds are done by the norm that follows them, in float32: the block hands the
    last delta on as `pending`, and the next norm (the next layer's, or the model's
    final one) adds it.

    A part that said at bind time that it can take its norm into its own kernels
    (`Part.fuse_norm`) is run through `forward_fused` for steps of up to its
    `fused_rows` rows: it reads the residual's rounded copy and row statistics that the
    part before it left (`RowStats`), adds its own delta into the residual and leaves the
    same for the part after it, so that neither the norm nor the add needs a kernel of
    its own.  Each half of the block decides for itself; a part without the protocol is
    given normed rows and returns a delta, as ever.

    block_params: `residual_scale` m (default 1): x += m * mixer(norm(x)); x += m * feed_forward(norm(x)).  The deltas are
    handed on with their multiplier (`ScaledDelta`) and the norm that adds them multiplies, in float32; the few-row path,
    whose products add into the stream themselves, is not taken then.  A layer without a feed-forward is
    x += m * mixer(norm(x)) alone.
    """

    graph_safe = True
    accepts_row_stats = True
    accepts_scaled = True
    optional_feed_forward = True
    kernel_files = None  # (its parts' few-row path: not said)

    def __init__(self, spec, mixer, feed_forward, mixer_norm, ff_norm):
        super().__init__(spec, mixer, feed_forward, mixer_norm, ff_norm)
        self.scale = float(spec.block_params.get("residual_scale", 1.0))
        if (feed_forward is None) != (ff_norm is None):
            raise ValueError("a pre-norm layer has a feed-forward and its norm, or neither")
        from .base import Part

        joins = [type(p).fuse_norm is not Part.fuse_norm for p in (mixer, feed_forward) if p is not None]
        if self.scale != 1.0 or feed_forward is None or not any(joins):
            # the few-row path is the only thing the block launches beyond its parts' kernels, and no part here joins it
            self.kernel_files = ()

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        plain = self.scale == 1.0
        self.fuse_mixer = plain and bool(self.mixer.fuse_norm(self.mixer_norm))
        self.fuse_feed_forward = plain and self.feed_forward is not None and bool(self.feed_forward.fuse_norm(self.ff_norm))

    def _scaled(self, delta):
        return delta if self.scale == 1.0 else ScaledDelta(delta, self.scale)

    @staticmethod
    def _for(norm, pending):
        return as_delta(pending, scaled=norm.accepts_scaled)

    def forward(self, ctx, residual, pending, cache, owns_cache=True):
        rt = ctx.rt
        t, d = residual.shape
        if self.fuse_mixer and t <= self.mixer.fused_rows and not isinstance(pending, ScaledDelta):
            pending = self.mixer.forward_fused(ctx, residual, pending, self.mixer_norm, cache, owns_cache)
        else:
            xn = rt.workspace.get("block.normed", (t, d), rt.dtype)
            self.mixer_norm.forward(residual, self._for(self.mixer_norm, pending), xn)
            pending = self._scaled(self.mixer.forward(ctx, xn, cache, owns_cache))
        if self.feed_forward is None:
            return pending
        if self.fuse_feed_forward and t <= self.feed_forward.fused_rows:
            return self.feed_forward.forward_fused(ctx, residual, pending, self.ff_norm)
        xn = rt.workspace.get("block.normed", (t, d), rt.dtype)
        self.ff_norm.forward(residual, self._for(self.ff_norm, pending), xn)
        return self._scaled(self.feed_forward.forward(ctx, xn))


@register_block("parallel")
class ParallelBlock(Block):
    """x += mixer(norm1(x)) + feed_forward(norm2(x)): both norms read the same x, and the two outputs are summed before
    they are added to the stream.  The block hands both on (`DeltaPair`); the next norm adds them in float32.  Two layer
    norms of equal size and eps share their mean and variance and are written by one kernel.  A layer without a
    feed-forward is x += mixer(norm1(x)).  A layer with a feed-forward but no norm of its own for it has ONE norm whose
    output both halves read: x += mixer(norm1(x)) + feed_forward(norm1(x)).
    """

    graph_safe = True
    accepts_pairs = True
    optional_feed_forward = True

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        both = getattr(self.mixer_norm, "shares_statistics_with", None)
        self.one_kernel = self.ff_norm is not None and both is not None and both(self.ff_norm)

    def forward(self, ctx, residual, pending, cache, owns_cache=True):
        rt = ctx.rt
        t, d = residual.shape
        pairs = self.mixer_norm.accepts_pairs
        xn = rt.workspace.get("block.normed", (t, d), rt.dtype)
        if self.feed_forward is None:
            self.mixer_norm.forward(residual, as_delta(pending, pairs), xn)
            return self.mixer.forward(ctx, xn, cache, owns_cache)
        if self.ff_norm is None:  # one norm, read by both halves
            xf = xn
            self.mixer_norm.forward(residual, as_delta(pending, pairs), xn)
        elif self.one_kernel:
            xf = rt.workspace.get("block.normed_ff", (t, d), rt.dtype)
            self.mixer_norm.forward_both(self.ff_norm, residual, as_delta(pending, pairs), xn, xf)
        else:
            xf = rt.workspace.get("block.normed_ff", (t, d), rt.dtype)
            self.mixer_norm.forward(residual, as_delta(pending, pairs), xn)
            self.ff_norm.forward(residual, None, xf)
        # The two halves read different rows and share no scratch memory.  In a captured step they run side by side, as
        # two branches of the graph: the step's chain of dependent kernels is then the mixer's alone.  (When a step is
        # launched plainly, the second stream's events would cost the host more than they save.)
        import torch

        if torch.cuda.is_current_stream_capturing():
            main, side = torch.cuda.current_stream(), rt.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                b = self.feed_forward.forward(ctx, xf)
            a = self.mixer.forward(ctx, xn, cache, owns_cache)
            main.wait_stream(side)
            return DeltaPair(a, b)
        a = self.mixer.forward(ctx, xn, cache, owns_cache)
        return DeltaPair(a, self.feed_forward.forward(ctx, xf))
