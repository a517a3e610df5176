"""How a mixer, a feed-forward and their norms are arranged in a layer.

``PreNormBlock``: h += mixer(norm1(h)); h += ffn(norm2(h)) (src/dense.rs:380-390).
``ParallelBlock``: x = norm(h); h += factor * (mixer(x) + ffn(x)): one norm, both sublayers read it; or two norms of
the same stream, one for each sublayer.
The residual stream is float32.  A block receives the stream together with a
pending delta (the previous block's last output, not yet added) so that every
add is fused with the norm that follows it; it returns the stream and its own
pending delta.
"""
from __future__ import annotations

from .base import ParamSpec, Part, ScaledSum


class PreNormBlock(Part):
    """``norm2`` and ``ffn`` may both be None (a layer of a mixer alone: what the mixer gives is the block's pending
    delta).  ``input_conv`` (a ``ShortConv`` with ``residual``): what the mixer reads is x + conv(x) of the normed rows,
    a short causal convolution over time whose last inputs are part of every request's state; it is the first thing the
    block remembers, before what its mixer remembers."""

    graph_safe = True

    def __init__(self, norm1, mixer, norm2=None, ffn=None, input_conv=None):
        if (norm2 is None) != (ffn is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        self.norm1, self.mixer, self.norm2, self.ffn, self.input_conv = norm1, mixer, norm2, ffn, input_conv

    def children(self):
        return [p for p in (self.norm1, self.input_conv, self.mixer, self.norm2, self.ffn) if p is not None]

    def cache_specs(self):
        return (self.input_conv.cache_specs() if self.input_conv is not None else []) + self.mixer.cache_specs()

    def forward(self, h, pending, batch, cache):
        tap = self.ctx.tap
        h, x = self.norm1.forward(h, pending)
        if tap is not None:
            tap("residual", h)      # the stream as this block finds it: everything before it has been added
            tap("norm1", x)
        if self.input_conv is not None:
            views = list(cache) if isinstance(cache, (tuple, list)) else [cache]
            x = self.input_conv.forward(x, batch, views[0], self.ctx.workspace.get("conv_in", tuple(x.shape), x.dtype))
            cache = None if len(views) == 1 else (views[1] if len(views) == 2 else tuple(views[1:]))
            if tap is not None:
                tap("conv_in", x)
        a = self.mixer.forward(x, batch, cache)
        if tap is not None and not isinstance(a, ScaledSum):
            tap("mixer_out", a)
        if self.ffn is None:
            return h, a
        h, x = self.norm2.forward(h, a)
        if tap is not None:
            tap("norm2", x)
        m = self.ffn.forward(x, batch)
        if tap is not None:
            tap("ffn_out", m)
        return h, m


class ParallelBlock(Part):
    """One norm whose rows the mixer and the feed-forward both read; what they give is added to the stream together,
    times ``factor``: h <- h + factor * (mixer(norm(h)) + ffn(norm(h))).  ``ffn`` may be None (a layer of a mixer
    alone).  With ``norm2`` the feed-forward reads a norm of its own, of the same stream:
    h <- h + factor * (mixer(norm(h)) + ffn(norm2(h))); both norms come from one kernel, which forms the rows' mean of
    squares once.  The sum is formed in float by the norm that adds it (the next block's, or the model's last)."""

    graph_safe = True

    def __init__(self, norm, mixer, ffn=None, factor: float = 1.0, norm2=None, mixer_scale: str | None = None,
                 ffn_scale: str | None = None, width: int = 0):
        if norm2 is not None and ffn is None:
            raise ValueError("a second norm goes with a feed-forward")
        if ffn_scale is not None and ffn is None:
            raise ValueError("a feed-forward's scale goes with a feed-forward")
        if (mixer_scale is not None or ffn_scale is not None) and (width <= 0 or factor != 1.0):
            raise ValueError("scale vectors need the width, and take the place of a factor")
        self.norm, self.mixer, self.ffn, self.factor, self.norm2 = norm, mixer, ffn, float(factor), norm2
        # tensor names of learned vectors of the stream's width ("layer scale"): the mixer's result and the feed-forward's
        # are each multiplied by its own, number by number, before they are added to the stream
        self.mixer_scale, self.ffn_scale, self.width = mixer_scale, ffn_scale, int(width)
        self.mixer_vector = self.ffn_vector = None

    def param_specs(self):
        return [ParamSpec(n, (self.width,), "norm", "float32") for n in (self.mixer_scale, self.ffn_scale) if n is not None]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        if self.mixer_scale is not None:
            self.mixer_vector = tensors[self.mixer_scale].contiguous()
        if self.ffn_scale is not None:
            self.ffn_vector = tensors[self.ffn_scale].contiguous()

    def children(self):
        return [p for p in (self.norm, self.norm2, self.mixer, self.ffn) if p is not None]

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, h, pending, batch, cache):
        tap = self.ctx.tap
        if self.norm2 is not None:
            h, x, x_ffn = self.norm.forward(h, pending, also=self.norm2)
        else:
            h, x = self.norm.forward(h, pending)
            x_ffn = x
        if tap is not None:
            tap("residual", h)
            tap("norm1", x)
            if self.norm2 is not None:
                tap("norm2", x_ffn)
        a = self.mixer.forward(x, batch, cache)
        if tap is not None and not isinstance(a, ScaledSum):
            tap("mixer_out", a)
        m = None
        if self.ffn is not None:
            m = self.ffn.forward(x_ffn, batch)
            if tap is not None:
                tap("ffn_out", m)
        if self.mixer_vector is None and self.ffn_vector is None and not isinstance(a, ScaledSum):
            return h, ScaledSum(a, m, self.factor)
        # the mixer's share (itself perhaps a weighted sum of two mixers) under its vector, the feed-forward's under its own
        if isinstance(a, ScaledSum):
            if self.factor != 1.0:
                raise ValueError("a mixer that hands on a weighted sum goes with scale vectors, not with a factor")
            if a.vector is not None or a.third is not None:
                raise ValueError("a mixer hands on at most two weighted terms")
            return h, ScaledSum(a.first, a.second, a.factor, a.ratio, vector=self.mixer_vector, third=m, third_vector=self.ffn_vector)
        return h, ScaledSum(a, None, 1.0, 1.0, vector=self.mixer_vector, third=m, third_vector=self.ffn_vector)
