"""The step before a pass of a group of layers that runs several times in a row with the same weights.

    x <- W_in [x; x0] + step[t]

x is the stream as the layers before left it, x0 the embedding's output (the token rows before any layer touched them),
[x; x0] the two side by side (x first), W_in [width, 2 * width], and step[t] a learned vector of pass t, added after
the product.  The first pass takes this step like every other.  The sum that the layer before left to be added to the
stream is formed in float on the way into the product's input; the product's result is the new stream, in float.

A schedule holds one ``LoopEntry`` for every pass, each followed by the group's layers with that pass's caches.  The
entries of one loop share their tensors: the first one declares and binds them, the others name it as ``owner``.
The embedding must be built with ``keep_rows``: its kernel leaves x0 in the compute dtype for this step.
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part
from .norm import _terms


class LoopEntry(Part):
    graph_safe = True

    def __init__(self, in_name: str, step_name: str, width: int, times: int, index: int, owner: "LoopEntry | None" = None):
        if not 0 <= index < times:
            raise ValueError(f"pass {index} of {times}")
        self.in_name, self.step_name = in_name, step_name
        self.width, self.times, self.index, self.owner = int(width), int(times), int(index), owner
        self.w_in = self.steps = None

    def param_specs(self):
        if self.owner is not None:
            return []
        return [ParamSpec(self.in_name, (self.width, 2 * self.width)),
                ParamSpec(self.step_name, (self.times, self.width), "linear", "float32")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        if self.owner is None:
            self.w_in = tensors[self.in_name].contiguous()
            self.steps = tensors[self.step_name].contiguous()

    def linear_weights(self):
        return [self.w_in] if self.owner is None else []

    def forward(self, h, pending, batch, cache=None):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        src = self.owner if self.owner is not None else self
        rows = batch.per_step.get("embedding_rows")
        if rows is None:
            raise RuntimeError("a loop's entry needs the embedding's rows: build the embedding with keep_rows")
        tap = self.ctx.tap
        first, second, factor, ratio = _terms(pending)
        both = ws.get("loop_in", (h.shape[0], 2 * self.width), dt)
        ops.stream_concat(h, first, rows, both, delta2=second, mult=factor, mult2=ratio, write_h=tap is not None)
        if tap is not None:
            tap("residual", h)      # the stream as the layers before left it
            tap("loop_in", both)
        ops.linear(both, src.w_in, h, ws, batch.status)      # the product's rows are the new stream, in float
        ops.add_bias(h, src.steps[self.index])
        if tap is not None:
            tap("loop_out", h)
        return h, None
