"""RMSNorm fused with the residual add.

RMSNorm(v; w, eps) = v * rsqrt(mean(v^2) + eps) * w over the last axis, with the
plain weight (src/dense.rs:382,385-391).  The residual stream is float32; the
kernel adds the pending delta, stores the sum back and writes the normalised rows
in the compute dtype.  The weight is held in float32 (exact for a bfloat16
checkpoint) so both paths read the same numbers.
"""
from __future__ import annotations

from .base import Norm, ParamSpec, ScaledSum


def _terms(delta):
    """(first, second, factor, ratio) of what is to be added to the stream: factor * (first + ratio * second)."""
    if isinstance(delta, ScaledSum):
        if delta.vector is not None or delta.third is not None:
            raise ValueError("this norm adds factor * (first + ratio * second) only: no vectors, no third term")
        return delta.first, delta.second, delta.factor, delta.ratio
    return delta, None, 1.0, 1.0


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, name: str, width: int, eps: float, out_scale: float = 1.0):
        self.name, self.width, self.eps = name, int(width), float(eps)
        # what the normed rows are multiplied with besides the weight (a model that scales its logits: the factor goes
        # through the head's product, so it may as well be put on the rows the head reads); folded into the weight, in float
        self.out_scale = float(out_scale)
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.width,), "norm", "float32")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = tensors[self.name].contiguous()
        if self.out_scale != 1.0:
            self.weight = (self.weight * self.out_scale).contiguous()

    def forward(self, h, delta, also=None):
        """``also``: a second norm of the same rows (same eps) with its own weight; the mean of squares is formed once and
        (h, x, x of the second norm) comes back."""
        x = self.ctx.workspace.get("norm_out", (h.shape[0], self.width), self.ctx.dtype)
        first, second, factor, ratio = _terms(delta)
        if also is None:
            self.ctx.ops.add_rmsnorm(h, first, self.weight, self.eps, x, delta2=second, mult=factor, mult2=ratio)
            return h, x
        if also.eps != self.eps or also.width != self.width:
            raise ValueError("two norms of the same rows in one pass need the same eps and width")
        x2 = self.ctx.workspace.get("norm_out_second", (h.shape[0], self.width), self.ctx.dtype)
        self.ctx.ops.add_rmsnorm(h, first, self.weight, self.eps, x, delta2=second, mult=factor, mult2=ratio,
                                 weight2=also.weight, x2_out=x2)
        return h, x, x2

    def forward_rows(self, h, delta, rows):
        x = self.ctx.workspace.get("norm_rows_out", (rows.shape[0], self.width), self.ctx.dtype)
        first, second, factor, ratio = _terms(delta)
        self.ctx.ops.add_rmsnorm(h, first, self.weight, self.eps, x, rows=rows, delta2=second, mult=factor, mult2=ratio)
        return x


class GroupRMSNorm(Norm):
    """The stream's norm in ``groups`` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps), the whole
    times the weight; fused with the add of what is pending, which may carry a vector for every term (a layer that scales
    its mixer's and its feed-forward's results number by number): v = h + vector * (factor * (first + ratio * second)) +
    third_vector * third, formed in float.  One group is the plain RMS norm."""

    graph_safe = True

    def __init__(self, name: str, width: int, eps: float, groups: int = 1, out_scale: float = 1.0):
        if groups < 1 or width % groups:
            raise ValueError(f"a row of {width} numbers does not split into {groups} equal parts")
        self.name, self.width, self.eps, self.groups = name, int(width), float(eps), int(groups)
        self.out_scale = float(out_scale)     # folded into the weight, in float (a model that scales its logits)
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.width,), "norm", "float32")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = tensors[self.name].contiguous()
        if self.out_scale != 1.0:
            self.weight = (self.weight * self.out_scale).contiguous()

    @staticmethod
    def _all_terms(delta):
        """(d1, d2, d3, m1, m2, va, vb) of v = h + va * (m1 * d1 + m2 * d2) + vb * d3."""
        if isinstance(delta, ScaledSum):
            first, second, m1, m2 = delta.first, delta.second, delta.factor, delta.factor * delta.ratio
            if first is None:
                first, second, m1, m2 = second, None, m2, 0.0
            return first, second, delta.third, m1, m2, delta.vector, delta.third_vector
        return delta, None, None, 1.0, 0.0, None, None

    def forward(self, h, delta, also=None):
        x = self.ctx.workspace.get("norm_out", (h.shape[0], self.width), self.ctx.dtype)
        if also is None:
            self.ctx.ops.add_group_rmsnorm(h, self._all_terms(delta), self.weight, self.eps, self.groups, x)
            return h, x
        if also.eps != self.eps or also.width != self.width or getattr(also, "groups", 1) != self.groups:
            raise ValueError("two norms of the same rows in one pass need the same eps, width and groups")
        x2 = self.ctx.workspace.get("norm_out_second", (h.shape[0], self.width), self.ctx.dtype)
        self.ctx.ops.add_group_rmsnorm(h, self._all_terms(delta), self.weight, self.eps, self.groups, x, weight2=also.weight, x2_out=x2)
        return h, x, x2

    def forward_rows(self, h, delta, rows):
        x = self.ctx.workspace.get("norm_rows_out", (rows.shape[0], self.width), self.ctx.dtype)
        self.ctx.ops.add_group_rmsnorm(h, self._all_terms(delta), self.weight, self.eps, self.groups, x, rows=rows)
        return x
