"""Mixers whose memory is a matrix a head that is stepped from token to token:  S_t = diag(a_t) S_(t-1) + k_t v_t^T,
o_t = S_t^T q_t, with S (K x V, float32, kept transposed) in a state slot of the request.

``StateSpaceMixer`` (the state-space-duality layer, "Mamba-2"): one input product laid out [z | x | B | C | dt]; x, B and
C pass a short causal convolution and silu; per head a = exp(-exp(A_log) dt) with dt = softplus(dt + dt_bias), k = dt B,
q = C, v = x (B and C are shared by the heads of a group), y = o + D x; y * silu(z) is RMS-normed in ``norm_groups`` equal
parts and projected out.

``GatedLinearMixer`` (linear attention whose forget gate also decides what is written, "HGRN2"): q = silu(W_q h),
v = W_v h, f = low + (1 - low) sigmoid(W_f h + b) per head and channel; a = f, k = 1 - f; every head's o is RMS-normed
over its V numbers with one weight shared by the heads, and projected out.

Step sizes, decays, gates, the state and the norms are float whatever the run's dtype; the products and the convolution
run in the compute dtype.  Tensor names below ``prefix`` are parameters of both.
"""
from __future__ import annotations

import torch

from .base import CacheSpec, Mixer, ParamSpec
from .conv import ShortConv


class StateSpaceMixer(Mixer):
    graph_safe = True
    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
             "norm": "norm", "out": "o"}

    def __init__(self, prefix: str, width: int, heads: int, vdim: int, state: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float, names: dict | None = None):
        if heads % groups or (heads * vdim) % norm_groups:
            raise ValueError("heads must divide into groups, and heads * vdim into norm_groups")
        self.prefix, self.width = prefix, int(width)
        self.heads, self.vdim, self.state, self.groups = int(heads), int(vdim), int(state), int(groups)
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        self.inner = self.heads * self.vdim
        self.conv_channels = self.inner + 2 * self.groups * self.state
        self.names = {k: f"{prefix}.{v}" for k, v in {**self.NAMES, **(names or {})}.items()}
        self.conv = ShortConv(self.names["conv"], self.conv_channels, conv_taps, self.names["conv_bias"], activation="silu")

    def children(self):
        return [self.conv]

    def cache_specs(self):
        return self.conv.cache_specs() + [CacheSpec("state", state_shape=(self.heads, self.vdim, self.state), state_dtype="float32")]

    def param_specs(self):
        n = self.names
        return [ParamSpec(n["in"], (2 * self.inner + 2 * self.groups * self.state + self.heads, self.width)),
                ParamSpec(n["dt_bias"], (self.heads,), "linear", "float32"),
                ParamSpec(n["a_log"], (self.heads,), "linear", "float32"),
                ParamSpec(n["skip"], (self.heads,), "ones", "float32"),
                ParamSpec(n["norm"], (self.inner,), "norm", "float32"),
                ParamSpec(n["out"], (self.width, self.inner))]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        n = self.names
        self.w_in, self.w_out = tensors[n["in"]].contiguous(), tensors[n["out"]].contiguous()
        self.dt_bias, self.a_log = tensors[n["dt_bias"]].contiguous(), tensors[n["a_log"]].contiguous()
        self.skip, self.norm_w = tensors[n["skip"]].contiguous(), tensors[n["norm"]].contiguous()

    def linear_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        conv_cache, state_cache = cache
        n, inner, cc = x.shape[0], self.inner, self.conv_channels
        proj = ws.get("ssm_in", (n, self.w_in.shape[0]), dt)
        ops.linear(x, self.w_in, proj, ws, batch.status)
        tap = self.ctx.tap
        if tap is not None:
            tap("ssm_in", proj)
        conv = ws.get("ssm_conv", (n, cc), dt)
        self.conv.forward(proj[:, inner:inner + cc], batch, conv_cache, conv)
        if tap is not None:
            tap("ssm_conv", conv)
        y = ws.get("recurrence_out", (n, inner), torch.float32)
        ops.recurrence_ssd(conv, proj[:, inner + cc:], self.dt_bias, self.a_log, self.skip, state_cache.state, y, batch,
                           state_cache.slots, self.heads, self.groups, self.state, self.vdim, workspace=ws)
        if tap is not None:
            tap("recurrence_out", y)
        gated = ws.get("recurrence_normed", (n, inner), dt)
        ops.group_rmsnorm(y, self.norm_w, self.eps, gated, self.norm_groups, gate=proj[:, :inner])
        if tap is not None:
            tap("recurrence_normed", gated)
        out = ws.get("mixer_out", (n, self.width), dt)
        ops.linear(gated, self.w_out, out, ws, batch.status)
        return out


class GatedLinearMixer(Mixer):
    graph_safe = True
    NAMES = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "out": "o"}

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, eps: float, names: dict | None = None,
                 out_name: str = "mixer_out"):
        self.prefix, self.width = prefix, int(width)
        self.heads, self.dim, self.vdim, self.eps = int(heads), int(dim), int(vdim), float(eps)
        self.names = {k: f"{prefix}.{v}" for k, v in {**self.NAMES, **(names or {})}.items()}
        self.out_name = out_name

    def cache_spec(self):
        return CacheSpec("state", state_shape=(self.heads, self.vdim, self.dim), state_dtype="float32")

    def param_specs(self):
        n, hk, hv = self.names, self.heads * self.dim, self.heads * self.vdim
        return [ParamSpec(n["q"], (hk, self.width)), ParamSpec(n["f"], (hk, self.width)), ParamSpec(n["v"], (hv, self.width)),
                ParamSpec(n["f_bias"], (hk,), "linear", "float32"), ParamSpec(n["lower"], (hk,), "zeros", "float32"),
                ParamSpec(n["norm"], (self.vdim,), "norm", "float32"), ParamSpec(n["out"], (self.width, hv))]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        n = self.names
        self.w_qfv = torch.cat([tensors.pop(n["q"]), tensors.pop(n["f"]), tensors.pop(n["v"])], dim=0).contiguous()
        self.w_out = tensors[n["out"]].contiguous()
        self.f_bias, self.lower = tensors[n["f_bias"]].contiguous(), tensors[n["lower"]].contiguous()
        self.norm_w = tensors[n["norm"]].contiguous()

    def linear_weights(self):
        return [self.w_qfv, self.w_out]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, hk, hv = x.shape[0], self.heads * self.dim, self.heads * self.vdim
        proj = ws.get("gla_in", (n, 2 * hk + hv), dt)
        ops.linear(x, self.w_qfv, proj, ws, batch.status)
        tap = self.ctx.tap
        if tap is not None:
            tap("gla_in", proj)
        o = ws.get("gla_recurrence_out", (n, hv), torch.float32)
        ops.recurrence_gate(proj[:, :hk], proj[:, hk:2 * hk], proj[:, 2 * hk:], self.f_bias, self.lower, cache.state, o, batch,
                            cache.slots, self.heads, self.dim, self.vdim, workspace=ws)
        if tap is not None:
            tap("gla_recurrence_out", o)
        normed = ws.get("gla_normed", (n, hv), dt)
        ops.group_rmsnorm(o, self.norm_w, self.eps, normed, self.heads)
        if tap is not None:
            tap("gla_normed", normed)
        out = ws.get(self.out_name, (n, self.width), dt)
        ops.linear(normed, self.w_out, out, ws, batch.status)
        if tap is not None:
            tap("gla_proj", out)
        return out


class DecayLinearMixer(Mixer):
    """Linear attention with a learned decay a head and channel and a bonus for the current token ("RWKV" time mixing):

        every projection reads its own mix of the token's input and the previous token's: x + (x' - x) * mu_s, s in r, k, v, g, w
        r, k, v = W_r, W_k, W_v of their mixes (heads x dim each), gate = silu(W_g mix_g)
        a_t = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))                         per head and channel
        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,  S_t = diag(a_t) S_(t-1) + k_t v_t^T

    every head's o is RMS-normed over its own numbers, the heads side by side are multiplied by a weight and by the gate, and
    projected out.  A request remembers the last token's input (compute dtype) and S (float32, zero at the start).  The
    mixes, the decay, the state and the norm are float whatever the run's dtype."""

    graph_safe = True
    NAMES = {"mu": "mu.{s}", "r": "r", "k": "k", "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "out": "o"}
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, prefix: str, width: int, heads: int, dim: int, rank: int, eps: float, names: dict | None = None,
                 out_name: str = "mixer_out"):
        self.prefix, self.width = prefix, int(width)
        self.heads, self.dim, self.rank, self.eps = int(heads), int(dim), int(rank), float(eps)
        self.inner = self.heads * self.dim
        self.names = {k: f"{prefix}.{v}" for k, v in {**self.NAMES, **(names or {})}.items()}
        self.out_name = out_name

    def cache_specs(self):
        return [CacheSpec("state", state_shape=(self.width,), state_dtype="compute"),
                CacheSpec("state", state_shape=(self.heads, self.dim, self.dim), state_dtype="float32")]

    def param_specs(self):
        n = self.names
        specs = [ParamSpec(n["mu"].format(s=s), (self.width,), "linear", "float32") for s in self.MIXES]
        specs += [ParamSpec(n[s], (self.inner, self.width)) for s in ("r", "k", "v", "g")]
        specs += [ParamSpec(n["w1"], (self.rank, self.width)), ParamSpec(n["w2"], (self.inner, self.rank)),
                  ParamSpec(n["w0"], (self.inner,), "linear", "float32"), ParamSpec(n["u"], (self.heads, self.dim), "linear", "float32"),
                  ParamSpec(n["norm"], (self.inner,), "norm", "float32"), ParamSpec(n["out"], (self.width, self.inner))]
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        n = self.names
        self.mu = torch.stack([tensors.pop(n["mu"].format(s=s)) for s in self.MIXES]).contiguous()
        self.w = {s: tensors[n[s]].contiguous() for s in ("r", "k", "v", "g", "w1", "w2")}
        # r, k, v and g have one shape and each its own input: in bfloat16 they are one batched product of the library
        self.w_four = torch.stack([self.w[s] for s in ("r", "k", "v", "g")]).transpose(1, 2) if ctx.dtype == torch.bfloat16 else None
        self.w0, self.u = tensors[n["w0"]].contiguous(), tensors[n["u"]].contiguous()
        self.norm_w, self.w_out = tensors[n["norm"]].contiguous(), tensors[n["out"]].contiguous()

    def linear_weights(self):
        return list(self.w.values()) + [self.w_out]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        last_cache, state_cache = cache
        n, inner = x.shape[0], self.inner
        tap = self.ctx.tap
        mixes = ws.get("shift_mixes", (len(self.MIXES), n, self.width), dt)
        ops.token_shift_mix(x, self.mu, mixes, last_cache.state, batch, last_cache.slots)
        if tap is not None:
            tap("shift_mixes", mixes)
        proj = ws.get("decay_in", (5, n, inner), dt)       # r, k, v, g and the decay's raw numbers
        if self.w_four is not None:
            torch.bmm(mixes[:4], self.w_four, out=proj[:4])
        else:       # (the 32-bit path: every product on the FMA units in ascending k)
            for i, s in enumerate(("r", "k", "v", "g")):
                ops.linear(mixes[i], self.w[s], proj[i], ws, batch.status)
        low = ws.get("decay_low", (n, self.rank), dt)
        ops.linear(mixes[4], self.w["w1"], low, ws, batch.status)
        ops.unary_act(low, low, "tanh")
        ops.linear(low, self.w["w2"], proj[4], ws, batch.status)
        if tap is not None:
            tap("decay_in", proj)
        o = ws.get("decay_recurrence_out", (n, inner), torch.float32)
        ops.recurrence_decay(proj[0], proj[1], proj[4], proj[2], self.w0, self.u, state_cache.state, o, batch, state_cache.slots,
                             self.heads, self.dim, self.dim, workspace=ws)
        if tap is not None:
            tap("decay_recurrence_out", o)
        normed = ws.get("decay_normed", (n, inner), dt)
        ops.group_rmsnorm(o, self.norm_w, self.eps, normed, self.heads, gate=proj[3], gate_after=True)
        if tap is not None:
            tap("decay_normed", normed)
        out = ws.get(self.out_name, (n, self.width), dt)
        ops.linear(normed, self.w_out, out, ws, batch.status)
        if tap is not None:
            tap("decay_proj", out)
        return out


class ParallelMixer(Mixer):
    """Two mixers side by side on the same input: left_scale * left(x) + right_scale * right(x).  The sum is handed on
    unformed (``ScaledSum``): the norm that adds it to the stream forms it in float."""

    graph_safe = True

    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0):
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)

    def children(self):
        return [self.left, self.right]

    def cache_specs(self):
        return self.left.cache_specs() + self.right.cache_specs()

    @staticmethod
    def _views(views, count):
        return None if count == 0 else (views[0] if count == 1 else tuple(views))

    def forward(self, x, batch, cache):
        from .base import ScaledSum
        views = list(cache) if isinstance(cache, (tuple, list)) else [cache]
        nl, nr = len(self.left.cache_specs()), len(self.right.cache_specs())
        a = self.left.forward(x, batch, self._views(views[:nl], nl))
        b = self.right.forward(x, batch, self._views(views[nl:nl + nr], nr))
        tap = self.ctx.tap
        if tap is not None:
            tap("left_out", a)
            tap("right_out", b)
        return ScaledSum.weighted(a, self.left_scale, b, self.right_scale)
