"""A routed feed-forward (mixture of experts) with an optional shared expert.

    z = W_router x                      in float32, whatever the activations' type
    E(x) = the ``top`` experts with the largest z; weight_e = softmax over those z alone
    y = sum over e in E(x) of weight_e * expert_e(x)  (+ shared(x))
    expert(x) = down(act(gate x) * (up x)), no biases

The experts' weights are kept stacked, [experts, 2 * inner, width] and [experts, width, inner]; an expert's gate and
up rows come in blocks of 64 gate rows each followed by their 64 up rows (plain concatenation when the inner size
is no multiple of 64), as the dense feed-forward keeps them.  A step sorts its (row, choice) pairs by expert on the
device and the experts' products run over their runs of rows: in bfloat16 on the tcgen05 tensor cores
(``csrc/kernels/moe_tcgen05.cu``; with blocks of 64 the gate/up product forms act(gate) * up in its epilogue), in
float32 on the FMA units with every sum in ascending k (``csrc/kernels/moe.cu``).  Nothing waits for the host, so
decode steps can be captured in graphs.  The shared expert is a gated feed-forward like any other.

Options, each a parameter:
``scoring="sigmoid"``: an expert's score is s = sigmoid(z); the choice goes by s + correction (a tensor ``correction``, one
    number an expert, when ``correction_name`` is given) among the experts of the ``keep_groups`` best of ``groups`` equal
    groups of neighbouring experts (a group's worth is the sum of its two largest corrected scores; experts of other groups
    cannot be chosen); the weights are the chosen s over their sum, times ``route_scale``.
``activation="swish_clamp"`` with ``activation_args=(limit, alpha)``: an expert's pointwise part is
    g = min(gate x, limit), u = clamp(up x, -limit, limit), g * sigmoid(alpha * g) * (u + 1).
``normalize=False`` (sigmoid scoring): a chosen expert's weight is its score itself (times ``route_scale``), not its share of
    the chosen scores' sum.
``gated=False``: an expert has no gate, expert(x) = down(act(up x)) with a one-argument activation (``activation="relu2"``:
    the square of max(., 0)); ``names`` are then (up, down).
``weight_input=True``: a chosen expert's weight multiplies what the expert READS, y = sum of expert_e(weight_e * x), not what
    it gives (for an expert that is not linear in its input this is another function): the rows are weighted while they
    are brought into the experts' order, and the experts' results are added as they are.
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec


class RoutedFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, width: int, inner: int, n_experts: int, top: int, activation: str = "silu",
                 shared: FeedForward | None = None, router_name: str = "router", expert_name: str = "e{index}",
                 names: tuple = ("gate", "up", "down"), activation_args: tuple = (), scoring: str = "softmax",
                 correction_name: str | None = None, groups: int = 1, keep_groups: int = 1, route_scale: float = 1.0,
                 normalize: bool = True, gated: bool = True, weight_input: bool = False):
        if not 0 < top <= n_experts:
            raise ValueError(f"a row cannot take {top} of {n_experts} experts")
        if top > 32:
            raise ValueError("at most 32 experts a row")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown scoring {scoring!r}")
        if scoring == "softmax" and (correction_name is not None or groups != 1 or route_scale != 1.0):
            raise ValueError("a correction, groups and a factor go with sigmoid scoring")
        if groups < 1 or n_experts % groups or not 1 <= keep_groups <= groups or keep_groups * (n_experts // groups) < top:
            raise ValueError(f"{groups} groups of which {keep_groups} are kept do not fit {n_experts} experts of which {top} are chosen")
        if not gated and (activation != "relu2" or len(names) != 2):
            raise ValueError("an expert without a gate has the activation 'relu2' and two tensors (up, down)")
        if gated and (activation == "relu2" or len(names) != 3):
            raise ValueError("a gated expert has a two-argument activation and three tensors (gate, up, down)")
        if not normalize and scoring != "sigmoid":
            raise ValueError("weights that are not normalised go with sigmoid scoring")
        self.normalize, self.gated, self.weight_input = bool(normalize), bool(gated), bool(weight_input)
        self.activation_args = tuple(activation_args)
        self.scoring, self.groups, self.keep_groups, self.route_scale = scoring, int(groups), int(keep_groups), float(route_scale)
        self.correction_name = f"{prefix}.{correction_name}" if correction_name else None
        self.correction = None
        self.prefix, self.width, self.inner = prefix, int(width), int(inner)
        self.n_experts, self.top, self.activation = int(n_experts), int(top), activation
        self.shared = shared
        self.router = f"{prefix}.{router_name}"
        self.expert_names = [tuple(f"{prefix}.{expert_name.format(index=e)}.{n}" for n in names) for e in range(self.n_experts)]
        self.w_router = self.w_gate_up = self.w_down = None

    def children(self):
        return [self.shared] if self.shared is not None else []

    def param_specs(self):
        specs = [ParamSpec(self.router, (self.n_experts, self.width), "linear", "float32")]
        if self.correction_name:
            specs.append(ParamSpec(self.correction_name, (self.n_experts,), "linear", "float32"))
        for names in self.expert_names:
            specs += [ParamSpec(n, (self.inner, self.width)) for n in names[:-1]] + [ParamSpec(names[-1], (self.width, self.inner))]
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.w_router = tensors[self.router].contiguous()
        if self.correction_name:
            self.correction = tensors[self.correction_name].contiguous()
        gu, down = [], []
        self.block = 64 if self.inner % 64 == 0 else 0
        if not self.gated:
            self.block = 0
            self.w_gate_up = torch.stack([tensors.pop(up) for up, _ in self.expert_names]).contiguous()      # [experts, inner, width]
            self.w_down = torch.stack([tensors.pop(d) for _, d in self.expert_names]).contiguous()
            return
        for gate, up, d in self.expert_names:
            g, u = tensors.pop(gate), tensors.pop(up)
            if self.block:
                g, u = g.view(self.inner // 64, 64, self.width), u.view(self.inner // 64, 64, self.width)
                gu.append(torch.stack([g, u], dim=1).reshape(2 * self.inner, self.width))
            else:
                gu.append(torch.cat([g, u], dim=0))
            down.append(tensors.pop(d))
        self.w_gate_up = torch.stack(gu).contiguous()      # [experts, 2 * inner, width]
        self.w_down = torch.stack(down).contiguous()       # [experts, width, inner]

    def forward(self, x, batch=None):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, top, e = x.shape[0], self.top, self.n_experts
        ids = ws.get("moe_ids", (n, top), torch.int32)
        weights = ws.get("moe_weights", (n, top), torch.float32)
        ops.moe_route(x, self.w_router, top, ids, weights, ws.get("moe_logits", (n, e), torch.float32), scoring=self.scoring,
                      correction=self.correction, groups=self.groups, keep=self.keep_groups, route_scale=self.route_scale,
                      normalize=self.normalize)
        tap = self.ctx.tap
        if tap is not None:
            tap("moe_ids", ids)
            tap("moe_weights", weights)
        offsets = ws.get("moe_offsets", (e + 1,), torch.int32)
        pairs = ws.get("moe_sorted", (n * top,), torch.int32)
        where = ws.get("moe_where", (n * top,), torch.int32)
        ops.moe_sort(ids, e, offsets, pairs, where)
        if tap is not None:
            tap("moe_sorted", pairs)
        act = ws.get("moe_act", (n * top, self.inner), dt)
        y = ws.get("moe_expert_out", (n * top, self.width), dt)
        tensor_cores = (dt == torch.bfloat16 and ops.use_tcgen05_experts and batch is not None
                        and ops.moe_gemm_tcgen05_supported(self.w_gate_up.shape[1], self.width)
                        and ops.moe_gemm_tcgen05_supported(self.width, self.inner))
        rows = None
        if tensor_cores or self.weight_input:
            rows = ws.get("moe_rows", (n * top, self.width), dt)
            if self.weight_input:
                ops.moe_gather_scaled(x, pairs, weights, top, rows)
            else:
                ops.moe_gather(x, pairs, top, rows)
            if tap is not None:
                tap("moe_rows", rows)
        if not self.gated:
            # up product, the activation (in the tensor-core product's epilogue), down product
            if tensor_cores:
                ops.moe_gemm_tcgen05(rows, self.w_gate_up, act, offsets, batch.status, unary=self.activation)
            else:
                if rows is not None:
                    ops.moe_gemm(rows, self.w_gate_up, act, offsets)
                else:
                    ops.moe_gemm(x, self.w_gate_up, act, offsets, sorted_pairs=pairs, top=top)
                ops.unary_act(act, act, self.activation)
            if tap is not None:
                tap("moe_act", act)
            if tensor_cores:
                ops.moe_gemm_tcgen05(act, self.w_down, y, offsets, batch.status)
            else:
                ops.moe_gemm(act, self.w_down, y, offsets)
        elif tensor_cores:
            if self.block:
                ops.moe_gemm_tcgen05(rows, self.w_gate_up, act, offsets, batch.status, gated=True, activation=self.activation,
                                     args=self.activation_args)
            else:
                gu = ws.get("moe_gate_up", (n * top, 2 * self.inner), dt)
                ops.moe_gemm_tcgen05(rows, self.w_gate_up, gu, offsets, batch.status)
                if tap is not None:
                    tap("moe_gate_up", gu)
                ops.swiglu(gu, act, 0, self.activation, self.activation_args)
            if tap is not None:
                tap("moe_act", act)
            ops.moe_gemm_tcgen05(act, self.w_down, y, offsets, batch.status)
        else:
            gu = ws.get("moe_gate_up", (n * top, 2 * self.inner), dt)
            if rows is not None:
                ops.moe_gemm(rows, self.w_gate_up, gu, offsets)
            else:
                ops.moe_gemm(x, self.w_gate_up, gu, offsets, sorted_pairs=pairs, top=top)
            if tap is not None:
                tap("moe_gate_up", gu)
            ops.swiglu(gu, act, self.block, self.activation, self.activation_args)
            if tap is not None:
                tap("moe_act", act)
            ops.moe_gemm(act, self.w_down, y, offsets)
        if tap is not None:
            tap("moe_expert_out", y)
        shared = self.shared.forward(x, batch, out_name="ffn_shared_out") if self.shared is not None else None
        if tap is not None and shared is not None:
            tap("moe_shared_out", shared)
        out = ws.get("ffn_out", (n, self.width), dt)
        ops.moe_combine(y, where, None if self.weight_input else weights, shared, out)
        return out
