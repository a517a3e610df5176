"""A plain, slow implementation of the Sosuvik decoder: float64, whole sequences, no cache.

One function per mechanism, written from the design's equations in this file's own notation; it shares no code with
the package.  ``config`` is the dictionary of a config.json, ``w`` maps tensor names to float64 tensors.  With
``bf16=True`` the places where the serving path rounds (products' results and activations) are rounded to bfloat16
too, so that two bfloat16 evaluations can be compared.

Notation: T tokens, D width, H query heads, G key/value heads, d query/key size, dv value size, r latent size,
dr rotated size.
"""
import math

import torch


def rnd(x, bf16):
    return x.to(torch.bfloat16).to(torch.float64) if bf16 else x


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# ------------------------------------------------------------------------------------------------------ rotation

def frequencies(rot):
    """(f [dims / 2], m): the angle of pair i at position p is p * f[i]; cosines and sines are multiplied by m.
    Unscaled f[i] = base^(-2i / dims).  Scaled: pairs that turn more than `fast` times in `original` positions keep
    their frequency, pairs that turn less than `slow` times are slowed by `factor`, a linear ramp over the pair index
    lies between; m = 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims) if dims else i
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_that_turns(times):
        return dims * math.log(sc["original"] / (2.0 * math.pi * times)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_that_turns(sc["fast"])), 0)
    hi = min(math.ceil(pair_that_turns(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot, neighbours):
    """x [..., T, n]: the first rot.dims numbers are turned by the position's angles, the rest pass.  Pairs are
    (i, i + dims / 2), or with ``neighbours`` (2i, 2i + 1); (u, v) -> (u cos a - v sin a, v cos a + u sin a)."""
    dims = rot["dims"]
    if dims == 0:
        return x
    f, m = frequencies(rot)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(a) * m, torch.sin(a) * m
    out = x.clone()
    first = slice(0, dims, 2) if neighbours else slice(0, dims // 2)
    second = slice(1, dims, 2) if neighbours else slice(dims // 2, dims)
    u, v = x[..., first], x[..., second]
    out[..., first] = u * c - v * s
    out[..., second] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------------ mixers

def sees(T, chunk=None, start=0):
    """[T, T] bool: query i reads key j iff j <= i and, with chunks, both lie in the same chunk of positions
    (chunks counted from position 0)."""
    i = torch.arange(start, start + T).unsqueeze(1)
    j = torch.arange(start, start + T).unsqueeze(0)
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_with_sink(scores):
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)): one more term of score 0, which carries no value."""
    top = scores.max(-1, keepdim=True).values.clamp(min=0.0)
    e = torch.exp(scores - top)
    return e / (torch.exp(-top) + e.sum(-1, keepdim=True))


def chunked_attention(x, w, prefix, m, bf16=False):
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(x @ w[f"{prefix}.q"].T, bf16).view(T, H, d).transpose(0, 1)
    k = rnd(x @ w[f"{prefix}.k"].T, bf16).view(T, G, d).transpose(0, 1)
    v = rnd(x @ w[f"{prefix}.v"].T, bf16).view(T, G, dv).transpose(0, 1)
    q = rnd(rotate(q, pos, m["rot"], False), bf16)
    k = rnd(rotate(k, pos, m["rot"], False), bf16)
    k = k.repeat_interleave(H // G, dim=0)          # query head h reads key/value head h // (H / G)
    v = v.repeat_interleave(H // G, dim=0)
    s = (q @ k.transpose(1, 2)) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    s = s.masked_fill(~sees(T, (m.get("mask") or {}).get("size")), -math.inf)
    p = softmax_with_sink(s)
    o = rnd((p @ v).transpose(0, 1).reshape(T, H * dv), bf16)
    return rnd(o @ w[f"{prefix}.o"].T, bf16)


def rotated_latent_attention(x, w, prefix, m, eps, bf16=False):
    T = x.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = rnd(x @ w[f"{prefix}.q"].T, bf16).view(T, H, d + dr).transpose(0, 1)     # a head: [d that meet the latent | dr rotated]
    down = rnd(x @ w[f"{prefix}.dkv"].T, bf16)                                  # [r | dr]
    c = rnd(rms_norm(down[:, :r], w[f"{prefix}.dkv.norm"], eps), bf16)          # the latent
    shared = rnd(rotate(down[:, r:], pos, m["rot"], True), bf16)                # one rotated key part for all heads
    q_turned = rnd(rotate(q[..., d:], pos, m["rot"], True), bf16)
    k = (c @ w[f"{prefix}.uk"].T).view(T, H, d).transpose(0, 1)
    v = (c @ w[f"{prefix}.uv"].T).view(T, H, dv).transpose(0, 1)
    s = (q[..., :d] @ k.transpose(1, 2) + q_turned @ shared.T.unsqueeze(0)) * m["scale"]
    s = s.masked_fill(~sees(T), -math.inf)
    p = torch.softmax(s, dim=-1)
    o = rnd((p @ v).transpose(0, 1).reshape(T, H * dv), bf16)
    return rnd(o @ w[f"{prefix}.o"].T, bf16)


# ------------------------------------------------------------------------------------------------------ experts

def choose_experts(z, correction, router):
    """z [T, E] router logits -> (ids [T, top], weights [T, top]).  Scores s = sigmoid(z); the choice goes by s + correction
    among the experts of the `keep` best groups (a group's worth: the sum of its two largest corrected scores, or its one);
    weights = chosen s / (their sum + 1e-20) * scale."""
    E, top = router["experts"], router["top"]
    s = torch.sigmoid(z)
    c = s + correction
    groups = router.get("groups")
    if groups and groups["count"] > 1:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        worth = c.view(-1, n, per).topk(min(2, per), dim=-1).values.sum(-1)
        kept = torch.zeros_like(worth, dtype=torch.bool).scatter_(1, worth.topk(keep, dim=-1).indices, True)
        c = c.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
    ids = c.topk(top, dim=-1).indices
    chosen = s.gather(1, ids)
    return ids, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * router.get("scale", 1.0)


def choice_margin(z, correction, router):
    """[T]: how far a row's choice is from another one: the smallest of the gap between the last chosen and the first
    unchosen corrected score (among the kept groups) and the gap between the last kept and the first dropped group's worth.
    Infinite where there is nothing to choose.  (A test in reduced precision leaves rows with a small margin out.)"""
    E, top = router["experts"], router["top"]
    c = torch.sigmoid(z) + correction
    margin = torch.full((z.shape[0],), math.inf, dtype=z.dtype)
    groups = router.get("groups")
    if groups and groups["count"] > 1:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        worth = c.view(-1, n, per).topk(min(2, per), dim=-1).values.sum(-1)
        ranked = worth.sort(-1, descending=True)
        if keep < n:
            margin = ranked.values[:, keep - 1] - ranked.values[:, keep]
        kept = torch.zeros_like(worth, dtype=torch.bool).scatter_(1, ranked.indices[:, :keep], True)
        c = c.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
    ranked = c.sort(-1, descending=True).values
    if top < E:
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])     # (infinite when the next one is out)
    return margin


def clamped_expert(x, gate, up, down, limit, bf16=False):
    g = rnd(x @ gate.T, bf16).clamp(max=limit)
    u = rnd(x @ up.T, bf16).clamp(-limit, limit)
    return rnd(rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0), bf16) @ down.T, bf16)


def grouped_experts(x, w, prefix, mlp, bf16=False, margins_out=None):
    z = x @ w[f"{prefix}.router"].T
    ids, weights = choose_experts(z, w[f"{prefix}.correction"], mlp["router"])
    if margins_out is not None:
        margins_out.append(choice_margin(z, w[f"{prefix}.correction"], mlp["router"]))
    out = torch.zeros_like(x)
    for e in range(mlp["router"]["experts"]):
        rows, slot = torch.nonzero(ids == e, as_tuple=True)
        if rows.numel():
            y = clamped_expert(x[rows], w[f"{prefix}.e{e}.gate"], w[f"{prefix}.e{e}.up"], w[f"{prefix}.e{e}.down"],
                               mlp["expert"]["limit"], bf16)
            out[rows] += weights[rows, slot].unsqueeze(-1) * y
    return rnd(out, bf16)


# ------------------------------------------------------------------------------------------------------ the model

def order_of_runs(config):
    """[(layer, pass or None)]: ``pass`` is set for the first layer of a pass of the loop (where the embedding's output
    is mixed back in)."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(config, w, tokens, bf16=False, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream after every layer run;
    ``margins_out``: one that receives every routed layer run's ``choice_margin``."""
    eps = config["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    for i, t in order_of_runs(config):
        if t is not None:
            x = rnd(torch.cat([x, x0], dim=-1), bf16) @ w["loop.in"].T + w["loop.step"][t]
        layer, p = config["layers"][i], f"l{i}"
        h = rnd(rms_norm(x, w[f"{p}.norm1"], eps), bf16)
        if layer["type"] == "attention":
            total = chunked_attention(h, w, f"{p}.mix", layer["mixer"], bf16)
        elif layer["type"] == "latent_attention":
            total = rotated_latent_attention(h, w, f"{p}.mix", layer["mixer"], eps, bf16)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            h2 = rnd(rms_norm(x, w[f"{p}.norm2"], eps), bf16)
            total = total + grouped_experts(h2, w, f"{p}.mlp", layer["mlp"], bf16, margins_out)
        x = x + total
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rnd(rms_norm(x, w["final.norm"], eps), bf16)
    return x @ w["head"].T * config.get("logit_scale", 1.0)
