"""A plain, slow implementation of the Reverax decoder: float64, whole sequences, no cache.

One function per mechanism, written from the design's equations in this file's own notation; it shares no code with
the package.  ``config`` is the dictionary of a config.json, ``w`` maps tensor names to float64 tensors.  With
``bf16=True`` the places where the serving path rounds (products' results and activations) are rounded to bfloat16
too, so that two bfloat16 evaluations can be compared.

Notation: T tokens, D width, H query heads, G key/value heads, d query/key size, dv value size.
"""
import math

import torch


def rnd(x, bf16):
    return x.to(torch.bfloat16).to(torch.float64) if bf16 else x


def rms(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, weight, eps, groups):
    """The row in ``groups`` equal consecutive parts, each over its own root mean square; then times the weight."""
    t, d = x.shape
    return rms(x.reshape(t, groups, d // groups), eps).reshape(t, d) * weight


def turn(x, positions, base, dims, neighbours, sign=1.0):
    """x [T, heads, n]: the first ``dims`` numbers of a head are turned by sign * position * base^(-2i/dims); pairs are
    (i, i + dims/2), or with ``neighbours`` (2i, 2i + 1); (u, v) -> (u cos a - v sin a, v cos a + u sin a)."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    a = sign * positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    first = slice(0, dims, 2) if neighbours else slice(0, dims // 2)
    second = slice(1, dims, 2) if neighbours else slice(dims // 2, dims)
    out = x.clone()
    u, v = x[..., first], x[..., second]
    out[..., first] = u * c - v * s
    out[..., second] = v * c + u * s
    return out


def project(h, w, name, bf16, bias=True):
    y = h @ w[name].T
    if bias:
        y = rnd(y, bf16) + w[name + ".b"]
    return rnd(y, bf16)


def visible(t, window):
    """[T, T] bool: query i (rows) reads key j (columns) when j <= i and, with a window, i - j < window."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    ok = j <= i
    if window:
        ok &= (i - j) < window
    return ok


# ------------------------------------------------------------------------------------------------- attention mixers

def talking_attention(h, w, p, m, bf16):
    """Grouped-query attention, neighbours rotated, whose scaled scores are mixed over the heads before the softmax:
    s'_h = sum_g talk[h, g] s_g."""
    t = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    q = turn(project(h, w, f"{p}.q", bf16).reshape(t, H, d), pos, m["rot"]["base"], m["rot"]["dims"], True)
    k = turn(project(h, w, f"{p}.k", bf16).reshape(t, G, d), pos, m["rot"]["base"], m["rot"]["dims"], True)
    v = project(h, w, f"{p}.v", bf16).reshape(t, G, dv)
    q, k = rnd(q, bf16), rnd(k, bf16)
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("ihc,jhc->hij", q, k[:, kv_of]) * m["scale"]
    s = torch.einsum("hg,gij->hij", w[f"{p}.talk"], s)
    s = s.masked_fill(~visible(t, 0), -math.inf)
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhc->ihc", a, v[:, kv_of])
    return rnd(rnd(o, bf16).reshape(t, H * dv) @ w[f"{p}.o"].T, bf16)


def windowed_attention(h, w, p, m, eps, bf16):
    """Grouped-query attention with normed q and k (one weight for all heads), halves rotated, values turned by their
    own position and the result turned back by the query's, capped scores, a window, and a learned sink a head in the
    softmax's denominator."""
    t = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    pos = torch.arange(t)
    q = rms(project(h, w, f"{p}.q", bf16).reshape(t, H, d), eps) * w[f"{p}.q.norm"]
    k = rms(project(h, w, f"{p}.k", bf16).reshape(t, G, d), eps) * w[f"{p}.k.norm"]
    q, k = rnd(turn(q, pos, base, dims, False), bf16), rnd(turn(k, pos, base, dims, False), bf16)
    v = rnd(turn(project(h, w, f"{p}.v", bf16).reshape(t, G, dv), pos, base, dv, False), bf16)
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("ihc,jhc->hij", q, k[:, kv_of]) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    window = (m.get("mask") or {}).get("size", 0)
    s = s.masked_fill(~visible(t, window), -math.inf)
    sink = w[f"{p}.sink"][:, None, None].expand(H, t, 1)
    a = torch.softmax(torch.cat([s, sink], dim=-1), dim=-1)[..., :t]
    o = torch.einsum("hij,jhc->ihc", a, v[:, kv_of])
    o = turn(o, pos, base, dv, False, sign=-1.0)
    return rnd(rnd(o, bf16).reshape(t, H * dv) @ w[f"{p}.o"].T, bf16)


def time_mix(h, w, p, m, eps, bf16, state_out=None):
    """Linear attention with a decay a head and channel and a bonus for the current token:
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,  S_t = diag(w_t) S_(t-1) + k_t v_t^T,  S_0 = 0,
    every projection reading its own mix of the token's and the previous token's input."""
    t, D = h.shape
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, D, dtype=h.dtype), h[:-1]], dim=0)

    def mixed(s):
        return rnd(h + (before - h) * w[f"{p}.mu.{s}"], bf16)
    r = project(mixed("r"), w, f"{p}.r", bf16, bias=False).reshape(t, H, d)
    k = project(mixed("k"), w, f"{p}.k", bf16, bias=False).reshape(t, H, d)
    v = project(mixed("v"), w, f"{p}.v", bf16, bias=False).reshape(t, H, d)
    g = project(mixed("g"), w, f"{p}.g", bf16, bias=False)
    gate = rnd(g * torch.sigmoid(g), bf16)
    low = rnd(torch.tanh(project(mixed("w"), w, f"{p}.w1", bf16, bias=False)), bf16)
    decay = torch.exp(-torch.exp(project(low, w, f"{p}.w2", bf16, bias=False) + w[f"{p}.w0"])).reshape(t, H, d)
    u = w[f"{p}.u"]
    S = torch.zeros(H, d, d, dtype=torch.float64)
    o = torch.zeros(t, H, d, dtype=torch.float64)
    for i in range(t):
        kv = k[i, :, :, None] * v[i, :, None, :]
        o[i] = torch.einsum("hc,hce->he", r[i], S + u[:, :, None] * kv)
        S = decay[i, :, :, None] * S + kv
    if state_out is not None:
        state_out.append(S)
    y = rms(o, eps).reshape(t, H * d) * w[f"{p}.norm"] * gate
    return rnd(rnd(y, bf16) @ w[f"{p}.o"].T, bf16)


# ------------------------------------------------------------------------------------------------- feed-forwards

def gated_dense(h, w, p, bf16):
    g = rnd(h @ w[f"{p}.gate"].T, bf16)
    u = rnd(h @ w[f"{p}.up"].T, bf16)
    return rnd(rnd(g * torch.sigmoid(g) * u, bf16) @ w[f"{p}.down"].T, bf16)


def squared_relu_experts(h, w, p, mlp, bf16, margins_out=None):
    """Scores sigmoid(router h); every row takes its ``top`` best experts; a chosen expert reads score * h and
    computes down(relu(up x)^2); the experts' results are added."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ w[f"{p}.router"].T)
    best, ids = torch.sort(s, dim=-1, descending=True, stable=True)
    if margins_out is not None:
        margins_out.append(best[:, top - 1] - best[:, top] if top < n else torch.full((h.shape[0],), math.inf, dtype=s.dtype))
    out = torch.zeros_like(h)
    for e in range(n):
        rows, place = torch.nonzero(ids[:, :top] == e, as_tuple=True)
        if rows.numel():
            x = rnd(best[rows, place, None] * h[rows], bf16)
            a = rnd(torch.relu(rnd(x @ w[f"{p}.e{e}.up"].T, bf16)) ** 2, bf16)
            out[rows] += rnd(a @ w[f"{p}.e{e}.down"].T, bf16)
    return rnd(out, bf16)


# ------------------------------------------------------------------------------------------------- the model

def forward(config, w, tokens, bf16=False, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream after every layer;
    ``margins_out``: one that receives, for every routed layer, each row's distance between the last chosen and the
    first refused score."""
    eps, groups = config["norm"]["eps"], config["norm"].get("groups", 1)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}"
        h = rnd(group_norm(x, w[f"{p}.norm1"], eps, groups), bf16)
        m = layer["mixer"]
        if layer["type"] == "attention":
            a = talking_attention(h, w, f"{p}.mix", m, bf16)
        elif layer["type"] == "parallel":
            a = (m["left_scale"] * windowed_attention(h, w, f"{p}.mix.left", m["left"], eps, bf16)
                 + m["right_scale"] * time_mix(h, w, f"{p}.mix.right", m["right"], eps, bf16))
        else:
            raise ValueError(layer["type"])
        total = a * w[f"{p}.ls1"]
        mlp = layer.get("mlp")
        if mlp:
            h2 = rnd(group_norm(x, w[f"{p}.norm2"], eps, groups), bf16)
            f = gated_dense(h2, w, f"{p}.mlp", bf16) if mlp["kind"] == "dense" else squared_relu_experts(h2, w, f"{p}.mlp", mlp, bf16, margins_out)
            total = total + f * w[f"{p}.ls2"]
        x = x + total
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rnd(group_norm(x, w["final.norm"], eps, groups), bf16)
    return x @ w["embed"].T * config.get("logit_scale", 1.0)
