"""Grouped-query attention over the paged cache.

q, k, v projections -> per-head RMSNorm of q and k (optional) -> rotation of q
and k -> keys and values into the request's pages -> softmax(scale q k^T + causal
mask [+ window]) v -> output projection (src/dense.rs:139-270).  Query head i
reads kv head i // (heads / kv_heads); scale = head_dim^-0.5 unless given.  The
three projections are one matrix product over the concatenated weights
[q; k; v]; each output row is the same dot product as with separate weights.
With ``bias`` the projections take ``<prefix>.bias`` tensors, added to the rounded
product as the reference does (src/weights.rs:96,198-200); the output
projection's is optional in a checkpoint.
"""
from __future__ import annotations

import torch

from .base import CacheSpec, Mixer, ParamSpec


class AttentionMixer(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, head_dim: int, position,
                 qk_norm_eps: float | None = None, window: int = 0, scale: float | None = None,
                 bias: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.prefix, self.width = prefix, int(width)
        self.heads, self.kv_heads, self.head_dim = int(heads), int(kv_heads), int(head_dim)
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = int(window)
        self.scale = (float(scale) if scale is not None else self.head_dim ** -0.5) * float(getattr(position, "score_scale", 1.0))
        self.bias = bool(bias)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.b_qkv = self.b_o = None

    def children(self):
        return [self.position]

    def cache_spec(self):
        return CacheSpec("paged", kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def graph_key(self, shape):
        # the one launch shape of a decode step that follows the lengths: into how many blocks the keys are split
        return (self.ctx.ops.decode_attention_splits(shape.n_seqs, self.kv_heads, self.head_dim, self.heads // self.kv_heads,
                                                     shape.max_seq_len, self.ctx.dtype),)

    def param_specs(self):
        p, hd = self.prefix, self.head_dim
        specs = [ParamSpec(f"{p}.q_proj.weight", (self.heads * hd, self.width)),
                 ParamSpec(f"{p}.k_proj.weight", (self.kv_heads * hd, self.width)),
                 ParamSpec(f"{p}.v_proj.weight", (self.kv_heads * hd, self.width)),
                 ParamSpec(f"{p}.o_proj.weight", (self.width, self.heads * hd))]
        if self.qk_norm_eps is not None:
            specs += [ParamSpec(f"{p}.q_norm.weight", (hd,), "norm", "float32"),
                      ParamSpec(f"{p}.k_norm.weight", (hd,), "norm", "float32")]
        if self.bias:
            specs += [ParamSpec(f"{p}.q_proj.bias", (self.heads * hd,), "linear", "float32"),
                      ParamSpec(f"{p}.k_proj.bias", (self.kv_heads * hd,), "linear", "float32"),
                      ParamSpec(f"{p}.v_proj.bias", (self.kv_heads * hd,), "linear", "float32"),
                      ParamSpec(f"{p}.o_proj.bias", (self.width,), "linear", "float32", optional=True)]
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        p = self.prefix
        self.w_qkv = torch.cat([tensors.pop(f"{p}.q_proj.weight"), tensors.pop(f"{p}.k_proj.weight"),
                                tensors.pop(f"{p}.v_proj.weight")], dim=0).contiguous()
        self.w_o = tensors[f"{p}.o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[f"{p}.q_norm.weight"].contiguous()
            self.k_norm = tensors[f"{p}.k_norm.weight"].contiguous()
        if self.bias:
            self.b_qkv = torch.cat([tensors.pop(f"{p}.q_proj.bias"), tensors.pop(f"{p}.k_proj.bias"),
                                    tensors.pop(f"{p}.v_proj.bias")]).contiguous()
            self.b_o = tensors.get(f"{p}.o_proj.bias")

    def linear_weights(self):
        return [self.w_qkv, self.w_o]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n = x.shape[0]
        nq, nkv, hd = self.heads, self.kv_heads, self.head_dim
        q = ws.get("q_rot", (n, nq * hd), dt)
        angles = self.position.angles(batch)
        projection = None
        qkv = ws.get("qkv", (n, (nq + 2 * nkv) * hd), dt)
        ops.linear(x, self.w_qkv, qkv, ws, batch.status)
        if self.b_qkv is not None:
            ops.add_bias(qkv, self.b_qkv)
        tap = self.ctx.tap
        if tap is not None:
            tap("qkv", qkv)
        if ops.decode_takes_projection(batch, dt, hd, nq // nkv, cache.page_size, self.position.rotary_dim, angles):
            # decoding: the attention kernel norms, rotates and stores its own token while it waits for its keys
            projection = (qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, angles, not cache.read_only)
        else:
            ops.qk_rope_cache(qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, self.position.inv_freq,
                              self.position.rotary_dim, batch.positions, batch.seq_index, cache.block_table,
                              cache.page_size, cache.k_pool, cache.v_pool, q, nq, nkv, hd, not cache.read_only,
                              batch.status, angles)
        if tap is not None and projection is None:
            tap("q_rot", q)
        o = ws.get("attn_out", (n, nq * hd), dt)
        ops.attention(q, cache.k_pool, cache.v_pool, batch, cache.block_table, cache.page_size, o, nq, nkv, hd,
                      cache.window, self.scale, ws, projection=projection)
        if tap is not None:
            tap("attn_out", o)
        y = ws.get("mixer_out", (n, self.width), dt)
        ops.linear(o, self.w_o, y, ws, batch.status)
        if self.b_o is not None:
            ops.add_bias(y, self.b_o)
        return y


class GatedAttentionMixer(Mixer):
    """Grouped-query attention with the options some designs add to it, each a parameter:

    ``dim`` / ``vdim``: query/key and value heads of different sizes (the cache's heads take the larger, the rest is zeros);
    ``whole_norm_eps``: q and k are RMS-normed over the WHOLE projection, all heads at once, with weights of the
        projection's size, before they are split into heads and rotated (None: no norm);
    ``sink``: the softmax's denominator has one more term, exp(0): p_j = exp(s_j) / (1 + sum_j exp(s_j)), a key that every
        query may give weight to and that has no value;
    ``gate``: the concatenated heads are multiplied with sigmoid(W_g x), number by number, before the output product;
    ``scale``: of the scores; ``position``: the rotation (over the first ``rotary_dim`` numbers of a head, halves paired);
    ``softcap`` > 0: a scaled score s becomes softcap * tanh(s / softcap) before the softmax;
    ``chunk`` > 0: positions form chunks of that many, counted from the sequence's start, and a query at position i reads
        key j <= i only if floor(i / chunk) = floor(j / chunk) (whatever way the prompt was cut into steps);
    ``bias``: q, k and v take a bias each (the tensor's name with ``.b`` added), added to the product in float;
    ``head_norm_eps``: every q and k head is RMS-normed over its own ``dim`` numbers, with ONE weight of ``dim`` numbers
        for all heads (tensors ``q.norm``, ``k.norm``), before the rotation (None: no such norm);
    ``sink="learned"``: the sink's score is a learned number a head (tensor ``sink``) instead of 0; it is not scaled or capped;
    ``value_position``: a second rotation, over all ``vdim`` numbers of a value head: a value is cached turned by its own
        position, and a head's result (the weighted sum of such values) is turned back by the query's position;
    ``head_pad``: the cache's head size is the next one the tensor-core attention kernels are built for (16, 32, 64, 96,
        128) instead of max(dim, vdim); the padding is zeros.

    The four products that read the layer's input (q, k, v, gate) are one product over stacked weights.
    """

    graph_safe = True
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, position, scale: float,
                 whole_norm_eps: float | None = None, sink: bool = False, gate: bool = False, window: int = 0,
                 names: dict | None = None, out_name: str = "mixer_out", softcap: float = 0.0, chunk: int = 0, bias: bool = False,
                 head_norm_eps: float | None = None, value_position=None, head_pad: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if whole_norm_eps is not None and head_norm_eps is not None:
            raise ValueError("q and k are normed over the whole projection or head by head, not both")
        if value_position is not None and (value_position.rotary_dim != vdim or vdim % 2):
            raise ValueError("the values' rotation is over all of an even number of value numbers")
        self.prefix, self.width = prefix, int(width)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.head_dim = max(self.dim, self.vdim)     # of the cache, of q as the attention kernels read it, and of their output
        if head_pad:
            self.head_dim = next((s for s in (16, 32, 64, 96, 128) if s >= self.head_dim), self.head_dim)
        self.bias, self.head_norm_eps, self.value_position = bool(bias), head_norm_eps, value_position
        # the options that the general split kernel takes (the whole-projection kernel takes none of them)
        self.by_heads = self.bias or head_norm_eps is not None or value_position is not None or bool(getattr(position, "interleaved", False))
        self.position = position
        self.scale = float(scale) * float(getattr(position, "score_scale", 1.0))
        if sink not in (False, True, "learned"):
            raise ValueError("sink is False, True (a score of 0) or 'learned'")
        self.learned_sink = sink == "learned"
        self.whole_norm_eps, self.sink, self.gate, self.window = whole_norm_eps, bool(sink), bool(gate), int(window)
        self.softcap, self.chunk = float(softcap), int(chunk)
        if self.softcap < 0 or self.chunk < 0:
            raise ValueError("softcap and chunk are positive, or 0 for none")
        self.names = {k: f"{prefix}.{v}" for k, v in {**self.NAMES, **(names or {})}.items()}
        self.out_name = out_name
        self.q_norm = self.k_norm = self.sinks = None

    def children(self):
        return [self.position] + ([self.value_position] if self.value_position is not None else [])

    def cache_spec(self):
        return CacheSpec("paged", kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def graph_key(self, shape):
        return (self.ctx.ops.decode_attention_splits(shape.n_seqs, self.kv_heads, self.head_dim, self.heads // self.kv_heads,
                                                     shape.max_seq_len, self.ctx.dtype, self.chunk),)

    def param_specs(self):
        n, qd, kd = self.names, self.heads * self.dim, self.kv_heads * self.dim
        specs = [ParamSpec(n["q"], (qd, self.width)), ParamSpec(n["k"], (kd, self.width)),
                 ParamSpec(n["v"], (self.kv_heads * self.vdim, self.width)), ParamSpec(n["o"], (self.width, self.heads * self.vdim))]
        if self.whole_norm_eps is not None:
            specs += [ParamSpec(n["q_norm"], (qd,), "norm", "float32"), ParamSpec(n["k_norm"], (kd,), "norm", "float32")]
        if self.head_norm_eps is not None:
            specs += [ParamSpec(n["q_norm"], (self.dim,), "norm", "float32"), ParamSpec(n["k_norm"], (self.dim,), "norm", "float32")]
        if self.bias:
            specs += [ParamSpec(n["q"] + ".b", (qd,), "linear", "float32"), ParamSpec(n["k"] + ".b", (kd,), "linear", "float32"),
                      ParamSpec(n["v"] + ".b", (self.kv_heads * self.vdim,), "linear", "float32")]
        if self.learned_sink:
            specs.append(ParamSpec(n["sink"], (self.heads,), "linear", "float32"))
        if self.gate:
            specs.append(ParamSpec(n["g"], (self.heads * self.vdim, self.width)))
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        n = self.names
        stack = [tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"])] + ([tensors.pop(n["g"])] if self.gate else [])
        self.w_in = torch.cat(stack, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.whole_norm_eps is not None or self.head_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()
        self.b_in = None
        if self.bias:
            self.b_in = torch.cat([tensors.pop(n["q"] + ".b"), tensors.pop(n["k"] + ".b"), tensors.pop(n["v"] + ".b")]).contiguous()
        if self.learned_sink:
            self.sinks = tensors[n["sink"]].contiguous()
        elif self.sink:
            self.sinks = torch.zeros(self.heads, dtype=torch.float32, device=ctx.device)

    def linear_weights(self):
        return [self.w_in, self.w_o]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, nq, nkv, hd = x.shape[0], self.heads, self.kv_heads, self.head_dim
        proj = ws.get("qkvg", (n, self.w_in.shape[0]), dt)
        ops.linear(x, self.w_in, proj, ws, batch.status)
        tap = self.ctx.tap
        if tap is not None:
            tap("qkv", proj)
        q = ws.get("q_rot", (n, nq * hd), dt)
        turned = self.value_position.angles(batch) if self.value_position is not None else None
        if self.by_heads:
            qkv = proj if not self.gate else proj[:, :(nq + nkv) * self.dim + nkv * self.vdim]
            ops.heads_rope_cache(qkv, self.b_in, self.q_norm, self.k_norm, self.head_norm_eps or 0.0, self.position.angles(batch),
                                 self.position.rotary_dim, bool(getattr(self.position, "interleaved", False)), turned,
                                 bool(getattr(self.value_position, "interleaved", False)), batch.positions, batch.seq_index,
                                 cache.block_table, cache.page_size, cache.k_pool, cache.v_pool, q, nq, nkv, self.dim, self.vdim, hd,
                                 not cache.read_only, batch.status)
        else:
            ops.qk_whole_norm_rope_cache(proj, self.q_norm, self.k_norm, self.whole_norm_eps or 0.0, self.position.inv_freq,
                                         self.position.rotary_dim, batch.positions, batch.seq_index, cache.block_table, cache.page_size,
                                         cache.k_pool, cache.v_pool, q, nq, nkv, self.dim, self.vdim, hd, not cache.read_only,
                                         batch.status, self.position.angles(batch))
        if tap is not None:
            tap("q_rot", q)
        o = ws.get("attn_out", (n, nq * hd), dt)
        ops.attention(q, cache.k_pool, cache.v_pool, batch, cache.block_table, cache.page_size, o, nq, nkv, hd, cache.window,
                      self.scale, ws, sinks=self.sinks, chunk=self.chunk, softcap=self.softcap)
        if tap is not None:
            tap("attn_out", o)
        if turned is not None:
            # every head's sum of values that were turned by their own positions is turned back by the query's (and narrowed)
            back = ws.get("attn_turned_back", (n, nq * self.vdim), dt)
            ops.unrotate_heads(o, turned, bool(getattr(self.value_position, "interleaved", False)), back, nq, self.vdim, hd)
            o, hd = back, self.vdim
            if tap is not None:
                tap("attn_turned_back", o)
        if self.gate:
            gated = o if hd == self.vdim else ws.get("attn_gated", (n, nq * self.vdim), dt)
            ops.sigmoid_gate(o, hd, proj[:, (nq + nkv) * self.dim + nkv * self.vdim:], gated, nq, self.vdim)
            o = gated
            if tap is not None:
                tap("attn_gated", o)
        elif hd != self.vdim:
            # (a copy into a buffer of its own: with one head, reshape would hand the product a view with gaps between rows)
            narrow = ws.get("attn_narrow", (n, nq * self.vdim), dt)
            narrow.view(n, nq, self.vdim).copy_(o.view(n, nq, hd)[:, :, :self.vdim])
            o = narrow
        y = ws.get(self.out_name, (n, self.width), dt)
        ops.linear(o, self.w_o, y, ws, batch.status)
        if tap is not None:
            tap("attn_proj", y)
        return y


class TalkingAttentionMixer(Mixer):
    """Grouped-query attention whose scaled scores are mixed over the heads before the softmax ("talking heads"):
    s'_h = sum_g talk[h, g] s_g with a learned ``talk`` [heads, heads]; causal (or a window), ordinary softmax.  q, k and v
    may take biases; q and k are rotated over the first ``rotary_dim`` numbers of a head as ``position`` says (neighbours or
    halves paired); query/key heads of ``dim`` and value heads of ``vdim`` numbers.  A token's row of scores needs all
    heads' scores of the same key, so this mixer has attention kernels of its own (``csrc/kernels/attention_talk.cu``)."""

    graph_safe = True
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "talk": "talk"}

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, position, scale: float,
                 bias: bool = False, window: int = 0, names: dict | None = None, out_name: str = "mixer_out"):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if heads > 32:
            raise ValueError("scores are mixed over at most 32 heads")
        self.prefix, self.width = prefix, int(width)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        # of the cache and of q as the kernels read it: the larger of the two sizes, padded with zeros to the next multiple of 16
        # (what the tensor-core kernel takes)
        self.head_dim = -(-max(self.dim, self.vdim) // 16) * 16
        self.position, self.scale = position, float(scale) * float(getattr(position, "score_scale", 1.0))
        self.bias, self.window = bool(bias), int(window)
        self.names = {k: f"{prefix}.{v}" for k, v in {**self.NAMES, **(names or {})}.items()}
        self.out_name = out_name

    def children(self):
        return [self.position]

    def cache_spec(self):
        return CacheSpec("paged", kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def graph_key(self, shape):
        # the one launch shape of a decode step that follows the lengths: into how many blocks the keys are split
        return (self.ctx.ops.talk_splits(shape.n_seqs, shape.max_seq_len, self.window),)

    def param_specs(self):
        n, qd, kd, vd = self.names, self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        specs = [ParamSpec(n["q"], (qd, self.width)), ParamSpec(n["k"], (kd, self.width)), ParamSpec(n["v"], (vd, self.width)),
                 ParamSpec(n["o"], (self.width, self.heads * self.vdim)),
                 ParamSpec(n["talk"], (self.heads, self.heads), "linear", "float32")]
        if self.bias:
            specs += [ParamSpec(n["q"] + ".b", (qd,), "linear", "float32"), ParamSpec(n["k"] + ".b", (kd,), "linear", "float32"),
                      ParamSpec(n["v"] + ".b", (vd,), "linear", "float32")]
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        n = self.names
        self.w_in = torch.cat([tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"])], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.talk = tensors[n["talk"]].contiguous()
        self.b_in = None
        if self.bias:
            self.b_in = torch.cat([tensors.pop(n["q"] + ".b"), tensors.pop(n["k"] + ".b"), tensors.pop(n["v"] + ".b")]).contiguous()

    def linear_weights(self):
        return [self.w_in, self.w_o]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, nq, nkv, hd = x.shape[0], self.heads, self.kv_heads, self.head_dim
        proj = ws.get("qkv", (n, self.w_in.shape[0]), dt)
        ops.linear(x, self.w_in, proj, ws, batch.status)
        tap = self.ctx.tap
        if tap is not None:
            tap("qkv", proj)
        q = ws.get("q_rot", (n, nq * hd), dt)
        ops.heads_rope_cache(proj, self.b_in, None, None, 0.0, self.position.angles(batch), self.position.rotary_dim,
                             bool(getattr(self.position, "interleaved", False)), None, False, batch.positions, batch.seq_index,
                             cache.block_table, cache.page_size, cache.k_pool, cache.v_pool, q, nq, nkv, self.dim, self.vdim, hd,
                             not cache.read_only, batch.status)
        if tap is not None:
            tap("q_rot", q)
        o = ws.get("attn_out", (n, nq * self.vdim), dt)
        ops.attention_talk(q, cache.k_pool, cache.v_pool, self.talk, batch, cache.block_table, cache.page_size, o, nq, nkv, hd,
                           self.dim, self.vdim, cache.window, self.scale, ws)
        if tap is not None:
            tap("attn_out", o)
        y = ws.get(self.out_name, (n, self.width), dt)
        ops.linear(o, self.w_o, y, ws, batch.status)
        if tap is not None:
            tap("attn_proj", y)
        return y
