"""Attention through a cached latent, without positions.

    c_q = RMSNorm(W_dq x)          q_h = W_uq,h c_q                      (heads h, ``dim`` numbers each)
    c   = RMSNorm(W_dkv x)         k_h = W_uk,h c,   v_h = W_uv,h c      (``vdim`` numbers a value)
    s_h[i, j] = scale * q_h[i] . k_h[j]      over the keys j <= i of the window (i - j < window; 0: all)
    o_h = softmax(s_h) v_h * sigmoid(W_g x)_h        y = W_o [o_1 .. o_H]

Only c is kept per token (``kv_rank`` numbers in one pool of pages: ``CacheSpec(values=False)``).  Keys and
values are never formed: since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, the query is carried into the latent's space
(one small product a head), attention runs there with c as key and as value of every head (one kv head of
size kv_rank: the framework's attention kernels, with the same pool as keys and values), and W_uv,h is applied
to the result.  A step's work then follows the latents it reads, not heads * head size.

The three products that read x (W_dq, W_dkv, W_g) are one product over the stacked weights.  A mixer built with
``own_latent=False`` has no W_dkv: its schedule entry names the cache of the layer whose latents it reads, with its
own W_uk, W_uv, queries and window.

Options, each a parameter:
``q_rank=0``: no query latent; q = W_q x straight from the layer's input (tensor ``q``).
``rot_dim`` > 0 with a ``position``: a query head is [dim numbers that meet the latent | rot_dim rotated numbers], W_dkv has
    kv_rank + rot_dim rows, and the last rot_dim of them (not normed) are one rotated key part that all heads share:
        s_h[i, j] = scale * (q_h[i, :dim] . k_h[j] + rot(q_h[i, dim:]) . rot(kr[j]))
    The page row of a token is then [c | rot(kr) | zeros], padded to a head size the attention kernels take; a query row is
    [W_uk,h^T q_h[:dim] | rot(q_h[dim:]) | zeros], so the score is still one dot product a key, and the values are the
    row's first kv_rank numbers.
``gated=False``: no output gate.
"""
from __future__ import annotations

import torch

from .base import CacheSpec, Mixer, ParamSpec


class LatentAttentionMixer(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, eps: float,
                 scale: float | None = None, window: int = 0, cache_window: int | None = None, own_latent: bool = True,
                 gated: bool = True, rot_dim: int = 0, position=None):
        self.prefix, self.width = prefix, int(width)
        self.rot_dim, self.position = int(rot_dim), position
        if self.rot_dim and (position is None or position.rotary_dim != self.rot_dim):
            raise ValueError("a rotated part needs a position encoding that rotates exactly that part")
        if self.rot_dim and not own_latent:
            raise ValueError("a mixer with a rotated key part keeps its own latents")
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(scale) if scale is not None else self.dim ** -0.5
        self.window = int(window)
        # how long the cache keeps a latent: the widest window of the layers that read it (0: for ever)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.own_latent, self.gated = bool(own_latent), bool(gated)
        # numbers of a page row: the latent alone, or [latent | rotated key part] padded with zeros to a head size that
        # the tensor-core attention kernels take (beyond those sizes: to a multiple of 16)
        self.row = self.kv_rank
        if self.rot_dim:
            need = self.kv_rank + self.rot_dim
            self.row = next((s for s in (16, 32, 64, 96, 128) if s >= need), -(-need // 16) * 16)

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_spec(self):
        return CacheSpec("paged", kv_heads=1, head_dim=self.row, window=self.cache_window, values=False)

    def heads_a_call(self) -> int:
        """How many heads one attention launch takes: all of them share the one latent "kv head", and the kernels take
        groups of up to 16 query heads (the tensor-core kernels by their tiles; the FMA kernel runs a warp a head and
        has registers for 16 of them in a block).  More heads go in several launches over the same latents."""
        return min(self.heads, 16)

    def graph_key(self, shape):
        return (self.ctx.ops.decode_attention_splits(shape.n_seqs, 1, self.row, self.heads_a_call(), shape.max_seq_len,
                                                     self.ctx.dtype),)

    def param_specs(self):
        p = self.prefix
        qd = self.heads * (self.dim + self.rot_dim)
        if self.q_rank:
            specs = [ParamSpec(f"{p}.dq", (self.q_rank, self.width)),
                     ParamSpec(f"{p}.dq.norm", (self.q_rank,), "norm", "float32"),
                     ParamSpec(f"{p}.uq", (qd, self.q_rank))]
        else:
            specs = [ParamSpec(f"{p}.q", (qd, self.width))]
        if self.own_latent:
            specs += [ParamSpec(f"{p}.dkv", (self.kv_rank + self.rot_dim, self.width)),
                      ParamSpec(f"{p}.dkv.norm", (self.kv_rank,), "norm", "float32")]
        specs += [ParamSpec(f"{p}.uk", (self.heads * self.dim, self.kv_rank)),
                  ParamSpec(f"{p}.uv", (self.heads * self.vdim, self.kv_rank))]
        if self.gated:
            specs.append(ParamSpec(f"{p}.g", (self.heads, self.width)))
        specs.append(ParamSpec(f"{p}.o", (self.width, self.heads * self.vdim)))
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        p = self.prefix
        down = [tensors.pop(f"{p}.dq" if self.q_rank else f"{p}.q")]
        if self.own_latent:
            down.append(tensors.pop(f"{p}.dkv"))
            self.kv_norm = tensors[f"{p}.dkv.norm"].contiguous()
        else:
            self.kv_norm = None
        if self.gated:
            down.append(tensors.pop(f"{p}.g"))
        self.w_down = torch.cat(down, dim=0).contiguous()          # rows: [query latent, or queries | key/value latent (| key part) | gates]
        self.q_norm = tensors[f"{p}.dq.norm"].contiguous() if self.q_rank else None
        self.w_uq = tensors[f"{p}.uq"].contiguous() if self.q_rank else None
        # W_uk,h^T: [heads, kv_rank, dim], the matrix that carries head h's query into the latent's space
        self.w_uk_t = tensors.pop(f"{p}.uk").view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors.pop(f"{p}.uv").view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()

    def linear_weights(self):
        return [w for w in (self.w_down, self.w_uq, self.w_o) if w is not None]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, H, r, rot, row = x.shape[0], self.heads, self.kv_rank, self.rot_dim, self.row
        qh = self.dim + rot                      # numbers of a query head
        tap = self.ctx.tap
        kv = (r + rot) if self.own_latent else 0
        proj = ws.get("latent_down", (n, self.w_down.shape[0]), dt)
        ops.linear(x, self.w_down, proj, ws, batch.status)
        if tap is not None:
            tap("latent_down", proj)
        write = self.own_latent and not cache.read_only
        first = self.q_rank if self.q_rank else H * qh      # columns of proj before the key/value latent's
        if self.q_rank:
            cq = ws.get("latent_q", (n, self.q_rank), dt)
            # (with a rotated part the latent goes into its page together with that part, below)
            ops.latent_norms(proj, self.q_rank, kv if not rot else 0, self.q_norm, self.kv_norm, self.eps, cq,
                             cache.k_pool if write and not rot else None, batch.positions, batch.seq_index, cache.block_table,
                             cache.page_size, batch.status)
            if tap is not None:
                tap("latent_q", cq)
            q = ws.get("q_heads", (n, H * qh), dt)
            ops.linear(cq, self.w_uq, q, ws, batch.status)
            q = q.view(n, H, qh)
        else:
            q = proj[:, :first].unflatten(1, (H, qh))
        if tap is not None:
            tap("q_heads", q.reshape(n, H * qh))
        q_lat = ws.get("q_rot", (n, H * row), dt)
        ops.linear_heads(q[:, :, :self.dim], self.w_uk_t, q_lat.view(n, H, row)[:, :, :r])
        if rot:
            ops.latent_rope(proj[:, first:first + kv], r, rot, self.position.interleaved, self.kv_norm,
                            self.eps, q, self.dim, H, q_lat, row, self.position.angles(batch), cache.k_pool if write else None,
                            batch.positions, batch.seq_index, cache.block_table, cache.page_size, batch.status)
        if tap is not None:
            tap("q_latent", q_lat)
        o_lat = ws.get("attn_out", (n, H * row), dt)
        step = self.heads_a_call()
        if step >= H:
            ops.attention(q_lat, cache.k_pool, cache.k_pool, batch, cache.block_table, cache.page_size, o_lat, H, 1, row,
                          self.window, self.scale, ws)
        else:
            for h0 in range(0, H, step):
                hc = min(step, H - h0)
                q_part = ws.get("q_rot_part", (n, hc * row), dt)
                o_part = ws.get("attn_out_part", (n, hc * row), dt)
                q_part.view(n, hc, row).copy_(q_lat.view(n, H, row)[:, h0:h0 + hc])
                ops.attention(q_part, cache.k_pool, cache.k_pool, batch, cache.block_table, cache.page_size, o_part, hc, 1, row,
                              self.window, self.scale, ws)
                o_lat.view(n, H, row)[:, h0:h0 + hc].copy_(o_part.view(n, hc, row))
        if tap is not None:
            tap("attn_out", o_lat)
        o = ws.get("attn_heads", (n, H * self.vdim), dt)
        ops.linear_heads(o_lat.view(n, H, row)[:, :, :r], self.w_uv, o.view(n, H, self.vdim))
        if tap is not None:
            tap("attn_values", o)
        if self.gated:
            ops.gate_heads(o, proj[:, first + kv:], H, self.vdim)
        if tap is not None:
            tap("attn_heads", o)
        y = ws.get("mixer_out", (n, self.width), dt)
        ops.linear(o, self.w_o, y, ws, batch.status)
        return y
