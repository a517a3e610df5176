"""Token embedding and the output head.

h = embed_tokens.weight[ids] (src/weights.rs:203-204); logits = x . lm_head^T, or
x . embed_tokens^T when the head is tied (src/dense.rs:358-362,392-396).  Logits
come out in float32 in every run, and only for the rows that are asked for.
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, name: str, vocab: int, width: int, scale: float = 1.0, keep_rows: bool = False):
        self.name, self.vocab, self.width = name, int(vocab), int(width)
        self.scale = float(scale)   # a token's row is multiplied with this on its way into the stream (in float); a head
        self.weight = None          # tied to this table reads it unscaled
        # the embedding's output is read again later in the step (the stream itself is overwritten as layers add to it): the
        # kernel leaves the rows once more, in the compute dtype, as ``batch.per_step["embedding_rows"]``
        self.keep_rows = bool(keep_rows)

    def param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.width), "embedding")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = tensors[self.name].contiguous()

    def forward(self, ids, batch=None):
        """Rows of the table for ``ids``; where the batch says so (``from_last``) a token's id is the one the last
        step's sampling left on the device for its sequence."""
        h = self.ctx.workspace.get("residual", (ids.shape[0], self.width), torch.float32)
        rows = None
        if self.keep_rows:
            if batch is None:
                raise ValueError("an embedding that keeps its rows for later layers needs the batch to leave them with")
            rows = self.ctx.workspace.get("embedding_rows", (ids.shape[0], self.width), self.weight.dtype)
            batch.per_step["embedding_rows"] = rows
        if batch is not None and batch.last_tokens is not None:
            self.ctx.ops.embedding(ids, self.weight, h, batch.from_last, batch.seq_index, batch.slots, batch.last_tokens,
                                   scale=self.scale, rows_out=rows)
        else:
            self.ctx.ops.embedding(ids, self.weight, h, scale=self.scale, rows_out=rows)
        return h


class PositionedEmbedding(TokenEmbedding):
    """Token rows plus a learned vector per position: h[t] = table[id_t] + positions_table[p_t], p_t counted from 0
    in each sequence, added unscaled in float.  ``max_positions`` rows: the longest sequence the model takes."""

    def __init__(self, name: str, vocab: int, width: int, position_name: str, max_positions: int):
        super().__init__(name, vocab, width)
        self.position_name, self.max_positions = position_name, int(max_positions)
        self.position_table = None

    def param_specs(self):
        return super().param_specs() + [ParamSpec(self.position_name, (self.max_positions, self.width), "embedding")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.position_table = tensors[self.position_name].contiguous()

    def forward(self, ids, batch=None):
        if batch is None:
            raise ValueError("an embedding with learned positions needs the batch's positions")
        h = self.ctx.workspace.get("residual", (ids.shape[0], self.width), torch.float32)
        last = batch.last_tokens is not None
        self.ctx.ops.embedding(ids, self.weight, h, batch.from_last if last else None, batch.seq_index if last else None,
                               batch.slots if last else None, batch.last_tokens, pos_table=self.position_table,
                               positions=batch.positions)
        return h


class OutputHead(Part):
    graph_safe = True

    """``name`` of its own weight, or ``tied_to`` an embedding whose table it reads."""

    def __init__(self, vocab: int, width: int, name: str | None = None, tied_to: TokenEmbedding | None = None):
        if (name is None) == (tied_to is None):
            raise ValueError("an output head has either its own weight or a tied embedding")
        self.name, self.tied_to, self.vocab, self.width = name, tied_to, int(vocab), int(width)
        self.weight = None

    def param_specs(self):
        return [] if self.name is None else [ParamSpec(self.name, (self.vocab, self.width), "linear")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = self.tied_to.weight if self.name is None else tensors[self.name].contiguous()

    def linear_weights(self):
        return [self.weight]

    def forward(self, x, batch=None):
        logits = self.ctx.workspace.get("logits", (x.shape[0], self.vocab), torch.float32)
        self.ctx.ops.linear(x, self.weight, logits, self.ctx.workspace, batch.status if batch is not None else None)
        return logits
