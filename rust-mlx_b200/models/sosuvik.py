"""The Sosuvik decoder put together from parts.

Token embedding; layers with two RMS norms of the same stream, one feeding the mixer and one a feed-forward of routed
experts, whose outputs are added to the stream together: x <- x + (mixer(norm1(x)) + ff(norm2(x))).  A mixer is either
grouped-query attention (rotation over part of a head with scaled frequencies, scores through softcap * tanh(s / softcap),
a query reading only its own chunk of positions, a sink of score 0 in the softmax's denominator) or attention through a
cached latent with one rotated key part that all heads share (neighbouring numbers paired).  The experts clamp their gate
and up numbers and are chosen by sigmoid scores with a correction, among the best groups of experts.  A run of layers may
loop: it runs several times in a row with the same weights, every pass with caches of its own and behind a ``LoopEntry``
that mixes the embedding's output back into the stream.  A last RMS norm, an output head of its own, logits times a factor.
Tensors: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.sosuvik import SosuvikConfig
from ..parts.attention import GatedAttentionMixer
from ..parts.base import LayerCall
from ..parts.block import ParallelBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.latent_attention import LatentAttentionMixer
from ..parts.loop import LoopEntry
from ..parts.norm import RMSNorm
from ..parts.position import RotaryEmbedding
from ..parts.routed import RoutedFeedForward
from ..registry import register_architecture
from .spec import ModelSpec

SWISH_ALPHA = 1.702     # the experts' g * sigmoid(alpha * g): fixed by the design


def _mixer(prefix: str, c: SosuvikConfig, layer):
    m = layer.mixer
    if layer.type == "attention":
        position = RotaryEmbedding(m.dim, m.rot.base, rotary_dim=m.rot.dims, scaling=m.rot.scaling_dict(), factor_on="rotated")
        return GatedAttentionMixer(prefix, c.width, m.heads, m.kv_heads, m.dim, m.vdim, position, m.scale, sink=True,
                                   softcap=m.softcap, chunk=m.chunk)
    position = RotaryEmbedding(m.rot_dim, m.rot.base, rotary_dim=m.rot_dim, scaling=m.rot.scaling_dict(), factor_on="rotated",
                               interleaved=True)
    return LatentAttentionMixer(prefix, c.width, m.heads, m.dim, m.vdim, 0, m.kv_rank, c.eps, scale=m.scale, gated=False,
                                rot_dim=m.rot_dim, position=position if m.rot_dim else None)


def _feed_forward(prefix: str, width: int, f):
    if f is None:
        return None
    return RoutedFeedForward(prefix, width, f.ff, f.experts, f.top, activation="swish_clamp", activation_args=(f.limit, SWISH_ALPHA),
                             scoring="sigmoid", correction_name="correction", groups=f.groups, keep_groups=f.keep,
                             route_scale=f.scale)


def build_sosuvik(config: SosuvikConfig) -> ModelSpec:
    c = config
    embedding = TokenEmbedding("embed", c.vocab, c.width, keep_rows=c.loop is not None)
    blocks = []
    for i, layer in enumerate(c.layers):
        ffn = _feed_forward(f"l{i}.mlp", c.width, layer.mlp)
        blocks.append(ParallelBlock(RMSNorm(f"l{i}.norm1", c.width, c.eps), _mixer(f"l{i}.mix", c, layer), ffn,
                                    norm2=RMSNorm(f"l{i}.norm2", c.width, c.eps) if ffn is not None else None))
    # the order of the runs: layers before the loop, the loop's passes (each behind its entry, each with caches of its
    # own), the layers after it
    schedule, next_cache = [], 0

    def run(i):
        nonlocal next_cache
        schedule.append(LayerCall(i, next_cache))
        next_cache += 1
    if c.loop is None:
        for i in range(len(c.layers)):
            run(i)
    else:
        lp = c.loop
        for i in range(lp.start):
            run(i)
        first = None
        for t in range(lp.times):
            entry = LoopEntry("loop.in", "loop.step", c.width, lp.times, t, owner=first)
            first = first or entry
            blocks.append(entry)
            schedule.append(LayerCall(len(blocks) - 1, None))
            for i in range(lp.start, lp.stop):
                run(i)
        for i in range(lp.stop, len(c.layers)):
            run(i)
    spec = ModelSpec(config=c, embedding=embedding, blocks=blocks, schedule=schedule,
                     final_norm=RMSNorm("final.norm", c.width, c.eps, out_scale=c.logit_scale),
                     head=OutputHead(c.vocab, c.width, name="head"), vocab_size=c.vocab, eos_token_ids=tuple(c.eos_token_id))
    spec.check_schedule()
    return spec


register_architecture("Sosuvik", SosuvikConfig, build_sosuvik, model_types=("sosuvik",))
