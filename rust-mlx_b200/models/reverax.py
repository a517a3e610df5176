"""The Reverax decoder put together from parts.

Token embedding; layers x <- x + (s1 * mixer(norm1(x)) + s2 * ff(norm2(x))) with two norms of the same stream, each a
norm in groups (the row in equal consecutive parts, each over its own root mean square), and two learned vectors s1, s2
that scale the mixer's and the feed-forward's results number by number.  A mixer is either attention whose scores are
mixed over the heads before the softmax (biases, neighbours rotated over part of a head), or two mixers side by side on
the same input: windowed attention (biases, q and k normed head by head with one weight, halves rotated, values turned
by their own position and the result turned back, capped scores, a learned sink a head) beside linear attention with a
learned decay and a bonus for the current token, whose projections read mixes of the token's and the previous token's
input.  A feed-forward is gated and dense, or routed experts without a gate (squared relu) that read the row times its
sigmoid score, or absent.  A layer may use an earlier layer's tensors with caches and states of its own: the schedule
then names that layer's block again with new cache ids.  A last norm, the embedding's table as the head, logits times a
factor.  Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.mix.*``,
``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.reverax import ReveraxConfig
from ..parts.attention import GatedAttentionMixer, TalkingAttentionMixer
from ..parts.base import LayerCall
from ..parts.block import ParallelBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.feedforward import SwiGLUFeedForward
from ..parts.norm import GroupRMSNorm
from ..parts.position import RotaryEmbedding
from ..parts.recurrent import DecayLinearMixer, ParallelMixer
from ..parts.routed import RoutedFeedForward
from ..registry import register_architecture
from .spec import ModelSpec


def _mixer(prefix: str, c: ReveraxConfig, layer, index: int):
    m = layer.mixer
    if layer.type == "attention":
        position = RotaryEmbedding(m.dim, m.rot.base, rotary_dim=m.rot.dims, interleaved=True)
        return TalkingAttentionMixer(prefix, c.width, m.heads, m.kv_heads, m.dim, m.vdim, position, m.scale, bias=True)
    a, r = m.left, m.right
    if r.rank <= 0:
        raise ValueError(f"layers[{index}].mixer.right: the decay's inner size is not known: neither config.json ('rank') nor a "
                         f"checkpoint's '{prefix}.right.w1' gives it")
    left = GatedAttentionMixer(f"{prefix}.left", c.width, a.heads, a.kv_heads, a.dim, a.vdim,
                               RotaryEmbedding(a.dim, a.rot.base, rotary_dim=a.rot.dims), a.scale, sink="learned", window=a.window,
                               softcap=a.softcap, bias=True, head_norm_eps=c.eps,
                               value_position=RotaryEmbedding(a.vdim, a.rot.base, rotary_dim=a.vdim), head_pad=True,
                               out_name="left_out")
    right = DecayLinearMixer(f"{prefix}.right", c.width, r.heads, r.dim, r.rank, c.eps, out_name="right_out")
    return ParallelMixer(left, right, m.left_scale, m.right_scale)


def _feed_forward(prefix: str, width: int, f):
    if f is None:
        return None
    if f.kind == "dense":
        return SwiGLUFeedForward(prefix, width, f.ff, activation="silu", names=("gate", "up", "down"))
    return RoutedFeedForward(prefix, width, f.ff, f.experts, f.top, activation="relu2", names=("up", "down"), scoring="sigmoid",
                             normalize=False, gated=False, weight_input=True)


def build_reverax(config: ReveraxConfig) -> ModelSpec:
    c = config
    embedding = TokenEmbedding("embed", c.vocab, c.width)
    blocks, block_of = [], {}
    for i, layer in enumerate(c.layers):
        if layer.weights_of is not None:
            continue
        ffn = _feed_forward(f"l{i}.mlp", c.width, layer.mlp)
        block_of[i] = len(blocks)
        blocks.append(ParallelBlock(GroupRMSNorm(f"l{i}.norm1", c.width, c.eps, c.norm_groups), _mixer(f"l{i}.mix", c, layer, i), ffn,
                                    norm2=GroupRMSNorm(f"l{i}.norm2", c.width, c.eps, c.norm_groups) if ffn is not None else None,
                                    mixer_scale=f"l{i}.ls1", ffn_scale=f"l{i}.ls2" if ffn is not None else None, width=c.width))
    # every layer of the configuration is a run of its owner's block with caches of its own
    schedule, next_cache = [], 0
    for i in range(len(c.layers)):
        block = blocks[block_of[c.owner(i)]]
        count = len(block.cache_specs())
        ids = tuple(range(next_cache, next_cache + count))
        next_cache += count
        schedule.append(LayerCall(block_of[c.owner(i)], ids[0] if count == 1 else ids))
    spec = ModelSpec(config=c, embedding=embedding, blocks=blocks, schedule=schedule,
                     final_norm=GroupRMSNorm("final.norm", c.width, c.eps, c.norm_groups, out_scale=c.logit_scale),
                     head=OutputHead(c.vocab, c.width, tied_to=embedding), vocab_size=c.vocab, eos_token_ids=tuple(c.eos_token_id))
    spec.check_schedule()
    return spec


register_architecture("Reverax", ReveraxConfig, build_reverax, model_types=("reverax",))
