"""Sebavik assembled from parts, and its entry in the architecture registry.

A decoder of pre-norm blocks whose sublayers' outputs enter the stream through a stored scale per
channel and one constant factor (``ScaledResidualBlock``).  What a sublayer reads is its normed input
plus a short causal convolution of it over time; after the feed-forward every layer adds a gated
projection of a small per-token vector (``TokenSide``); what a layer hands on is a weighted sum of the
embedding's output and all layers' results so far (``DepthMix``).  The embedding adds a row of a second
table chosen by a hash of the previous and the current token.  The mixer is grouped-query softmax
attention without rotation (``ScoredAttention``): biased projections, capped scores, a learned
logarithmic penalty on distance, a window beside which the sequence's first positions stay visible, a
learned sink in the softmax's denominator, and values mixed with those of the first such layer.  The
feed-forward is a clamped gated one, or a routed one whose weights are the softmax over the chosen
logits; it may be absent.  The head is the embedding table.

Tensor names: ``embed``, ``bigram``, ``side.embed``, ``final.norm`` and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.canon1``, ``l<i>.canon2``, ``l<i>.dwa``,
``l<i>.side.{gate, proj, norm}``, ``l<i>.mix.*`` and ``l<i>.mlp.*``.  Matrices are stored [out, in].
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sebavik import SebavikConfig
from ..parts.block import DepthMix, ScaledResidualBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.norm import RMSNorm
from ..parts.routed_ffn import ClampedGLU, RoutedFFN
from ..parts.scored_attention import ScoredAttention
from ..parts.token_side import TokenSide, TokenSideTable
from .decoder import DecoderModel, LayerRun

BLOCK_NAMES = {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "feed_forward": "mlp", "scale_1": "ls1",
               "scale_2": "ls2", "conv_1": "canon1", "conv_2": "canon2", "side": "side"}
GLU_ALPHA = 1.702  # the dense feed-forward's sigmoid: g * sigmoid(1.702 g) * (u + 1)


def build_sebavik(config: SebavikConfig) -> DecoderModel:
    c = config
    layers = len(c.layers)
    table = TokenSideTable(c.vocab, layers, c.side_dim) if c.side_dim else None
    blocks, schedule = [], []
    entries = 0
    mixing_seen = False
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        value_mix = None
        if m.v_mix:
            value_mix = "mix" if mixing_seen else "source"
            mixing_seen = True
        mixer = ScoredAttention(c.width, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, c.eps, softcap=m.softcap,
                                sink="learned", window=m.window, keep_first=m.keep_first, bias=True, distance_log=True,
                                value_mix=value_mix)
        ffn = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ffn = ClampedGLU(c.width, layer.mlp.ff, layer.mlp.limit, GLU_ALPHA)
        elif layer.mlp is not None:
            ffn = RoutedFFN(c.width, layer.mlp.experts, layer.mlp.top, layer.mlp.ff, 0.0, 0.0, correction=False,
                            scoring="softmax_top", activation="silu")
        side = TokenSide(c.width, table, i, c.eps) if table is not None else None
        block = ScaledResidualBlock(c.width, mixer, ffn, RMSNorm(c.width, c.eps, suffix=""),
                                    RMSNorm(c.width, c.eps, suffix="") if ffn is not None else None, BLOCK_NAMES,
                                    mult=c.residual_mult, layer_scale=True, taps=c.canon_taps, side=side,
                                    depth=DepthMix(i, layers))
        blocks.append(block)
        cache_entry = entries
        entries += 1
        state_entry = None
        if block.state_need() is not None:
            state_entry = entries
            entries += 1
        schedule.append(LayerRun(i, cache_entry, True, state_entry))
    b = c.bigram
    embedding = TokenEmbedding(c.vocab, c.width, tensor="embed", scale=c.embedding_scale,
                               pair_table="bigram" if b is not None else None, pair_buckets=b.buckets if b else 0,
                               pair_mul_prev=b.mul_prev if b else 0, pair_mul_cur=b.mul_cur if b else 0)
    head = OutputHead(c.vocab, c.width, RMSNorm(c.width, c.eps, suffix=""), tied_to=embedding, norm_name="final.norm")
    # a checkpoint may carry the tensors of what a layer's configuration leaves out: the norm, scale and
    # convolution of an absent feed-forward, the mixing factor of a layer that does not mix its values
    unused = set()
    for i, layer in enumerate(c.layers):
        if layer.mlp is None:
            unused.update(f"l{i}.{BLOCK_NAMES[k]}" for k in ("ffn_norm", "scale_2", "conv_2"))
        if not layer.mixer.v_mix:
            unused.add(f"l{i}.{BLOCK_NAMES['mixer']}.{ScoredAttention.NAMES['vmix']}")
    return DecoderModel(c, embedding, blocks, head, schedule=schedule, block_prefix="l{}", embed_prefix="",
                        shared_parts=[table] if table is not None else [], ignorable=unused.__contains__)


register_architecture("Sebavik", SebavikConfig.from_json, build_sebavik)
