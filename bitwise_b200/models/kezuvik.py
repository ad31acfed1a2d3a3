"""Kezuvik assembled from parts, and its entry in the architecture registry.

A decoder whose layers carry a layer norm (a weight, no bias) before and after each sublayer, with a
constant factor on what a sublayer adds: ``x += m * norm1b(mixer(norm1(x)))``, ``x += m * norm2b(ff(norm2(
x)))`` (``SandwichBlock``; the factor rides on the later norm's weight).  Three kinds of mixer, in any order:

* ``latent_attention``: queries through a latent of their own, keys and values from one cached latent per
  position plus a rotated key part that the heads share; the rotation pairs entry i with entry i + dims / 2;
  ordinary causal softmax; a gate per entry of the heads' outputs;
* ``latent_attention_2``: the same with rescaled rotary frequencies where the configuration gives a
  rescaling, a learned sink per head in the softmax's denominator and a gate per head;
* ``attention``: grouped-query attention inside a window, with biased projections, a short causal
  convolution over time on q, k and v, q and k divided by their root mean square per head, no rotation,
  and a gate per entry.

The feed-forward is the dense gated one with the tanh form of GELU, or absent.  The head is the
embedding table after a last layer norm, and the logits are capped by ``cap * tanh(z / cap)``.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``,
``l<i>.norm2b``, ``l<i>.mix.*`` (see the mixers), ``l<i>.mlp.{gate, up, down}``.  Matrices are stored
[out, in].
"""
from __future__ import annotations

from ..config.kezuvik import KezuvikConfig
from ..config.registry import register_architecture
from ..parts.block import SandwichBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.latent_attention import LatentAttention
from ..parts.mlp import SwiGLU
from ..parts.norm import LayerNorm
from ..parts.rope import HalfRotaryEncoding, RampScaling
from ..parts.scored_attention import ScoredAttention
from .decoder import DecoderModel, LayerRun

BLOCK_NAMES = {"mixer_norm": "norm1", "mixer_post": "norm1b", "mixer": "mix", "ffn_norm": "norm2", "ffn_post": "norm2b",
               "feed_forward": "mlp"}
ROT_GAIN_COEFFICIENT = 0.1  # cos and sin of rescaled frequencies carry 0.1 * ln(factor) + 1


def build_kezuvik(config: KezuvikConfig) -> DecoderModel:
    c = config

    def norm(gain: float = 1.0):
        return LayerNorm(c.width, c.eps, suffix="", gain=gain)

    rotaries = {}   # one table per (turned entries, base, rescaling)
    blocks, schedule = [], []
    entries = 0
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        if m.latent:
            sc = m.rot_scaling
            scaling = RampScaling(sc.factor, sc.original, sc.fast, sc.slow, ROT_GAIN_COEFFICIENT) if sc is not None else None
            key = (m.rot_dims, m.rot_base, scaling.key() if scaling is not None else None)
            if key not in rotaries:
                rotaries[key] = HalfRotaryEncoding(m.rot_dims, m.rot_base, scaling)
            second = m.kind == "latent_attention_2"
            mixer = LatentAttention(c.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.scale, c.eps,
                                    position=rotaries[key], q_rank=m.q_rank, sink=second,
                                    gate="head" if second else "entry", stack_inputs=True)
        else:
            mixer = ScoredAttention(c.width, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, c.eps, conv_taps=m.conv or 0,
                                    qk_norm="unit", window=m.window, bias=True, gate="entry")
        ffn = SwiGLU(c.width, layer.ff, names=("gate", "up", "down"), suffix="", activation="gelu_tanh") if layer.ff else None
        blocks.append(SandwichBlock(c.width, mixer, ffn, norm(), norm(c.residual_mult), norm() if ffn else None,
                                    norm(c.residual_mult) if ffn else None, BLOCK_NAMES))
        cache_entry, state_entry = entries, None
        entries += 1
        if mixer.state_need() is not None:
            state_entry = entries
            entries += 1
        schedule.append(LayerRun(i, cache_entry, True, state_entry))
    embedding = TokenEmbedding(c.vocab, c.width, tensor="embed")
    head = OutputHead(c.vocab, c.width, norm(), tied_to=embedding, norm_name="final.norm", softcap=c.logit_softcap)
    return DecoderModel(c, embedding, blocks, head, schedule=schedule, position_encodings=list(rotaries.values()),
                        block_prefix="l{}", embed_prefix="")


register_architecture("Kezuvik", KezuvikConfig.from_json, build_kezuvik)
