"""Small Kezuvik configurations for the tests, and weights for them.

The configurations differ from one another in every size and in the order of their layers: widths that
are no multiple of 8, one head and many, windows shorter and longer than a page and than the prompts,
convolutions of one to five taps or none, rotated parts of which only some entries turn, rescaled rotary
frequencies whose ramp covers all, some or none of the pairs, a layer without feed-forward, a model
without a cap on the logits or with a residual factor of one.  Weights are drawn so that scores, gates and
activations are of order one (the softmax is far from flat, sinks and gates matter).
"""
import numpy as np
import torch

from bitwise_b200.config.kezuvik import KezuvikConfig, KezuvikLayerConfig, KezuvikMixerConfig, RotScalingConfig


def latent(kind="latent_attention", heads=3, dim=16, rot_dim=8, vdim=16, kv_rank=40, q_rank=24, scale=0.2, base=10000.0,
           dims=None, scaling=None):
    return KezuvikMixerConfig(kind, heads, dim, vdim, scale, rot_dim=rot_dim, kv_rank=kv_rank, q_rank=q_rank, rot_base=base,
                              rot_dims=dims if dims is not None else rot_dim, rot_scaling=scaling)


def window(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, conv=3, size=20):
    return KezuvikMixerConfig("attention", heads, dim, vdim, scale, kv_heads=kv_heads, conv=conv, window=size)


L = KezuvikLayerConfig

CONFIGS = {
    # all three mixers; the tensor-core kernels take these shapes on the serving precision
    "a": KezuvikConfig(vocab=131, width=64, eps=1e-5, residual_mult=0.6, logit_softcap=12.0, layers=(
        L(window(heads=4, kv_heads=2, dim=32, vdim=16, scale=0.7, conv=3, size=24), 96),
        L(latent("latent_attention_2", heads=2, dim=16, rot_dim=16, vdim=24, kv_rank=48, q_rank=40, scale=0.17, base=5000.0,
                 scaling=RotScalingConfig(4.0, 64.0, 8.0, 0.5)), 80),
        L(latent(heads=5, dim=16, rot_dim=8, vdim=16, kv_rank=40, q_rank=24, scale=0.21, base=200000.0), 96),
        L(window(heads=2, kv_heads=1, dim=16, vdim=32, scale=0.9, conv=5, size=7), None))),
    # odd sizes everywhere, one head, only part of the rotated entries turn, a window of one page exactly, one tap
    # (a factor per channel, no state), no cap, a residual factor of one, a latent layer without feed-forward
    "b": KezuvikConfig(vocab=97, width=50, eps=1e-6, residual_mult=1.0, logit_softcap=None, layers=(
        L(latent(heads=1, dim=10, rot_dim=6, vdim=7, kv_rank=33, q_rank=9, scale=0.3, base=100.0, dims=4), 36),
        L(window(heads=3, kv_heads=3, dim=10, vdim=6, scale=1.1, conv=1, size=16), 28),
        L(latent("latent_attention_2", heads=3, dim=6, rot_dim=10, vdim=12, kv_rank=70, q_rank=19, scale=0.25, base=777.0,
                 scaling=RotScalingConfig(1.5, 32.0, 4.0, 2.0)), None),
        L(window(heads=6, kv_heads=2, dim=12, vdim=10, scale=0.8, conv=2, size=33), 20))),
    # the second latent kind without a rescaling, the first with one; a window longer than any prompt of the tests; no
    # convolution; many heads; value size 1 (a gate per entry and a gate per head are then the same shape)
    "c": KezuvikConfig(vocab=64, width=48, eps=1e-5, residual_mult=0.35, logit_softcap=3.0, layers=(
        L(latent("latent_attention_2", heads=4, dim=8, rot_dim=4, vdim=1, kv_rank=24, q_rank=16, scale=0.35, base=50.0), 40),
        L(latent(heads=12, dim=8, rot_dim=8, vdim=4, kv_rank=136, q_rank=8, scale=0.3, base=10000.0,
                 scaling=RotScalingConfig(8.0, 16.0, 1.0, 0.25)), 24),
        L(window(heads=8, kv_heads=1, dim=8, vdim=8, scale=1.3, conv=None, size=500), 24))),
}


def random_weights(config, seed, std=None):
    """name -> bfloat16 CPU tensor."""
    from bitwise_b200.config.registry import lookup_architecture
    g = torch.Generator().manual_seed(seed)
    specs = lookup_architecture("Kezuvik").build(config).param_specs()
    out = {}
    for s in specs:
        if s.name.endswith(".sink"):
            t = torch.randn(s.shape, generator=g) * 1.5 + 1.0
        elif s.name.endswith(".b"):
            t = torch.randn(s.shape, generator=g) * 0.5
        elif s.name.endswith(".conv"):
            t = torch.randn(s.shape, generator=g) * 0.6
        elif len(s.shape) == 1:
            t = 1.0 + 0.2 * torch.randn(s.shape, generator=g)
        elif s.name == "embed":
            t = torch.randn(s.shape, generator=g)
        else:
            t = torch.randn(s.shape, generator=g) * (std or 1.6 / np.sqrt(s.shape[1]))
        out[s.name] = t.to(torch.bfloat16)
    return out


def tokens(config, n, seed):
    return np.random.default_rng(seed).integers(0, config.vocab, n).tolist()
