"""Small Sebavik configurations for the tests, and weights for them.

The configurations differ from one another in every size and use every branch: one and several
key/value heads, value sizes unlike the key size, windows of several sizes in one model (several
page groups) and none, kept first keys that fill less than a page, more than a page and more than
the window, none kept, layers that mix their values with an earlier layer's (the first of which is
not the model's first layer) beside layers that do not, dense and routed feed-forwards and none in
any order, one expert chosen, all experts chosen, convolutions of one to five taps and none, with
and without the second embedding table and the per-layer token input, a width that is no multiple
of 8, forty query heads on one key/value head.  No two sizes of a configuration are equal by
accident (heads, experts, taps, kept keys and choices all differ).  Weights are drawn so that
scores are of order one to ten (caps bite, the softmax is far from flat, the sink and the distance
term matter) and so that clamps of the dense feed-forward are reached.
"""
import numpy as np
import torch

from bitwise_b200.config.sebavik import BigramConfig, SebavikConfig, SebavikLayerConfig, SebavikMixerConfig, SebavikMlpConfig


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, window=None, keep_first=0, v_mix=False):
    return SebavikMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap,
                              window=window, keep_first=keep_first if window else 0, v_mix=v_mix)


def dense(ff, limit):
    return SebavikMlpConfig("dense", ff, limit)


def moe(experts, top, ff):
    return SebavikMlpConfig("moe", ff, None, experts, top)


def layer(mixer, mlp=None):
    return SebavikLayerConfig(mixer, mlp)


CONFIGS = {
    # two key/value heads, values wider than keys, two windows and a layer without one, kept keys inside the
    # first page, a layer between the mixing layers that does not mix, three taps
    "a": SebavikConfig(vocab=101, width=64, eps=1e-5, residual_mult=0.5, embedding_scale=2.0,
                       bigram=BigramConfig(53, 7, 13), canon_taps=3, side_dim=6, layers=(
        layer(attention(4, 2, 16, 24, 0.3, softcap=5.0, window=20, keep_first=3), moe(5, 2, 24)),
        layer(attention(4, 2, 16, 24, 0.25, window=33, keep_first=5, v_mix=True), dense(96, 1.5)),
        layer(attention(6, 1, 8, 40, 0.4, softcap=12.0), None),
        layer(attention(8, 2, 32, 24, 0.2, softcap=9.0, window=20, keep_first=3, v_mix=True), moe(3, 3, 16)),
        layer(attention(2, 2, 16, 24, 0.3, window=7, v_mix=True), dense(40, 0.7)))),
    # odd sizes: a width that is no multiple of 8, one key/value head and as many as heads, kept keys beyond a
    # page and beyond the window, five taps, one expert chosen, no second table, no token input, factor 1
    "b": SebavikConfig(vocab=67, width=50, eps=1e-6, residual_mult=1.0, embedding_scale=1.0, canon_taps=5, layers=(
        layer(attention(3, 1, 10, 12, 0.4, softcap=30.0, window=9, keep_first=18, v_mix=True), dense(36, 2.0)),
        layer(attention(2, 2, 36, 12, 0.2, window=40, keep_first=1), moe(4, 1, 20)),
        layer(attention(5, 1, 20, 12, 0.35, softcap=4.0, v_mix=True), moe(6, 4, 12)),
        layer(attention(3, 3, 24, 28, 0.3, window=64, keep_first=17), None))),
    # forty query heads on one key/value head, a window that ends inside a key tile, one tap (a factor per
    # channel, no state), a token input of one number, large multipliers of the second table
    "c": SebavikConfig(vocab=64, width=64, eps=1e-5, residual_mult=0.25, embedding_scale=8.0,
                       bigram=BigramConfig(7, 1000003, 999983), canon_taps=1, side_dim=1, layers=(
        layer(attention(40, 1, 8, 16, 0.5, softcap=8.0, window=33, keep_first=2, v_mix=True), dense(64, 1.0)),
        layer(attention(8, 4, 32, 4, 0.2, window=130, keep_first=40), moe(2, 2, 72)),
        layer(attention(3, 1, 24, 16, 0.3, v_mix=True), None))),
}

# Combinations at the edges of what the cache manager and the blocks see: no window anywhere, no convolution
# (no state of the blocks) and no second table (no state at all), windows only, a window of one key.
EDGE_CONFIGS = {
    "no_state": SebavikConfig(vocab=50, width=32, eps=1e-5, residual_mult=0.7, embedding_scale=0.5, side_dim=4, layers=(
        layer(attention(2, 1, 16, 16, 0.3), dense(24, 1.0)), layer(attention(2, 2, 8, 8, 0.3, softcap=3.0), moe(3, 2, 8)))),
    "windows_only": SebavikConfig(vocab=50, width=32, eps=1e-5, residual_mult=0.7, embedding_scale=0.5,
                                  bigram=BigramConfig(11, 3, 5), canon_taps=2, layers=(
        layer(attention(2, 1, 16, 16, 0.3, window=1, keep_first=1, v_mix=True), dense(24, 1.0)),
        layer(attention(4, 1, 8, 16, 0.3, window=5, v_mix=True), None),
        layer(attention(2, 2, 16, 8, 0.3, softcap=2.0, window=48, keep_first=33), moe(4, 3, 8)))),
    "taps_only": SebavikConfig(vocab=50, width=40, eps=1e-5, residual_mult=1.5, embedding_scale=0.5, canon_taps=4, layers=(
        layer(attention(2, 1, 16, 16, 0.3, window=16, keep_first=16), None),
        layer(attention(1, 1, 24, 8, 0.3), dense(16, 0.5)))),
}


def random_weights(config, seed, scores=1.0):
    """name -> bfloat16 CPU tensor.  ``scores``: a factor on the query and key projections."""
    from bitwise_b200.config.registry import lookup_architecture
    g = torch.Generator().manual_seed(seed)
    specs = lookup_architecture("Sebavik").build(config).param_specs()
    out = {}
    for s in specs:
        last = s.name.rsplit(".", 1)[-1]
        rand = lambda *shape: torch.randn(shape or s.shape, generator=g)
        if last in ("canon1", "canon2"):
            t = rand() * 0.5
        elif last == "dwa":
            t = 0.3 * rand()
            t[-1] += 1.0                                   # mostly the layer's own result, some of every earlier one
        elif last == "vmix":
            t = 0.2 + 0.6 * torch.rand(s.shape, generator=g)
        elif last == "r1":
            t = 0.6 * rand()                               # either sign: far keys are pushed away or pulled near
        elif last == "r2":
            t = 0.05 + 2.0 * torch.rand(s.shape, generator=g)
        elif last == "sink":
            t = 2.0 * rand()
        elif last == "b":
            t = 0.5 * rand()
        elif last in ("ls1", "ls2") or last.startswith("norm") or s.name == "final.norm":
            t = 1.0 + 0.25 * rand()
        elif s.name in ("embed", "bigram", "side.embed"):
            t = rand()
        elif last in ("q", "k") and ".mix." in s.name:
            t = rand() * (scores * 2.0 / np.sqrt(s.shape[1]))
        elif last == "router":
            t = rand() * (3.0 / np.sqrt(s.shape[1]))       # logits well apart: no choice hangs on rounding
        else:
            t = rand() * (1.6 / np.sqrt(s.shape[1]))
        out[s.name] = t.to(torch.bfloat16)
    return out


def as_float64(weights):
    """The weights as the plain implementation reads them: name -> float64 numpy array."""
    return {n: t.to(torch.float64).numpy() for n, t in weights.items()}


def tokens(config, n, seed):
    return np.random.default_rng(seed).integers(0, config.vocab, n).tolist()
