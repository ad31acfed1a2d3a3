"""The Sebavik design in float64 on the CPU: one function per mechanism, whole sequences, no cache.

Slow and plain on purpose: it shares no code with the package and is what the package's kernels,
cache and step function are compared with.  ``cfg`` is the dictionary of config.json, ``w`` maps
tensor names to float64 (integer tables: int) numpy arrays.

Notation: a sequence has T tokens at positions 0 .. T - 1; rows of an array are positions.
"""
from __future__ import annotations

import math

import numpy as np


# What a serving precision stores between two matrix products is rounded to it; the plain implementation rounds
# nothing unless a test asks for it, to learn how large an error rounding alone causes for given weights:
# ``with rounding(fn): forward(...)`` applies ``fn`` to what every matrix product reads besides the stream (the
# normed input of a sublayer, queries, keys, values, the weighted values, the activated inner rows) and to
# nothing that the design keeps in 32-bit (norms, scores, weights of the softmax, routers, the stream).
_stored = [lambda a: a]


class rounding:
    def __init__(self, fn):
        self.fn = fn

    def __enter__(self):
        _stored.append(self.fn)

    def __exit__(self, *exc):
        _stored.pop()


def stored(a):
    return _stored[-1](a)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
    """Every row divided by sqrt(mean(row^2) + eps)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def embed_tokens(cfg, w, tokens):
    """Token rows times the scale, plus the bigram table's row of (previous token, token)."""
    e = cfg["embedding"]
    x = w["embed"][tokens] * e.get("scale", 1.0)
    b = e.get("bigram")
    if b:
        x = x + w["bigram"][pair_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x


def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """The second table's row per position: a hash of the previous and the current token, the last row at position 0."""
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets for t, tok in enumerate(tokens)]


def time_conv(h, taps_w):
    """h + conv(h), conv(h)_t = sum_j taps_w[:, j] h_(t - taps + 1 + j), zeros before position 0."""
    T = h.shape[0]
    taps = taps_w.shape[1]
    out = h.copy()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += taps_w[:, j] * h[s]
    return out


def visible(i, j, size, keep):
    """Whether position i sees position j: not later, and inside the window or among the kept first ones."""
    return j <= i and (size is None or i - j < size or j < keep)


def windowed_sink_attention(q, k, v, scale, cap, r1, r2, sink, size, keep):
    """q [T, H, D], k [T, G, D], v [T, G, V]; r1, r2, sink [H].  Returns [T, H, V].

    score(i, j) = cap * tanh(q_i . k_j * scale / cap) - r1 * ln(1 + r2 * (i - j)) over the visible j; the
    softmax's denominator holds exp(sink) besides, which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, size, keep)]
            s = (k[js, g] @ q[i, hd]) * scale
            if cap:
                s = cap * np.tanh(s / cap)
            s = s - r1[hd] * np.log1p(r2[hd] * (i - np.array(js, dtype=np.float64)))
            top = max(s.max(), sink[hd])
            e = np.exp(s - top)
            den = e.sum() + math.exp(sink[hd] - top)
            out[i, hd] = (e / den) @ v[js, g]
    return out


def mix_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def attention(m, w, p, h, v_first, first_mixing):
    """One attention mixer over the rows ``h``.  Returns (output, the values as cached)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + ".q"].T + w[p + ".q.b"]
    k = h @ w[p + ".k"].T + w[p + ".k.b"]
    v = h @ w[p + ".v"].T + w[p + ".v.b"]
    if m.get("v_mix") and not first_mixing:
        v = mix_values(v, v_first, float(w[p + ".vmix"]))
    mask = m.get("mask") or {}
    out = windowed_sink_attention(stored(q).reshape(T, H, D), stored(k).reshape(T, G, D), stored(v).reshape(T, G, V), m["scale"],
                                  m.get("softcap"), w[p + ".r1"], w[p + ".r2"], w[p + ".sink"], mask.get("size"),
                                  mask.get("keep_first", 0))
    return stored(out.reshape(T, H * V)) @ w[p + ".o"].T, v


def dense_ff(mlp, w, p, h):
    limit = mlp["limit"]
    g = np.minimum(stored(h @ w[p + ".gate"].T), limit)
    u = np.clip(stored(h @ w[p + ".up"].T), -limit, limit)
    return stored(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + ".down"].T


def route(z, top):
    """Per row: the ``top`` largest logits (the lower index on a tie) and the softmax over them."""
    chosen = np.zeros((z.shape[0], top), dtype=np.int64)
    weights = np.zeros((z.shape[0], top))
    for t in range(z.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-z[t, e], e))[:top]
        zz = z[t, order]
        e = np.exp(zz - zz.max())
        chosen[t], weights[t] = order, e / e.sum()
    return chosen, weights


def moe_ff(mlp, w, p, h):
    top = mlp["router"]["top"]
    chosen, weights = route(h @ w[p + ".router"].T, top)
    out = np.zeros((h.shape[0], w[p + ".e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            q = f"{p}.e{e}"
            a = stored(w[q + ".gate"] @ h[t])
            y = stored((a * sigmoid(a)) * stored(w[q + ".up"] @ h[t]))
            out[t] += wt * (w[q + ".down"] @ y)
    return out


def token_side(cfg, w, layer, tokens, x):
    """The per-layer token input: what is added to the stream (before the residual factor)."""
    dim = cfg["token_side"]["dim"]
    p = f"l{layer}.side"
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = stored(gelu_tanh(stored(x) @ w[p + ".gate"].T) * e)
    y = g @ w[p + ".proj"].T
    return rms_unit(y, cfg["norm"]["eps"]) * w[p + ".norm"]


def depth_average(history, a):
    """sum_j a[j] * history[j] over everything so far: the embedding's output and every layer's result."""
    return sum(float(a[j]) * history[j] for j in range(len(history)))


def forward(cfg, w, tokens, collect=None):
    """Logits [T, vocab] of one sequence.  ``collect``: a list that receives the stream after every layer."""
    tokens = list(tokens)
    eps = cfg["norm"]["eps"]
    mult = cfg.get("residual_mult", 1.0)
    canon = cfg.get("canon")
    x = embed_tokens(cfg, w, tokens)
    history = [x]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = rms_norm(x, w[p + ".norm1"], eps)
        if canon:
            h = time_conv(h, w[p + ".canon1"])
        h = stored(h)
        m = layer["mixer"]
        y, v = attention(m, w, p + ".mix", h, v_first, v_first is None)
        if m.get("v_mix") and v_first is None:
            v_first = v
        x = x + mult * (y * w[p + ".ls1"])
        if layer.get("mlp"):
            h = rms_norm(x, w[p + ".norm2"], eps)
            if canon:
                h = time_conv(h, w[p + ".canon2"])
            h = stored(h)
            mlp = layer["mlp"]
            y = dense_ff(mlp, w, p + ".mlp", h) if mlp["kind"] == "dense" else moe_ff(mlp, w, p + ".mlp", h)
            x = x + mult * (y * w[p + ".ls2"])
        if cfg.get("token_side"):
            x = x + mult * token_side(cfg, w, i, tokens, x)
        history.append(x)
        x = depth_average(history, w[p + ".dwa"])
        if collect is not None:
            collect.append(x)
    x = stored(rms_norm(x, w["final.norm"], eps))
    return x @ w["embed"].T
