"""The Kezuvik design stated plainly: whole sequences, no cache, no batching, float64 on the CPU.

One function per mechanism, written from the design's equations and sharing nothing with the
package: the tests compare the package's kernels, cache and scheduler with these.

Notation: x is [tokens, width]; a weight W is stored [out, in] and applied as ``x @ W.T``; ``w``
is a dict name -> tensor; ``cfg`` is the model's config.json as a dict.

* layer norm without bias: ``(x - mean) / sqrt(var + eps) * g`` (var = mean of squared deviations)
* root-mean-square norm: ``x / sqrt(mean(x^2) + eps)`` (times a weight where there is one)
* rotation, half layout: entry i of a vector is paired with entry i + dims / 2; the pair at position
  p turns by ``p * f_i``; with a rescaling of the frequencies, low frequencies are divided by a
  factor, a ramp blends between, and cos and sin carry a constant gain
* latent attention: keys and values of all heads are made from one latent vector per token plus one
  rotated key part that every head shares; queries pass a latent of their own
* window attention with biased projections, a causal convolution over time on q, k and v and unit
  norms per head of q and k
* an output gate from the mixer's input on the heads' outputs, per entry or per head
* a layer is ``x += m * post1(mixer(pre1(x)))``, ``x += m * post2(ff(pre2(x)))``, all four layer norms
* the logits are capped by ``cap * tanh(z / cap)``
"""
import contextlib
import math

import torch

F64 = torch.float64

_ROUND = None


@contextlib.contextmanager
def rounding(fn):
    """Inside the block, what the serving precision stores in 16 bits between its kernels (the sublayers' inputs,
    projections, cached vectors, the heads' outputs) is passed through ``fn``: the plain result then shows how large
    an error rounding alone causes."""
    global _ROUND
    _ROUND, old = fn, _ROUND
    try:
        yield
    finally:
        _ROUND = old


def stored(x):
    return _ROUND(x) if _ROUND is not None else x


def layer_norm(x, g, eps):
    mean = x.mean(-1, keepdim=True)
    d = x - mean
    var = (d * d).mean(-1, keepdim=True)
    return d / torch.sqrt(var + eps) * g


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """The angle per position of every pair, and the gain on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turns_to_index(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_index(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns_to_index(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(v, positions, rot):
    """v: [tokens, ..., n]; of the first ``dims`` entries, i and i + dims / 2 turn together; the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    f, gain = rotary_frequencies(rot)
    out = v.clone()
    p = torch.as_tensor(positions, dtype=F64).reshape((-1,) + (1,) * (v.dim() - 1))
    for i in range(half):
        a = p * f[i]
        c, s = (torch.cos(a) * gain)[..., 0], (torch.sin(a) * gain)[..., 0]
        u, t = v[..., i], v[..., i + half]
        out[..., i] = u * c - t * s
        out[..., i + half] = t * c + u * s
    return out


def causal_conv(u, taps_w):
    """u: [tokens, channels]; taps_w: [channels, taps]; y_t = sum_j w[:, j] u_(t - taps + 1 + j)."""
    n, taps = u.shape[0], taps_w.shape[1]
    y = torch.zeros_like(u)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    return y


def softmax_rows(scores, visible, sink=None):
    """scores, visible: [heads, tokens, tokens]; sink: [heads] logits joining the denominator, or None."""
    s = scores.masked_fill(~visible, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.reshape(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.reshape(-1, 1, 1) - m)
    return e / den


def latent_mixer(h, w, pre, m, eps, positions, second):
    """``second``: the kind with rescaled frequencies, a sink per head and a gate per head."""
    n = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = stored(unit_rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"])
    q = stored(cq @ w[pre + "uq"].T).reshape(n, H, dim + rd)
    d = h @ w[pre + "dkv"].T
    c = stored(unit_rms(d[:, :rank], eps) * w[pre + "dkv.norm"])
    k_rot = stored(rotate_half(d[:, rank:], positions, m["rot"]))
    q_rot = stored(rotate_half(q[:, :, dim:], positions, m["rot"]))
    k = (c @ w[pre + "uk"].T).reshape(n, H, dim)
    v = (c @ w[pre + "uv"].T).reshape(n, H, vd)
    scores = (torch.einsum("ihd,jhd->hij", q[:, :, :dim], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    pos = torch.as_tensor(positions)
    visible = (pos[None, :] <= pos[:, None])[None].expand(H, n, n)
    p = softmax_rows(scores, visible, w[pre + "sink"] if second else None)
    o = torch.einsum("hij,jhd->ihd", p, v)
    g = torch.sigmoid(h @ w[pre + "g"].T)
    o = stored(stored(o) * (g[:, :, None] if second else g.reshape(n, H, vd)))
    return o.reshape(n, H * vd) @ w[pre + "o"].T


def window_mixer(h, w, pre, m, eps, positions):
    n = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def project(name):
        u = h @ w[pre + name].T + w[pre + name + ".b"]
        return causal_conv(u, w[pre + name + ".conv"]) if m.get("conv") else u

    q = stored(unit_rms(project("q").reshape(n, H, dim), eps))
    k = stored(unit_rms(project("k").reshape(n, G, dim), eps))
    v = stored(project("v").reshape(n, G, vd))
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    pos = torch.as_tensor(positions)
    dist = pos[:, None] - pos[None, :]
    visible = dist >= 0
    if m.get("mask"):
        visible = visible & (dist < m["mask"]["size"])
    p = softmax_rows(scores, visible[None].expand(H, n, n))
    o = stored(torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * vd))
    return stored(o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    return stored(gelu_tanh(stored(h @ w[pre + "gate"].T)) * stored(h @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [tokens, vocab] of one whole sequence; ``layers_out``: a list that receives the stream after
    every layer."""
    w = {k: v.to(F64) for k, v in weights.items() if v.dtype != torch.int32}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    positions = list(range(len(tokens)))
    x = w["embed"][torch.as_tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = stored(layer_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "attention":
            y = window_mixer(h, w, p + "mix.", layer["mixer"], eps, positions)
        else:
            y = latent_mixer(h, w, p + "mix.", layer["mixer"], eps, positions, layer["type"] == "latent_attention_2")
        x = x + mult * layer_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            y = dense_ff(stored(layer_norm(x, w[p + "norm2"], eps)), w, p + "mlp.")
            x = x + mult * layer_norm(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    z = stored(layer_norm(x, w["final.norm"], eps)) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
