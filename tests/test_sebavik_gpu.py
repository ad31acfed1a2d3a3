"""Sebavik on the device against the plain implementation (tests/plain_sebavik.py).

Each mechanism alone (the embedding with its second table and the previous token across steps,
the norm with the convolution over time and its state, biased projections with mixed values on
their way into the pages, attention with cap, logarithmic distance term, learned sink, window and
kept first keys, the clamped and the routed feed-forward, the token input with the depth average),
with inputs made so that a key far away, a key at a window's edge, a kept first key or the sink
decides the result; then whole models of several shapes in both precisions, the same requests cut
in every way (whole, token by token, portions down to two tokens, mixed batches over a pool whose
pages and slots are used again), long decoding, and greedy generation through the engine and its
scheduler and through the command line.
"""
import math

import numpy as np
import pytest
import torch

import plain_sebavik as P
import replay_patterns as R
from sebavik_configs import CONFIGS, EDGE_CONFIGS, as_float64, random_weights, tokens

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}   # relative to the largest reference value
SEQ = 1 << 20                                  # the tile height that lists whole sequences


def ops_of(dtype):
    from bitwise_b200.kernels.ops import get_ops
    return get_ops(dtype)


def act(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def f64(t):
    return t.detach().to(torch.float64).cpu().numpy()


def close(got, want, dtype, what="", factor=1.0):
    got = f64(got) if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: {got.shape} against {want.shape}"
    err = float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
    assert err <= TOL[dtype] * factor, f"{what}: relative error {err:.3g}"


class Batch:
    """What the kernels read of a step: rows of sequences, their tokens, positions, slots and tiles."""

    def __init__(self, seqs, slots=None, toks=None):
        # seqs: list of (first position, rows); one block-table row each
        pos, row_seq, seq_pos0, seq_row0 = [], [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(seqs):
            seq_pos0.append(p0), seq_row0.append(r)
            pos += list(range(p0, p0 + cnt))
            row_seq += [s] * cnt
            r += cnt
        self.i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.n, self.seqs = r, seqs
        self.pos, self.row_seq = self.i32(pos), self.i32(row_seq)
        self.seq_pos0, self.seq_row0 = self.i32(seq_pos0), self.i32(seq_row0 + [r])
        self.seq_slot = self.i32(list(slots) if slots is not None else list(range(len(seqs))))
        self.tokens = self.i32(list(toks)) if toks is not None else None
        self.max_keys = max(pos) + 1

    def query_tiles(self, tile_rows):
        t_seq, t_row0, t_rows = [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(self.seqs):
            for a in range(0, cnt, tile_rows):
                t_seq.append(s), t_row0.append(r + a), t_rows.append(min(tile_rows, cnt - a))
            r += cnt
        return self.i32(t_seq), self.i32(t_row0), self.i32(t_rows), len(t_seq)


def pages_in_no_order(seqs, total, page, g):
    """A block table [seqs, blocks] over a pool of ``total`` pages handed out in no order."""
    blocks = (max(p0 + cnt for p0, cnt in seqs) + page - 1) // page
    perm = torch.randperm(total, generator=g)[:len(seqs) * blocks]
    return perm.to(torch.int32).reshape(len(seqs), blocks).to(DEV)


def fill_pages(seq_tensors, table, page, kv_heads, size, dtype):
    cache = torch.zeros(int(table.max()) + 2, kv_heads, page, size, dtype=act(dtype), device=DEV)
    for s, t in enumerate(seq_tensors):
        idx = torch.arange(t.shape[0])
        cache[table[s].long()[idx // page], :, idx % page, :] = t.to(act(dtype)).to(DEV)
    return cache


def in_portions(total, cuts, rest):
    """Row counts of two sequences per step until both have ``total`` rows: ``cuts``, then ``rest`` again and again."""
    at, cuts, out = [0, 0], list(cuts), []
    while at[0] < total or at[1] < total:
        c = cuts.pop(0) if cuts else rest
        step = []
        for s in range(2):
            n = min(c[s], total - at[s])
            if n:
                step.append((s, at[s], n))
                at[s] += n
        if step:
            out.append(step)
    return out


CUTS = [(1, 0), (1, 0), (2, 3), (1, 1), (6, 2), (2, 1), (1, 9), (7, 1), (3, 2)]   # sequence 1 begins at the third step


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab,buckets,mul_prev,mul_cur,scale", [(50, 30, 7, 3, 5, 0.5), (264, 300, 509, 37, 11, 1.0),
                                                                       (64, 1000, 1, 1000003, 999983, 8.0),
                                                                       (1500, 5000, 9973, 2000003, 3, 0.25)])
def test_embedding_with_second_table_and_previous_token_across_steps(dtype, width, vocab, buckets, mul_prev, mul_cur, scale):
    """Two sequences in portions through dirty slots: a portion's first row finds its previous token in the slot."""
    ops = ops_of(dtype)
    T = 29
    g = torch.Generator().manual_seed(width)
    table = torch.randn(vocab, width, generator=g).to(act(dtype))
    pair = torch.randn(buckets + 1, width, generator=g).to(act(dtype))
    seq_toks = [torch.randint(0, vocab, (T,), generator=g).tolist() for _ in range(2)]
    seq_toks[0][:3] = [vocab - 1, vocab - 1, vocab - 1]       # the largest products of the hash
    want = [f64(table)[t] * scale + f64(pair)[P.pair_rows(t, buckets, mul_prev, mul_cur)] for t in seq_toks]
    last = torch.full((4, 1), vocab - 1, dtype=torch.int32, device=DEV)   # dirty slots
    got = [np.zeros((T, width)) for _ in range(2)]
    for step in in_portions(T, CUTS, (5, 6)):
        b = Batch([(p0, n) for _, p0, n in step], slots=[3 - 2 * s for s, _, _ in step],
                  toks=[t for s, p0, n in step for t in seq_toks[s][p0:p0 + n]])
        out = torch.empty(b.n, width, device=DEV)
        ops.embed_pair(table.to(DEV), pair.to(DEV), b, last, out, scale, buckets, mul_prev, mul_cur)
        ops.last_token_update(b, last, b.query_tiles(SEQ))
        r = 0
        for s, p0, n in step:
            got[s][p0:p0 + n] = f64(out[r:r + n])
            r += n
    for s in range(2):
        close(got[s], want[s], "float32", f"sequence {s}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,taps", [(50, 5), (64, 3), (256, 4), (1500, 2), (40, 1), (96, 16)])
def test_norm_and_convolution_over_time_with_state_across_steps(dtype, width, taps):
    """Both sublayers' inputs of two sequences in portions (single rows, pairs, portions shorter and longer than the
    taps); the second sequence starts late in a slot that someone else left dirty."""
    ops = ops_of(dtype)
    T = 41
    g = torch.Generator().manual_seed(width + taps)
    xs = [[torch.randn(T, width, generator=g) * 3 for _ in range(2)] for _ in range(2)]     # [sequence][sublayer]
    nw = [1 + 0.3 * torch.randn(width, generator=g) for _ in range(2)]
    cw = [0.6 * torch.randn(width, taps, generator=g) for _ in range(2)]
    want = [[P.time_conv(P.rms_norm(f64(xs[s][k]), f64(nw[k]), 1e-5), f64(cw[k])) for k in range(2)] for s in range(2)]
    state = torch.full((3, max(taps - 1, 1), 2 * width), 1e3, device=DEV) if taps > 1 else None
    got = [[np.zeros((T, width)) for _ in range(2)] for _ in range(2)]
    for step in in_portions(T, CUTS, (5, 6)):
        b = Batch([(p0, n) for _, p0, n in step], slots=[2 - s for s, _, _ in step])
        normed = torch.empty(b.n, 2 * width, device=DEV)
        for k in range(2):
            x = torch.cat([xs[s][k][p0:p0 + n] for s, p0, n in step]).to(DEV)
            out = torch.empty(b.n, width, dtype=act(dtype), device=DEV)
            ops.norm_conv(x, nw[k].to(DEV), 1e-5, cw[k].t().contiguous().to(DEV), state, k * width, b, out, normed, k * width)
            r = 0
            for s, p0, n in step:
                got[s][k][p0:p0 + n] = f64(out[r:r + n])
                r += n
        if taps > 1:
            ops.conv_state_update(normed, state, b, taps, b.query_tiles(SEQ))
    for s in range(2):
        for k in range(2):
            close(got[s][k], want[s][k], dtype, f"sequence {s}, sublayer {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,taps", [(260, 4), (258, 3), (72, 5), (1100, 2), (36, 1)])
def test_norm_and_convolution_over_time_in_long_steps(dtype, width, taps):
    """Steps of more than a thousand rows, where a block of the kernel takes several rows: sequences of one to 1,400
    rows side by side, so that portions begin and end at every place of a block's rows, cut once in the middle (the
    second step reads the state that the first one left in dirty slots)."""
    ops = ops_of(dtype)
    lengths, first = [1400, 3, 1, 905, 8, 2], [700, 2, 1, 500, 5, 1]
    g = torch.Generator().manual_seed(width * taps)
    xs = [torch.randn(L, width, generator=g) * 2 for L in lengths]
    nw, cw = 1 + 0.3 * torch.randn(width, generator=g), 0.6 * torch.randn(width, taps, generator=g)
    want = [P.time_conv(P.rms_norm(f64(x), f64(nw), 1e-5), f64(cw)) for x in xs]
    state = torch.full((len(lengths) + 1, max(taps - 1, 1), width), 1e3, device=DEV) if taps > 1 else None
    got = [np.zeros((L, width)) for L in lengths]
    steps = [[(s, 0, f) for s, f in enumerate(first)],
             [(s, f, L - f) for s, (L, f) in enumerate(zip(lengths, first)) if L > f]]
    for step in steps:
        b = Batch([(p0, n) for _, p0, n in step], slots=[len(lengths) - s for s, _, _ in step])
        x = torch.cat([xs[s][p0:p0 + n] for s, p0, n in step]).to(DEV)
        normed = torch.full((b.n, width), float("nan"), device=DEV)
        out = torch.empty(b.n, width, dtype=act(dtype), device=DEV)
        ops.norm_conv(x, nw.to(DEV), 1e-5, cw.t().contiguous().to(DEV), state, 0, b, out, normed, 0)
        if taps > 1:
            ops.conv_state_update(normed, state, b, taps, b.query_tiles(SEQ))
        r = 0
        for s, p0, n in step:
            got[s][p0:p0 + n] = f64(out[r:r + n])
            r += n
    for s in range(len(lengths)):
        close(got[s], want[s], dtype, f"sequence {s}")
    if taps > 1:
        assert torch.isfinite(state[1:]).all()                 # every slot's rows were written from rows that were kept


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,entries", [(50, 4), (256, 6), (1500, 2)])
def test_scaled_sums_token_input_and_depth_average(dtype, width, entries):
    ops = ops_of(dtype)
    n, dim, vocab = 7, 6, 19
    g = torch.Generator().manual_seed(width)
    rnd = lambda *s: torch.randn(*s, generator=g)
    x, d, scale = rnd(n, width), rnd(n, width), rnd(width)
    got, rounded = x.clone().to(DEV), torch.empty(n, width, dtype=act(dtype), device=DEV)
    ops.scaled_add(got, scale.to(DEV), d.to(DEV), rounded)
    close(got, f64(x) + f64(scale) * f64(d), "float32", "x + s d")
    assert torch.equal(rounded, got.to(act(dtype)))
    same = got.clone()
    ops.scaled_add(same, None, None, rounded)               # nothing added, the rounded copy alone
    assert torch.equal(same, got)
    # the gate of the token input: gelu_tanh(t) * the token's slice of the shared table
    t, table = rnd(n, dim) * 2, rnd(vocab, 3 * dim).to(act(dtype))
    toks = torch.randint(0, vocab, (n,), generator=g).to(torch.int32)
    gated = torch.empty(n, dim, dtype=act(dtype), device=DEV)
    ops.token_gate(t.to(DEV), table.to(DEV), 2 * dim, toks.to(DEV), gated)
    close(gated, P.gelu_tanh(f64(t)) * f64(table)[toks.long().numpy(), 2 * dim:3 * dim], dtype, "gate")
    # x += mult * norm(y) w, the history's entry, then the weighted sum over the history so far
    hist = [rnd(n, width) for _ in range(entries - 1)]
    y, w, mix = rnd(n, width) * 5, 1 + 0.3 * rnd(width), rnd(entries)
    history = torch.full((n, (entries + 1) * width), 7e3, device=DEV)    # one entry more than is used
    ops.copy_history(hist[0].to(DEV), history)
    for j in range(1, entries - 1):
        history[:, j * width:(j + 1) * width] = hist[j].to(DEV)
    got = x.clone().to(DEV)
    ops.normed_add_mix(got, y.to(DEV), w.to(DEV), 1e-5, 0.3, history, entries - 1, mix.to(DEV))
    own = f64(x) + 0.3 * P.rms_unit(f64(y), 1e-5) * f64(w)
    close(history[:, (entries - 1) * width:entries * width], own, "float32", "the layer's result in the history")
    close(got, P.depth_average([f64(h) for h in hist] + [own], f64(mix)), "float32", "depth average", 4.0)
    got = x.clone().to(DEV)                                  # the sum alone, and the average alone
    ops.normed_add_mix(got, y.to(DEV), w.to(DEV), 1e-5, 0.3, None, 0, None)
    close(got, own, "float32", "x + mult norm(y)")
    got = x.clone().to(DEV)
    ops.normed_add_mix(got, None, None, 0.0, 1.0, history, entries - 1, mix.to(DEV))
    close(got, P.depth_average([f64(h) for h in hist] + [f64(x)], f64(mix)), "float32", "average alone", 4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 24), (3, 1, 10, 12), (8, 1, 64, 80), (2, 2, 36, 4), (5, 5, 8, 40)])
def test_biased_projections_and_mixed_values_into_the_pages(dtype, heads, kv_heads, dim, vdim):
    """The first mixing layer stores its values and keeps them in 32-bit; a later layer stores (1 - lambda) v + lambda
    v_first.  Two sequences in one step, pages in no order."""
    ops = ops_of(dtype)
    page, lam = 16, 0.37
    g = torch.Generator().manual_seed(dim * vdim)
    seqs = [(5, 30), (40, 3)]
    b = Batch(seqs)
    cols = heads * dim + kv_heads * (dim + vdim)
    table = pages_in_no_order(seqs, 9, page, g)
    bias = torch.randn(cols, generator=g)
    lam_t = torch.tensor([lam], device=DEV)
    first = torch.empty(b.n, kv_heads * vdim, device=DEV)
    us = [torch.randn(b.n, cols, generator=g) * 2 for _ in range(2)]
    for layer, u in enumerate(us):
        kc = torch.zeros(10, kv_heads, page, dim, dtype=act(dtype), device=DEV)
        vc = torch.zeros(10, kv_heads, page, vdim, dtype=act(dtype), device=DEV)
        q = torch.empty(b.n, heads * dim, dtype=act(dtype), device=DEV)
        extra = {"v_keep": first} if layer == 0 else {"vmix_src": first, "vmix_lambda": lam_t}
        ops.qkv_prepare(u.to(DEV), None, None, None, None, 1e-5, None, None, b, table, kc, vc, q, heads, kv_heads, dim, vdim,
                        bias=bias.to(DEV), **extra)
        y = f64(u) + f64(bias)
        v = y[:, (heads + kv_heads) * dim:]
        if layer == 0:
            v_first = v
            close(first, v, "float32", "the first layer's values in 32-bit")
        else:
            v = P.mix_values(v, v_first, lam)
        close(q, y[:, :heads * dim], dtype, f"queries of layer {layer}")
        r = 0
        for s, (p0, n) in enumerate(seqs):
            idx = torch.arange(p0, p0 + n)
            blocks, slots = table[s].cpu().long()[idx // page], idx % page
            close(kc.cpu()[blocks, :, slots, :].reshape(n, -1), y[r:r + n, heads * dim:(heads + kv_heads) * dim], dtype, "keys")
            close(vc.cpu()[blocks, :, slots, :].reshape(n, -1), v[r:r + n], dtype, f"values of layer {layer}")
            r += n


# (the serving precision runs shapes with sizes in steps of 16 on the tensor cores, the others on the CUDA cores)
ATTENTION_SHAPES = [(4, 2, 16, 24), (8, 1, 64, 80), (3, 3, 40, 8), (40, 1, 8, 16), (2, 1, 96, 200), (6, 2, 64, 32), (2, 2, 32, 256)]


def rounded(dtype, g, *shape):
    """Random values that the cache holds exactly in this precision, as float64 numpy."""
    return f64(torch.randn(*shape, generator=g).to(act(dtype)))


def run_attention(ops, dtype, q, kc, vc, table, p0, n, heads, kv_heads, dim, vdim, scale, cap, r1, r2, sink, window, keep):
    b = Batch([(p0, n)])
    out = torch.empty(n, heads * vdim, dtype=act(dtype), device=DEV)
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    ops.scored_attention(torch.tensor(q[p0:p0 + n].reshape(n, -1)).to(act(dtype)).to(DEV).contiguous(), kc, vc, table, out, heads,
                         kv_heads, dim, vdim, scale, cap or 0.0, True, None, window or 0, b, dist_a=dev(r1), dist_b=dev(r2),
                         sinks=dev(sink), keep_first=keep)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", ATTENTION_SHAPES)
@pytest.mark.parametrize("cap", [None, 6.0])
def test_far_keys_learned_sink_and_distance_term(dtype, heads, kv_heads, dim, vdim, cap):
    """No window.  One query is scaled so that a key hundreds of positions back takes nearly all its weight in spite
    of the distance term; another sees only very negative scores, so that the sink takes nearly all of it; a head
    with a negative first number is pulled toward far keys."""
    ops = ops_of(dtype)
    page, T = 16, 700
    g = torch.Generator().manual_seed(heads * dim)
    q, k, v = rounded(dtype, g, T, heads, dim), rounded(dtype, g, T, kv_heads, dim), rounded(dtype, g, T, kv_heads, vdim)
    scale = 1.0 / math.sqrt(dim)
    to_act = lambda a: f64(torch.tensor(a).to(act(dtype)))
    k[5] = to_act(q[690, 0] * 3)                          # a far key that query 690 of head 0 agrees with
    q[650] = to_act(-np.abs(q[650]) * (40 / math.sqrt(dim)))
    k[:651] = np.abs(k[:651])                             # every score of row 650 is very negative
    r1 = np.linspace(-0.3, 0.9, heads)
    r2 = np.linspace(0.05, 2.5, heads)
    sink = np.linspace(-2.0, 3.0, heads)
    want = P.windowed_sink_attention(q, k, v, scale, cap, r1, r2, sink, None, 0)
    table = pages_in_no_order([(0, T)], 60, page, g)
    kc = fill_pages([torch.tensor(k)], table, page, kv_heads, dim, dtype)
    vc = fill_pages([torch.tensor(v)], table, page, kv_heads, vdim, dtype)
    for p0, n in ((0, T), (600, 100), (649, 2), (690, 1), (650, 1), (0, 1), (1, 2)):
        out = run_attention(ops, dtype, q, kc, vc, table, p0, n, heads, kv_heads, dim, vdim, scale, cap, r1, r2, sink, None, 0)
        close(out, want[p0:p0 + n].reshape(n, -1), dtype, f"rows {p0}..{p0 + n - 1}", 2.0)
    assert cap or np.abs(want[650]).max() < 0.05 * np.abs(v).max(), "the sink did not take the weight"
    # without the sink's own number the denominator would hold 1: the learned number must matter at position 0
    s0 = float(q[0, 0] @ k[0, 0]) * scale
    s0 = cap * math.tanh(s0 / cap) if cap else s0
    assert np.allclose(want[0, 0], v[0, 0] * math.exp(s0) / (math.exp(s0) + math.exp(sink[0])))


def window_case(dtype, g, T, heads, kv_heads, dim, vdim, window, keep, cap):
    """Queries, keys and values of one sequence in which single keys at the edges decide their rows, and the plain result."""
    q, k, v = rounded(dtype, g, T, heads, dim), rounded(dtype, g, T, kv_heads, dim), rounded(dtype, g, T, kv_heads, vdim)
    scale = 1.0 / math.sqrt(dim)
    to_act = lambda a: f64(torch.tensor(a).to(act(dtype)))
    marked = {}
    for i, j in ((200, 200 - window + 1), (250, 250 - window), (280, keep - 1), (290, keep), (window + keep + 3, keep),
                 (270, 270 - window + 1)):
        if 0 <= j <= i < T and i not in marked:
            q[i] = to_act(np.tile(k[j, 0] * (14.0 / (float(k[j, 0] @ k[j, 0]) * scale)), (heads, 1)))   # a score of 14
            marked[i] = j
    r1, r2, sink = np.linspace(-0.2, 0.6, heads), np.linspace(0.1, 1.5, heads), np.linspace(-1.0, 1.0, heads)
    want = P.windowed_sink_attention(q, k, v, scale, cap, r1, r2, sink, window, keep)
    # the marked key decides its row where it is seen, and does not where it is hidden
    for i, j in marked.items():
        near = np.abs(want[i, 0] - v[j, 0]).max() < 0.25 * np.abs(v).max()
        assert near == P.visible(i, j, window, keep) or dim < 16, (i, j)
    return q, k, v, scale, r1, r2, sink, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 96, 24), (3, 1, 10, 12), (8, 1, 64, 80), (2, 2, 32, 32), (40, 1, 8, 16)])
@pytest.mark.parametrize("window,keep", [(7, 0), (33, 2), (80, 4), (96, 20), (9, 18), (1, 1), (64, 16), (130, 40), (16, 17)])
def test_window_edges_and_kept_first_keys(dtype, heads, kv_heads, dim, vdim, window, keep):
    """The key just outside a query's window is made to agree with it strongly (it would take all the weight if it
    were seen), the key just inside another query's window likewise (it must take it); the same for the last kept
    first key and the first key that is not kept.  Pages that the window has passed are given back (table entries
    -1) but for those of the kept keys.  Prompt portions and single rows."""
    ops = ops_of(dtype)
    page, T, cap = 16, 300, 30.0
    g = torch.Generator().manual_seed(dim + window + keep)
    q, k, v, scale, r1, r2, sink, want = window_case(dtype, g, T, heads, kv_heads, dim, vdim, window, keep, cap)
    table = pages_in_no_order([(0, T)], 30, page, g)
    kc = fill_pages([torch.tensor(k)], table, page, kv_heads, dim, dtype)
    vc = fill_pages([torch.tensor(v)], table, page, kv_heads, vdim, dtype)
    portions = [(0, T), (190, 70), (199, 2), (250, 1), (280, 1), (290, 1), (270, 1), (keep, 1), (max(keep - 1, 0), 2),
                (window - 1, 2), (window + keep + 3, 1), (0, 1)]
    for p0, n in portions:
        tb = table.clone()
        first_needed = p0 - window + 1
        kept_blocks = (keep + page - 1) // page
        if first_needed >= page:
            tb[0, kept_blocks:max(kept_blocks, first_needed // page)] = -1
        out = run_attention(ops, dtype, q, kc, vc, tb, p0, n, heads, kv_heads, dim, vdim, scale, cap, r1, r2, sink, window, keep)
        close(out, want[p0:p0 + n].reshape(n, -1), dtype, f"rows {p0}..{p0 + n - 1}", 2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_of_unequal_sequences_in_one_step(dtype):
    """Three sequences in one step (a long portion, a pair, a single row deep in its context) give what each gives alone."""
    ops = ops_of(dtype)
    heads, kv_heads, dim, vdim, page, window, keep = 6, 2, 32, 16, 16, 50, 5
    g = torch.Generator().manual_seed(11)
    lens = [90, 200, 333]
    ks, vs = [rounded(dtype, g, n, kv_heads, dim) for n in lens], [rounded(dtype, g, n, kv_heads, vdim) for n in lens]
    qs = [rounded(dtype, g, n, heads, dim) for n in lens]
    r1, r2, sink = np.linspace(0.1, 0.7, heads), np.linspace(0.2, 1.0, heads), np.linspace(-1.0, 2.0, heads)
    table = pages_in_no_order([(0, n) for n in lens], 70, page, g)
    kc = fill_pages([torch.tensor(a) for a in ks], table, page, kv_heads, dim, dtype)
    vc = fill_pages([torch.tensor(a) for a in vs], table, page, kv_heads, vdim, dtype)
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    alone = [P.windowed_sink_attention(qs[s], ks[s], vs[s], 0.2, 9.0, r1, r2, sink, window, keep) for s in range(3)]
    for seqs in ([(20, 70), (198, 2), (332, 1)], [(89, 1), (199, 1), (332, 1)], [(0, 3), (0, 1), (100, 60)]):
        b = Batch(seqs)
        qrows = np.concatenate([qs[s][p0:p0 + n].reshape(n, -1) for s, (p0, n) in enumerate(seqs)])
        out = torch.empty(b.n, heads * vdim, dtype=act(dtype), device=DEV)
        ops.scored_attention(torch.tensor(qrows).to(act(dtype)).to(DEV).contiguous(), kc, vc, table, out, heads, kv_heads, dim, vdim,
                             0.2, 9.0, True, None, window, b, dist_a=dev(r1), dist_b=dev(r2), sinks=dev(sink), keep_first=keep)
        want = np.concatenate([alone[s][p0:p0 + n].reshape(n, -1) for s, (p0, n) in enumerate(seqs)])
        close(out, want, dtype, str(seqs), 2.0)


def test_tensor_core_attention_agrees_with_the_plain_kernel():
    """bfloat16: the same step on both kernels (prompt portion, then single rows spread over spans)."""
    ops = ops_of("bfloat16")
    heads, kv_heads, dim, vdim, page, T = 8, 2, 64, 64, 16, 600
    g = torch.Generator().manual_seed(5)
    k = torch.randn(T, kv_heads, dim, generator=g).to(torch.bfloat16)
    v = torch.randn(T, kv_heads, vdim, generator=g).to(torch.bfloat16)
    table = pages_in_no_order([(0, T)], 40, page, g)
    kc, vc = fill_pages([k], table, page, kv_heads, dim, "bfloat16"), fill_pages([v], table, page, kv_heads, vdim, "bfloat16")
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    r1, r2, sink = dev(np.linspace(-0.2, 0.8, heads)), dev(np.linspace(0.1, 2.0, heads)), dev(np.linspace(-2.0, 2.0, heads))
    for seqs in ([(100, 500)], [(599, 1)], [(0, 40)]):
        b = Batch(seqs)
        q = torch.randn(b.n, heads * dim, generator=g).to(torch.bfloat16).to(DEV)
        outs = []
        for plain in (False, True):
            ops.plain_mixers(plain)
            try:
                both = []
                for window, keep in ((0, 0), (100, 7), (300, 40)):
                    o = torch.empty(b.n, heads * vdim, dtype=torch.bfloat16, device=DEV)
                    ops.scored_attention(q, kc, vc, table, o, heads, kv_heads, dim, vdim, 0.125, 12.0, True, None, window, b,
                                         dist_a=r1, dist_b=r2, sinks=sink, keep_first=keep)
                    both.append(o.float())
            finally:
                ops.plain_mixers(False)
            outs.append(both)
        for a, c in zip(*outs):
            assert float((a - c).abs().max()) <= 0.02 * float(c.abs().max())


@pytest.mark.parametrize("experts,top", [(8, 4), (5, 1), (3, 3), (64, 6), (2, 1), (1, 1)])
def test_router_takes_the_largest_logits_and_softmax_over_them(experts, top):
    ops = ops_of("float32")
    g = torch.Generator().manual_seed(experts)
    n = 37
    z = torch.randn(n, experts, generator=g) * 3
    if experts > 2:
        z[0, 1:3] = z[0].max() + 1.0                       # a tie at the top: the lower index comes first
        z[1] = -40.0 + torch.arange(experts) * 1e-3        # all very negative: the weights still sum to one
    chosen = torch.empty(n, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(n, top, dtype=torch.float32, device=DEV)
    ops.route(z.to(DEV), None, 1, 1, top, 1.0, chosen, weights, softmax_top=True)
    want_c, want_w = P.route(f64(z), top)
    assert chosen.cpu().tolist() == want_c.tolist()
    close(weights, want_w, "float32", "weights")
    assert np.allclose(f64(weights).sum(1), 1.0, atol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,inner,experts,top", [(50, 19, 5, 2), (72, 40, 3, 3), (192, 64, 8, 4), (64, 24, 4, 1)])
def test_routed_and_clamped_feed_forward(dtype, width, inner, experts, top):
    """The routed feed-forward as its kernels run it (route, lists, grouped products, silu gate, the weighted sum
    scaled per channel into the stream), and the dense one with its clamps reached on both sides."""
    ops = ops_of(dtype)
    g = torch.Generator().manual_seed(width + top)
    n = 150 if width < 100 else 700
    rnd = lambda *s: torch.randn(*s, generator=g)
    h = rnd(n, width).to(act(dtype))
    w = {"p.router": (rnd(experts, width) * 3 / math.sqrt(width)).to(act(dtype))}
    for e in range(experts):
        w[f"p.e{e}.gate"] = (rnd(inner, width) * 2 / math.sqrt(width)).to(act(dtype))
        w[f"p.e{e}.up"] = (rnd(inner, width) * 2 / math.sqrt(width)).to(act(dtype))
        w[f"p.e{e}.down"] = (rnd(width, inner) / math.sqrt(inner)).to(act(dtype))
    scale, x = rnd(width), rnd(n, width)
    want = f64(x) + f64(scale) * P.moe_ff({"router": {"top": top}}, {k_: f64(t) for k_, t in w.items()}, "p", f64(h))
    hd = h.to(DEV)
    z = torch.empty(n, experts, device=DEV)
    ops.linear(hd, w["p.router"].to(DEV), z)
    chosen = torch.empty(n, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(n, top, dtype=torch.float32, device=DEV)
    ops.route(z, None, 1, 1, top, 1.0, chosen, weights, softmax_top=True)
    off = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    tiles = torch.empty(2, experts + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(n * top, dtype=torch.int32, device=DEV)
    place = torch.empty(n * top, dtype=torch.int32, device=DEV)
    ops.group_rows(chosen, experts, off, tiles, order, place)
    w1 = torch.stack([torch.cat([w[f"p.e{e}.gate"], w[f"p.e{e}.up"]], 0) for e in range(experts)]).contiguous().to(DEV)
    w2 = torch.stack([w[f"p.e{e}.down"] for e in range(experts)]).contiguous().to(DEV)
    gate_up = torch.empty(n * top, 2 * inner, dtype=act(dtype), device=DEV)
    sorted_x = torch.empty(n * top, width, dtype=act(dtype), device=DEV)
    ops.grouped_linear(hd, w1, gate_up, n * top, lists=(off, tiles, order), order_div=top, sorted_x=sorted_x)
    hh = torch.empty(n * top, inner, dtype=act(dtype), device=DEV)
    ops.swiglu(gate_up, hh)
    y = torch.empty(n * top, width, dtype=torch.float32, device=DEV)
    ops.grouped_linear(hh, w2, y, n * top, lists=(off, tiles, order), gather=False)
    got = x.clone().to(DEV)
    ops.combine(got, None, y, place, weights, top, scale=scale.to(DEV))
    close(got, want, dtype, "x + s * routed(h)", 2.0)
    # the dense feed-forward: min(gate, limit), clamp(up, -limit, limit), g sigmoid(1.702 g) (u + 1)
    dw = {"d.gate": w["p.e0.gate"] * 2, "d.up": w["p.e0.up"] * 2, "d.down": w["p.e0.down"]}
    limit = 0.8
    gu = torch.empty(n, 2 * inner, dtype=act(dtype), device=DEV)
    ops.linear(hd, torch.cat([dw["d.gate"], dw["d.up"]], 0).contiguous().to(DEV), gu)
    assert float((gu[:, :inner] > limit).float().mean()) > 0.02 and float((gu[:, inner:] < -limit).float().mean()) > 0.02
    a = torch.empty(n, inner, dtype=act(dtype), device=DEV)
    ops.glu_clamped(gu, a, limit, 1.702)
    out = torch.empty(n, width, device=DEV)
    ops.linear(a, dw["d.down"].to(DEV), out)
    close(out, P.dense_ff({"limit": limit}, {k_: f64(t) for k_, t in dw.items()}, "d", f64(h)), dtype, "dense", 2.0)


# ---------------------------------------------------------------------------------------------
# whole models

_models, _plain = {}, {}
WEIGHT_SEED = 7


def model_of(name, dtype):
    from bitwise_b200 import Model
    if (name, dtype) not in _models:
        _models[(name, dtype)] = Model.from_tensors(CONFIGS[name], random_weights(CONFIGS[name], WEIGHT_SEED), dtype=dtype, device=DEV)
    return _models[(name, dtype)]


def to_bf16(a):
    return torch.tensor(np.asarray(a)).to(torch.bfloat16).to(torch.float64).numpy()


def plain_pair(cfg, W, toks, collect=None, collect_rounded=None):
    """The plain logits of one request, and the plain logits with everything rounded to bfloat16 that the serving
    precision stores in it: the second shows how large an error rounding alone causes for these weights."""
    exact = P.forward(cfg.to_json(), W, toks, collect)
    with P.rounding(to_bf16):
        rounded_ = P.forward(cfg.to_json(), W, toks, collect_rounded)
    return exact, rounded_


def plain_logits(name, toks, rounded_too=False):
    key = (name, tuple(toks))
    if key not in _plain:
        _plain[key] = plain_pair(CONFIGS[name], as_float64(random_weights(CONFIGS[name], WEIGHT_SEED)), toks)
    return _plain[key] if rounded_too else _plain[key][0]


# lengths around the pages' (16), the key tiles' and the windows' edges of each configuration
LENGTHS = {"a": [70, 45, 5, 300, 64, 17, 1, 131], "b": [100, 9, 330, 1, 65, 33], "c": [40, 290, 3, 17, 132]}


def requests_of(name):
    return {f"{name}-{i}": tokens(CONFIGS[name], n, i) for i, n in enumerate(LENGTHS[name])}


def row_errors(got, want):
    """Per position: root mean square of the difference over that of the reference row."""
    return np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))


def assess(errors, dtype, what, rounding_alone=None):
    """float32: every position within the tolerance.  bfloat16: against the errors that rounding alone causes in the
    plain implementation for the same weights and tokens (``rounding_alone``, per position): the mean, the 95th
    percentile and the worst position may be twice to three times that and no more.  (Rounding turns a router's close
    call now and then, which is a step in the output and no error of arithmetic; it does so in both.)"""
    errors = np.concatenate([np.atleast_1d(e) for e in errors])
    if dtype == "float32":
        assert errors.max() <= 4 * TOL[dtype], f"{what}: worst relative error {errors.max():.3g}"
        return
    base = np.concatenate([np.atleast_1d(e) for e in rounding_alone])
    assert len(base) == len(errors)
    q = lambda e: float(np.quantile(e, 0.95))
    assert errors.mean() <= 2 * base.mean() + 0.01 and q(errors) <= 2 * q(base) + 0.02 and errors.max() <= 3 * base.max() + 0.05, \
        f"{what}: mean relative error {errors.mean():.3g} (rounding alone: {base.mean():.3g}), 95th percentile " \
        f"{q(errors):.3g} ({q(base):.3g}), worst {errors.max():.3g} ({base.max():.3g})"


def compare(name, dtype, got_by_request):
    errors, base = [], []
    for rid, toks in requests_of(name).items():
        want, rounded_ = plain_logits(name, toks, rounded_too=True)
        got = got_by_request[rid]
        assert got.shape == want.shape
        errors.append(row_errors(got, want))
        base.append(row_errors(rounded_, want))
    assess(errors, dtype, f"{name} {dtype} against the plain implementation", base)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts_and_layers(name, dtype):
    model = model_of(name, dtype)
    reqs = requests_of(name)
    steps = R.whole(reqs)
    compare(name, dtype, R.collect(steps, R.run_in_process(model, steps, 384), CONFIGS[name].vocab))
    # the stream after every layer, for one request
    toks = next(iter(reqs.values()))
    want, want_rounded = [], []
    plain_pair(CONFIGS[name], as_float64(random_weights(CONFIGS[name], WEIGHT_SEED)), toks, want, want_rounded)
    seen = []
    for b in model.decoder.blocks:
        def fwd(ctx, x, cache, orig=b.forward):
            orig(ctx, x, cache)
            seen.append(x[:ctx.n].clone())
        b.forward = fwd
    try:
        model.logits(toks)
    finally:
        for b in model.decoder.blocks:
            del b.forward
    assert len(seen) == len(want)
    for i, (got, w, wr) in enumerate(zip(seen, want, want_rounded)):
        assess([row_errors(got.float().cpu().numpy(), w)], dtype, f"stream after layer {i}", [row_errors(wr, w)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cut_gives_the_same_logits(name, dtype):
    model = model_of(name, dtype)
    reqs = requests_of(name)
    vocab = CONFIGS[name].vocab
    base = R.collect(R.whole(reqs), R.run_in_process(model, R.whole(reqs), 384), vocab)
    patterns = {"tail": (R.tail_one_by_one(reqs, tail=40), 384), "portions": (R.portions(reqs), 384),
                "pairs": (R.portions(reqs, sizes=(2,)), 384), "mixed": (R.mixed(reqs, 704, seed=3), 704),
                "mixed-tight": (R.mixed(reqs, 448, seed=4), 448)}
    for pname, (steps, pool) in patterns.items():
        for graphs in ((None, False) if dtype == "bfloat16" and pname in ("tail", "mixed") else (None,)):
            got = R.collect(steps, R.run_in_process(model, steps, pool, use_graphs=graphs), vocab)
            compare(name, dtype, got)
            # between two cuts only rounding differs: far less than between precision and plain
            errs = np.concatenate([row_errors(got[rid], base[rid]) for rid in reqs])
            assert errs.max() <= (1e-5 if dtype == "float32" else 0.02), f"{name} {dtype} {pname}: cuts differ by {errs.max():.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(EDGE_CONFIGS))
def test_layer_combinations_at_the_edges(name, dtype):
    """Models without any state, with windows only (one of a single key), with the convolution as the only state."""
    from bitwise_b200 import Model
    cfg = EDGE_CONFIGS[name]
    W = random_weights(cfg, 3)
    model = Model.from_tensors(cfg, W, dtype=dtype, device=DEV)
    reqs = {f"{name}{i}": tokens(cfg, n, i) for i, n in enumerate([37, 70, 5, 1, 18])}
    want, base = {}, {}
    for rid, t in reqs.items():
        want[rid], rounded_ = plain_pair(cfg, as_float64(W), t)
        base[rid] = row_errors(rounded_, want[rid])
    for steps, pool in ((R.whole(reqs), 128), (R.portions(reqs, sizes=(3, 2, 11, 1)), 128), (R.mixed(reqs, 192, seed=5), 192)):
        got = R.collect(steps, R.run_in_process(model, steps, pool), cfg.vocab)
        assess([row_errors(got[rid], want[rid]) for rid in reqs], dtype, f"{name} {dtype}", [base[rid] for rid in reqs])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_first_key_decides_after_long_decoding(dtype):
    """One layer whose window is long passed while a kept first key holds what the last positions ask for: the query
    and key projections are the identity on a few channels, one early token's embedding is large there, and so is
    the embedding of the token that is decoded last.  Hidden (one position beyond the kept ones), the same key
    changes nothing."""
    from bitwise_b200 import Model
    from sebavik_configs import attention, dense, layer
    from bitwise_b200.config.sebavik import SebavikConfig
    cfg = SebavikConfig(vocab=40, width=32, eps=1e-5, residual_mult=1.0, embedding_scale=1.0, canon_taps=0, layers=(
        layer(attention(2, 1, 16, 16, 1.0, softcap=50.0, window=24, keep_first=3), dense(24, 1.0)),))
    W = random_weights(cfg, 5)
    eye = torch.zeros(16, 32)
    eye[:4, :4] = torch.eye(4)
    W["l0.mix.q"], W["l0.mix.k"] = torch.cat([eye, eye]).to(torch.bfloat16), eye.to(torch.bfloat16)
    W["l0.mix.q.b"], W["l0.mix.k.b"] = torch.zeros(32).to(torch.bfloat16), torch.zeros(16).to(torch.bfloat16)
    W["l0.norm1"] = torch.ones(32).to(torch.bfloat16)
    W["l0.mix.r1"] = torch.tensor([0.25, -0.25]).to(torch.bfloat16)
    W["embed"][:, :4] *= 0.05
    W["embed"][38, :4], W["embed"][39, :4] = torch.tensor([9.0, 0, 0, 0]).to(torch.bfloat16), torch.tensor([9.0, 0, 0, 0]).to(torch.bfloat16)
    model = Model.from_tensors(cfg, W, dtype=dtype, device=DEV)
    base = [t % 38 for t in tokens(cfg, 200, 1)]
    outs = {}
    for where in (2, 3):                                    # the last kept position, and the first that is not kept
        toks = list(base)
        toks[where], toks[-1] = 38, 39
        want, rounded_ = plain_pair(cfg, as_float64(W), toks)
        steps = R.tail_one_by_one({"r": toks}, tail=150)
        got = R.collect(steps, R.run_in_process(model, steps, 256), cfg.vocab)["r"]
        assess([row_errors(got, want)], dtype, f"marked key at {where}", [row_errors(rounded_, want)])
        outs[where] = want[-1]
    plain = list(base)
    plain[-1] = 39
    unmarked = P.forward(cfg.to_json(), as_float64(W), plain)[-1]
    assert np.abs(outs[3] - unmarked).max() < 1e-9 * np.abs(unmarked).max() + 1e-9, "a hidden key changed the logits"
    assert np.abs(outs[2] - unmarked).max() > 0.05 * np.abs(unmarked).max(), "the kept key did not decide"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_reused_pages(dtype):
    # one request decoded token by token from position 3 to past 600 (pages, key tiles, windows and the kept first
    # keys' edge are crossed one position at a time) while others come and go in the pool and in the slots
    name = "a"
    model = model_of(name, dtype)
    toks = tokens(CONFIGS[name], 620, 99)
    others = {f"o{i}": tokens(CONFIGS[name], n, 50 + i) for i, n in enumerate([30, 64, 100, 7, 65, 120])}
    from bitwise_b200.engine.replay import make_replay_stepper
    from bitwise_b200.engine.step import StepEntry
    stepper = make_replay_stepper(model, 640 + 128 + 64, max_live=3)
    queue = list(others.items())
    live = None
    errors, base = [], []
    want, want_rounded = plain_logits(name, toks, rounded_too=True)
    out = stepper.run([StepEntry("long", toks[:3], [2])])
    for p in range(3, len(toks)):
        entries = [StepEntry("long", toks[p:p + 1], [0])]
        if live is None and queue and p % 7 == 0:
            live = [queue.pop(0), 0]
        if live is not None:
            (rid, ot), at = live
            c = min(len(ot) - at, 1 + p % 9)
            entries.append(StepEntry(rid, ot[at:at + c], [c - 1]))
            live[1] += c
        out = stepper.run(entries).float().cpu().numpy()
        errors.append(row_errors(out[0], want[p]))
        base.append(row_errors(want_rounded[p], want[p]))
        if live is not None:
            w, wr = plain_logits(name, live[0][1], rounded_too=True)
            errors.append(row_errors(out[1], w[live[1] - 1]))
            base.append(row_errors(wr[live[1] - 1], w[live[1] - 1]))
            if live[1] == len(live[0][1]):
                stepper.finish(live[0][0])
                live = None
    assert not queue
    stepper.finish("long")
    assert stepper.manager.all_free()
    assess(errors, dtype, "long decoding", base)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    name = "a"
    model = model_of(name, dtype)
    cfg = CONFIGS[name]
    prompts = [tokens(cfg, n, 200 + i) for i, n in enumerate([5, 40, 17, 1, 33])]
    new = 12
    # a pool that does not hold all requests at once and a token budget below the longest prompt
    eng = Engine(model, EngineConfig(num_blocks=12, block_size=16, max_batched_tokens=24, max_num_seqs=3))
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=new, ignore_eos=True))
    W = as_float64(random_weights(cfg, WEIGHT_SEED))
    for prompt, out in zip(prompts, got):
        assert len(out) == new
        seq = list(prompt)
        for t in out:
            row = P.forward(cfg.to_json(), W, seq)[-1]
            if dtype == "float32":
                assert t == int(row.argmax()) or row.max() - row[t] < 1e-4 * np.abs(row).max()
            else:
                assert row.max() - row[t] <= 0.05 * np.abs(row).max(), "the chosen token is no near-maximum"
            seq.append(t)
    assert eng.manager.all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_simulated_traces_reproduce_requests_run_alone(dtype):
    # the engine's simulator: random requests, budgets and pools, preemption with recomputation; a request's tokens
    # and the fingerprint of its logits must be those it yields alone on an idle engine
    from bitwise_b200.engine.simulate import run_traces
    out = run_traces(model_of("a", dtype), traces=8, seed=5)
    assert out.traces == 8 and out.requests_checked > 10
    assert out.violations == 0, (out.token_mismatch, out.fingerprint_mismatch, out.hangs, out.leaks)


def test_command_line_random_folder_replay_and_generation(tmp_path):
    """``bitwise_b200 random`` writes a Sebavik folder from a config.json; ``bin/trace_run`` replays a mixed schedule
    on it and ``bitwise_b200 generate`` decodes greedily: both as a user calls them, both against the plain
    implementation on the folder's own tensors."""
    import json
    import os
    import subprocess
    import sys
    from bitwise_b200.weights.safetensors_io import SafetensorsFile
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CONFIGS["b"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_json()))
    folder = tmp_path / "model"
    run = lambda *a, **k: subprocess.run([sys.executable, *a], capture_output=True, text=True, timeout=900, **k)
    p = run(os.path.join(root, "bin", "bitwise_b200"), "random", "--config", str(tmp_path / "config.json"), "--seed", "11",
            "--out", str(folder), "--dtype", "bfloat16", "--std", "0.3", "--norm-jitter", "0.2")
    assert p.returncode == 0, p.stderr[-2000:]
    f = SafetensorsFile(str(folder / "model.safetensors"))
    W = {n: f.tensor(n).to(torch.float64).numpy() for n in f.names()}
    raw = json.load(open(folder / "config.json"))
    reqs = {f"q{i}": tokens(cfg, n, 300 + i) for i, n in enumerate([33, 70, 2, 19])}
    steps = R.mixed(reqs, 192, seed=8)
    out = tmp_path / "out"
    p = run(os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
            "--max-tokens", "192", input="".join(json.dumps(s) + "\n" for s in steps))
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    outs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg.vocab) for s in steps}
    got = R.collect(steps, outs, cfg.vocab)
    for rid, toks in reqs.items():
        want = P.forward(raw, W, toks)
        assert np.abs(got[rid] - want).max() <= 1e-4 * np.abs(want).max(), rid
    prompt = reqs["q3"]
    p = run(os.path.join(root, "bin", "bitwise_b200"), "generate", "--model", str(folder), "--dtype", "float32",
            "--max-new-tokens", "6", "--ignore-eos", "--temperature", "0", "--prompt-ids", ",".join(map(str, prompt)))
    assert p.returncode == 0, p.stderr[-2000:]
    seq = list(prompt)
    for t in json.loads(p.stdout.strip().split("\n")[0])["tokens"]:
        row = P.forward(raw, W, seq)[-1]
        assert t == int(row.argmax()) or row.max() - row[t] < 1e-4 * np.abs(row).max()
        seq.append(t)
