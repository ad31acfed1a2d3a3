"""Kezuvik on the device against the plain implementation (tests/plain_kezuvik.py).

Each new mechanism alone (the rotation in the half layout with rescaled frequencies on its way into the pages and
on the queries, the layer norm after a sublayer, gates, the GELU feed-forward step and the cap, latent attention
with a sink where one far key among hundreds or the sink decides), then whole models of several shapes in both
precisions, the same requests cut in every way (whole, token by token, portions down to two tokens, mixed batches
over a pool whose pages and slots are used again), a key just inside and just outside a window in a prompt and in
decoding, long decoding, and greedy generation through the engine and its scheduler and through the command line.
"""
import json
import math

import numpy as np
import pytest
import torch

import plain_kezuvik as P
import replay_patterns as R
from kezuvik_configs import CONFIGS, L, latent, random_weights, tokens, window
from bitwise_b200.config.kezuvik import KezuvikConfig

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}   # relative to the largest reference value
F64 = torch.float64
WEIGHT_SEED = 3
_models, _plain = {}, {}


def to_bf16(a):
    return a.to(torch.bfloat16).to(F64)


def ops_of(dtype):
    from bitwise_b200.kernels.ops import get_ops
    return get_ops(dtype)


def act(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def close(got, want, dtype, what="", factor=1.0):
    got = got.detach().to(F64).cpu() if isinstance(got, torch.Tensor) else torch.as_tensor(got, dtype=F64)
    want = torch.as_tensor(want, dtype=F64)
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    err = float((got - want).abs().max() / max(float(want.abs().max()), 1e-30))
    assert err <= TOL[dtype] * factor, f"{what}: relative error {err:.3g}"


class Batch:
    """What the kernels read of a step: rows of sequences with their positions, and query tiles."""

    def __init__(self, seqs):
        # seqs: list of (first position, rows); one block-table row each
        pos, row_seq, seq_pos0, seq_row0 = [], [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(seqs):
            seq_pos0.append(p0), seq_row0.append(r)
            pos += list(range(p0, p0 + cnt))
            row_seq += [s] * cnt
            r += cnt
        self.i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.n, self.seqs, self.positions = r, seqs, pos
        self.pos, self.row_seq = self.i32(pos), self.i32(row_seq)
        self.seq_pos0, self.seq_row0 = self.i32(seq_pos0), self.i32(seq_row0 + [r])
        self.max_keys = max(pos) + 1

    def query_tiles(self, tile_rows):
        t_seq, t_row0, t_rows = [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(self.seqs):
            for a in range(0, cnt, tile_rows):
                t_seq.append(s), t_row0.append(r + a), t_rows.append(min(tile_rows, cnt - a))
            r += cnt
        return self.i32(t_seq), self.i32(t_row0), self.i32(t_rows), len(t_seq)


def scattered_table(seqs, page, g, spare=5):
    """A block table [seqs, blocks] over a pool whose pages are handed out in no order."""
    blocks = (max(p0 + cnt for p0, cnt in seqs) + page - 1) // page
    perm = torch.randperm(len(seqs) * blocks + spare, generator=g)[:len(seqs) * blocks]
    return perm.to(torch.int32).reshape(len(seqs), blocks).to(DEV)


ROTS = [(8, 8, 100.0, None), (16, 16, 5000.0, (4.0, 64.0, 8.0, 0.5)), (6, 4, 777.0, (1.5, 32.0, 4.0, 2.0)), (32, 32, 50000.0, None),
        (12, 2, 20.0, (2.0, 8.0, 1.0, 0.5))]


def rot_of(dims, base, sc):
    rot = {"dims": dims, "base": base}
    if sc:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
    return rot


def encoding_of(dims, base, sc, positions):
    from bitwise_b200.parts.rope import HalfRotaryEncoding, RampScaling
    return HalfRotaryEncoding(dims, base, RampScaling(*sc) if sc else None, positions=positions)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rot_dim,dims,base,sc", ROTS)
@pytest.mark.parametrize("rank,heads,dim", [(40, 3, 16), (33, 1, 10), (136, 12, 8)])
def test_half_layout_rotation_into_the_pages_and_on_the_queries(dtype, rot_dim, dims, base, sc, rank, heads, dim):
    ops = ops_of(dtype)
    g = torch.Generator().manual_seed(rank + rot_dim)
    seqs = [(0, 5), (37, 4), (250, 1), (15, 20)]
    b = Batch(seqs)
    page = 16
    table = scattered_table(seqs, page, g)
    cos, sin = encoding_of(dims, base, sc, 300).rotary_tables(DEV)
    rot = rot_of(dims, base, sc)
    # the down projection's rows may be columns of a wider product
    wide = torch.randn(b.n, rank + rot_dim + 7, generator=g).to(DEV)
    d = wide[:, :rank + rot_dim]
    w = (1.0 + 0.2 * torch.randn(rank, generator=g)).to(DEV)
    cache = torch.zeros(int(table.max()) + 1, page, rank + rot_dim, dtype=act(dtype), device=DEV)
    ops.latent_store(d, w, 1e-5, b.pos, b.row_seq, cos, sin, table, cache, rank, rot_dim, half_layout=True)
    # the same with the queries' latent taken from the columns behind, normed in the same kernel
    again = torch.zeros_like(cache)
    qw = (1.0 + 0.2 * torch.randn(7, generator=g)).to(DEV)
    q_lat = torch.zeros(b.n, 7, dtype=act(dtype), device=DEV)
    ops.latent_store(wide, w, 1e-5, b.pos, b.row_seq, cos, sin, table, again, rank, rot_dim, half_layout=True, q_latent=(qw, q_lat))
    assert torch.equal(again, cache)
    close(q_lat, P.unit_rms(wide[:, rank + rot_dim:].to(F64).cpu(), 1e-5) * qw.to(F64).cpu(), dtype, "the queries' latent")
    d64 = d.to(F64).cpu()
    want = torch.cat([P.unit_rms(d64[:, :rank], 1e-5) * w.to(F64).cpu(), P.rotate_half(d64[:, rank:], b.positions, rot)], 1)
    rows = [cache[int(table[int(b.row_seq[r]), p // page]), p % page] for r, p in enumerate(b.positions)]
    close(torch.stack(rows), want, dtype, "stored latent and rotated key part")
    # the queries' rotated parts, from [dim | rot_dim] per head into [rank | rot_dim] per head
    q = torch.randn(b.n, heads * (dim + rot_dim), generator=g).to(act(dtype)).to(DEV)
    out = torch.zeros(b.n, heads * (rank + rot_dim), dtype=act(dtype), device=DEV)
    ops.rotate_heads(q, heads, dim + rot_dim, dim, rot_dim, out, rank + rot_dim, rank, b.pos, cos, sin, half_layout=True)
    want_q = P.rotate_half(q.to(F64).cpu().reshape(b.n, heads, dim + rot_dim)[..., dim:], b.positions, rot)
    close(out.reshape(b.n, heads, rank + rot_dim)[..., rank:], want_q, dtype, "rotated query parts")
    assert float(out.reshape(b.n, heads, rank + rot_dim)[..., :rank].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,rows", [(50, 7), (256, 33), (1500, 4), (8, 1)])
def test_layer_norm_after_a_sublayer(dtype, width, rows):
    ops = ops_of(dtype)
    g = torch.Generator().manual_seed(width)
    d = (torch.randn(rows, width, generator=g) * 3.0 + 1.5).to(DEV)
    x0 = torch.randn(rows, width, generator=g).to(DEV)
    w = (0.7 * (1.0 + 0.2 * torch.randn(width, generator=g))).to(DEV)
    w2 = (1.0 + 0.2 * torch.randn(width, generator=g)).to(DEV)
    want_x = x0.to(F64).cpu() + P.layer_norm(d.to(F64).cpu(), w.to(F64).cpu(), 1e-5)
    x = x0.clone()
    ops.layernorm_residual(d, w, 1e-5, x)
    close(x, want_x, "float32", "stream after the norm")
    x = x0.clone()
    xn = torch.zeros(rows, width, dtype=act(dtype), device=DEV)
    ops.layernorm_residual(d, w, 1e-5, x, next_weight=w2, next_eps=1e-6, next_out=xn)
    close(x, want_x, "float32", "stream after the norm, with the next norm")
    close(xn, P.layer_norm(want_x, w2.to(F64).cpu(), 1e-6), dtype, "the next sublayer's input")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gates_gelu_step_and_cap(dtype):
    ops = ops_of(dtype)
    g = torch.Generator().manual_seed(5)
    for n, heads, vdim in [(9, 3, 20), (1, 1, 7), (40, 8, 16)]:
        v = torch.randn(n, heads * vdim, generator=g).to(act(dtype)).to(DEV)
        for group in (1, vdim):
            wide = (torch.randn(n, heads * vdim // group + 3, generator=g) * 3.0).to(DEV)
            logits = wide[:, 3:]                                   # columns of a wider product
            got = v.clone()
            ops.sigmoid_gate(got, logits, group)
            want = v.to(F64).cpu() * torch.sigmoid(logits.to(F64).cpu()).repeat_interleave(group, dim=1)
            close(got, want, dtype, f"gate per {'entry' if group == 1 else 'head'}")
    gate_up = (torch.randn(13, 2 * 37, generator=g) * 2.5).to(act(dtype)).to(DEV)
    h = torch.zeros(13, 37, dtype=act(dtype), device=DEV)
    ops.glu_gelu(gate_up, h)
    gu = gate_up.to(F64).cpu()
    close(h, P.gelu_tanh(gu[:, :37]) * gu[:, 37:], dtype, "gelu(gate) * up")
    z = (torch.randn(5, 301, generator=g) * 40.0).to(DEV)
    want = 7.5 * torch.tanh(z.to(F64).cpu() / 7.5)
    ops.softcap_rows(z, 7.5)
    close(z, want, "float32", "capped logits")
    assert float(z.abs().max()) <= 7.5


@pytest.mark.parametrize("m", [1, 8, 16, 40, 128, 300, 1100])
@pytest.mark.parametrize("width,inter", [(256, 320), (512, 1408), (64, 64)])
def test_gelu_in_the_epilogue_of_the_gate_and_up_product(m, width, inter):
    """The serving precision applies the gated step in the product's epilogue; the bits are those of the product
    followed by the stand-alone kernel, for steps of few rows, of a tile's rows and of many tiles."""
    ops = ops_of("bfloat16")
    assert ops.fuses_swiglu(width, inter, activation="gelu_tanh")
    g = torch.Generator().manual_seed(m + inter)
    x = torch.randn(m, width, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inter, width, generator=g) * 2.0 / math.sqrt(width)).to(torch.bfloat16).to(DEV)
    up = (torch.randn(inter, width, generator=g) / math.sqrt(width)).to(torch.bfloat16).to(DEV)
    fused = torch.zeros(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(x, ops.interleave_gate_up(gate, up), fused, activation="gelu_tanh")
    gate_up = torch.zeros(m, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, torch.cat([gate, up]).contiguous(), gate_up)
    apart = torch.zeros(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.glu_gelu(gate_up, apart)
    assert torch.equal(fused, apart)
    x64 = x.to(F64).cpu()
    want = P.gelu_tanh(to_bf16(x64 @ gate.to(F64).cpu().T)) * to_bf16(x64 @ up.to(F64).cpu().T)
    close(fused, want, "bfloat16", "gelu(gate) * up")
    silu = torch.zeros(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(x, ops.interleave_gate_up(gate, up), silu)          # the other activation is still itself
    g64 = to_bf16(x64 @ gate.to(F64).cpu().T)
    close(silu, g64 * torch.sigmoid(g64) * to_bf16(x64 @ up.to(F64).cpu().T), "bfloat16", "silu(gate) * up")


def run_latent_attention(ops, dtype, q, cache, table, batch, heads, rank, rot_dim, scale, sinks):
    out = torch.zeros(batch.n, heads * rank, dtype=act(dtype), device=DEV)
    ops.latent_attention(q, cache, table, out, heads, rank, rot_dim, scale, batch, 0, sinks=sinks)
    return out


def plain_latent_attention(q, keys_of_row, heads, rank, scale, sinks):
    """q: [n, heads, rank + rot]; keys_of_row[r]: [keys, rank + rot] (float64); the weighted sums of latents."""
    outs = []
    for r, keys in enumerate(keys_of_row):
        s = (q[r] @ keys.T) * scale
        p = P.softmax_rows(s[:, None, :], torch.ones(heads, 1, keys.shape[0], dtype=torch.bool),
                           sinks if sinks is not None else None)[:, 0, :]
        outs.append((p @ keys[:, :rank]).reshape(-1))
    return torch.stack(outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank,rot_dim", [(2, 48, 16), (3, 33, 6), (12, 136, 8), (5, 40, 8)])
@pytest.mark.parametrize("sink", [None, "learned", "high"])
def test_a_far_key_among_hundreds_and_the_sink(dtype, heads, rank, rot_dim, sink):
    """One sequence of 700 cached positions whose key at position 3 points along the queries, scaled so that its score
    stands out: it must carry most of the weight for rows of a prompt's portion and for single decoded rows (whose
    keys are spread over spans), among other sequences in the same step.  A sink near the largest score takes its share
    of the denominator; a sink far above it takes everything."""
    ops = ops_of(dtype)
    g = torch.Generator().manual_seed(heads * rank)
    dk, page, T = rank + rot_dim, 16, 700
    seqs_fill = [(0, T), (0, 260), (0, 300)]
    table = scattered_table(seqs_fill, page, g)
    cache = torch.zeros(int(table.max()) + 1, page, dk, dtype=act(dtype), device=DEV)
    keys = [torch.randn(n, dk, generator=g) * 0.5 for _, n in seqs_fill]
    direction = torch.randn(dk, generator=g)
    direction /= direction.norm()
    keys[0][3] = direction * 12.0
    for s, k in enumerate(keys):
        idx = torch.arange(k.shape[0])
        cache[table[s].long()[idx // page], idx % page] = k.to(act(dtype)).to(DEV)
    stored_keys = [cache[table[s].long()[torch.arange(k.shape[0]) // page], torch.arange(k.shape[0]) % page].to(F64).cpu()
                   for s, k in enumerate(keys)]
    scale = 0.5
    sinks = None
    if sink == "learned":
        sinks = torch.tensor([12.0 * 3.0 * scale * (0.8 + 0.05 * h) for h in range(heads)])
    elif sink == "high":
        sinks = torch.full((heads,), 60.0)
    sinks_dev = sinks.to(DEV) if sinks is not None else None
    for seqs in ([(680, 20), (85, 5), (0, 0)], [(699, 1), (89, 1), (299, 1)], [(3, 1), (40, 1), (256, 1)], [(0, 4), (255, 3), (290, 10)]):
        seqs = [(p0, n) for p0, n in seqs]
        live = [(s, p0, n) for s, (p0, n) in enumerate(seqs) if n]
        b = Batch([(p0, n) for _, p0, n in live])
        tbl = table[[s for s, _, _ in live]].contiguous()
        q = torch.randn(b.n, heads, dk, generator=g) * 0.3
        q += direction * 3.0                                    # every query looks for the marked key
        qd = q.reshape(b.n, heads * dk).to(act(dtype)).to(DEV)
        got = run_latent_attention(ops, dtype, qd, cache, tbl, b, heads, rank, rot_dim, scale, sinks_dev)
        q64 = qd.to(F64).cpu().reshape(b.n, heads, dk)
        keys_of_row = [stored_keys[live[int(b.row_seq[r])][0]][:p + 1] for r, p in enumerate(b.positions)]
        want = plain_latent_attention(q64, keys_of_row, heads, rank, scale, sinks.to(F64) if sinks is not None else None)
        close(got, want, dtype, f"rows {seqs}", factor=2.0)
        marked = stored_keys[0][3, :rank]
        first = [r for r in range(b.n) if int(b.row_seq[r]) == 0 and live[0][0] == 0 and b.positions[r] >= 3]
        if first and sink is None:
            share = (want[first[0]].reshape(heads, rank) @ marked) / (marked @ marked)
            assert float(share.min()) > 0.8, "the far key does not carry the weight"
        if sink == "high":
            assert float(got.abs().max()) < 1e-6


# ---------------------------------------------------------------------------------------------
def model_of(name, dtype):
    from bitwise_b200 import Model
    if (name, dtype) not in _models:
        _models[(name, dtype)] = Model.from_tensors(CONFIGS[name], random_weights(CONFIGS[name], WEIGHT_SEED), dtype=dtype, device=DEV)
    return _models[(name, dtype)]


def plain_pair(cfg, W, toks, collect=None):
    """The plain logits of one request, and the plain logits with everything rounded to bfloat16 that the serving
    precision stores in it: the second shows how large an error rounding alone causes for these weights."""
    exact = P.forward(cfg.to_json(), W, toks, collect).numpy()
    with P.rounding(to_bf16):
        rounded_ = P.forward(cfg.to_json(), W, toks).numpy()
    return exact, rounded_


def plain_logits(name, toks, rounded_too=False):
    key = (name, tuple(toks))
    if key not in _plain:
        _plain[key] = plain_pair(CONFIGS[name], random_weights(CONFIGS[name], WEIGHT_SEED), toks)
    return _plain[key] if rounded_too else _plain[key][0]


# lengths around the pages' (16), the key tiles' and spans' (32, 256) and the windows' edges of each configuration
LENGTHS = {"a": [70, 45, 5, 300, 64, 17, 1, 131], "b": [100, 9, 330, 1, 65, 33], "c": [40, 290, 3, 17, 132]}


def requests_of(name):
    return {f"{name}-{i}": tokens(CONFIGS[name], n, i) for i, n in enumerate(LENGTHS[name])}


def row_errors(got, want):
    """Per position: root mean square of the difference over that of the reference row."""
    return np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))


def assess(errors, dtype, what, rounding_alone=None):
    """float32: every position within the tolerance.  bfloat16: against the errors that rounding alone causes in the
    plain implementation for the same weights and tokens (``rounding_alone``, per position): the mean, the 95th
    percentile and the worst position may be twice to three times that and no more."""
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
    if dtype == "float32":                                   # the stream after every layer, for one request
        from bitwise_b200.engine.replay import make_replay_stepper
        from bitwise_b200.engine.step import StepEntry
        toks = reqs[f"{name}-1"]
        want = []
        P.forward(CONFIGS[name].to_json(), random_weights(CONFIGS[name], WEIGHT_SEED), toks, want)
        caught = []
        originals = [b.forward for b in model.decoder.blocks]
        try:
            for b, orig in zip(model.decoder.blocks, originals):
                b.forward = lambda ctx, x, cache, _o=orig: (_o(ctx, x, cache), caught.append(x.detach().clone()))
            make_replay_stepper(model, 384, use_graphs=False).run([StepEntry("r", toks, [])])
        finally:
            for b in model.decoder.blocks:
                del b.forward
        assert len(caught) == len(want)
        for i, (got, w) in enumerate(zip(caught, want)):
            close(got, w, "float32", f"stream after layer {i}", factor=4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cut_gives_the_same_logits(name, dtype):
    model = model_of(name, dtype)
    reqs = requests_of(name)
    vocab = CONFIGS[name].vocab
    whole = R.collect(R.whole(reqs), R.run_in_process(model, R.whole(reqs), 384), vocab)
    cuts = {"token by token": (R.tail_one_by_one(reqs, 40), 384), "portions": (R.portions(reqs), 384),
            "portions of two": (R.portions(reqs, sizes=(2,)), 384), "mixed": (R.mixed(reqs, 512, seed=7), 512),
            "mixed, a tight pool": (R.mixed(reqs, 400, seed=8, max_live=3), 400)}
    for what, (steps, pool) in cuts.items():
        got = R.collect(steps, R.run_in_process(model, steps, pool, max_live=4), vocab)
        compare(name, dtype, got)
        for rid in reqs:                                      # and against the whole prompt, beyond rounding nothing
            err = np.abs(got[rid] - whole[rid]).max() / np.abs(whole[rid]).max()
            assert err <= (1e-4 if dtype == "float32" else 0.08), (what, rid, err)


def window_model(dtype, size, conv):
    """One window layer whose query and key projections are the identity on the head's channels: a token whose
    embedding is large along one channel is looked for by another such token."""
    from bitwise_b200 import Model
    cfg = KezuvikConfig(vocab=40, width=32, eps=1e-5, residual_mult=1.0, logit_softcap=None, layers=(
        L(window(heads=2, kv_heads=1, dim=16, vdim=16, scale=2.0, conv=conv, size=size), 24),))
    W = random_weights(cfg, 5)
    eye = torch.zeros(16, 32)
    eye[:, :16] = torch.eye(16)
    W["l0.mix.q"], W["l0.mix.k"] = torch.cat([eye, eye]).to(torch.bfloat16), eye.to(torch.bfloat16)
    W["l0.mix.q.b"], W["l0.mix.k.b"] = torch.zeros(32).to(torch.bfloat16), torch.zeros(16).to(torch.bfloat16)
    W["l0.norm1"] = torch.ones(32).to(torch.bfloat16)
    if conv:
        for n in ("q", "k", "v"):                              # the last tap alone: the convolution passes its input on
            W[f"l0.mix.{n}.conv"][:, :-1] = 0
            W[f"l0.mix.{n}.conv"][:, -1] = 1
    W["embed"][38], W["embed"][39] = W["embed"][38] * 0.05, W["embed"][39] * 0.05
    W["embed"][38, 0], W["embed"][39, 0] = 1.0, 1.0
    return cfg, W, Model.from_tensors(cfg, W, dtype=dtype, device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size,conv", [(24, None), (16, 2), (33, None), (1, None), (130, 3)])
def test_a_key_just_inside_and_just_outside_the_window(dtype, size, conv):
    cfg, W, model = window_model(dtype, size, conv)
    total = 200
    base = [t % 38 for t in tokens(cfg, total, 1)]
    plain = list(base)
    plain[-1] = 39
    unmarked = P.forward(cfg.to_json(), W, plain)[-1].numpy()
    for tail in (0, 150):                                     # the last position in a prompt's portion, and decoded alone
        outs = {}
        for dist in (size - 1, size):                         # the last position that the window sees, and the next
            if dist == 0:
                continue                                      # (a window of one sees the position itself only)
            toks = list(plain)
            toks[total - 1 - dist] = 38
            want, rounded_ = plain_pair(cfg, W, toks)
            steps = R.tail_one_by_one({"r": toks}, tail=tail) if tail else R.portions({"r": toks}, sizes=(61, 2, 90, 47))
            got = R.collect(steps, R.run_in_process(model, steps, 256), cfg.vocab)["r"]
            assess([row_errors(got, want)], dtype, f"marked key at distance {dist}", [row_errors(rounded_, want)])
            outs[dist] = (want[-1], got[-1])
        want_out, got_out = outs[size]
        assert np.abs(want_out - unmarked).max() < 1e-9 * np.abs(unmarked).max() + 1e-9, "a key outside the window changed the logits"
        if size - 1 in outs:
            want_in, got_in = outs[size - 1]
            assert np.abs(want_in - unmarked).max() > 0.04 * np.abs(unmarked).max(), "the key inside the window did not decide"
            gap = np.abs(want_in - want_out).max()
            assert np.abs(got_in - want_in).max() < 0.25 * gap and np.abs(got_out - want_out).max() < 0.25 * gap


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_decides_in_a_latent_layer_after_long_decoding(dtype):
    """One latent layer whose projections pass the first channels on: the key of an early token whose embedding is large
    along one channel is what a last token of the same kind looks for, across hundreds of positions."""
    from bitwise_b200 import Model
    cfg = KezuvikConfig(vocab=40, width=32, eps=1e-5, residual_mult=0.8, logit_softcap=20.0, layers=(
        L(latent("latent_attention_2", heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=16, q_rank=16, scale=0.5, base=100.0), 24),))
    W = random_weights(cfg, 6)
    eye = torch.zeros(16, 32)
    eye[:, :16] = torch.eye(16)
    W["l0.mix.dq"] = eye.to(torch.bfloat16)
    W["l0.mix.dkv"] = torch.cat([eye, torch.zeros(8, 32)]).to(torch.bfloat16)           # no rotated key part
    uq = torch.zeros(2, 24, 16)
    uq[:, :16] = torch.eye(16)
    W["l0.mix.uq"], W["l0.mix.uk"] = uq.reshape(48, 16).to(torch.bfloat16), torch.cat([torch.eye(16)] * 2).to(torch.bfloat16)
    for n in ("l0.norm1", "l0.mix.dq.norm", "l0.mix.dkv.norm"):
        W[n] = torch.ones_like(W[n])
    W["l0.mix.sink"] = torch.tensor([2.0, -1.0]).to(torch.bfloat16)
    W["embed"][38], W["embed"][39] = W["embed"][38] * 0.05, W["embed"][39] * 0.05
    W["embed"][38, 0], W["embed"][39, 0] = 1.0, 1.0
    model = Model.from_tensors(cfg, W, dtype=dtype, device=DEV)
    base = [t % 38 for t in tokens(cfg, 600, 1)]
    toks = list(base)
    toks[2], toks[-1] = 38, 39
    plain = list(base)
    plain[-1] = 39
    want, rounded_ = plain_pair(cfg, W, toks)
    unmarked = P.forward(cfg.to_json(), W, plain)[-1].numpy()
    assert np.abs(want[-1] - unmarked).max() > 0.05 * np.abs(unmarked).max(), "the far key did not decide"
    for steps in (R.tail_one_by_one({"r": toks}, tail=330), R.portions({"r": toks}, sizes=(250, 2, 300, 31, 17))):
        got = R.collect(steps, R.run_in_process(model, steps, 640), cfg.vocab)["r"]
        assess([row_errors(got, want)], dtype, "a far key in a latent layer", [row_errors(rounded_, want)])
        assert np.abs(got[-1] - want[-1]).max() < 0.25 * np.abs(want[-1] - unmarked).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_reused_pages(dtype):
    # one request decoded token by token from position 3 to past 600 (pages, key tiles, spans and windows are crossed one
    # position at a time) while others come and go in the pool and in the slots
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
    W = random_weights(cfg, WEIGHT_SEED)
    for prompt, out in zip(prompts, got):
        assert len(out) == new
        seq = list(prompt)
        for t in out:
            row = P.forward(cfg.to_json(), W, seq)[-1].numpy()
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
    """``bitwise_b200 random`` writes a Kezuvik folder from a config.json; ``bin/trace_run`` replays a mixed schedule
    on it and ``bitwise_b200 generate`` decodes greedily: both as a user calls them, both against the plain
    implementation on the folder's own tensors."""
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
    W = {n: f.tensor(n).clone() for n in f.names()}
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
        want = P.forward(raw, W, toks).numpy()
        assert np.abs(got[rid] - want).max() <= 1e-4 * np.abs(want).max(), rid
    prompt = reqs["q3"]
    p = run(os.path.join(root, "bin", "bitwise_b200"), "generate", "--model", str(folder), "--dtype", "float32",
            "--max-new-tokens", "6", "--ignore-eos", "--temperature", "0", "--prompt-ids", ",".join(map(str, prompt)))
    assert p.returncode == 0, p.stderr[-2000:]
    seq = list(prompt)
    for t in json.loads(p.stdout.strip().split("\n")[0])["tokens"]:
        row = P.forward(raw, W, seq)[-1].numpy()
        assert t == int(row.argmax()) or row.max() - row[t] < 1e-4 * np.abs(row).max()
        seq.append(t)
