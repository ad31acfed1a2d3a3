"""Kezuvik without a device: configuration, registry, declared tensors, cache needs, the rotary tables with
rescaled frequencies, the plain implementation's own properties (one per mechanism), and the engine's host
side (pages that windows give back, slots with the convolutions' state, every cut) on the stand-in kernels."""
import json
import math

import numpy as np
import pytest
import torch

import plain_kezuvik as P
import replay_patterns as R
from cpu_ops import CpuOps
from kezuvik_configs import CONFIGS, random_weights, tokens
from bitwise_b200 import Model
from bitwise_b200.config import ConfigError, architecture_of
from bitwise_b200.config.kezuvik import KezuvikConfig
from bitwise_b200.models.kezuvik import build_kezuvik
from bitwise_b200.parts import PagedKVNeed, PagedLatentNeed, SlotStateNeed
from bitwise_b200.parts.rope import HalfRotaryEncoding, RampScaling

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_config_round_trip_and_registry(name):
    cfg = CONFIGS[name]
    raw = json.loads(json.dumps(cfg.to_json()))
    assert raw["architecture"] == "Kezuvik"
    arch = architecture_of(raw)
    assert arch.name == "Kezuvik"
    assert arch.config_from_json(raw) == cfg


def test_config_optional_keys_and_errors():
    base = CONFIGS["a"].to_json()
    d = json.loads(json.dumps(base))
    d.pop("logit_softcap"), d.pop("residual_mult")
    d["layers"][0]["mixer"].pop("conv"), d["layers"][0]["mixer"].pop("mask"), d["layers"][1]["mixer"]["rot"].pop("scaling")
    cfg = KezuvikConfig.from_json(d)
    assert cfg.logit_softcap is None and cfg.residual_mult == 1.0
    assert cfg.layers[0].mixer.conv is None and cfg.layers[0].mixer.window is None and cfg.layers[1].mixer.rot_scaling is None
    for change, word in [(lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
                         (lambda d: d["layers"][1].update(type="other"), "unknown type"),
                         (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "not supported"),
                         (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
                         (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
                         (lambda d: d["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
                         (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
                         (lambda d: d.update(logit_softcap=0.0), "logit_softcap"),
                         (lambda d: d["norm"].pop("eps"), "eps"),
                         (lambda d: d.pop("width"), "width")]:
        d = json.loads(json.dumps(base))
        change(d)
        with pytest.raises(ConfigError, match=word):
            KezuvikConfig.from_json(d)


def test_declared_tensors_and_cache_needs():
    cfg = CONFIGS["a"]
    model = build_kezuvik(cfg)
    specs = {s.name: tuple(s.shape) for s in model.param_specs()}
    assert specs["embed"] == (131, 64) and specs["final.norm"] == (64,) and "head" not in specs
    # the window layer: biased projections with taps, no norm weights, a gate per entry
    assert specs["l0.mix.q"] == (128, 64) and specs["l0.mix.k.b"] == (64,) and specs["l0.mix.v.conv"] == (32, 3)
    assert specs["l0.mix.g"] == (64, 64) and specs["l0.mix.o"] == (64, 64) and "l0.mix.q.norm" not in specs
    # the second latent kind: a sink and a gate per head; the first: a gate per entry and no sink
    assert specs["l1.mix.sink"] == (2,) and specs["l1.mix.g"] == (2, 64) and specs["l1.mix.dkv"] == (48 + 16, 64)
    assert specs["l1.mix.uq"] == (2 * 32, 40) and specs["l1.mix.dq.norm"] == (40,) and specs["l1.mix.dkv.norm"] == (48,)
    assert specs["l2.mix.g"] == (5 * 16, 64) and "l2.mix.sink" not in specs and specs["l2.mix.uv"] == (80, 40)
    # a layer without feed-forward has neither its norms nor its matrices
    assert "l3.norm2" not in specs and "l3.norm2b" not in specs and "l3.mlp.gate" not in specs and "l3.norm1b" in specs
    assert specs["l0.mlp.gate"] == (96, 64) and specs["l0.mlp.down"] == (64, 96)
    needs = model.cache_needs()
    assert needs == [PagedKVNeed(2, 32, 24, v_dim=16), SlotStateNeed((2, 128 + 64 + 32), torch.float32),
                     PagedLatentNeed(48, 16, None), PagedLatentNeed(40, 8, None),
                     PagedKVNeed(1, 16, 7, v_dim=32), SlotStateNeed((4, 32 + 16 + 32), torch.float32)]
    # one tap is a factor per channel and keeps no state; no taps at all neither
    assert [type(n).__name__ for n in build_kezuvik(CONFIGS["b"]).cache_needs()].count("SlotStateNeed") == 1
    assert all(not isinstance(n, SlotStateNeed) for n in build_kezuvik(CONFIGS["c"]).cache_needs())
    # the residual factor rides on the norm after the sublayer
    W = random_weights(cfg, 1)
    m = Model.from_tensors(cfg, W, dtype="float32", device="cpu", ops=CpuOps("float32"))
    blk = m.decoder.blocks[0]
    assert torch.allclose(blk.mixer_post.weight, W["l0.norm1b"].float() * 0.6)
    assert torch.allclose(blk.mixer_norm.weight, W["l0.norm1"].float())


@pytest.mark.parametrize("dims,base,sc", [(16, 5000.0, (4.0, 64.0, 8.0, 0.5)), (8, 10000.0, (8.0, 16.0, 1.0, 0.25)),
                                          (10, 777.0, (1.5, 32.0, 4.0, 2.0)), (32, 50000.0, (2.0, 2048.0, 32.0, 1.0)),
                                          (4, 50.0, None), (6, 1e6, (3.0, 1e9, 2.0, 1.0)), (6, 20.0, (3.0, 1.0, 64.0, 32.0))])
def test_rotary_tables_with_rescaled_frequencies(dims, base, sc):
    rot = {"dims": dims, "base": base}
    if sc:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
    enc = HalfRotaryEncoding(dims, base, RampScaling(*sc) if sc else None, positions=50)
    enc.reserve(300)                                              # grown in two pieces
    f, gain = P.rotary_frequencies(rot)
    assert np.allclose(enc.freq64, f, rtol=1e-13)
    p = np.arange(300)[:, None]
    cos, sin = enc._cos, enc._sin
    assert cos.shape == (300, dims // 2) and cos.dtype == np.float32
    assert np.abs(cos - np.cos(p * np.array(f)) * gain).max() < 1e-6 and np.abs(sin - np.sin(p * np.array(f)) * gain).max() < 1e-6
    if sc:
        # pairs before the ramp keep their frequency, pairs behind it are divided by the factor
        plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        assert all(a <= b * (1 + 1e-12) and a >= b / sc[0] * (1 - 1e-12) for a, b in zip(f, plain))
        assert math.isclose(gain, 0.1 * math.log(sc[0]) + 1.0)
    if sc == (3.0, 1e9, 2.0, 1.0):
        assert np.allclose(f, plain)                                # the ramp begins behind the last pair
    if sc == (3.0, 1.0, 64.0, 32.0):
        # the ramp is over before the first pair: all pairs but the one at its foot are divided
        assert np.allclose(f[1:], np.array(plain[1:]) / 3.0) and f[0] == plain[0]


def test_plain_rotation_in_the_half_layout():
    g = torch.Generator().manual_seed(0)
    v = torch.randn(9, 3, 12, generator=g, dtype=F64)
    rot = {"dims": 8, "base": 100.0}
    pos = list(range(20, 29))
    out = P.rotate_half(v, pos, rot)
    assert torch.equal(out[..., 8:], v[..., 8:])                                    # entries beyond dims pass
    for i in range(4):                                                              # pair i is (i, i + 4): lengths stay
        assert torch.allclose(out[..., i] ** 2 + out[..., i + 4] ** 2, v[..., i] ** 2 + v[..., i + 4] ** 2)
    assert torch.allclose(P.rotate_half(v, [0] * 9, rot), v)
    # a dot product of two turned vectors depends on the distance only
    a, b = torch.randn(1, 8, generator=g, dtype=F64), torch.randn(1, 8, generator=g, dtype=F64)
    d1 = (P.rotate_half(a, [7], rot) * P.rotate_half(b, [3], rot)).sum()
    d2 = (P.rotate_half(a, [104], rot) * P.rotate_half(b, [100], rot)).sum()
    assert torch.allclose(d1, d2)
    # with a rescaling both cos and sin carry the gain: lengths grow by it
    rot2 = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 16.0, "fast": 4.0, "slow": 0.5}}
    out2 = P.rotate_half(v, pos, rot2)
    gain = 0.1 * math.log(4.0) + 1.0
    assert torch.allclose(out2[..., 0] ** 2 + out2[..., 4] ** 2, gain ** 2 * (v[..., 0] ** 2 + v[..., 4] ** 2))


def test_plain_convolution_softmax_sink_and_window():
    g = torch.Generator().manual_seed(1)
    u = torch.randn(6, 3, generator=g, dtype=F64)
    w = torch.randn(3, 4, generator=g, dtype=F64)
    y = P.causal_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0])                                     # zeros before the start
    assert torch.allclose(y[5], w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4] + w[:, 3] * u[5])
    s = torch.randn(2, 5, 5, generator=g, dtype=F64)
    vis = torch.tril(torch.ones(5, 5, dtype=torch.bool))[None].expand(2, 5, 5)
    p = P.softmax_rows(s, vis)
    assert torch.allclose(p.sum(-1), torch.ones(2, 5, dtype=F64)) and bool((p[:, 0, 1:] == 0).all())
    sink = torch.tensor([0.3, -50.0], dtype=F64)
    ps = P.softmax_rows(s, vis, sink)
    e = torch.exp(s[0, 4])
    assert torch.allclose(ps[0, 4], e / (e.sum() + math.exp(0.3)))                   # the sink counts once, unscaled
    assert torch.allclose(ps[1], p[1])                                               # a sink far below changes nothing
    assert float(P.softmax_rows(s, vis, torch.tensor([60.0, 60.0], dtype=F64)).max()) < 1e-20
    assert math.isclose(float(P.gelu_tanh(torch.tensor(1.0, dtype=F64))), 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715)))


def test_plain_forward_is_causal_and_uses_every_mechanism():
    cfg = CONFIGS["a"]
    W = {k: v.to(F64) for k, v in random_weights(cfg, 3).items()}
    toks = tokens(cfg, 60, 1)
    raw = cfg.to_json()
    full = P.forward(raw, W, toks)
    assert torch.allclose(full[:41], P.forward(raw, W, toks[:41]))                 # later tokens change nothing earlier
    assert float(full.abs().max()) < 12.0                                          # the cap
    for name in ("l1.mix.sink", "l0.mix.g", "l1.mix.g", "l2.mix.g", "l0.mix.k.b", "l0.mix.v.conv", "l3.mix.q.conv", "l2.mix.dq.norm",
                 "l1.mix.dkv.norm", "l0.norm1b", "l2.norm2b", "final.norm", "l1.mlp.up"):
        W2 = dict(W)
        W2[name] = W[name] + 0.5
        assert not torch.allclose(full, P.forward(raw, W2, toks)), name
    # the window: position 59 of layer 3 (window 7) sees 53 .. 59; the first layer (window 24) 36 .. 59; the other layers all
    other = list(toks)
    other[0] = (toks[0] + 1) % cfg.vocab
    assert not torch.allclose(full[59], P.forward(raw, W, other)[59])               # the latent layers see the first token
    only_windows = json.loads(json.dumps(raw))
    only_windows["layers"] = [raw["layers"][0], raw["layers"][3]]
    W3 = {k.replace("l3.", "l1."): v for k, v in W.items() if not k.startswith(("l1.", "l2."))}
    a, b = P.forward(only_windows, W3, toks), P.forward(only_windows, W3, other)
    reach = (24 - 1) + (7 - 1) + (3 - 1) + (5 - 1)                                   # windows and convolutions of both layers
    assert torch.allclose(a[reach + 1:], b[reach + 1:]) and not torch.allclose(a[reach], b[reach])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cut_on_the_stand_in(name):
    cfg = CONFIGS[name]
    W = random_weights(cfg, 3)
    model = Model.from_tensors(cfg, W, dtype="float32", device="cpu", ops=CpuOps("float32"))
    reqs = {f"{name}{i}": tokens(cfg, n, i) for i, n in enumerate([37, 70, 5, 1, 18])}
    want = {rid: P.forward(cfg.to_json(), W, t).numpy() for rid, t in reqs.items()}
    for steps, pool in ((R.whole(reqs), 128), (R.tail_one_by_one(reqs, 9), 128), (R.portions(reqs, sizes=(3, 2, 11, 1)), 128),
                        (R.portions(reqs, sizes=(2,)), 128), (R.mixed(reqs, 192, seed=5), 192)):
        got = R.collect(steps, R.run_in_process(model, steps, pool), cfg.vocab)
        for rid in reqs:
            err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
            assert err < 2e-4, (rid, err)


def test_window_layers_give_pages_back_while_latent_layers_keep_theirs():
    from bitwise_b200.engine.replay import make_replay_stepper
    from bitwise_b200.engine.step import StepEntry
    cfg = CONFIGS["a"]
    model = Model.from_tensors(cfg, random_weights(cfg, 3), dtype="float32", device="cpu", ops=CpuOps("float32"))
    stepper = make_replay_stepper(model, 256, 16, max_live=2)
    toks = tokens(cfg, 200, 4)
    stepper.run([StepEntry("r", toks[:150], [149])])
    groups = stepper.manager.groups
    windows = sorted(g.window for g in groups if g.window)
    assert windows == [7, 24] and any(g.window is None for g in groups)
    from bitwise_b200.cache import FREED
    tables = stepper.manager.get("r").tables
    held = {g.window: sum(1 for p in tables[i] if p != FREED) for i, g in enumerate(groups)}
    assert held[None] == 10 and held[7] <= 2 and held[24] <= 3
    stepper.finish("r")
    assert stepper.manager.all_free()


def test_folder_round_trip(tmp_path):
    import os
    from bitwise_b200.weights.safetensors_io import SafetensorsFile
    cfg = CONFIGS["b"]
    folder = Model.write_random_folder(str(tmp_path / "m"), cfg, seed=4, std=0.3, norm_jitter=0.2)
    stored = json.load(open(os.path.join(folder, "config.json")))
    assert {k: v for k, v in stored.items() if k != "torch_dtype"} == cfg.to_json()
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    assert tuple(tensors["l2.mix.sink"].shape) == (3,) and tuple(tensors["l2.mix.g"].shape) == (3, 50)
    toks = tokens(cfg, 40, 2)
    got = Model.load(folder, "float32", device="cpu", ops=CpuOps("float32")).logits(toks)
    want = P.forward(stored, tensors, toks).numpy()
    assert np.abs(got - want).max() < 2e-4 * np.abs(want).max()
