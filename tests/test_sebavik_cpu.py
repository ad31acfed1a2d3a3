"""Sebavik without a device: configuration, registry, declared tensors, run order, cache needs,
the plain implementation's own properties (one per mechanism), the cache manager's kept first
pages, and the engine's host side (pages, slots, the previous token, the convolutions' state and
the first mixing layer's values across steps) on the stand-in kernels."""
import json
import math

import numpy as np
import pytest
import torch

import plain_sebavik as P
import replay_patterns as R
from cpu_ops import CpuOps
from sebavik_configs import CONFIGS, EDGE_CONFIGS, as_float64, random_weights, tokens
from bitwise_b200 import Model
from bitwise_b200.cache import FREED, CacheManager, GroupSpec
from bitwise_b200.cache.manager import groups_from_needs
from bitwise_b200.config import ConfigError, architecture_of
from bitwise_b200.config.sebavik import SebavikConfig
from bitwise_b200.models.sebavik import build_sebavik
from bitwise_b200.parts import PagedKVNeed, SlotStateNeed


@pytest.mark.parametrize("name", sorted(CONFIGS) + sorted(EDGE_CONFIGS))
def test_config_round_trip_and_registry(name):
    cfg = CONFIGS.get(name) or EDGE_CONFIGS[name]
    raw = json.loads(json.dumps(cfg.to_json()))
    assert raw["architecture"] == "Sebavik"
    arch = architecture_of(raw)
    assert arch.name == "Sebavik"
    assert arch.config_from_json(raw) == cfg


def test_config_optional_keys_and_errors():
    base = CONFIGS["a"].to_json()
    # what the file leaves out does not exist: no second table, no convolution, no token input, no cap, no window
    d = json.loads(json.dumps(base))
    d["embedding"].pop("bigram"), d.pop("canon"), d.pop("token_side")
    d["layers"][0]["mixer"].pop("softcap"), d["layers"][0]["mixer"].pop("mask")
    cfg = SebavikConfig.from_json(d)
    assert cfg.bigram is None and cfg.canon_taps == 0 and cfg.side_dim == 0
    assert cfg.layers[0].mixer.softcap is None and cfg.layers[0].mixer.window is None and cfg.layers[0].mixer.keep_first == 0
    for change, word in [(lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
                         (lambda d: d["layers"][1].update(type="other"), "unknown type"),
                         (lambda d: d["layers"][0]["mlp"].update(kind="gated"), "not supported"),
                         (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "choices"),
                         (lambda d: d["layers"][1]["mlp"].pop("limit"), "limit"),
                         (lambda d: d["layers"][3]["mixer"].update(vdim=8), "mix their values"),
                         (lambda d: d["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
                         (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
                         (lambda d: d["norm"].pop("eps"), "eps"),
                         (lambda d: d.pop("width"), "width")]:
        d = json.loads(json.dumps(base))
        change(d)
        with pytest.raises(ConfigError, match=word):
            SebavikConfig.from_json(d)


def test_declared_tensors_run_order_and_cache_needs():
    cfg = CONFIGS["a"]
    model = build_sebavik(cfg)
    names = {s.name: s.shape for s in model.param_specs()}
    assert names["embed"] == (101, 64) and names["bigram"] == (54, 64) and names["side.embed"] == (101, 30)
    assert names["final.norm"] == (64,) and "head" not in names and "lm_head.weight" not in names
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mix.q.b"] == (64,) and names["l0.mix.v.b"] == (48,) and names["l0.mix.o"] == (64, 96)
    assert names["l0.mix.r1"] == (4,) and names["l0.mix.r2"] == (4,) and names["l0.mix.sink"] == (4,)
    assert "l0.mix.vmix" not in names and names["l1.mix.vmix"] == () and names["l3.mix.vmix"] == ()
    assert names["l0.mlp.router"] == (5, 64) and names["l0.mlp.e4.gate"] == (24, 64) and names["l0.mlp.e4.down"] == (64, 24)
    assert names["l1.mlp.gate"] == (96, 64) and names["l1.mlp.down"] == (64, 96)
    assert names["l0.canon1"] == (64, 3) and names["l0.canon2"] == (64, 3) and names["l0.ls2"] == (64,)
    assert names["l2.canon1"] == (64, 3) and "l2.canon2" not in names and "l2.norm2" not in names and "l2.ls2" not in names
    assert names["l0.dwa"] == (2,) and names["l4.dwa"] == (6,)
    assert names["l3.side.gate"] == (6, 64) and names["l3.side.proj"] == (64, 6) and names["l3.side.norm"] == (64,)
    # a stored tensor that the configuration leaves no use for is passed over when a folder is loaded
    assert model.ignorable_tensor("l2.norm2") and model.ignorable_tensor("l0.mix.vmix") and not model.ignorable_tensor("l0.norm2")
    # every layer owns pages and, with more than one tap, a state slot entry for both sublayers' last inputs
    runs = [(r.block, r.cache, r.owns_cache, r.state) for r in model.schedule]
    assert runs == [(0, 0, True, 1), (1, 2, True, 3), (2, 4, True, 5), (3, 6, True, 7), (4, 8, True, 9)]
    needs = model.cache_needs()
    assert needs[0] == PagedKVNeed(2, 16, 20, v_dim=24, keep_first=3) and needs[1] == SlotStateNeed((2, 128), torch.float32)
    assert needs[4] == PagedKVNeed(1, 8, None, v_dim=40) and needs[5] == SlotStateNeed((2, 64), torch.float32)
    assert needs[8] == PagedKVNeed(2, 16, 7, v_dim=24, keep_first=0)
    assert SlotStateNeed((1,), torch.int32) in needs          # the previous token
    groups = groups_from_needs(needs)
    assert [(g.window, g.keep_first, g.entries) for g in groups] == [(None, 0, (4,)), (7, 0, (8,)), (20, 3, (0, 6)), (33, 5, (2,))]
    assert model.graph_safe()
    # one tap is a factor per channel and needs no state; no second table: no previous token
    edge = build_sebavik(EDGE_CONFIGS["no_state"])
    assert not any(isinstance(n, SlotStateNeed) for n in edge.cache_needs())


def test_kept_first_pages_stay_while_the_window_passes():
    m = CacheManager([GroupSpec(20, (0,), 18)], [8], 16, 2)   # 18 kept keys: two pages
    m.begin("r")
    assert m.ensure("r", 100)
    m.advance("r", 90)            # the next query reads keys from 71 on: pages 0 .. 3 are passed, 0 and 1 are kept
    assert m.get("r").tables[0][:5] == [0, 1, FREED, FREED, 4]
    assert m.available(0) == 8 - 7 + 2
    m.begin("s")                  # the freed pages go to another request
    assert m.ensure("s", 40) and sorted(m.get("s").tables[0]) == [2, 3, 7]
    m.check_consistency()
    m.release("r")
    m.release("s")
    assert m.all_free()
    # kept keys that fill less than a page keep that page; none kept: none stays
    m = CacheManager([GroupSpec(5, (0,), 3), GroupSpec(5, (1,), 0)], [4, 4], 16, 1)
    m.begin("r")
    assert m.ensure("r", 64)
    m.advance("r", 60)
    assert m.get("r").tables[0] == [0, FREED, FREED, 3] and m.get("r").tables[1] == [FREED, FREED, FREED, 3]
    m.release("r")
    assert m.all_free()


# -- the plain implementation's own properties -------------------------------------------------
def test_plain_embedding_rows_of_the_second_table():
    assert P.pair_rows([5, 9, 9, 0], 7, 3, 2) == [7, (5 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7, (9 * 3) % 7]
    cfg = {"embedding": {"scale": 0.5, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 2}}}
    w = {"embed": np.arange(20.0).reshape(10, 2), "bigram": 100.0 + np.arange(16.0).reshape(8, 2)}
    x = P.embed_tokens(cfg, w, [5, 9])
    assert np.allclose(x[0], w["embed"][5] * 0.5 + w["bigram"][7]) and np.allclose(x[1], w["embed"][9] * 0.5 + w["bigram"][5])
    assert np.allclose(P.embed_tokens({"embedding": {}}, w, [3]), w["embed"][3])


def test_plain_convolution_over_time():
    rng = np.random.default_rng(0)
    h, c = rng.standard_normal((7, 3)), rng.standard_normal((3, 4))
    y = P.time_conv(h, c)
    assert np.allclose(y[0], h[0] + c[:, 3] * h[0])                              # zeros before the start
    assert np.allclose(y[5], h[5] + sum(c[:, j] * h[2 + j] for j in range(4)))
    assert np.allclose(P.time_conv(h, c[:, :1]), h * (1 + c[:, 0]))              # one tap: a factor per channel


def test_plain_window_kept_first_keys_sink_and_distance():
    assert [j for j in range(10) if P.visible(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(10) if P.visible(9, j, None, 0)] == list(range(10))
    assert [j for j in range(4) if P.visible(2, j, 1, 0)] == [2]
    rng = np.random.default_rng(1)
    q, k, v = rng.standard_normal((12, 2, 4)), rng.standard_normal((12, 1, 4)), rng.standard_normal((12, 1, 5))
    r1, r2, sink = np.array([0.5, -0.2]), np.array([1.5, 0.3]), np.array([0.7, -1.0])
    out = P.windowed_sink_attention(q, k, v, 0.3, None, r1, r2, sink, 3, 2)
    k2, v2 = k.copy(), v.copy()
    k2[2:7], v2[2:7] = 99.0, 99.0                 # position 9 sees 0, 1 and 7 .. 9
    out2 = P.windowed_sink_attention(q, k2, v2, 0.3, None, r1, r2, sink, 3, 2)
    assert np.allclose(out[9:], out2[9:]) and not np.allclose(out[8], out2[8])
    # position 0 sees itself and the sink: its weight is e^s / (e^s + e^sink); no distance term at distance 0
    s = float(q[0, 1] @ k[0, 0]) * 0.3
    assert np.allclose(out[0, 1], v[0, 0] * math.exp(s) / (math.exp(s) + math.exp(-1.0)))
    # zero queries: the weights are (1 + r2 d)^(-r1) over the visible keys, the sink counts once with exp(sink)
    flat = P.windowed_sink_attention(np.zeros_like(q), k, v, 0.3, 5.0, r1, r2, sink, None, 0)
    d = np.arange(11, -1, -1.0)
    wts = (1 + 1.5 * d) ** -0.5
    assert np.allclose(flat[11, 0], (wts[:, None] * v[:, 0]).sum(0) / (wts.sum() + math.exp(0.7)))
    # the cap bounds the product's part of a score, not the distance term and not the sink
    big = P.windowed_sink_attention(1e3 * q, k, v, 0.3, 0.01, r1, r2, sink, None, 0)
    assert np.abs(big[11, 0] - flat[11, 0]).max() < 0.05 * np.abs(v).max()
    # a very large sink takes all the weight
    gone = P.windowed_sink_attention(q, k, v, 0.3, None, r1, r2, np.array([60.0, 60.0]), 3, 2)
    assert np.abs(gone).max() < 1e-12


def test_plain_feed_forwards_router_and_mixing():
    rng = np.random.default_rng(2)
    z = np.array([[0.1, 2.0, -1.0, 2.0, 0.5]])
    chosen, weights = P.route(z, 3)
    assert chosen.tolist() == [[1, 3, 4]]          # the lower index first on a tie
    e = np.exp(np.array([2.0, 2.0, 0.5]) - 2.0)
    assert np.allclose(weights[0], e / e.sum()) and np.isclose(weights.sum(), 1.0)
    assert np.allclose(P.route(z, 1)[1], 1.0)
    # the dense feed-forward's clamps: the gate from above only, the other factor on both sides
    w = {"p.gate": np.eye(3), "p.up": np.eye(3), "p.down": np.eye(3)}
    h = np.array([[5.0, -5.0, 0.5]])
    y = P.dense_ff({"limit": 1.0}, w, "p", h)[0]
    sg = lambda g: g / (1 + math.exp(-1.702 * g))
    assert np.allclose(y, [sg(1.0) * 2.0, sg(-5.0) * 0.0, sg(0.5) * 1.5])
    assert np.allclose(P.mix_values(np.ones(3), np.zeros(3), 0.25), 0.75)
    hist = [rng.standard_normal((2, 3)) for _ in range(3)]
    assert np.allclose(P.depth_average(hist, [0.5, -1.0, 2.0]), 0.5 * hist[0] - hist[1] + 2 * hist[2])
    assert np.isclose(P.gelu_tanh(np.array(1.0)), 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715)))


def test_plain_forward_is_causal_and_uses_every_mechanism():
    cfg = CONFIGS["a"]
    W = as_float64(random_weights(cfg, 3))
    toks = tokens(cfg, 60, 1)
    full = P.forward(cfg.to_json(), W, toks)
    assert np.allclose(full[:41], P.forward(cfg.to_json(), W, toks[:41]))        # later tokens change nothing earlier
    # each tensor that only one mechanism reads changes the logits
    for name in ("bigram", "side.embed", "l4.mix.vmix", "l3.mix.sink", "l0.mix.r1", "l4.dwa", "l2.canon1", "l0.ls2", "l1.mix.k.b"):
        W2 = dict(W)
        W2[name] = W[name] + 0.5
        assert not np.allclose(full, P.forward(cfg.to_json(), W2, toks)), name
    W2 = dict(W)
    W2["l1.mix.vmix"] = np.array(0.9)             # the first mixing layer's own factor is idle
    assert np.allclose(full, P.forward(cfg.to_json(), W2, toks))
    W2["l3.mix.vmix"] = np.array(1.0)             # layer 3's values are then layer 1's: its own projection is idle
    W3 = dict(W2)
    W3["l3.mix.v"], W3["l3.mix.v.b"] = W["l3.mix.v"] * 0.0, W["l3.mix.v.b"] + 3.0
    assert np.allclose(P.forward(cfg.to_json(), W2, toks), P.forward(cfg.to_json(), W3, toks))


# -- the engine's host side on the stand-in kernels ---------------------------------------------
@pytest.mark.parametrize("name", sorted(CONFIGS) + sorted(EDGE_CONFIGS))
def test_every_cut_on_the_stand_in(name):
    cfg = CONFIGS.get(name) or EDGE_CONFIGS[name]
    W = random_weights(cfg, 3)
    model = Model.from_tensors(cfg, W, dtype="float32", device="cpu", ops=CpuOps("float32"))
    reqs = {f"{name}{i}": tokens(cfg, n, i) for i, n in enumerate([37, 70, 5, 1, 18])}
    want = {rid: P.forward(cfg.to_json(), as_float64(W), t) for rid, t in reqs.items()}
    for steps, pool in ((R.whole(reqs), 128), (R.tail_one_by_one(reqs, 9), 128), (R.portions(reqs, sizes=(3, 2, 11, 1)), 128),
                        (R.portions(reqs, sizes=(2,)), 128), (R.mixed(reqs, 192, seed=5), 192)):
        got = R.collect(steps, R.run_in_process(model, steps, pool), cfg.vocab)
        for rid in reqs:
            err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
            assert err < 2e-4, (rid, err)


def test_folder_round_trip_with_scalars_and_idle_tensors(tmp_path):
    """A random folder of the design is written and loaded again; a scalar tensor is stored like any other.  A folder
    may hold the tensors of sublayers that the configuration leaves out and the first mixing layer's idle factor, or
    lack that factor: both load, and give the same logits."""
    import os
    from bitwise_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = CONFIGS["a"]
    folder = Model.write_random_folder(str(tmp_path / "m"), cfg, seed=4, std=0.3, norm_jitter=0.2)
    stored = json.load(open(os.path.join(folder, "config.json")))
    assert {k: v for k, v in stored.items() if k != "torch_dtype"} == cfg.to_json()
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    assert tuple(tensors["l3.mix.vmix"].shape) == () and tuple(tensors["l4.dwa"].shape) == (6,)
    assert bool((tensors["l0.mix.r2"] >= 0).all())                       # the factor inside the logarithm
    toks = tokens(cfg, 40, 2)
    first = Model.load(folder, "float32", device="cpu", ops=CpuOps("float32")).logits(toks)
    want = P.forward(cfg.to_json(), as_float64(tensors), toks)
    assert np.abs(first - want).max() < 2e-4 * np.abs(want).max()
    tensors.pop("l1.mix.vmix", None)                                     # layer 1 is the first that mixes
    tensors["l0.mix.vmix"] = torch.tensor(0.5)                           # layer 0 does not mix at all
    tensors["l2.norm2"], tensors["l2.ls2"], tensors["l2.canon2"] = torch.ones(64), torch.ones(64), torch.zeros(64, 3)
    write_safetensors(path, list(tensors.items()))
    again = Model.load(folder, "float32", device="cpu", ops=CpuOps("float32")).logits(toks)
    assert np.array_equal(first, again)
